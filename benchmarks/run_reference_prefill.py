"""Runs the reference project's own prefill benchmark (profiling/bench_prefill.py, unmodified) on this GPU.

The reference checkout is looked up as ``TTCD_REFERENCE_ROOT``, a ``reference`` directory beside this repository, or
``baseline/_ref`` (its installed packages plus a copy of its ``profiling`` directory).  Every argument is handed to
the reference script as is, e.g.

    python benchmarks/run_reference_prefill.py --config configs/ipttcd/ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k.json \
        --name v9 --seqlens 65536 --modes eval_nomask_cache train_fwd --patch none
    python benchmarks/run_reference_prefill.py ... --patch fused_conv      # its fused Triton attention + Triton conv

One setting is applied before the script starts: under transformers >= 5 the upstream classes' list-form
``_tied_weights_keys`` raises in ``post_init``; the equivalent dict form is set on the classes (no computation changes).
"""
from __future__ import annotations

import os
import runpy
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def reference_root() -> Path | None:
    for c in (os.environ.get("TTCD_REFERENCE_ROOT"), str(ROOT.parent / "reference"), str(ROOT / "baseline" / "_ref")):
        if c and (Path(c) / "profiling" / "bench_prefill.py").is_file() and (Path(c) / "custom_models").is_dir():
            return Path(c)
    return None


def main():
    root = reference_root()
    if root is None:
        raise SystemExit("reference checkout with profiling/bench_prefill.py not found")
    sys.path[:0] = [str(root), str(root / "profiling")]
    for k in [k for k in sys.modules if k.split(".")[0] in ("custom_models", "flame", "fla")]:
        del sys.modules[k]
    import custom_models  # noqa: F401  (registers the upstream model types)
    import transformers
    if int(transformers.__version__.split(".")[0]) >= 5:
        from transformers import PreTrainedModel
        for mod_name, mod in list(sys.modules.items()):
            if not mod_name.startswith(("custom_models", "fla.models")):
                continue
            for obj in vars(mod).values():
                if isinstance(obj, type) and issubclass(obj, PreTrainedModel) and isinstance(
                        obj.__dict__.get("_tied_weights_keys"), (list, tuple)):
                    obj._tied_weights_keys = {"lm_head.weight": "model.embeddings.weight"}
    script = root / "profiling" / "bench_prefill.py"
    sys.argv = [str(script), *sys.argv[1:]]
    runpy.run_path(str(script), run_name="__main__")


if __name__ == "__main__":
    main()
