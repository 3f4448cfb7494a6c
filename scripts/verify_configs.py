"""Installation check: every model config JSON under ``configs/`` resolves to one of this package's model types
through ``transformers.AutoConfig``, and (with ``--build``) a shrunken copy of each family's model constructs and
runs one forward on CPU (reference scripts/verify_extract.py:23-53 checks its own registration the same way).

    python scripts/verify_configs.py            # prints a JSON summary, exits 1 on any failure
    python scripts/verify_configs.py --build
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

SHRINK = {"hidden_size": 64, "num_hidden_layers": 2, "num_heads": 4, "num_kv_heads": 2, "intermediate_size": 128,
          "vocab_size": 256, "max_position_embeddings": 512, "head_dim": 16}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--configs", default=str(ROOT / "configs"))
    ap.add_argument("--build", action="store_true", help="also build a shrunken model per model_type and run a forward")
    args = ap.parse_args(argv)
    import torch
    from transformers import AutoConfig

    import ttcd_b200.models as models
    from ttcd_b200.train.engine import build_model, load_model_config
    known = set(models.MODEL_CLASSES)
    report, failures, built = {}, [], {}
    for path in sorted(Path(args.configs).rglob("*.json")):
        rel = str(path.relative_to(args.configs))
        try:
            raw = json.loads(path.read_text())
            mtype = raw.get("model_type")
            if mtype not in known:
                report[rel] = {"model_type": mtype, "status": "not a model type of this package"}
                continue
            cfg = AutoConfig.from_pretrained(str(path))
            report[rel] = {"model_type": cfg.model_type, "class": type(cfg).__name__, "status": "ok"}
            if args.build and mtype not in built:
                small = {k: v for k, v in SHRINK.items() if hasattr(cfg, k)}
                if getattr(cfg, "ttt_layers", None):
                    small["ttt_layers"] = [1]
                for key in ("window_size", "window_size_student", "ttt_chunk"):
                    if isinstance(getattr(cfg, key, None), int):
                        small[key] = min(getattr(cfg, key), 32 if key != "ttt_chunk" else 16)
                model = build_model(load_model_config(str(path), **small), "cpu", torch.float32, seed=0)
                ids = torch.randint(0, small.get("vocab_size", 256), (1, 64))
                loss = model(input_ids=ids, labels=ids).loss
                built[mtype] = {"config": rel, "params": sum(p.numel() for p in model.parameters()), "loss": float(loss)}
        except Exception as e:  # noqa: BLE001  (report and continue with the next file)
            report[rel] = {"status": f"{type(e).__name__}: {e}"}
            failures.append(rel)
    print(json.dumps({"model_types": sorted(known), "configs": report, "built": built, "failures": failures}, indent=2))
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
