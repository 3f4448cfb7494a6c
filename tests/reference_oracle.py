"""Loads the upstream reference model classes on CPU for parity tests.

The reference calls three GPU-only functions on its forward path (flash-attn, a Triton rotary
kernel and a Triton swiglu).  They are replaced here by dense PyTorch equivalents so the model
can run forward and backward on the CPU; nothing else is modified.  Tests that use this oracle
are skipped when the reference tree is not present.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

# the upstream checkout: TTCD_REFERENCE_ROOT, else a `reference` directory beside this repository
REFERENCE_ROOT = Path(os.environ.get("TTCD_REFERENCE_ROOT", str(Path(__file__).resolve().parents[2] / "reference")))


def available() -> bool:
    return (REFERENCE_ROOT / "custom_models").is_dir()


def _dense_flash_attn(q, k, v, causal=True, window_size=(-1, -1), **_):
    B, Tq, H, D = q.shape
    Tk, HK = k.shape[1], k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // HK, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // HK, 1)
    s = qf @ kf.transpose(-1, -2) * D ** -0.5
    i = torch.arange(Tq)[:, None] + (Tk - Tq)
    j = torch.arange(Tk)[None, :]
    mask = j <= i
    if window_size[0] >= 0:
        mask &= j >= i - window_size[0]
    s = s.masked_fill(~mask, float("-inf"))
    return (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3).to(q.dtype)


def load():
    """Returns the reference ``custom_models`` package with CPU-capable stand-ins installed."""
    # The reference owns the module name ``custom_models`` inside a test process (HF looks model
    # classes up through sys.modules); this repo's compat package of the same name is tested in
    # a subprocess.
    for k in [k for k in sys.modules if k == "custom_models" or k.startswith("custom_models.")]:
        if not str(getattr(sys.modules[k], "__file__", "")).startswith(str(REFERENCE_ROOT)):
            del sys.modules[k]
    sys.path.insert(0, str(REFERENCE_ROOT))
    try:
        import fla.layers.attn as fla_attn
        import fla.modules.rotary as fla_rotary
        import custom_models as ref_cm  # noqa: F401
        from custom_models.ipttcd import modeling_ipttcdv9 as m9
        from custom_models.ipttcd import modeling_ipttcdv9_lowcopy as m9l
        from custom_models.ipttcd import modeling_ipttcdv9_lowcopy_scanfuse as m9s
        from custom_models.ipttt import modeling_ipttt as mt
    finally:
        sys.path.remove(str(REFERENCE_ROOT))

    fla_attn.flash_attn_func = _dense_flash_attn

    def rotary_cpu(x, cos, sin, interleaved=False, seqlen_offsets=0, cu_seqlens=None, **_):
        T = x.shape[1]
        off = int(seqlen_offsets) if not torch.is_tensor(seqlen_offsets) else int(seqlen_offsets.max())
        return fla_rotary.rotary_embedding_ref(x, cos[off:off + T], sin[off:off + T], interleaved)

    fla_rotary.rotary_embedding = rotary_cpu
    for mod in (m9, m9l, m9s, mt):
        mod.swiglu = lambda a, b: F.silu(a) * b
        if hasattr(mod, "swiglu_linear"):
            mod.swiglu_linear = lambda a, b, w, bias=None: F.linear(F.silu(a) * b, w, bias)
    return dict(v9=m9s, v9_base=m9, v9_lowcopy=m9l, ipttt=mt, fla_attn=fla_attn)
