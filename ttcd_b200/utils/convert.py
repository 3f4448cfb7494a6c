"""Checkpoint conversion and merging tools (HF <-> DCP), same command lines as the reference.

* ``convert_hf_causal_lm_to_dcp``: HF Llama-family checkpoint (Qwen3 / SmolLM2 / Llama) -> this framework's
  parameter names -> DCP directory of raw keys (flame/utils/convert_qwen_to_ipttcd_dcp.py).  TTT-only
  parameters keep the target's initialisation; embeddings are resized by partial copy; a tied ``lm_head`` is
  written as its own tensor.
* ``convert_model_to_dcp`` / ``convert_dcp_to_hf``: generic round trip (flame/utils/convert_hf_to_dcp.py,
  convert_dcp_to_hf.py).
* ``convert_transformer_to_ipttcd_dcp``: copy a trained ``transformer`` checkpoint of this framework into an
  IP-TTCD model by equal keys (flame/utils/convert_transformer_to_ipttcdv3_dcp.py).
* ``merge_checkpoints``: SMA / EMA / WMA averaging over step checkpoints (flame/utils/checkpoint_merge.py).
"""
from __future__ import annotations

import json
import os
import re
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp

from ..train.checkpoint import checkpoint_keys, detect_model_prefix, load_model_weights
from ..train.engine import load_model_config

_HF_RULES: list[tuple[re.Pattern, str]] = [
    (re.compile(r"^model\.embed_tokens\.weight$"), "model.embeddings.weight"),
    (re.compile(r"^model\.norm\.weight$"), "model.norm.weight"),
    (re.compile(r"^lm_head\.weight$"), "lm_head.weight"),
    (re.compile(r"^model\.layers\.(\d+)\.self_attn\.([qkvo]_proj)\.(weight|bias)$"), r"model.layers.\1.attn.\2.\3"),
    (re.compile(r"^model\.layers\.(\d+)\.self_attn\.([qk]_norm)\.weight$"), r"model.layers.\1.attn.\2.weight"),
    (re.compile(r"^model\.layers\.(\d+)\.input_layernorm\.weight$"), r"model.layers.\1.attn_norm.weight"),
    (re.compile(r"^model\.layers\.(\d+)\.post_attention_layernorm\.weight$"), r"model.layers.\1.mlp_norm.weight"),
    (re.compile(r"^model\.layers\.(\d+)\.mlp\.(gate_proj|up_proj|down_proj)\.weight$"), r"model.layers.\1.mlp.\2.weight"),
]


def map_hf_key(key: str) -> str | None:
    """HF Llama-family parameter name -> this framework's name (None when there is no counterpart)."""
    for pattern, repl in _HF_RULES:
        if pattern.match(key):
            return pattern.sub(repl, key)
    return None


def _copy_resized(name: str, src: torch.Tensor, dst: torch.Tensor) -> bool:
    """Copy ``src`` into ``dst``; vocabulary matrices of different height are copied row-prefix-wise."""
    if src.shape == dst.shape:
        dst.copy_(src.to(dst.dtype))
        return True
    if name in ("model.embeddings.weight", "lm_head.weight") and src.dim() == 2 and src.shape[1] == dst.shape[1]:
        rows = min(src.shape[0], dst.shape[0])
        dst[:rows].copy_(src[:rows].to(dst.dtype))
        return True
    return False


def _build_target(config_path: str, vocab_size: int | None = None, dtype=torch.float32):
    from transformers import AutoModelForCausalLM
    cfg = load_model_config(config_path)
    if vocab_size is not None:
        cfg.vocab_size = max(cfg.vocab_size, vocab_size)
    torch.manual_seed(0)
    model = AutoModelForCausalLM.from_config(cfg).to(dtype)
    return cfg, model


def _raw_state_dict(model, untie: bool = True) -> dict[str, torch.Tensor]:
    sd = {k: v.detach().clone() for k, v in model.state_dict().items() if "rotary" not in k}
    if untie and "lm_head.weight" not in sd:
        sd["lm_head.weight"] = sd["model.embeddings.weight"].clone()
    return sd


def save_raw_dcp(state_dict: dict[str, torch.Tensor], checkpoint: str, thread_count: int = 8) -> None:
    os.makedirs(checkpoint, exist_ok=True)
    dcp.save(state_dict, storage_writer=dcp.FileSystemWriter(checkpoint, thread_count=thread_count), no_dist=True)


def convert_hf_causal_lm_to_dcp(model: str, config: str, checkpoint: str, tokenizer: str | None = None,
                                source_state_dict: dict | None = None) -> dict:
    """HF checkpoint ``model`` -> target built from ``config`` -> DCP at ``checkpoint``.  Returns a report."""
    vocab = None
    if tokenizer:
        from transformers import AutoTokenizer
        vocab = len(AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=True))
    if source_state_dict is None:
        from transformers import AutoModelForCausalLM
        src_model = AutoModelForCausalLM.from_pretrained(model, torch_dtype=torch.float32)
        source_state_dict = src_model.state_dict()
    cfg, target = _build_target(config, vocab)
    tgt_sd = target.state_dict()
    copied, skipped = [], []
    with torch.no_grad():
        for key, tensor in source_state_dict.items():
            name = map_hf_key(key)
            if name is None or name not in tgt_sd or not _copy_resized(name, tensor, tgt_sd[name]):
                if name == "lm_head.weight" and getattr(cfg, "tie_word_embeddings", False):
                    continue
                skipped.append(key)
                continue
            copied.append(name)
        if getattr(cfg, "ttt_output_use_teacher_conv", False):
            # continued training starts from an exact copy of the base model: the teacher conv that feeds
            # the output path must be the identity tap
            for m in target.modules():
                conv = getattr(m, "ttt_teacher_conv", None)
                if conv is not None:
                    conv.weight.zero_()
                    tap = conv.kernel_size[0] - 1 if conv.padding[0] == 0 else conv.kernel_size[0] // 2
                    conv.weight[:, 0, tap] = 1.0
    sd = _raw_state_dict(target)
    if "lm_head.weight" in source_state_dict and not getattr(cfg, "tie_word_embeddings", False):
        pass
    save_raw_dcp(sd, checkpoint)
    untouched = sorted(set(tgt_sd) - set(copied))
    return {"copied": len(copied), "skipped_source_keys": skipped, "target_only_keys": untouched, "checkpoint": checkpoint}


def convert_model_to_dcp(model: str, checkpoint: str) -> None:
    """A saved model of this framework (``save_pretrained`` directory) -> DCP of raw keys."""
    from transformers import AutoModelForCausalLM
    m = AutoModelForCausalLM.from_pretrained(model)
    save_raw_dcp(_raw_state_dict(m), checkpoint)


def convert_dcp_to_hf(path: str, step: int | None, config: str, tokenizer: str | None = None, output: str | None = None) -> str:
    """DCP checkpoint (either key convention) -> ``save_pretrained`` directory."""
    ckpt = os.path.join(path, "checkpoint", f"step-{step}") if step is not None else path
    cfg, model = _build_target(config)
    load_model_weights(model, ckpt)
    out = output or path
    model.save_pretrained(out, safe_serialization=True)
    if tokenizer:
        from transformers import AutoTokenizer
        AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=True).save_pretrained(out)
    return out


def convert_transformer_to_ipttcd_dcp(source: str, config: str, checkpoint: str, tokenizer: str | None = None) -> dict:
    """Equal-key copy of a ``transformer`` checkpoint (HF dir or DCP) into an IP-TTCD model, saved as DCP."""
    vocab = None
    if tokenizer:
        from transformers import AutoTokenizer
        vocab = len(AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=True))
    cfg, target = _build_target(config, vocab)
    tgt_sd = target.state_dict()
    if os.path.isfile(os.path.join(source, ".metadata")):
        keys = checkpoint_keys(source)
        prefix = detect_model_prefix(keys)
        wanted = {prefix + k: torch.empty_like(v) for k, v in tgt_sd.items() if prefix + k in keys}
        dcp.load(wanted, checkpoint_id=source, no_dist=True)
        src_sd = {k[len(prefix):]: v for k, v in wanted.items()}
    else:
        from transformers import AutoModelForCausalLM
        src_sd = AutoModelForCausalLM.from_pretrained(source).state_dict()
    copied = []
    with torch.no_grad():
        for k, v in src_sd.items():
            if k in tgt_sd and _copy_resized(k, v, tgt_sd[k]):
                copied.append(k)
    save_raw_dcp(_raw_state_dict(target), checkpoint)
    return {"copied": len(copied), "target_only_keys": sorted(set(tgt_sd) - set(copied))}


def merge_weights(steps: list[int], merge_type: str, alpha: float = 0.9) -> list[float]:
    """Averaging coefficients over ``sorted(steps)``: simple, exponential, or LR-weighted moving average."""
    steps = sorted(steps)
    n = len(steps)
    if merge_type == "sma":
        return [1.0 / n] * n
    if merge_type == "ema":
        return [(alpha if i > 0 else 1.0) * (1.0 - alpha) ** (n - i - 1) for i in range(n)]
    if merge_type == "wma":
        total, start = max(steps), min(steps)
        span = total - start + 1

        def ratio(s: int) -> float:
            if s < start:
                return 1.0
            if s >= total:
                return alpha
            return 1.0 + (alpha - 1.0) * (s - start) / (span - 1)

        w = []
        for i in range(1, n):
            w.append(ratio(steps[i]) if i == n - 1 else ratio(steps[i]) - ratio(steps[i + 1]))
        return [1.0 - sum(w)] + w
    raise ValueError(f"unknown merge type {merge_type!r}")


def merge_checkpoints(path: str, output_path: str, steps: list[int], weights: list[float], config: str,
                      tokenizer: str | None = None, only_mlp: bool = False) -> str:
    """Weighted average of step checkpoints (optionally only the MLP tensors; the rest from the last step)."""
    steps = sorted(steps)
    cfg, model = _build_target(config)
    acc: dict[str, torch.Tensor] = {}
    for step, w in zip(steps, weights):
        load_model_weights(model, os.path.join(path, "checkpoint", f"step-{step}"))
        for k, v in model.state_dict().items():
            if only_mlp and ".mlp." not in k:
                acc[k] = v.detach().float().clone()           # last step wins
            else:
                acc[k] = acc.get(k, 0) + v.detach().float() * w
    with torch.no_grad():
        for k, v in model.state_dict().items():
            v.copy_(acc[k].to(v.dtype))
    model.save_pretrained(output_path, safe_serialization=True)
    if tokenizer:
        from transformers import AutoTokenizer
        AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=True).save_pretrained(output_path)
    Path(output_path, "merge_info.json").write_text(json.dumps({"steps": steps, "weights": weights, "only_mlp": only_mlp}))
    return output_path


def strip_legacy_buffers(state_dict: dict) -> dict:
    """Drop ``*.ttt_lr`` buffers written by old checkpoints (flame/utils/legacy_state_dict.py)."""
    return {k: v for k, v in state_dict.items() if not k.endswith(".ttt_lr")}
