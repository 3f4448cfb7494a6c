"""Shared pieces of the evaluation scripts: model loading (HF directory, or config JSON + DCP checkpoint in
either key convention — training checkpoints prefix keys with ``model.``, step-0 conversions do not;
reference scripts/eval_niah.py:79-110), RoPE-scaling overrides, and a greedy decoder that drives the
model's own prefill + windowed KV cache (reference scripts/eval_ruler.py:145-178)."""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def add_model_args(ap):
    ap.add_argument("--config", default=None, help="model config JSON (with --checkpoint)")
    ap.add_argument("--checkpoint", default=None, help="DCP checkpoint directory")
    ap.add_argument("--hf_model", default=None, help="save_pretrained directory (instead of --config/--checkpoint)")
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--rope_scaling_type", default=None, help="e.g. yarn / linear / dynamic")
    ap.add_argument("--rope_scaling_factor", type=float, default=None)
    ap.add_argument("--rope_scaling_original_max_pos", type=int, default=None)


def load_model(args, dtype=torch.bfloat16):
    import ttcd_b200.models  # noqa: F401  (registers the model types)
    from ttcd_b200.train.checkpoint import load_model_weights
    from ttcd_b200.train.engine import build_model, load_model_config
    overrides = {}
    if args.rope_scaling_type:
        scaling = {"rope_type": args.rope_scaling_type, "factor": args.rope_scaling_factor or 1.0}
        if args.rope_scaling_original_max_pos:
            scaling["original_max_position_embeddings"] = args.rope_scaling_original_max_pos
        overrides["rope_scaling"] = scaling
    device = torch.device(args.device)
    if args.hf_model:
        from transformers import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(args.hf_model, torch_dtype=dtype, **overrides)
    else:
        if not (args.config and args.checkpoint):
            raise SystemExit("give --hf_model, or --config and --checkpoint")
        cfg = load_model_config(args.config, **overrides)
        model = build_model(cfg, "cpu", torch.float32, seed=0)
        missing = load_model_weights(model, args.checkpoint)
        if missing:
            print(f"[eval] {len(missing)} tensors not in the checkpoint (kept at init): {missing[:4]} ...")
    if device.type == "cpu":
        dtype = torch.float32
    return model.to(device=device, dtype=dtype).eval()


def load_tokenizer(path: str):
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(path, trust_remote_code=True)


@torch.no_grad()
def greedy_decode(model, input_ids: torch.Tensor, max_new_tokens: int, eos_ids: set[int] | None = None,
                  use_graph: bool = True) -> list[int]:
    """Batch-1 greedy decoding through the model's own ``generate`` (one prefill with the cache, then one token per
    step: a replayed CUDA graph on the native path unless ``use_graph`` is off); the tokens before the first
    end-of-sequence token are returned."""
    tokens = model.generate(input_ids, max_new_tokens=max_new_tokens, do_sample=False,
                            eos_token_id=sorted(eos_ids) if eos_ids else None, use_graph=use_graph)
    produced: list[int] = []
    for tok in tokens[0, input_ids.shape[1]:].tolist():
        if eos_ids and tok in eos_ids:
            break
        produced.append(tok)
    return produced


@torch.no_grad()
def token_nll(model, input_ids: torch.Tensor, chunk: int = 512) -> torch.Tensor:
    """Per-position negative log-likelihood [B, T-1], log-softmax taken 512 positions at a time
    (reference scripts/eval_token_ppl.py:163-207)."""
    logits = model(input_ids=input_ids, use_cache=False).logits[:, :-1]
    targets = input_ids[:, 1:]
    nll = torch.empty(targets.shape, dtype=torch.float32, device=input_ids.device)
    for c0 in range(0, targets.shape[1], chunk):
        lp = torch.log_softmax(logits[:, c0:c0 + chunk].float(), dim=-1)
        nll[:, c0:c0 + chunk] = -lp.gather(-1, targets[:, c0:c0 + chunk, None]).squeeze(-1)
    return nll
