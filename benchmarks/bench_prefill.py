"""Prefill / forward benchmark of a random-weight model built from a config JSON.

Modes, ablations, overrides and the timing protocol are those of the reference harness
(profiling/bench_prefill.py:111-195, 362-364): inputs ``randint(0, vocab, (B, L))`` with seed 1234, bf16,
CUDA events, median of ``--iters`` after ``--warmup``.

    python benchmarks/bench_prefill.py --config configs/ipttcd/ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k.json \
        --seq-len 65536 --batch 1 --modes eval_nomask_cache,train_fwd --ablation full --attn-impl fused

* modes: ``eval_mask_cache`` (mask of ones + KV cache + last-position logits), ``eval_nomask_cache``,
  ``eval_nocache``, ``train_fwd`` (training-mode forward, no grad), ``gen1`` (generate one token), ``gen64`` /
  ``gen64_eager`` (generate 64 tokens with the captured decode step / the eager loop; with ``gen1`` in the same run a
  ``decode`` row reports (gen64 - gen1) / 63 as ms per token), ``eval_ppl_style`` (all logits + 512-token chunked NLL).
* ablations: ``full``, ``no_ttt`` (blocks and MLPs treated as non-TTT: single attention), ``attn_only`` (dual
  attention kept, fast-weight scan off).
* ``--attn-impl fused|two_pass``: the one-pass dual-window kernel or two single-window calls (what the
  reference does without its patches).  The reference's other monkey patches (shared QKV, fused gate/up,
  Triton conv) have no switch here: those fusions are the only implementation.
* ``--override k=v`` edits config fields (JSON values).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

MODES = ("eval_mask_cache", "eval_nomask_cache", "eval_nocache", "train_fwd", "gen1", "gen64", "gen64_eager", "eval_ppl_style")


def apply_ablation(model, ablation: str) -> None:
    if ablation == "full":
        return
    if ablation not in ("no_ttt", "attn_only"):
        raise ValueError(f"unknown ablation {ablation!r}")
    for blk in model.model.layers:
        if ablation == "no_ttt" and hasattr(blk, "is_ttt_layer"):
            blk.is_ttt_layer = False
        if hasattr(blk, "mlp") and hasattr(blk.mlp, "is_ttt_layer"):
            blk.mlp.is_ttt_layer = False


@torch.no_grad()
def run_mode(model, input_ids, mode: str, iters: int, warmup: int) -> dict:
    dev = input_ids.device
    b, L = input_ids.shape

    def call():
        if mode == "eval_mask_cache":
            model.eval()
            return model(input_ids=input_ids, attention_mask=torch.ones(b, L, dtype=torch.long, device=dev), use_cache=True,
                         logits_to_keep=1)
        if mode == "eval_nomask_cache":
            model.eval()
            return model(input_ids=input_ids, use_cache=True, logits_to_keep=1)
        if mode == "eval_nocache":
            model.eval()
            return model(input_ids=input_ids, use_cache=False, logits_to_keep=1)
        if mode == "train_fwd":
            model.train()
            out = model(input_ids=input_ids, use_cache=False, logits_to_keep=1)
            model.eval()
            return out
        if mode == "gen1":
            model.eval()
            return model.generate(input_ids, max_new_tokens=1, do_sample=False)
        if mode in ("gen64", "gen64_eager"):
            model.eval()
            return model.generate(input_ids, max_new_tokens=64, do_sample=False, use_graph=mode == "gen64")
        if mode == "eval_ppl_style":
            model.eval()
            logits = model(input_ids=input_ids).logits[:, :-1]
            targets = input_ids[:, 1:]
            nll = torch.empty(targets.shape, dtype=torch.float32, device=dev)
            for c0 in range(0, targets.shape[1], 512):
                lp = torch.log_softmax(logits[:, c0:c0 + 512].float(), dim=-1)
                nll[:, c0:c0 + 512] = -lp.gather(-1, targets[:, c0:c0 + 512, None]).squeeze(-1)
            return nll.mean()
        raise ValueError(mode)

    for _ in range(warmup):
        call()
    torch.cuda.synchronize(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    times = []
    for _ in range(iters):
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        call()
        e.record()
        torch.cuda.synchronize(dev)
        times.append(a.elapsed_time(e))
    times.sort()
    med = times[len(times) // 2]
    return {"ms_median": round(med, 3), "ms_min": round(times[0], 3), "ms_max": round(times[-1], 3),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 1e9, 2), "tok_per_s": round(b * L / (med / 1e3))}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default=str(ROOT / "configs/ipttcd/ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k.json"))
    ap.add_argument("--seq-len", type=int, default=65536)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--modes", default="eval_nomask_cache")
    ap.add_argument("--ablation", default="full", choices=["full", "no_ttt", "attn_only"])
    ap.add_argument("--attn-impl", default="fused", choices=["fused", "two_pass"])
    ap.add_argument("--override", action="append", default=[], help="config field override k=v (JSON value)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--out", default=None, help="write the result rows to this JSON file")
    args = ap.parse_args(argv)

    from ttcd_b200 import ops
    from ttcd_b200.train.engine import build_model, load_model_config
    overrides = {}
    for item in args.override:
        k, _, v = item.partition("=")
        try:
            overrides[k] = json.loads(v)
        except json.JSONDecodeError:
            overrides[k] = v
    cfg = load_model_config(args.config, **overrides)
    if getattr(cfg, "max_position_embeddings", 0) < args.seq_len:
        cfg.max_position_embeddings = args.seq_len
    model = build_model(cfg, "cuda", torch.bfloat16, seed=0).eval()
    apply_ablation(model, args.ablation)
    ops.set_dual_attention_impl(args.attn_impl)
    g = torch.Generator().manual_seed(1234)
    input_ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq_len), generator=g).cuda()
    rows = []
    for mode in [m for m in args.modes.split(",") if m]:
        if mode not in MODES:
            raise SystemExit(f"unknown mode {mode!r}; choose from {MODES}")
        res = run_mode(model, input_ids, mode, args.iters, args.warmup)
        row = {"bench": "prefill", "mode": mode, "ablation": args.ablation, "attn_impl": args.attn_impl, "B": args.batch,
               "L": args.seq_len, "model": Path(args.config).stem, **res}
        print(json.dumps(row), flush=True)
        rows.append(row)
    by_mode = {r["mode"]: r for r in rows}
    for mode in ("gen64", "gen64_eager"):
        if mode in by_mode and "gen1" in by_mode:
            row = {"bench": "decode", "mode": mode, "B": args.batch, "L": args.seq_len, "model": Path(args.config).stem,
                   "ms_per_token": round((by_mode[mode]["ms_median"] - by_mode["gen1"]["ms_median"]) / 63, 3)}
            print(json.dumps(row), flush=True)
            rows.append(row)
    if args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
