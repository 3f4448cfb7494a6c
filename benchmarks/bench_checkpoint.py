"""Prefill / generate timing and attention-implementation A/B on a trained checkpoint with real prompts
(reference profiling/bench_real_ckpt.py:41-88 and profiling/ab_niah_fused.py:17-31).

Prompts come from a RULER-style ``validation.jsonl`` (``input`` [+ ``answer_prefix``], ``outputs``); the first one is a
warm-up.  Per prompt: one prefill with the cache and last-position logits, then greedy generation of ``--max_new``
tokens through the same decoder the evaluation scripts use.  With ``--ab`` the run is repeated with the dual-window
attention computed by two single-window calls instead of the fused kernel and the two sets of predictions are
compared (accuracy of each, number of identical strings).

    python benchmarks/bench_checkpoint.py --config cfg.json --checkpoint exp/run/checkpoint/step-10000 \
        --tokenizer tokenizers/Qwen3-0.6B-Base --data data/niah/qwen3/ctx65536/niah_single_1/validation.jsonl --n 8 --ab
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "scripts"))


def timed(fn, device):
    """(milliseconds, result): CUDA events on a GPU, wall clock on the host."""
    if device.type == "cuda":
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        a.record()
        out = fn()
        b.record()
        torch.cuda.synchronize(device)
        return a.elapsed_time(b), out
    import time
    t0 = time.perf_counter()
    out = fn()
    return (time.perf_counter() - t0) * 1e3, out


def load_prompts(path: str, n: int):
    prompts, refs = [], []
    with open(path) as f:
        for line in f:
            d = json.loads(line)
            prompts.append(d["input"] + (d.get("answer_prefix") or ""))
            refs.append(d.get("outputs", []))
            if len(prompts) >= n + 1:
                break
    return prompts, refs


@torch.no_grad()
def run(model, tok, prompts, refs, max_new: int, device, tag: str) -> dict:
    from eval_common import greedy_decode
    from eval_ruler import string_match_all
    eos = {tok.eos_token_id} if tok.eos_token_id is not None else None
    prefill, gen, lens, preds = [], [], [], []
    for i, prompt in enumerate(prompts):
        ids = tok(prompt, return_tensors="pt", add_special_tokens=False).input_ids.to(device)
        ms_p, _ = timed(lambda: model(input_ids=ids, use_cache=True, logits_to_keep=1), device)
        ms_g, out = timed(lambda: greedy_decode(model, ids, max_new, eos), device)
        if i == 0:
            continue                                  # warm-up prompt
        prefill.append(ms_p)
        gen.append(ms_g)
        lens.append(int(ids.shape[1]))
        preds.append(tok.decode(out, skip_special_tokens=True))
        print(f"[{tag}] prompt {i}: L={ids.shape[1]} prefill {ms_p:.1f} ms, prefill+{max_new} tokens {ms_g:.1f} ms", flush=True)
    med = lambda v: sorted(v)[len(v) // 2]  # noqa: E731
    res = {"tag": tag, "prefill_ms": prefill, "generate_ms": gen, "tokens": lens, "max_new": max_new, "predictions": preds,
           "accuracy": string_match_all(preds, refs[1:1 + len(preds)])}
    if prefill:
        res.update(median_prefill_ms=med(prefill), median_generate_ms=med(gen),
                   decode_ms_per_token=(med(gen) - med(prefill)) / max(1, max_new))
        print(f"[{tag}] median prefill {res['median_prefill_ms']:.1f} ms, decode {res['decode_ms_per_token']:.2f} ms/token, "
              f"accuracy {res['accuracy']:.1f}", flush=True)
    return res


def main(argv=None):
    from eval_common import add_model_args, load_model, load_tokenizer
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_model_args(ap)
    ap.add_argument("--data", required=True, help="validation.jsonl with `input` / `answer_prefix` / `outputs`")
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--max_new", type=int, default=64)
    ap.add_argument("--ab", action="store_true", help="repeat with two single-window attention calls and compare")
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from ttcd_b200 import ops
    device = torch.device(args.device)
    tok = load_tokenizer(args.tokenizer)
    model = load_model(args)
    prompts, refs = load_prompts(args.data, args.n)
    ops.set_dual_attention_impl("fused")
    results = {"fused": run(model, tok, prompts, refs, args.max_new, device, "fused")}
    if args.ab:
        ops.set_dual_attention_impl("two_pass")
        try:
            results["two_pass"] = run(model, tok, prompts, refs, args.max_new, device, "two_pass")
        finally:
            ops.set_dual_attention_impl("fused")
        a, b = results["fused"]["predictions"], results["two_pass"]["predictions"]
        results["identical_predictions"] = sum(x.strip() == y.strip() for x, y in zip(a, b))
        print(f"identical predictions: {results['identical_predictions']}/{len(a)}")
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(results, indent=1))
    return results


if __name__ == "__main__":
    main()
