"""Per-token divergence between two runs of a model on the same prompts: KL(p_a || p_b), total variation, top-1
flips and the largest logit difference (the model-level drift check of the reference, profiling/collect_kl_tv.py,
used there to show that the fused attention kernel does not change predictions).

    python scripts/collect_kl_tv.py --config cfg.json --checkpoint ckpt --tokenizer tok \
        --a fused --b two_pass --data_dir data/books_65k --seq_len 16384 --num_samples 8 --output drift.json

``--a/--b``: dual-attention implementations (fused | two_pass) to compare; with ``--checkpoint_b`` the second run
uses another checkpoint instead.  Random tokens are used when no ``--data_dir`` is given."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from eval_common import add_model_args, load_model, load_tokenizer


@torch.no_grad()
def logits_of(model, ids):
    return model(input_ids=ids, use_cache=False).logits.float()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_model_args(ap)
    ap.add_argument("--a", default="fused")
    ap.add_argument("--b", default="two_pass")
    ap.add_argument("--checkpoint_b", default=None)
    ap.add_argument("--data_dir", default=None)
    ap.add_argument("--seq_len", type=int, default=16384)
    ap.add_argument("--num_samples", type=int, default=8)
    ap.add_argument("--output", default="eval_results/kl_tv.json")
    args = ap.parse_args(argv)
    from ttcd_b200 import ops
    model_a = load_model(args)
    model_b = model_a
    if args.checkpoint_b:
        args_b = argparse.Namespace(**{**vars(args), "checkpoint": args.checkpoint_b})
        model_b = load_model(args_b)
    if args.data_dir:
        from eval_token_ppl import load_windows
        windows, _ = load_windows(args.data_dir, load_tokenizer(args.tokenizer), args.seq_len, args.num_samples, 0, 0, 0)
    else:
        g = torch.Generator().manual_seed(0)
        windows = torch.randint(0, model_a.config.vocab_size, (args.num_samples, args.seq_len), generator=g).tolist()
    kl, tv, flips, max_d, n = [], [], 0, 0.0, 0
    for w in windows:
        ids = torch.tensor([w], device=args.device)
        ops.set_dual_attention_impl(args.a if args.a in ("fused", "two_pass") else "fused")
        la = logits_of(model_a, ids)
        ops.set_dual_attention_impl(args.b if args.b in ("fused", "two_pass") else "fused")
        lb = logits_of(model_b, ids)
        pa, pb = torch.log_softmax(la, -1), torch.log_softmax(lb, -1)
        kl.append((pa.exp() * (pa - pb)).sum(-1).flatten().cpu())
        tv.append(0.5 * (pa.exp() - pb.exp()).abs().sum(-1).flatten().cpu())
        flips += int((la.argmax(-1) != lb.argmax(-1)).sum())
        max_d = max(max_d, float((la - lb).abs().max()))
        n += ids.numel()
    ops.set_dual_attention_impl("fused")
    kl, tv = torch.cat(kl), torch.cat(tv)
    q = lambda t, p: float(torch.quantile(t[:: max(1, t.numel() // 1_000_000)], p))  # noqa: E731
    res = {"tokens": n, "kl_mean": float(kl.mean()), "kl_p50": q(kl, 0.5), "kl_p99": q(kl, 0.99), "tv_mean": float(tv.mean()),
           "tv_p99": q(tv, 0.99), "top1_flip_rate": flips / max(1, n), "max_abs_logit_diff": max_d}
    Path(args.output).parent.mkdir(parents=True, exist_ok=True)
    Path(args.output).write_text(json.dumps(res, indent=1))
    print(json.dumps(res))


if __name__ == "__main__":
    main()
