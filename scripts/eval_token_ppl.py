"""Per-position perplexity on long documents (reference scripts/eval_token_ppl.py).

Documents come from ``shard_*.parquet`` files with a ``text`` column; each is tokenised and a window of
``--seq_len`` tokens is taken at ``--offset`` (or at a seeded random offset in ``[0, --offset_max]``, which
decouples the curve from the absolute position in the book; shorter documents are skipped).  Output JSON:
mean NLL per position, overall perplexity, and bucketed means (0-2k, 2k-4k, ... like the trainer's
``loss_by_pos`` metrics).

    python scripts/eval_token_ppl.py --config cfg.json --checkpoint exp/x/checkpoint/step-2000 \
        --tokenizer tokenizers/Qwen3-0.6B-Base --data_dir data/books_65k --seq_len 65536 --num_samples 50
"""
from __future__ import annotations

import argparse
import json
import math
import random
from pathlib import Path

import torch

from eval_common import add_model_args, load_model, load_tokenizer, token_nll


def load_windows(data_dir: str, tokenizer, seq_len: int, num_samples: int, offset: int, offset_max: int, seed: int):
    import pyarrow.parquet as pq
    rng = random.Random(seed)
    need = (offset_max if offset_max > 0 else offset) + seq_len
    windows, skipped = [], 0
    for shard in sorted(Path(data_dir).glob("shard_*.parquet")):
        for text in pq.read_table(shard, columns=["text"])["text"].to_pylist():
            if len(windows) >= num_samples:
                return windows, skipped
            toks = tokenizer.encode(text, add_special_tokens=False)
            if len(toks) < need:
                skipped += 1
                continue
            start = rng.randint(0, offset_max) if offset_max > 0 else offset
            windows.append(toks[start:start + seq_len])
    return windows, skipped


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_model_args(ap)
    ap.add_argument("--data_dir", default="data/books_65k")
    ap.add_argument("--seq_len", type=int, default=16384)
    ap.add_argument("--num_samples", type=int, default=50)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--offset", type=int, default=0)
    ap.add_argument("--offset_max", type=int, default=0)
    ap.add_argument("--offset_seed", type=int, default=0)
    ap.add_argument("--output", default="eval_results/token_ppl.json")
    args = ap.parse_args(argv)
    tok = load_tokenizer(args.tokenizer)
    model = load_model(args)
    windows, skipped = load_windows(args.data_dir, tok, args.seq_len, args.num_samples, args.offset, args.offset_max, args.offset_seed)
    if not windows:
        raise SystemExit(f"no document of at least {args.seq_len} tokens under {args.data_dir}")
    total = torch.zeros(args.seq_len - 1, dtype=torch.float64)
    for i in range(0, len(windows), args.batch_size):
        ids = torch.tensor(windows[i:i + args.batch_size], device=args.device)
        total += token_nll(model, ids).double().sum(0).cpu()
        print(f"[ppl] {min(i + args.batch_size, len(windows))}/{len(windows)} running nll {float(total.sum() / ((i + ids.shape[0]) * (args.seq_len - 1))):.4f}", flush=True)
    mean = (total / len(windows)).tolist()
    edges = [0, 2048, 4096, 8192, 16384, 32768, 65536, 131072]
    buckets = {f"{a}_{b}": sum(mean[a:b]) / len(mean[a:b]) for a, b in zip(edges[:-1], edges[1:]) if a < len(mean)}
    overall = sum(mean) / len(mean)
    Path(args.output).parent.mkdir(parents=True, exist_ok=True)
    Path(args.output).write_text(json.dumps({"seq_len": args.seq_len, "num_samples": len(windows), "skipped_short": skipped,
                                             "nll": overall, "ppl": math.exp(overall), "nll_by_bucket": buckets,
                                             "nll_per_position": mean}))
    print(f"[ppl] nll {overall:.4f} ppl {math.exp(overall):.3f} -> {args.output}")


if __name__ == "__main__":
    main()
