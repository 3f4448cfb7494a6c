"""Perplexity of a fixed final block as a function of how much same-document context precedes it
(reference scripts/eval_fixed_final_block_doc_ppl.py:276-466).

For every context length ``c`` the last ``c + final_block_size`` tokens of each long-enough document are fed to the
model and only the last ``final_block_size`` positions are scored, so every curve point scores the *same* tokens
with more or less history; contexts never cross a document boundary.

    # 1. pick documents once (parquet shards with a ``text`` column) and keep them as a manifest
    python scripts/eval_final_block_doc_ppl.py --tokenizer tok --data_files 'data/heldout/*.parquet' \
        --docs_manifest_out eval/docs.npz --stats_only --output_dir eval/ffb
    # 2. score models on the same manifest
    python scripts/eval_final_block_doc_ppl.py --tokenizer tok --docs_manifest_in eval/docs.npz --output_dir eval/ffb \
        --models "ttcd|exp/run/checkpoint|2000|configs/ipttcd/ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k.json" "base|hf|hf/qwen3"

Model specs are ``name|checkpoint_dir|step|config.json`` (DCP, loaded directly in either key convention) or
``name|hf|directory``.  Outputs: ``document_stats.json``, ``fixed_final_block_doc_ppl.json`` (meta, document stats,
per-model rows) and ``fixed_final_block_doc_ppl.csv`` (one row per context length, one column per model).  The
manifest is an ``.npz`` with ``flat_tokens`` (int32), ``lengths`` (int32) and ``document_stats_json``.
"""
from __future__ import annotations

import argparse
import glob
import json
import math
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

from eval_common import load_model, load_tokenizer

DEFAULT_CONTEXTS = [1024, 2048, 4096, 8192, 16384, 24576, 30720]


def quantiles(values) -> dict:
    if len(values) == 0:
        return {}
    arr = np.sort(np.asarray(values))
    pick = lambda q: int(arr[min(len(arr) - 1, int(q * (len(arr) - 1)))])  # noqa: E731
    return {"min": int(arr[0]), "p25": pick(0.25), "p50": pick(0.5), "p75": pick(0.75), "p90": pick(0.9), "p99": pick(0.99),
            "max": int(arr[-1])}


def select_documents(tokenizer, files: list[str], seq_len: int, token_budget: int, min_doc_tokens: int):
    """Document suffixes (≤ seq_len tokens, left-truncated) of every document with at least ``min_doc_tokens``
    tokens, in file order, until ``token_budget`` tokens are selected."""
    import pyarrow.parquet as pq
    docs, seen, eligible = [], [], []
    selected = 0
    side = getattr(tokenizer, "truncation_side", "right")
    tokenizer.truncation_side = "left"
    try:
        for path in files:
            pf = pq.ParquetFile(path)
            for g in range(pf.num_row_groups):
                texts = [t for t in pf.read_row_group(g, columns=["text"]).column("text").to_pylist() if t and t.strip()]
                if not texts:
                    continue
                enc = tokenizer(texts, add_special_tokens=False, return_attention_mask=False, truncation=True,
                                max_length=seq_len)["input_ids"]
                for ids in enc:
                    seen.append(len(ids))
                    if len(ids) < min_doc_tokens:
                        continue
                    eligible.append(len(ids))
                    docs.append(np.asarray(ids[-seq_len:], dtype=np.int32))
                    selected += len(docs[-1])
                    if selected >= token_budget:
                        break
                if selected >= token_budget:
                    break
            if selected >= token_budget:
                break
    finally:
        tokenizer.truncation_side = side
    stats = {"mode": "single_document", "num_files": len(files), "sampled_docs": len(seen),
             "sampled_doc_length_quantiles": quantiles(seen), "eligible_docs": len(docs),
             "eligible_total_tokens": int(sum(eligible)), "selected_total_tokens": int(selected),
             "min_doc_tokens": int(min_doc_tokens), "selected_doc_length_quantiles": quantiles([len(d) for d in docs])}
    for th in (2048, 4096, 8192, 16384, 32768):
        stats[f"sampled_docs_ge_{th}"] = int(sum(n >= th for n in seen))
        stats[f"eligible_docs_ge_{th}"] = int(sum(n >= th for n in eligible))
        stats[f"eligible_tokens_ge_{th}"] = int(sum(n for n in eligible if n >= th))
    return docs, stats


def save_manifest(path: str, docs, stats: dict) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    lengths = np.asarray([len(d) for d in docs], dtype=np.int32)
    flat = np.concatenate(docs).astype(np.int32) if docs else np.zeros(0, np.int32)
    np.savez_compressed(path, flat_tokens=flat, lengths=lengths, document_stats_json=np.array(json.dumps(stats)))


def load_manifest(path: str):
    data = np.load(path, allow_pickle=False)
    flat, lengths = data["flat_tokens"], data["lengths"]
    if int(lengths.sum()) != len(flat):
        raise ValueError(f"{path}: lengths sum to {int(lengths.sum())}, {len(flat)} tokens stored")
    ends = np.cumsum(lengths)
    docs = [flat[e - n:e].copy() for e, n in zip(ends.tolist(), lengths.tolist())]
    return docs, json.loads(str(data["document_stats_json"]))


@torch.no_grad()
def final_block_curve(model, docs, context_lens, block: int, batch_size: int, device: str) -> list[dict]:
    rows = []
    for ctx in context_lens:
        need = ctx + block
        pool = [d for d in docs if len(d) >= need]
        row = {"context_len": ctx, "final_block_size": block, "eval_len": need, "num_sequences": 0, "total_pred_tokens": 0,
               "avg_nll": None, "perplexity": None}
        if pool:
            nll_sum, count = 0.0, 0
            for i in range(0, len(pool), batch_size):
                ids = torch.from_numpy(np.stack([d[-need:] for d in pool[i:i + batch_size]]).astype(np.int64)).to(device)
                logits = model(input_ids=ids, use_cache=False).logits[:, ctx - 1:-1].float()   # predictors of the block
                logp = torch.log_softmax(logits, dim=-1)
                nll = -logp.gather(-1, ids[:, ctx:, None]).squeeze(-1)
                nll_sum += float(nll.double().sum())
                count += nll.numel()
            row.update(num_sequences=len(pool), total_pred_tokens=count, avg_nll=nll_sum / count,
                       perplexity=math.exp(nll_sum / count))
        print(f"[ffb] ctx={ctx} docs={len(pool)} ppl={row['perplexity']}", flush=True)
        rows.append(row)
    return rows


def parse_model_spec(spec: str):
    parts = spec.split("|")
    if len(parts) == 3 and parts[1] == "hf":
        return parts[0], {"hf_model": parts[2]}
    if len(parts) == 4:
        return parts[0], {"checkpoint": str(Path(parts[1]) / f"step-{int(parts[2])}"), "config": parts[3]}
    raise SystemExit(f"bad model spec {spec!r}: use 'name|checkpoint_dir|step|config.json' or 'name|hf|dir'")


def write_outputs(out_dir: Path, meta: dict, stats: dict, results: dict) -> None:
    (out_dir / "fixed_final_block_doc_ppl.json").write_text(
        json.dumps({"meta": meta, "document_stats": stats, "results": results}, indent=2) + "\n")
    names = list(results)
    lines = ["context_len," + ",".join(names)]
    for i, ctx in enumerate(meta["context_lens"]):
        cells = [results[n][i]["perplexity"] for n in names]
        lines.append(f"{ctx}," + ",".join("" if c is None else f"{c:.8f}" for c in cells))
    (out_dir / "fixed_final_block_doc_ppl.csv").write_text("\n".join(lines) + "\n")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--models", nargs="*", default=[])
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--seq_len", type=int, default=32768, help="longest document suffix kept")
    ap.add_argument("--final_block_size", type=int, default=1024)
    ap.add_argument("--context_lens", type=int, nargs="+", default=DEFAULT_CONTEXTS)
    ap.add_argument("--token_budget", type=int, default=20_000_000)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--min_doc_tokens_override", type=int, default=None)
    ap.add_argument("--docs_manifest_in", default=None)
    ap.add_argument("--docs_manifest_out", default=None)
    ap.add_argument("--data_files", nargs="*", default=None, help="parquet files or globs")
    ap.add_argument("--stats_only", action="store_true")
    args = ap.parse_args(argv)

    out_dir = Path(args.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    contexts = sorted({int(c) for c in args.context_lens})
    longest = contexts[-1] + args.final_block_size
    if contexts[0] < 1 or longest > args.seq_len:
        raise SystemExit(f"need 1 <= context and max(context_lens)+final_block_size <= seq_len ({longest} > {args.seq_len})")
    if args.docs_manifest_in:
        docs, stats = load_manifest(args.docs_manifest_in)
    else:
        files = sorted(f for pat in (args.data_files or []) for f in glob.glob(pat))
        if not files:
            raise SystemExit("give --docs_manifest_in or --data_files")
        min_tokens = args.min_doc_tokens_override if args.min_doc_tokens_override is not None else longest
        docs, stats = select_documents(load_tokenizer(args.tokenizer), files, args.seq_len, args.token_budget, min_tokens)
        if args.docs_manifest_out:
            save_manifest(args.docs_manifest_out, docs, stats)
    if not docs:
        raise SystemExit("no eligible document")
    (out_dir / "document_stats.json").write_text(json.dumps(stats, indent=2) + "\n")
    print(f"[ffb] {len(docs)} documents, {stats['selected_total_tokens'] / 1e6:.2f}M tokens")
    if args.stats_only:
        return
    dtype = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16}.get(
        args.dtype.lower(), torch.float32)
    results = {}
    for spec in args.models:
        name, where = parse_model_spec(spec)
        margs = SimpleNamespace(config=None, checkpoint=None, hf_model=None, device=args.device, rope_scaling_type=None,
                                rope_scaling_factor=None, rope_scaling_original_max_pos=None, **where)
        model = load_model(margs, dtype)
        results[name] = final_block_curve(model, docs, contexts, args.final_block_size, args.batch_size, args.device)
        del model
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    meta = {"tokenizer": args.tokenizer, "seq_len": args.seq_len, "final_block_size": args.final_block_size,
            "context_lens": contexts, "token_budget": args.token_budget, "num_documents": len(docs),
            "selected_total_tokens": stats["selected_total_tokens"], "min_doc_tokens": stats["min_doc_tokens"],
            "device": args.device, "dtype": args.dtype}
    write_outputs(out_dir, meta, stats, results)
    print(f"[ffb] wrote {out_dir}")


if __name__ == "__main__":
    main()
