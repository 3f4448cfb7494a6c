"""Merge evaluation outputs written by separate jobs.

``offset-shards``: per-seed outputs of ``eval_token_ppl.py`` (one JSON per seed of the random-offset evaluation)
into one per-position curve, each shard weighted by its sample count
(reference scripts/merge_offset_shards.py:19-58):

    python scripts/merge_eval_results.py offset-shards --inputs eval/ppl_seed{42,43,44}.json --output eval/ppl_merged.json

``final-block``: per-model outputs of ``eval_final_block_doc_ppl.py`` into one table, after checking that all of
them scored the same documents with the same settings (reference scripts/merge_fixed_final_block_doc_ppl.py:38-66):

    python scripts/merge_eval_results.py final-block --inputs eval/ffb_a eval/ffb_b --output_dir eval/ffb_all
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

SAME_META_KEYS = ("seq_len", "final_block_size", "context_lens", "selected_total_tokens", "min_doc_tokens", "num_documents")


def _curve_of(d: dict) -> list[float]:
    for key in ("nll_per_position", "avg_nll"):       # this repo's key, the reference's key
        if isinstance(d.get(key), list):
            return d[key]
    raise SystemExit("no per-position NLL list ('nll_per_position' or 'avg_nll') in the input")


def merge_offset_shards(inputs: list[str], output: str) -> dict:
    total, acc, first = 0, None, None
    for path in inputs:
        d = json.loads(Path(path).read_text())
        n, curve = int(d["num_samples"]), _curve_of(d)
        if acc is None:
            acc, first = [0.0] * len(curve), d
        if len(curve) != len(acc):
            raise SystemExit(f"{path}: {len(curve)} positions, the first shard has {len(acc)}")
        acc = [a + n * c for a, c in zip(acc, curve)]
        total += n
        print(f"  {path}: n={n} ppl={math.exp(sum(curve) / len(curve)):.3f}")
    mean = [a / total for a in acc]
    nll = sum(mean) / len(mean)
    out = {"seq_len": first["seq_len"], "num_samples": total, "offset_max": first.get("offset_max", 0), "merged_from": inputs,
           "nll_per_position": mean, "avg_nll": mean, "nll": nll, "ppl": math.exp(nll), "avg_ppl": math.exp(nll),
           "positions": list(range(1, len(mean) + 1))}
    Path(output).parent.mkdir(parents=True, exist_ok=True)
    Path(output).write_text(json.dumps(out))
    print(f"merged {len(inputs)} shards, n={total}, ppl={out['ppl']:.3f} -> {output}")
    return out


def merge_final_block(inputs: list[str], output_dir: str) -> dict:
    loaded = []
    for item in inputs:
        p = Path(item)
        p = p / "fixed_final_block_doc_ppl.json" if p.is_dir() else p
        payload = json.loads(p.read_text())
        if not payload.get("results"):
            raise SystemExit(f"{p}: no model results")
        loaded.append((p, payload))
    ref_path, ref = loaded[0]
    results = {}
    for p, payload in loaded:
        for key in SAME_META_KEYS:
            if payload["meta"].get(key) != ref["meta"].get(key):
                raise SystemExit(f"{p} and {ref_path} differ in meta[{key}]: {payload['meta'].get(key)} vs {ref['meta'].get(key)}")
        if payload["document_stats"] != ref["document_stats"]:
            raise SystemExit(f"{p} and {ref_path} scored different documents")
        for name, rows in payload["results"].items():
            if name in results:
                raise SystemExit(f"model name {name!r} appears twice")
            results[name] = rows
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "document_stats.json").write_text(json.dumps(ref["document_stats"], indent=2) + "\n")
    merged = {"meta": ref["meta"], "document_stats": ref["document_stats"], "results": results}
    (out / "fixed_final_block_doc_ppl.json").write_text(json.dumps(merged, indent=2) + "\n")
    names = list(results)
    lines = ["context_len," + ",".join(names)]
    for i, ctx in enumerate(ref["meta"]["context_lens"]):
        cells = [results[n][i]["perplexity"] for n in names]
        lines.append(f"{ctx}," + ",".join("" if c is None else f"{c:.8f}" for c in cells))
    (out / "fixed_final_block_doc_ppl.csv").write_text("\n".join(lines) + "\n")
    print(f"merged {len(names)} models -> {out}")
    return merged


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    a = sub.add_parser("offset-shards")
    a.add_argument("--inputs", nargs="+", required=True)
    a.add_argument("--output", required=True)
    b = sub.add_parser("final-block")
    b.add_argument("--inputs", nargs="+", required=True)
    b.add_argument("--output_dir", required=True)
    args = ap.parse_args(argv)
    if args.what == "offset-shards":
        merge_offset_shards(args.inputs, args.output)
    else:
        merge_final_block(args.inputs, args.output_dir)


if __name__ == "__main__":
    main()
