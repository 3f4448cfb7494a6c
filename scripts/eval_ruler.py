"""RULER-style long-context generation tasks (needle-in-a-haystack and friends): reference
scripts/eval_niah.py and scripts/eval_ruler.py.

Data layout: ``<data_dir>/<ctx_len>/<task>/validation.jsonl`` (also accepted: ``<data_dir>/ctx<ctx_len>/<task>/...`` as written
by ``gen_ruler_data.py``, and ``<data_dir>/<task>_<ctx_len>.jsonl``),
one JSON object per line with ``input``, ``outputs`` (list of reference strings), optional ``answer_prefix`` and
``index``.  The prompt is ``input`` (+ ``answer_prefix`` unless ``--no_answer_prefix``); decoding is greedy
through the model's own prefill + windowed cache; the score is RULER's ``string_match_all``: the mean over
samples of the fraction of references found (case-insensitive) in the prediction.

    python scripts/eval_ruler.py --data_dir data/niah/qwen3 --tasks niah_single_1 niah_multikey_1 \
        --ctx_lens 4096 16384 65536 --config cfg.json --checkpoint ckpt --tokenizer tok --output out.json
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from eval_common import add_model_args, greedy_decode, load_model, load_tokenizer

DEFAULT_TASKS = ["niah_single_1", "niah_single_2", "niah_single_3", "niah_multikey_1", "niah_multivalue", "niah_multiquery",
                 "vt", "cwe", "fwe", "qa_1", "qa_2"]
# tokens to generate per task family (RULER's settings)
MAX_NEW = {"niah": 128, "vt": 30, "cwe": 120, "fwe": 50, "qa": 32}


def string_match_all(preds: list[str], refs: list[list[str]]) -> float:
    if not preds:
        return 0.0
    per = [sum(1.0 for r in rs if r.lower() in p.lower()) / max(1, len(rs)) for p, rs in zip(preds, refs)]
    return 100.0 * sum(per) / len(per)


def find_file(data_dir: Path, task: str, ctx: int) -> Path | None:
    for cand in (data_dir / str(ctx) / task / "validation.jsonl", data_dir / f"ctx{ctx}" / task / "validation.jsonl",
                 data_dir / task / str(ctx) / "validation.jsonl",
                 data_dir / f"{task}_{ctx}.jsonl"):
        if cand.is_file():
            return cand
    return None


def run_file(model, tok, path: Path, device: str, max_new: int, max_samples: int | None, with_prefix: bool) -> dict:
    eos = {tok.eos_token_id} if tok.eos_token_id is not None else None
    preds, refs, idxs = [], [], []
    with path.open() as f:
        for line in f:
            if max_samples is not None and len(preds) >= max_samples:
                break
            d = json.loads(line)
            prompt = d["input"] + (d.get("answer_prefix") or "" if with_prefix else "")
            ids = tok(prompt, return_tensors="pt", add_special_tokens=False).input_ids.to(device)
            text = tok.decode(greedy_decode(model, ids, max_new, eos), skip_special_tokens=True)
            preds.append(text)
            refs.append(d["outputs"])
            idxs.append(d.get("index", len(idxs)))
    return {"n": len(preds), "accuracy": string_match_all(preds, refs), "predictions": preds, "references": refs, "indices": idxs}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_model_args(ap)
    ap.add_argument("--data_dir", required=True)
    ap.add_argument("--tasks", nargs="+", default=DEFAULT_TASKS)
    ap.add_argument("--ctx_lens", nargs="+", type=int, default=[4096, 8192, 16384, 32768, 65536])
    ap.add_argument("--max_samples", type=int, default=None)
    ap.add_argument("--max_new_tokens", type=int, default=None, help="override the per-task generation length")
    ap.add_argument("--no_answer_prefix", action="store_true")
    ap.add_argument("--output", required=True)
    ap.add_argument("--pred_dir", default=None, help="also write per-file predictions here")
    ap.add_argument("--save_preds", action="store_true", help="keep predictions inside the output JSON")
    args = ap.parse_args(argv)
    tok = load_tokenizer(args.tokenizer)
    model = load_model(args)
    results: dict[str, dict] = {}
    for ctx in args.ctx_lens:
        for task in args.tasks:
            path = find_file(Path(args.data_dir), task, ctx)
            if path is None:
                print(f"[ruler] no data for {task} @ {ctx}")
                continue
            family = next((k for k in MAX_NEW if task.startswith(k)), "niah")
            res = run_file(model, tok, path, args.device, args.max_new_tokens or MAX_NEW[family], args.max_samples,
                           not args.no_answer_prefix)
            print(f"[ruler] {task} @ {ctx}: {res['accuracy']:.1f} (n={res['n']})", flush=True)
            if args.pred_dir:
                out = Path(args.pred_dir) / f"{task}_{ctx}.jsonl"
                out.parent.mkdir(parents=True, exist_ok=True)
                out.write_text("\n".join(json.dumps({"index": i, "pred": p, "outputs": r})
                                         for i, p, r in zip(res["indices"], res["predictions"], res["references"])))
            if not args.save_preds:
                res = {"n": res["n"], "accuracy": res["accuracy"]}
            results.setdefault(str(ctx), {})[task] = res
    for ctx, tasks in results.items():
        tasks["average"] = sum(t["accuracy"] for t in tasks.values()) / max(1, len(tasks))
    Path(args.output).parent.mkdir(parents=True, exist_ok=True)
    Path(args.output).write_text(json.dumps(results, indent=1))


if __name__ == "__main__":
    main()
