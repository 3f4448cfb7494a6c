"""LongBench (English subset) evaluation (reference scripts/eval_longbench.py).

Per task: read ``<data_dir>/<task>.jsonl``, fill the task's prompt template (``--prompt_config`` JSON:
task -> template with ``{context}`` / ``{input}``), truncate prompts longer than ``--max_length`` tokens by
keeping the first and the last half (LongBench's convention: the question at the end survives), decode
greedily up to the task's limit (``--maxlen_config`` JSON), score with scripts/longbench_metrics.py.
Writes ``<output_pred_dir>/<task>.jsonl`` and one scores JSON."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from eval_common import add_model_args, greedy_decode, load_model, load_tokenizer
from longbench_metrics import DATASET2METRIC, scorer

ENGLISH_TASKS = list(DATASET2METRIC)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_model_args(ap)
    ap.add_argument("--data_dir", default="data/longbench/raw/data")
    ap.add_argument("--prompt_config", default="data/longbench/dataset2prompt.json")
    ap.add_argument("--maxlen_config", default="data/longbench/dataset2maxlen.json")
    ap.add_argument("--tasks", nargs="+", default=ENGLISH_TASKS)
    ap.add_argument("--max_length", type=int, default=31500)
    ap.add_argument("--num_per_task", type=int, default=0, help="0 = all")
    ap.add_argument("--start_idx", type=int, default=0)
    ap.add_argument("--end_idx", type=int, default=0, help="0 = to the end")
    ap.add_argument("--pred_filename", default="", help="suffix for per-task prediction files (sharded runs)")
    ap.add_argument("--output_pred_dir", required=True)
    ap.add_argument("--output_scores", required=True)
    args = ap.parse_args(argv)
    prompts = json.loads(Path(args.prompt_config).read_text())
    maxlens = json.loads(Path(args.maxlen_config).read_text())
    tok = load_tokenizer(args.tokenizer)
    model = load_model(args)
    eos = {tok.eos_token_id} if tok.eos_token_id is not None else None
    scores = {}
    Path(args.output_pred_dir).mkdir(parents=True, exist_ok=True)
    for task in args.tasks:
        path = Path(args.data_dir) / f"{task}.jsonl"
        if not path.is_file():
            print(f"[longbench] missing {path}")
            continue
        rows = [json.loads(line) for line in path.open()]
        rows = rows[args.start_idx:(args.end_idx or None)]
        if args.num_per_task:
            rows = rows[:args.num_per_task]
        preds, answers, classes = [], [], None
        out_path = Path(args.output_pred_dir) / f"{task}{args.pred_filename}.jsonl"
        with out_path.open("w") as out:
            for row in rows:
                ids = tok(prompts[task].format(**row), add_special_tokens=False).input_ids
                if len(ids) > args.max_length:
                    half = args.max_length // 2
                    ids = ids[:half] + ids[-half:]
                import torch
                gen = greedy_decode(model, torch.tensor([ids], device=args.device), int(maxlens[task]), eos)
                pred = tok.decode(gen, skip_special_tokens=True)
                preds.append(pred)
                answers.append(row["answers"])
                classes = row.get("all_classes")
                out.write(json.dumps({"pred": pred, "answers": row["answers"], "all_classes": classes, "length": row.get("length")}) + "\n")
        scores[task] = scorer(task, preds, answers, classes)
        print(f"[longbench] {task}: {scores[task]} (n={len(preds)})", flush=True)
    if scores:
        scores["average"] = round(sum(scores.values()) / len(scores), 2)
    Path(args.output_scores).parent.mkdir(parents=True, exist_ok=True)
    Path(args.output_scores).write_text(json.dumps(scores, indent=1))


if __name__ == "__main__":
    main()
