"""Scrape trainer logs for throughput: mean / median ``tps`` and ``mfu`` after a warm-up number of logged
steps (reference scripts/summarize_titan_step_metrics.py).

    python scripts/summarize_step_metrics.py exp/run/train.log --skip 5"""
import argparse
import json
import re
import statistics

LINE = re.compile(r"step:\s*(\d+).*?loss:\s*([0-9.eE+-]+).*?tps:\s*([0-9,]+).*?mfu:\s*([0-9.]+)%")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--skip", type=int, default=2, help="logged steps to drop from the start of each file")
    args = ap.parse_args(argv)
    for path in args.logs:
        rows = [(int(m[1]), float(m[2]), float(m[3].replace(",", "")), float(m[4])) for m in
                (LINE.search(line) for line in open(path, errors="replace")) if m]
        rows = rows[args.skip:]
        if not rows:
            print(json.dumps({"log": path, "steps": 0}))
            continue
        tps, mfu = [r[2] for r in rows], [r[3] for r in rows]
        print(json.dumps({"log": path, "steps": len(rows), "first_step": rows[0][0], "last_step": rows[-1][0],
                          "last_loss": rows[-1][1], "tps_mean": round(statistics.mean(tps), 1),
                          "tps_median": round(statistics.median(tps), 1), "mfu_mean": round(statistics.mean(mfu), 2)}))


if __name__ == "__main__":
    main()
