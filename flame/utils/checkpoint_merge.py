"""python -m flame.utils.checkpoint_merge --path RUN --output_path OUT --steps a b c --merge_type sma|ema|wma"""
import argparse

from ttcd_b200.utils.convert import merge_checkpoints, merge_weights


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--path", required=True)
    ap.add_argument("--output_path", required=True)
    ap.add_argument("--steps", type=int, nargs="+", required=True)
    ap.add_argument("--merge_type", choices=["sma", "ema", "wma"], default="sma")
    ap.add_argument("--alpha", type=float, default=0.9)
    ap.add_argument("--onlymlp", action="store_true")
    ap.add_argument("--config", required=True)
    ap.add_argument("--tokenizer", default=None)
    args = ap.parse_args(argv)
    steps = sorted(args.steps)
    weights = merge_weights(steps, args.merge_type, args.alpha)
    print(merge_checkpoints(args.path, args.output_path, steps, weights, args.config, args.tokenizer, args.onlymlp))


if __name__ == "__main__":
    main()
