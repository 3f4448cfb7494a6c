"""python -m flame.utils.convert_dcp_to_hf --path RUN --step N --config JSON --tokenizer TOK"""
import argparse

from ttcd_b200.utils.convert import convert_dcp_to_hf


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--path", required=True)
    ap.add_argument("--step", type=int, default=None)
    ap.add_argument("--config", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    print(convert_dcp_to_hf(args.path, args.step, args.config, args.tokenizer, args.output))


if __name__ == "__main__":
    main()
