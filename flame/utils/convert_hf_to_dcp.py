"""python -m flame.utils.convert_hf_to_dcp --model DIR --checkpoint OUT"""
import argparse

from ttcd_b200.utils.convert import convert_model_to_dcp


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--checkpoint", required=True)
    args = ap.parse_args(argv)
    convert_model_to_dcp(args.model, args.checkpoint)


if __name__ == "__main__":
    main()
