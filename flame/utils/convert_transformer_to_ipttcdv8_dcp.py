"""python -m flame.utils.convert_transformer_to_ipttcdvN_dcp --model SRC --config JSON --checkpoint OUT"""
import argparse
import json

from ttcd_b200.utils.convert import convert_transformer_to_ipttcd_dcp


def main(argv=None):
    ap = argparse.ArgumentParser(description="transformer checkpoint (HF dir or DCP) -> IP-TTCD DCP by equal keys")
    ap.add_argument("--model", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--checkpoint", required=True)
    args = ap.parse_args(argv)
    print(json.dumps(convert_transformer_to_ipttcd_dcp(args.model, args.config, args.checkpoint, args.tokenizer), indent=2)[:2000])


if __name__ == "__main__":
    main()
