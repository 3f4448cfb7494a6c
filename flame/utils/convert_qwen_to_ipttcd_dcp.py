"""python -m flame.utils.convert_qwen_to_ipttcd_dcp --model HF --config JSON --tokenizer TOK --checkpoint OUT"""
import argparse
import json

from ttcd_b200.utils.convert import convert_hf_causal_lm_to_dcp, map_hf_key as map_qwen_key_to_ipttcd  # noqa: F401


def main(argv=None):
    ap = argparse.ArgumentParser(description="HF Qwen3 / SmolLM2 / Llama checkpoint -> IP-TTCD DCP seed checkpoint")
    ap.add_argument("--model", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--checkpoint", required=True)
    args = ap.parse_args(argv)
    report = convert_hf_causal_lm_to_dcp(args.model, args.config, args.checkpoint, args.tokenizer)
    print(json.dumps({k: (v if not isinstance(v, list) else v[:20]) for k, v in report.items()}, indent=2))


if __name__ == "__main__":
    main()
