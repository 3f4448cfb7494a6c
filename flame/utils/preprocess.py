"""python -m flame.utils.preprocess --dataset NAME --tokenizer TOK --output DIR : offline tokenisation."""
import argparse


def tokenize_dataset(dataset, tokenizer, text_key="text", num_proc=8):
    def fn(batch):
        ids = tokenizer(batch[text_key], return_attention_mask=False)["input_ids"]
        return {"input_ids": ids, "bits_per_token": [len(t.encode("utf-8")) * 8 / max(1, len(i)) for t, i in zip(batch[text_key], ids)]}
    return dataset.map(fn, batched=True, num_proc=num_proc, remove_columns=dataset.column_names)


def main(argv=None):
    from datasets import load_dataset
    from transformers import AutoTokenizer
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--name", default=None)
    ap.add_argument("--split", default="train")
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--num_proc", type=int, default=8)
    args = ap.parse_args(argv)
    ds = load_dataset(args.dataset, args.name, split=args.split)
    tok = AutoTokenizer.from_pretrained(args.tokenizer, trust_remote_code=True)
    tokenize_dataset(ds, tok, num_proc=args.num_proc).save_to_disk(args.output)


if __name__ == "__main__":
    main()
