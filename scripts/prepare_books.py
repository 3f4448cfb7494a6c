"""Turn a corpus of long documents (one ``.txt`` file per document, or ``.jsonl`` with a ``text`` field) into the
``shard_*.parquet`` files (column ``text``) that the trainer's HF dataset path and scripts/eval_token_ppl.py read
(the role of the reference's scripts/prepare_books3.py).  Documents shorter than ``--min_chars`` are dropped.

    python scripts/prepare_books.py --input corpus/ --output data/books_65k --docs_per_shard 256 --min_chars 200000
"""
import argparse
import json
from pathlib import Path


def documents(root: Path):
    for path in sorted(root.rglob("*")):
        if path.suffix == ".txt":
            yield path.read_text(errors="replace")
        elif path.suffix == ".jsonl":
            with path.open() as f:
                for line in f:
                    if line.strip():
                        yield json.loads(line)["text"]


def main(argv=None):
    import pyarrow as pa
    import pyarrow.parquet as pq
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--docs_per_shard", type=int, default=256)
    ap.add_argument("--min_chars", type=int, default=0)
    args = ap.parse_args(argv)
    out = Path(args.output)
    out.mkdir(parents=True, exist_ok=True)
    buf, shard, kept, dropped = [], 0, 0, 0

    def flush():
        nonlocal buf, shard
        if buf:
            pq.write_table(pa.table({"text": buf}), out / f"shard_{shard:05d}.parquet")
            shard += 1
            buf = []

    for text in documents(Path(args.input)):
        if len(text) < args.min_chars:
            dropped += 1
            continue
        buf.append(text)
        kept += 1
        if len(buf) >= args.docs_per_shard:
            flush()
    flush()
    print(json.dumps({"documents": kept, "dropped_short": dropped, "shards": shard, "output": str(out)}))


if __name__ == "__main__":
    main()
