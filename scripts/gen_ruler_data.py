"""Synthetic long-context task data in the layout ``eval_ruler.py`` / ``eval_niah.py`` read:
``<save_dir>/ctx<N>/<task>/validation.jsonl``, one ``{"index", "input", "outputs", "answer_prefix", "length"}`` per line.

The reference generates these files with the RULER benchmark's ``prepare.py`` from a third-party checkout
(reference scripts/niah_gen_ruler.sh:29-56, scripts/ruler_gen_5tasks.sh:28-52); this script is a self-contained
generator of the same task families, with RULER's prompt wording, that needs nothing but a tokenizer:

* ``niah_single_1`` (repeated-sentence haystack, word key, number value), ``niah_single_2`` (prose haystack),
  ``niah_single_3`` (prose haystack, uuid value), ``niah_multikey_1`` (4 needles, 1 asked),
  ``niah_multivalue`` (1 key, 4 values, all asked), ``niah_multiquery`` (4 needles, 4 asked);
* ``vt`` (variable tracking: one chain of 5 assignments), ``cwe`` (10 common words among rare ones),
  ``fwe`` (three most frequent coded words of a Zipf-distributed stream).

The two question-answering tasks of RULER need SQuAD / HotpotQA and are not generated.  Every prompt is grown until
it just fits ``ctx - tokens_to_generate`` tokens of the given tokenizer.

    python scripts/gen_ruler_data.py --tokenizer tokenizers/Qwen3-0.6B-Base --save_dir data/niah/qwen3 \
        --ctx_lens 4096 16384 65536 --tasks niah_single_1 niah_multikey_1 vt --num_samples 100
"""
from __future__ import annotations

import argparse
import json
import random
import uuid
from pathlib import Path

ADJ = ("amber brisk calm dapper eager fuzzy gentle hollow ivory jolly keen lively mellow nimble odd placid quaint rustic "
       "silent tidy upbeat vivid witty young zesty ample bold crisp dusty elfin frail grand humble icy jaded lucid murky "
       "noble opaque proud quick rapid stout tense urban vast wary yearly zonal").split()
NOUN = ("anchor basket candle dolphin engine feather garden harbor island jacket kettle lantern meadow needle orchard "
        "pebble quiver ribbon saddle timber umbrella valley window yarn zipper antler beacon cradle dagger ember fossil "
        "glacier hammer inkwell jungle kernel ladder magnet nectar oyster pillar quartz rocket spindle tunnel urchin "
        "violin walnut yogurt").split()
NOISE = "The grass is green. The sky is blue. The sun is yellow. Here we go. There and back again."
TOKENS_TO_GENERATE = {"niah": 128, "vt": 30, "cwe": 120, "fwe": 50}

NIAH_TEMPLATE = ("Some special magic {kind} are hidden within the following text. Make sure to memorize it. I will quiz you "
                 "about the {kind} afterwards.\n{context}\nWhat are all the special magic {kind} for {query} mentioned in the "
                 "provided text?")
NIAH_PREFIX = " The special magic {kind} for {query} mentioned in the provided text are"
NEEDLE = "One of the special magic {kind} for {key} is: {value}."
VT_TEMPLATE = ("Memorize and track the chain(s) of variable assignment hidden in the following text.\n\n{context}\nQuestion: "
               "Find all variables that are assigned the value {query} in the text above.")
VT_PREFIX = " Answer: According to the chain(s) of variable assignment in the text above, {n} variables are assgined the value {query}, they are: "
CWE_TEMPLATE = ("Below is a numbered list of words. In these words, some appear more often than others. Memorize the ones that "
                "appear most often.\n{context}\nQuestion: What are the 10 most common words in the above list?")
CWE_PREFIX = " Answer: The top 10 words that appear most often in the list are:"
FWE_TEMPLATE = ("Read the following coded text and track the frequency of each coded word. Find the three most frequently "
                "appeared coded words. {context}\nQuestion: Do not provide any explanation. Please ignore the dots '....'. What "
                "are the three most frequently appeared words in the above coded text?")
FWE_PREFIX = " Answer: According to the coded text above, the three most frequently appeared words are:"

NIAH_TASKS = {  # haystack, value kind, needles (keys), values per key, keys asked
    "niah_single_1": ("noise", "numbers", 1, 1, 1), "niah_single_2": ("prose", "numbers", 1, 1, 1),
    "niah_single_3": ("prose", "uuids", 1, 1, 1), "niah_multikey_1": ("prose", "numbers", 4, 1, 1),
    "niah_multivalue": ("prose", "numbers", 1, 4, 1), "niah_multiquery": ("prose", "numbers", 4, 1, 4),
}
ALL_TASKS = list(NIAH_TASKS) + ["vt", "cwe", "fwe"]


def word(rng: random.Random) -> str:
    return f"{rng.choice(ADJ)}-{rng.choice(NOUN)}"


def prose_sentence(rng: random.Random) -> str:
    n = rng.randint(6, 14)
    words = [rng.choice(NOUN if i % 3 == 2 else ADJ) for i in range(n)]
    return " ".join(words).capitalize() + "."


def count_tokens(tok, text: str) -> int:
    return len(tok(text, add_special_tokens=False).input_ids)


def fit(build, tok, budget: int, lo: int = 1) -> int:
    """Largest size in [lo, ...] whose prompt ``build(size)`` has at most ``budget`` tokens (doubling, then bisection)."""
    if count_tokens(tok, build(lo)) > budget:
        return lo
    hi = lo * 2
    while count_tokens(tok, build(hi)) <= budget:
        lo, hi = hi, hi * 2
    while hi - lo > max(1, lo // 200):
        mid = (lo + hi) // 2
        if count_tokens(tok, build(mid)) <= budget:
            lo = mid
        else:
            hi = mid
    return lo


def make_niah(task: str, tok, budget: int, rng: random.Random) -> dict:
    haystack, kind, n_keys, n_vals, n_ask = NIAH_TASKS[task]
    keys = []
    while len(keys) < n_keys:
        k = word(rng)
        if k not in keys:
            keys.append(k)
    value = (lambda: str(uuid.UUID(int=rng.getrandbits(128)))) if kind == "uuids" else (lambda: str(rng.randint(10 ** 6, 10 ** 7 - 1)))
    values = {k: [value() for _ in range(n_vals)] for k in keys}
    needles = [NEEDLE.format(kind=kind, key=k, value=v) for k in keys for v in values[k]]
    asked = keys[:n_ask]
    query = asked[0] if len(asked) == 1 else ", ".join(asked[:-1]) + ", and " + asked[-1]
    seed = rng.getrandbits(32)

    def build(size: int) -> str:
        r = random.Random(seed)
        units = [NOISE] * size if haystack == "noise" else [prose_sentence(r) for _ in range(size)]
        for nd in needles:
            units.insert(r.randint(0, len(units)), nd)
        return NIAH_TEMPLATE.format(kind=kind, context=" ".join(units), query=query)

    size = fit(build, tok, budget)
    return {"input": build(size), "outputs": [v for k in asked for v in values[k]],
            "answer_prefix": NIAH_PREFIX.format(kind=kind, query=query)}


def make_vt(tok, budget: int, rng: random.Random, hops: int = 4) -> dict:
    names = []
    while len(names) < hops + 1:
        v = "".join(rng.choice("ABCDEFGHIJKLMNOPQRSTUVWXYZ") for _ in range(5))
        if v not in names:
            names.append(v)
    val = str(rng.randint(10000, 99999))
    chain = [f"VAR {names[0]} = {val}"] + [f"VAR {names[i + 1]} = VAR {names[i]} " for i in range(hops)]
    seed = rng.getrandbits(32)

    def build(size: int) -> str:
        r = random.Random(seed)
        units = [NOISE] * size
        spots = sorted(r.sample(range(size + 1), len(chain))) if size + 1 >= len(chain) else [0] * len(chain)
        for off, (pos, stmt) in enumerate(zip(spots, chain)):          # chain order is kept
            units.insert(pos + off, stmt)
        return VT_TEMPLATE.format(context=" ".join(units), query=val)

    size = fit(build, tok, budget, lo=len(chain))
    return {"input": build(size), "outputs": names, "answer_prefix": VT_PREFIX.format(n=len(names), query=val)}


def make_cwe(tok, budget: int, rng: random.Random, common_rep: int = 30, rare_rep: int = 3) -> dict:
    pool = sorted({f"{a}{n}" for a in ADJ for n in NOUN})
    rng.shuffle(pool)
    common = pool[:10]
    seed = rng.getrandbits(32)

    def build(size: int) -> str:
        r = random.Random(seed)
        words = common * common_rep + pool[10:10 + size] * rare_rep
        r.shuffle(words)
        return CWE_TEMPLATE.format(context=" ".join(f"{i + 1}. {w}" for i, w in enumerate(words)))

    size = min(fit(build, tok, budget), len(pool) - 10)
    return {"input": build(size), "outputs": common, "answer_prefix": CWE_PREFIX}


def make_fwe(tok, budget: int, rng: random.Random, alpha: float = 2.0, vocab: int = 2000) -> dict:
    coded = []
    while len(coded) < vocab:
        w = "".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(3, 8)))
        if w not in coded:
            coded.append(w)
    weights = [1.0 / (i + 1) ** alpha for i in range(vocab)]     # rank 0 stands for the dots and is not an answer
    seed = rng.getrandbits(32)

    def build(size: int) -> str:
        r = random.Random(seed)
        stream = r.choices(range(vocab), weights=weights, k=size)
        return FWE_TEMPLATE.format(context=" ".join("...." if i == 0 else coded[i] for i in stream))

    size = fit(build, tok, budget, lo=64)
    return {"input": build(size), "outputs": coded[1:4], "answer_prefix": FWE_PREFIX}


def make_sample(task: str, tok, ctx: int, rng: random.Random) -> dict:
    family = "niah" if task in NIAH_TASKS else task
    budget = ctx - TOKENS_TO_GENERATE[family]
    if family == "niah":
        d = make_niah(task, tok, budget, rng)
    elif task == "vt":
        d = make_vt(tok, budget, rng)
    elif task == "cwe":
        d = make_cwe(tok, budget, rng)
    elif task == "fwe":
        d = make_fwe(tok, budget, rng)
    else:
        raise SystemExit(f"unknown task {task!r}; choose from {ALL_TASKS}")
    d["length"] = count_tokens(tok, d["input"] + d["answer_prefix"])
    return d


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--save_dir", required=True)
    ap.add_argument("--ctx_lens", type=int, nargs="+", default=[4096, 8192, 16384, 32768, 65536])
    ap.add_argument("--tasks", nargs="+", default=list(NIAH_TASKS))
    ap.add_argument("--num_samples", type=int, default=100)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    from eval_common import load_tokenizer
    tok = load_tokenizer(args.tokenizer)
    for ctx in args.ctx_lens:
        for task in args.tasks:
            out = Path(args.save_dir) / f"ctx{ctx}" / task / "validation.jsonl"
            if out.is_file() and not args.overwrite and sum(1 for _ in out.open()) >= args.num_samples:
                print(f"[skip] {out}")
                continue
            out.parent.mkdir(parents=True, exist_ok=True)
            rng = random.Random(f"{args.seed}-{task}-{ctx}")
            with out.open("w") as f:
                for i in range(args.num_samples):
                    f.write(json.dumps({"index": i, **make_sample(task, tok, ctx, rng)}) + "\n")
            print(f"[done] {out}")


if __name__ == "__main__":
    main()
