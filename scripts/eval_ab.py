"""A/B sign-off of two execution paths of ONE model on real tasks: accuracy and prediction identity on RULER / NIAH
files, mean NLL on long documents, and the per-token divergence of the two paths' next-token distributions (the
reference's profiling/ab_niah_fused.py and profiling/eval_ab_extended.py, which compare its stock model with its
fused-attention patch on a trained checkpoint).

An arm is a comma list of switches:
    attn=fused|two_pass      one-pass dual-window kernel, or two single-window attention calls
    decode=graph|eager       captured decode step, or the eager token loop

    python scripts/eval_ab.py --config cfg.json --checkpoint ckpt --tokenizer tok \
        --arm_a attn=two_pass,decode=eager --arm_b attn=fused,decode=graph \
        --data_dir data/niah/qwen3 --tasks niah_single_1 niah_single_2 niah_multikey_1 niah_multiquery \
        --ctx_lens 32768 65536 --max_samples 25 --ppl_dir data/books_65k --ppl_docs 16 --kl_docs 8 --output ab.json

Every part is optional: without ``--data_dir`` the task suite is skipped, without ``--ppl_dir`` the NLL and KL passes
run on random tokens (``--seq_len``).  The summary line says whether the arms agree: identical predictions on every
sample, and the top-1 flip rate and NLL difference under ``--max_flip_rate`` / ``--max_nll_diff``."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from eval_common import add_model_args, load_model, load_tokenizer, token_nll


def parse_arm(text: str) -> dict:
    arm = {"attn": "fused", "decode": "graph"}
    for item in filter(None, text.split(",")):
        key, _, value = item.partition("=")
        if key not in arm or value not in {"attn": ("fused", "two_pass"), "decode": ("graph", "eager")}[key]:
            raise SystemExit(f"bad arm switch {item!r}")
        arm[key] = value
    return arm


class Arm:
    """Context manager that puts the library into an arm's settings and restores the defaults."""

    def __init__(self, arm: dict):
        self.arm = arm

    def __enter__(self):
        from ttcd_b200 import ops
        ops.set_dual_attention_impl(self.arm["attn"])
        return self

    def __exit__(self, *exc):
        from ttcd_b200 import ops
        ops.set_dual_attention_impl("fused")

    @property
    def use_graph(self) -> bool:
        return self.arm["decode"] == "graph"


def run_tasks(model, tok, args, arm: dict) -> dict:
    import eval_ruler as ruler
    out = {}
    eos = {tok.eos_token_id} if tok.eos_token_id is not None else None
    with Arm(arm) as a:
        for ctx in args.ctx_lens:
            for task in args.tasks:
                path = ruler.find_file(Path(args.data_dir), task, ctx)
                if path is None:
                    print(f"[ab] no data for {task} @ {ctx}")
                    continue
                preds, refs = [], []
                for line in path.read_text().splitlines()[: args.max_samples]:
                    d = json.loads(line)
                    prompt = d["input"] + (d.get("answer_prefix") or "")
                    ids = tok(prompt, return_tensors="pt", add_special_tokens=False).input_ids.to(args.device)
                    from eval_common import greedy_decode
                    toks = greedy_decode(model, ids, args.max_new_tokens, eos, use_graph=a.use_graph)
                    preds.append(tok.decode(toks, skip_special_tokens=True))
                    refs.append(d["outputs"])
                out[f"{task}@{ctx}"] = {"n": len(preds), "accuracy": ruler.string_match_all(preds, refs), "predictions": preds}
                print(f"[ab] {arm} {task}@{ctx}: {out[f'{task}@{ctx}']['accuracy']:.1f} (n={len(preds)})", flush=True)
    return out


def load_docs(args, tok, vocab: int, n: int) -> list[list[int]]:
    if args.ppl_dir:
        from eval_token_ppl import load_windows
        windows, _ = load_windows(args.ppl_dir, tok, args.seq_len, n, 0, 0, 0)
        return [list(w) for w in windows]
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, vocab, (n, args.seq_len), generator=g).tolist()


@torch.no_grad()
def nll_and_divergence(model, docs, args, arm_a: dict, arm_b: dict, kl_docs: int) -> dict:
    """Mean NLL per arm over every document; KL(p_a || p_b), top-1 flips and the largest logit gap over the first
    ``kl_docs`` of them (both arms' full logits of one document are alive at once there)."""
    nll = {"a": [], "b": []}
    kls, flips, positions, max_gap = [], 0, 0, 0.0
    for i, doc in enumerate(docs):
        ids = torch.tensor([doc], device=args.device)
        if i < kl_docs:
            with Arm(arm_a):
                la = model(input_ids=ids, use_cache=False).logits
            with Arm(arm_b):
                lb = model(input_ids=ids, use_cache=False).logits
            for c0 in range(0, la.shape[1], 2048):
                pa = torch.log_softmax(la[0, c0:c0 + 2048].float(), -1)
                pb = torch.log_softmax(lb[0, c0:c0 + 2048].float(), -1)
                kls.append((pa.exp() * (pa - pb)).sum(-1).cpu())
                flips += int((pa.argmax(-1) != pb.argmax(-1)).sum())
                max_gap = max(max_gap, float((la[0, c0:c0 + 2048].float() - lb[0, c0:c0 + 2048].float()).abs().max()))
                positions += pa.shape[0]
            for key, lg in (("a", la), ("b", lb)):
                lp_sum, n = 0.0, 0
                for c0 in range(0, lg.shape[1] - 1, 2048):
                    lp = torch.log_softmax(lg[0, c0:min(c0 + 2048, lg.shape[1] - 1)].float(), -1)
                    tgt = ids[0, c0 + 1:c0 + 1 + lp.shape[0]]
                    lp_sum += float(-lp.gather(-1, tgt[:, None]).sum())
                    n += lp.shape[0]
                nll[key].append(lp_sum / max(1, n))
            del la, lb
        else:
            for key, arm in (("a", arm_a), ("b", arm_b)):
                with Arm(arm):
                    nll[key].append(float(token_nll(model, ids).mean()))
    res = {"docs": len(docs), "mean_nll_a": sum(nll["a"]) / max(1, len(docs)), "mean_nll_b": sum(nll["b"]) / max(1, len(docs))}
    res["nll_diff"] = res["mean_nll_b"] - res["mean_nll_a"]
    if kls:
        kl = torch.cat(kls).double()
        q = lambda p: float(torch.quantile(kl[:: max(1, kl.numel() // 1_000_000)], p))  # noqa: E731
        res.update(kl_tokens=int(kl.numel()), kl_p50=q(0.5), kl_p90=q(0.9), kl_p99=q(0.99), kl_max=float(kl.max()),
                   top1_flip_rate=flips / max(1, positions), max_abs_logit_diff=max_gap)
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_model_args(ap)
    ap.add_argument("--arm_a", default="attn=two_pass,decode=eager")
    ap.add_argument("--arm_b", default="attn=fused,decode=graph")
    ap.add_argument("--data_dir", default=None)
    ap.add_argument("--tasks", nargs="+", default=["niah_single_1", "niah_single_2", "niah_multikey_1", "niah_multiquery"])
    ap.add_argument("--ctx_lens", nargs="+", type=int, default=[32768, 65536])
    ap.add_argument("--max_samples", type=int, default=25)
    ap.add_argument("--max_new_tokens", type=int, default=128)
    ap.add_argument("--ppl_dir", default=None)
    ap.add_argument("--seq_len", type=int, default=65536)
    ap.add_argument("--ppl_docs", type=int, default=16)
    ap.add_argument("--kl_docs", type=int, default=8)
    ap.add_argument("--max_flip_rate", type=float, default=5e-3)
    ap.add_argument("--max_nll_diff", type=float, default=1e-3)
    ap.add_argument("--output", default="eval_results/ab.json")
    args = ap.parse_args(argv)
    arm_a, arm_b = parse_arm(args.arm_a), parse_arm(args.arm_b)
    tok = load_tokenizer(args.tokenizer) if (args.data_dir or args.ppl_dir) else None
    model = load_model(args)
    report: dict = {"arm_a": arm_a, "arm_b": arm_b}
    agree = True
    if args.data_dir:
        res_a, res_b = run_tasks(model, tok, args, arm_a), run_tasks(model, tok, args, arm_b)
        rows, same_total, n_total = {}, 0, 0
        for key in res_a:
            a, b = res_a[key], res_b[key]
            same = sum(x.strip() == y.strip() for x, y in zip(a["predictions"], b["predictions"]))
            rows[key] = {"accuracy_a": a["accuracy"], "accuracy_b": b["accuracy"], "identical": same, "n": a["n"]}
            same_total, n_total = same_total + same, n_total + a["n"]
            flag = "" if a["accuracy"] == b["accuracy"] else "  <-- DIFF"
            print(f"{key:28s} a={a['accuracy']:5.1f} b={b['accuracy']:5.1f} identical={same}/{a['n']}{flag}")
        report["tasks"] = rows
        report["identical_predictions"] = [same_total, n_total]
        agree &= same_total == n_total
    if args.ppl_docs > 0:
        docs = load_docs(args, tok, model.config.vocab_size, args.ppl_docs)
        report["distribution"] = d = nll_and_divergence(model, docs, args, arm_a, arm_b, min(args.kl_docs, len(docs)))
        agree &= abs(d["nll_diff"]) <= args.max_nll_diff and d.get("top1_flip_rate", 0.0) <= args.max_flip_rate
        print(json.dumps(d))
    report["arms_agree"] = bool(agree)
    Path(args.output).parent.mkdir(parents=True, exist_ok=True)
    Path(args.output).write_text(json.dumps(report, indent=1))
    print(f"[ab] arms agree: {agree}")
    return report


if __name__ == "__main__":
    main()
