"""Tables (markdown on stdout, optional CSV) and figures (matplotlib when it is installed, plain SVG line charts
otherwise) from the JSON files the evaluation and benchmark scripts write.  One sub-command per result kind:

    python scripts/report_results.py niah --inputs base=eval/niah_base.json ttcd=eval/niah_ttcd.json [--fig out.png]
    python scripts/report_results.py token-ppl --inputs base=eval/ppl_base.json ttcd=eval/ppl_ttcd.json [--fig out.png]
    python scripts/report_results.py final-block --input eval/ffb_all/fixed_final_block_doc_ppl.json [--fig out.png]
    python scripts/report_results.py prefill --inputs 'results/*.json' [--fig out.png]

* ``niah``: accuracy per task and context length of ``eval_ruler.py`` / ``eval_niah.py`` outputs, one block per task
  with one row per model (the figure of the reference's scripts/plot_niah.py as a table).
* ``token-ppl``: mean NLL per position bucket (0-2K, 2K-4K, ...) of ``eval_token_ppl.py`` outputs
  (reference scripts/plot_token_ppl.py plots the same curves).
* ``final-block``: perplexity of the fixed final block per context length and model.
* ``prefill``: median milliseconds per (model, mode, sequence length) of ``benchmarks/bench_prefill.py --out`` files
  (reference profiling/summarize.py:10-44; the figure is the role of its profiling/plot_sweep.py / plot_bsz.py curves).

Without matplotlib a figure is written as ``<name>.svg`` by a small built-in SVG writer; the tables never need either.
"""
from __future__ import annotations

import argparse
import glob
import json
import math
from pathlib import Path

BUCKET_EDGES = [0, 2048, 4096, 8192, 16384, 32768, 65536, 131072]


def _named(items: list[str]) -> dict[str, Path]:
    out = {}
    for item in items:
        name, sep, path = item.partition("=")
        out[name if sep else Path(item).stem] = Path(path if sep else item)
    return out


def _table(header: list[str], rows: list[list]) -> str:
    fmt = lambda c: "-" if c is None else (f"{c:.2f}" if isinstance(c, float) else str(c))  # noqa: E731
    lines = ["| " + " | ".join(header) + " |", "|" + "---|" * len(header)]
    lines += ["| " + " | ".join(fmt(c) for c in r) + " |" for r in rows]
    return "\n".join(lines)


class _SvgAxes:
    """The few ``Axes`` calls the figures below make, drawn as a plain SVG file (line charts with markers, a legend,
    linear or log-2 x axis): the fallback when matplotlib cannot be imported."""
    COLORS = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#17becf", "#7f7f7f"]

    def __init__(self):
        self.series, self.xlog, self.xlabel, self.ylabel = [], False, "", ""

    def plot(self, x, y, marker=None, label=None, **_):
        pts = [(float(a), float(b)) for a, b in zip(x, y) if a is not None and b is not None]
        self.series.append((pts, bool(marker), label or f"series {len(self.series) + 1}"))
        return []

    def set_xscale(self, kind, base=2, **_):
        self.xlog = kind == "log"

    def set_xlabel(self, text):
        self.xlabel = text

    def set_ylabel(self, text):
        self.ylabel = text

    def grid(self, *_, **__):
        pass

    def legend(self, *_, **__):
        pass

    def save(self, path: Path, width=800, height=450) -> None:
        left, right, top, bottom = 70, 20, 20, 55
        fx = (lambda v: math.log2(v)) if self.xlog else (lambda v: v)
        pts = [(fx(a), b) for s_, _m, _l in self.series for a, b in s_ if not self.xlog or a > 0]
        if not pts:
            pts = [(0.0, 0.0), (1.0, 1.0)]
        x0, x1 = min(p[0] for p in pts), max(p[0] for p in pts)
        y0, y1 = min(p[1] for p in pts), max(p[1] for p in pts)
        x1, y1 = (x1 if x1 > x0 else x0 + 1.0), (y1 if y1 > y0 else y0 + 1.0)
        pad = 0.05 * (y1 - y0)
        y0, y1 = y0 - pad, y1 + pad
        sx = lambda v: left + (fx(v) - x0) / (x1 - x0) * (width - left - right)  # noqa: E731
        sy = lambda v: height - bottom - (v - y0) / (y1 - y0) * (height - top - bottom)  # noqa: E731
        out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="12">',
               f'<rect width="{width}" height="{height}" fill="white"/>']
        for i in range(6):                                           # horizontal grid lines and y tick labels
            v = y0 + (y1 - y0) * i / 5
            out.append(f'<line x1="{left}" y1="{sy(v):.1f}" x2="{width - right}" y2="{sy(v):.1f}" stroke="#dddddd"/>')
            out.append(f'<text x="{left - 6}" y="{sy(v) + 4:.1f}" text-anchor="end">{v:.3g}</text>')
        ticks = sorted({a for s_, _m, _l in self.series for a, _b in s_}) if self.xlog else [x0 + (x1 - x0) * i / 5 for i in range(6)]
        for v in ticks[:: max(1, len(ticks) // 10)]:
            if self.xlog and v <= 0:
                continue
            out.append(f'<line x1="{sx(v):.1f}" y1="{top}" x2="{sx(v):.1f}" y2="{height - bottom}" stroke="#eeeeee"/>')
            out.append(f'<text x="{sx(v):.1f}" y="{height - bottom + 16}" text-anchor="middle">{v:.6g}</text>')
        out.append(f'<rect x="{left}" y="{top}" width="{width - left - right}" height="{height - top - bottom}" fill="none" stroke="black"/>')
        for k, (series, marker, label) in enumerate(self.series):
            color = self.COLORS[k % len(self.COLORS)]
            series = [(a, b) for a, b in series if not self.xlog or a > 0]
            if series:
                path_pts = " ".join(f"{sx(a):.1f},{sy(b):.1f}" for a, b in series)
                out.append(f'<polyline points="{path_pts}" fill="none" stroke="{color}" stroke-width="1.6"/>')
                if marker:
                    out += [f'<circle cx="{sx(a):.1f}" cy="{sy(b):.1f}" r="3" fill="{color}"/>' for a, b in series]
            out.append(f'<rect x="{left + 10}" y="{top + 8 + 16 * k}" width="12" height="3" fill="{color}"/>')
            out.append(f'<text x="{left + 28}" y="{top + 14 + 16 * k}">{label}</text>')
        out.append(f'<text x="{(left + width - right) / 2:.0f}" y="{height - 12}" text-anchor="middle">{self.xlabel}</text>')
        out.append(f'<text x="16" y="{(top + height - bottom) / 2:.0f}" text-anchor="middle" '
                   f'transform="rotate(-90 16 {(top + height - bottom) / 2:.0f})">{self.ylabel}</text>')
        out.append("</svg>")
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text("\n".join(out))


def _figure(path: str | None, draw) -> None:
    """``draw(ax)`` into ``path`` with matplotlib, or, where it is not installed, as an SVG file beside it."""
    if not path:
        return
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        ax = _SvgAxes()
        draw(ax)
        target = Path(path).with_suffix(".svg")
        ax.save(target)
        print(f"(matplotlib is not installed: wrote {target} instead)")
        return
    fig, ax = plt.subplots(figsize=(8, 4.5), constrained_layout=True)
    draw(ax)
    ax.grid(True, alpha=0.3)
    ax.legend(frameon=False)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    fig.savefig(path, dpi=160)
    plt.close(fig)


def niah_tables(results: dict[str, dict]) -> tuple[str, dict]:
    """results: model name -> {ctx: {task: {"accuracy"}}}; returns markdown and {task: {model: {ctx: acc}}}."""
    ctxs = sorted({int(c) for r in results.values() for c in r})
    tasks = sorted({t for r in results.values() for per in r.values() for t in per})
    by_task, blocks = {}, []
    for task in tasks:
        rows = []
        for name, r in results.items():
            accs = {c: (r.get(str(c), {}).get(task)) for c in ctxs}
            accs = {c: (a["accuracy"] if isinstance(a, dict) else a) for c, a in accs.items()}
            by_task.setdefault(task, {})[name] = accs
            rows.append([name] + [None if accs[c] is None else float(accs[c]) for c in ctxs])
        blocks.append(f"**{task}**\n\n" + _table(["model"] + [str(c) for c in ctxs], rows))
    return "\n\n".join(blocks), by_task


def bucket_means(curve: list[float]) -> dict[str, float]:
    out = {}
    for a, b in zip(BUCKET_EDGES[:-1], BUCKET_EDGES[1:]):
        seg = curve[a:b]
        if seg:
            out[f"{a}-{b}"] = sum(seg) / len(seg)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("niah", "token-ppl"):
        p = sub.add_parser(name)
        p.add_argument("--inputs", nargs="+", required=True, help="name=path.json ...")
        p.add_argument("--fig", default=None)
    p = sub.add_parser("final-block")
    p.add_argument("--input", required=True)
    p.add_argument("--fig", default=None)
    p = sub.add_parser("prefill")
    p.add_argument("--fig", default=None)
    p.add_argument("--inputs", nargs="+", required=True, help="files or globs written by bench_prefill.py --out")
    args = ap.parse_args(argv)

    if args.what == "niah":
        results = {n: json.loads(p.read_text()) for n, p in _named(args.inputs).items()}
        text, by_task = niah_tables(results)
        print(text)
        avg = by_task.get("average")
        if avg:
            _figure(args.fig, lambda ax: [ax.plot(list(v), [v[c] for c in v], marker="o", label=n) for n, v in avg.items()]
                    and (ax.set_xscale("log", base=2), ax.set_xlabel("context length"), ax.set_ylabel("accuracy")))
    elif args.what == "token-ppl":
        curves = {}
        for n, p in _named(args.inputs).items():
            d = json.loads(p.read_text())
            curves[n] = d.get("nll_per_position") or d.get("avg_nll")
        buckets = {n: bucket_means(c) for n, c in curves.items()}
        cols = sorted({b for v in buckets.values() for b in v}, key=lambda s: int(s.split("-")[0]))
        rows = [[n] + [v.get(b) for b in cols] + [math.exp(sum(curves[n]) / len(curves[n]))] for n, v in buckets.items()]
        print(_table(["model"] + cols + ["ppl"], rows))

        def draw(ax):
            for n, c in curves.items():
                step = max(1, len(c) // 512)
                xs = list(range(0, len(c) - step + 1, step))
                ax.plot(xs, [sum(c[x:x + step]) / step for x in xs], lw=1.2, label=n)
            ax.set_xlabel("position")
            ax.set_ylabel("NLL")
        _figure(args.fig, draw)
    elif args.what == "final-block":
        d = json.loads(Path(args.input).read_text())
        ctxs = d["meta"]["context_lens"]
        rows = [[n] + [r["perplexity"] for r in rows_] for n, rows_ in d["results"].items()]
        print(_table(["model"] + [str(c) for c in ctxs], rows))

        def draw(ax):
            for n, rows_ in d["results"].items():
                pts = [(r["context_len"], r["perplexity"]) for r in rows_ if r["perplexity"] is not None]
                ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", label=n)
            ax.set_xscale("log", base=2)
            ax.set_xlabel("same-document context before the block")
            ax.set_ylabel("perplexity of the final block")
        _figure(args.fig, draw)
    else:
        cells: dict[tuple, dict[int, float]] = {}
        for pat in args.inputs:
            for path in sorted(glob.glob(pat)):
                try:
                    rows = json.loads(Path(path).read_text())
                except (OSError, json.JSONDecodeError):
                    continue
                for r in rows if isinstance(rows, list) else []:
                    if r.get("bench") != "prefill":
                        continue
                    label = r["model"] + ("" if r.get("ablation", "full") == "full" else f"[{r['ablation']}]")
                    label += "" if r.get("attn_impl", "fused") == "fused" else f"({r['attn_impl']})"
                    cells.setdefault((r["mode"], label), {})[int(r["L"])] = float(r["ms_median"])
        lens = sorted({L for v in cells.values() for L in v})
        for mode in sorted({m for m, _ in cells}):
            print(f"\n**{mode}** (median ms)\n")
            print(_table(["model"] + [f"L={L}" for L in lens],
                         [[label] + [v.get(L) for L in lens] for (m, label), v in sorted(cells.items()) if m == mode]))

        def draw(ax):            # one curve per (mode, model): median ms against the prompt length
            for (mode, label), v in sorted(cells.items()):
                xs = sorted(v)
                ax.plot(xs, [v[L] for L in xs], marker="o", label=f"{label} / {mode}")
            ax.set_xscale("log", base=2)
            ax.set_xlabel("prompt length")
            ax.set_ylabel("median ms")
        _figure(getattr(args, "fig", None), draw)


if __name__ == "__main__":
    main()
