"""Kernel microbenchmarks: tensor-core GEMM, dual-window attention, chunked depthwise conv.

Each number is the median of CUDA-event timings taken after warm-up, with an L2 flush (a 256 MiB
write) between timed iterations, and is reported with the achieved fraction of the measured peaks
in MEASURED_PEAKS.json (cuBLAS bf16 burst throughput and copy bandwidth).  Library baselines
(cuBLAS via torch.matmul, flash-attn 2) are timed the same way when importable.

    python benchmarks/bench_kernels.py [--what gemm,attn,conv,attn_bwd] [--seq 65536] [--batch 1]
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from ttcd_b200 import _native  # noqa: E402
from ttcd_b200.ops import cuda  # noqa: E402

BF = torch.bfloat16


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return d["bf16_tflops"], d["hbm_gbs"], "measured"
    return 1590.0, 6650.0, "fallback"


_flush = None


def timeit(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def emit(**kw):
    print(json.dumps(kw), flush=True)


def bench_gemm():
    tf_peak, _, src = peaks()
    shapes = [
        ("qkv 64K", 65536, 4096, 1024, False, False), ("o_proj 64K", 65536, 1024, 2048, False, False),
        ("gate_up 64K", 65536, 6144, 1024, False, False), ("down 64K", 65536, 1024, 3072, False, False),
        ("dgrad down", 65536, 3072, 1024, False, True), ("wgrad gate_up", 6144, 1024, 65536, True, True),
        ("lm_head chunk", 8192, 151936, 1024, False, False), ("square 8192", 8192, 8192, 8192, False, False),
    ]
    for name, M, N, K, a_t, b_row in shapes:
        a = torch.randn((K, M) if a_t else (M, K), device="cuda", dtype=BF)
        b = torch.randn((K, N) if b_row else (N, K), device="cuda", dtype=BF)
        al = a.t() if a_t else a
        bl = b if b_row else b.t()
        out = torch.empty(1, M, N, device="cuda", dtype=BF)
        ms = timeit(lambda: cuda.gemm(al, bl, out=out))
        ms_lib = timeit(lambda: torch.matmul(al, bl))
        tf = 2.0 * M * N * K / ms / 1e9
        emit(bench="gemm", shape=name, M=M, N=N, K=K, ms=round(ms, 4), tflops=round(tf, 1),
             frac_of_peak=round(tf / tf_peak, 3), peak_source=src, cublas_ms=round(ms_lib, 4),
             vs_cublas=round(ms_lib / ms, 3))


def _flash():
    try:
        from flash_attn import flash_attn_func
        return flash_attn_func
    except Exception:
        return None


def attn_flops(B, T, H, D, w):
    # causal sliding window: each query sees min(i+1, w) keys; 2 GEMMs x 2 flops
    keys = sum(min(i + 1, w) for i in (0, T - 1)) / 2 * T if w >= T else (w * (w + 1) / 2 + (T - w) * w)
    return 4.0 * B * H * D * keys


def bench_attn(seqs, batches, wt=8192, ws=4096, bwd=False):
    tf_peak, _, src = peaks()
    H, HK, D = 16, 8, 128
    fa = _flash()
    for B in batches:
        for T in seqs:
            q = torch.randn(B, T, H, D, device="cuda", dtype=BF, requires_grad=bwd)
            k = torch.randn(B, T, HK, D, device="cuda", dtype=BF, requires_grad=bwd)
            v = torch.randn(B, T, HK, D, device="cuda", dtype=BF, requires_grad=bwd)
            sc = D ** -0.5
            row = dict(bench="attn_bwd" if bwd else "attn_fwd", B=B, T=T, w_t=wt, w_s=ws, peak_source=src)
            if not bwd:
                with torch.no_grad():
                    ms_dual = timeit(lambda: cuda.attn_forward(q, k, v, wt, ws, sc, True))
                    ms_t = timeit(lambda: cuda.attn_forward(q, k, v, wt, wt, sc, False))
                    ms_s = timeit(lambda: cuda.attn_forward(q, k, v, ws, ws, sc, False))
                    from ttcd_b200 import ops
                    ms_lse = timeit(lambda: ops.lse_dual_window_attention(q, k, v, wt, ws, sc))
                fl = attn_flops(B, T, H, D, wt)
                row.update(fused_dual_ms=round(ms_dual, 3), teacher_only_ms=round(ms_t, 3),
                           two_calls_ms=round(ms_t + ms_s, 3), lse_variant_ms=round(ms_lse, 3), fused_tflops=round(fl / ms_dual / 1e9, 1),
                           frac_of_peak=round(fl / ms_dual / 1e9 / tf_peak, 3))
                if fa is not None:
                    with torch.no_grad():
                        ms_fa_t = timeit(lambda: fa(q, k, v, causal=True, window_size=(wt - 1, 0)))
                        ms_fa_s = timeit(lambda: fa(q, k, v, causal=True, window_size=(ws - 1, 0)))
                    row.update(fa2_teacher_ms=round(ms_fa_t, 3), fa2_two_calls_ms=round(ms_fa_t + ms_fa_s, 3),
                               speedup_vs_fa2_two_calls=round((ms_fa_t + ms_fa_s) / ms_dual, 2))
            else:
                o_t, o_s, _, _ = cuda._Attention.apply(q, k, v, wt, ws, sc, True)
                g_t, g_s = torch.randn_like(o_t), torch.randn_like(o_s)
                ms = timeit(lambda: torch.autograd.grad([o_t, o_s], [q, k, v], [g_t, g_s], retain_graph=True), iters=5)
                fl = 2.5 * attn_flops(B, T, H, D, wt) + 2.5 * attn_flops(B, T, H, D, ws)  # two separate backward passes
                row.update(fused_dual_bwd_ms=round(ms, 3), tflops=round(fl / ms / 1e9, 1))
                o1, _ = cuda._Attention.apply(q, k, v, wt, wt, sc, False)
                ms1 = timeit(lambda: torch.autograd.grad([o1], [q, k, v], [g_t], retain_graph=True), iters=5)
                fl1 = 2.5 * attn_flops(B, T, H, D, wt)  # algorithmic: 5 GEMMs
                row.update(single_window_bwd_ms=round(ms1, 3), single_tflops=round(fl1 / ms1 / 1e9, 1),
                           single_frac_of_peak=round(fl1 / ms1 / 1e9 / tf_peak, 3))
                if fa is not None:
                    ft = fa(q, k, v, causal=True, window_size=(wt - 1, 0))
                    fs = fa(q, k, v, causal=True, window_size=(ws - 1, 0))
                    ms_fa = timeit(lambda: torch.autograd.grad([ft, fs], [q, k, v], [g_t, g_s], retain_graph=True), iters=5)
                    row.update(fa2_two_bwd_ms=round(ms_fa, 3), speedup_vs_fa2=round(ms_fa / ms, 2))
            emit(**row)
            del q, k, v
            torch.cuda.empty_cache()


def bench_conv():
    _, bw_peak, src = peaks()
    for K in (5, 4):
        x = torch.randn(1, 16, 4096, 3072, device="cuda", dtype=BF)
        w = (torch.randn(3072, K, device="cuda") * 0.3).to(BF)
        with torch.no_grad():
            ms = timeit(lambda: cuda.dwconv_chunked(x, w, True))
        gb = 2 * x.numel() * 2 / 1e9
        row = dict(bench="dwconv_fwd", K=K, shape=list(x.shape), ms=round(ms, 4), gbs=round(gb / ms * 1e3, 1),
                   frac_of_copy_bw=round(gb / ms * 1e3 / bw_peak, 3), peak_source=src)
        xr = x.clone().requires_grad_()
        wr = w.clone().requires_grad_()
        y = cuda.dwconv_chunked(xr, wr, True)
        g = torch.randn_like(y)
        ms_b = timeit(lambda: torch.autograd.grad(y, [xr, wr], g, retain_graph=True), iters=5)
        row.update(bwd_ms=round(ms_b, 4))
        conv = torch.nn.Conv1d(3072, 3072, K, groups=3072, bias=False, device="cuda", dtype=BF)

        def cudnn_path():
            xf = x.view(16, 4096, 3072).transpose(1, 2)
            return conv(torch.nn.functional.pad(xf, (K - 1, 0))).transpose(1, 2)

        with torch.no_grad():
            row.update(cudnn_path_ms=round(timeit(cudnn_path), 4))
        emit(**row)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,attn,conv")
    ap.add_argument("--seq", default="65536")
    ap.add_argument("--batch", default="1")
    args = ap.parse_args()
    _native.load(required=True)
    what = args.what.split(",")
    seqs = [int(s) for s in args.seq.split(",")]
    batches = [int(s) for s in args.batch.split(",")]
    if "gemm" in what:
        bench_gemm()
    if "attn" in what:
        bench_attn(seqs, batches)
    if "attn_bwd" in what:
        bench_attn(seqs, batches, bwd=True)
    if "conv" in what:
        bench_conv()
    st = _native.device_status()
    if st:
        emit(error=f"device status {st}")


if __name__ == "__main__":
    main()
