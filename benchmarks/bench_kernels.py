"""Kernel microbenchmarks: tensor-core GEMM, dual-window attention, chunked depthwise conv.

Each number is the median of CUDA-event timings taken after warm-up, with an L2 flush (a 256 MiB
write) between timed iterations, and is reported with the achieved fraction of the measured peaks
in MEASURED_PEAKS.json (cuBLAS bf16 burst throughput and copy bandwidth).  Library baselines
(cuBLAS via torch.matmul, flash-attn 2) are timed the same way when importable.

    python benchmarks/bench_kernels.py [--what gemm,attn,conv,attn_bwd,misc,delta,ref,ref_misc] [--seq 65536] [--batch 1]

``--what ref`` times the reference project's own kernels on this GPU next to this library's: its fused dual-window
Triton kernel (profiling/fused_dual_attn.py:244-272), its LSE-combination variant on flash-attn 2
(profiling/lse_dual_attn.py:16-39), two flash-attn calls, and its Triton chunked depthwise conv
(profiling/fused_conv.py:51-61) against the cuDNN path.  They are imported, unmodified, from the reference checkout
(``TTCD_REFERENCE_ROOT``, a ``reference`` directory beside this repository, or ``baseline/_ref``).
``--what ref_misc`` does the same for its fla Triton add+RMSNorm, rotary, SwiGLU and fused linear-cross-entropy kernels
(fla/modules/{layernorm,rotary,activations,fused_linear_cross_entropy}.py).
``--what delta`` times the stages of the chunked delta rule (chunk-local kernels, chain kernels, the whole op forward +
backward) at the 340M shapes of the two delta families, 4096-token sequences, ``--batch`` sequences (16 in the model
benchmarks), beside the PyTorch statement of the rule and, when the reference checkout is importable, its Triton
``chunk_delta_rule`` / ``chunk_gated_delta_rule`` (fla/ops/delta_rule/chunk.py, fla/ops/gated_delta_rule/chunk.py);
``--what delta_stages`` times the kernels only (the small case for a profiler capture).
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
                o_t, o_s, _, _ = cuda._Attention.apply(q, k, v, wt, ws, sc, True, None, None)
                g_t, g_s = torch.randn_like(o_t), torch.randn_like(o_s)
                ms = timeit(lambda: torch.autograd.grad([o_t, o_s], [q, k, v], [g_t, g_s], retain_graph=True), iters=5)
                fl = 2.5 * attn_flops(B, T, H, D, wt) + 2.5 * attn_flops(B, T, H, D, ws)  # two separate backward passes
                row.update(fused_dual_bwd_ms=round(ms, 3), tflops=round(fl / ms / 1e9, 1))
                o1, _ = cuda._Attention.apply(q, k, v, wt, wt, sc, False, None, None)
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


def bench_misc():
    """Fast-weight scan, linear-cross-entropy, Newton-Schulz and add+RMSNorm at the flagship shapes against plain
    PyTorch statements of the same ops (cuBLAS matmuls, materialised logits)."""
    from ttcd_b200 import ops
    from ttcd_b200.ops import reference as ref
    torch.manual_seed(0)
    # --- fast-weight chunk scan: 1 x 16 chunks x 4096 tokens, d_i 3072, d_h 1024 (one TTT layer at 64K)
    b, T, C, d_i, d_h = 1, 16, 4096, 3072, 1024
    mk = lambda *sh, sc=1.0: (torch.randn(*sh, device="cuda") * sc).to(BF).requires_grad_()  # noqa: E731
    z_out, z_tgt, z_hat = mk(b, T, C, d_i, sc=0.3), mk(b, T, C, d_i, sc=0.3), mk(b, T, C, d_i, sc=0.3)
    beta = torch.sigmoid(torch.randn(b, T, C, 1, device="cuda")).to(BF).requires_grad_()
    w_down, w_upd = mk(d_h, d_i, sc=0.02), mk(d_i, d_h, sc=0.02)
    ins = [z_out, z_tgt, z_hat, beta, w_down, w_upd]

    def scan_fused():
        y = ops.ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_upd, lr=0.3, update_every=2)
        return torch.autograd.grad(y, ins, torch.ones_like(y))

    def scan_torch():
        y = ref.ttt_scan(z_out, z_tgt, z_hat, beta, w_down, w_upd, lr=0.3, update_every=2, state_dtype=torch.bfloat16)
        return torch.autograd.grad(y, ins, torch.ones_like(y))

    emit(bench="ttt_scan_fwd_bwd", shape=[b, T, C, d_i, d_h], fused_ms=round(timeit(scan_fused, iters=5), 3),
         torch_cublas_ms=round(timeit(scan_torch, iters=5), 3))
    del z_out, z_tgt, z_hat, beta, ins
    # --- linear-cross-entropy: 65536 tokens x 1024 -> 151936 classes
    n, hdim, vocab = 65536, 1024, 151936
    hid = (torch.randn(n, hdim, device="cuda") * 0.5).to(BF).requires_grad_()
    w = (torch.randn(vocab, hdim, device="cuda") * 0.02).to(BF).requires_grad_()
    labels = torch.randint(0, vocab, (n,), device="cuda")

    def lce():
        return torch.autograd.grad(ops.linear_cross_entropy(hid, labels, w), [hid, w])

    def lce_torch():                                  # chunked so that the fp32 logits fit: 8 x [8192, vocab]
        tot = 0.0
        gh = torch.zeros_like(hid)
        gw = torch.zeros_like(w, dtype=torch.float32)
        for c0 in range(0, n, 8192):
            hc = hid[c0:c0 + 8192].detach().requires_grad_()
            wc = w.detach().requires_grad_()
            loss = torch.nn.functional.cross_entropy((hc @ wc.t()).float(), labels[c0:c0 + 8192], reduction="sum") / n
            a, b_ = torch.autograd.grad(loss, [hc, wc])
            gh[c0:c0 + 8192] = a
            gw += b_
            tot += float(loss.detach())
        return tot

    emit(bench="linear_cross_entropy_fwd_bwd", tokens=n, hidden=hdim, vocab=vocab, fused_ms=round(timeit(lce, iters=3), 3),
         torch_cublas_ms=round(timeit(lce_torch, iters=3, warmup=1), 3), tflops=round(6 * n * hdim * vocab / 1e12, 1))
    del hid, w
    # --- Newton-Schulz (5 steps) on the model's matrices
    for shape in ((3072, 1024), (2048, 1024), (1024, 1024)):
        g = torch.randn(*shape, device="cuda").to(BF)
        with torch.no_grad():
            emit(bench="newton_schulz5", shape=list(shape), fused_ms=round(timeit(lambda: ops.newton_schulz(g)), 4),
                 torch_cublas_ms=round(timeit(lambda: ref.newton_schulz(g)), 4))
    # --- add + RMSNorm, 65536 x 1024
    _, bw_peak, src = peaks()
    x = torch.randn(65536, 1024, device="cuda").to(BF).requires_grad_()
    res = torch.randn(65536, 1024, device="cuda").to(BF)
    wn = torch.ones(1024, device="cuda", dtype=BF, requires_grad=True)
    with torch.no_grad():
        ms_f = timeit(lambda: ops.rmsnorm(x, wn, 1e-6, residual=res, prenorm=True))
    y, _ = ops.rmsnorm(x, wn, 1e-6, residual=res, prenorm=True)
    gy = torch.randn_like(y)
    ms_b = timeit(lambda: torch.autograd.grad(y, [x, wn], gy, retain_graph=True))
    gb_f = 4 * x.numel() * 2 / 1e9          # x, residual in; y, new residual out
    emit(bench="add_rmsnorm", shape=[65536, 1024], fwd_ms=round(ms_f, 4), fwd_frac_of_copy_bw=round(gb_f / ms_f * 1e3 / bw_peak, 3),
         bwd_ms=round(ms_b, 4), peak_source=src)


def _reference_profiling():
    """The reference checkout's ``profiling`` directory on sys.path; returns it, or None when it is not there."""
    import os
    cands = [os.environ.get("TTCD_REFERENCE_ROOT"), str(ROOT.parent / "reference"), str(ROOT / "baseline" / "_ref")]
    for c in cands:
        if c and (Path(c) / "profiling" / "fused_dual_attn.py").is_file():
            if c not in sys.path:
                sys.path.insert(0, c)
            return Path(c)
    return None


def bench_reference(seqs, batches, wt=8192, ws=4096):
    """The reference's kernels, run on this GPU, beside this library's (same inputs, same timing)."""
    root = _reference_profiling()
    if root is None:
        emit(bench="reference", error="reference checkout with profiling/ not found")
        return
    from profiling.fused_dual_attn import fused_dual_window_attn
    from profiling.lse_dual_attn import lse_dual_window_attn
    from profiling.fused_conv import causal_dwconv_chunked
    fa = _flash()
    H, HK, D = 16, 8, 128
    sc = D ** -0.5
    for B in batches:
        for T in seqs:
            q = torch.randn(B, T, H, D, device="cuda", dtype=BF)
            k = torch.randn(B, T, HK, D, device="cuda", dtype=BF)
            v = torch.randn(B, T, HK, D, device="cuda", dtype=BF)
            row = dict(bench="reference_attn_fwd", B=B, T=T, w_t=wt, w_s=ws)
            with torch.no_grad():
                ours = timeit(lambda: cuda.attn_forward(q, k, v, wt, ws, sc, True))
                row["ours_fused_ms"] = round(ours, 3)
                try:
                    o_ref = fused_dual_window_attn(q, k, v, wt, ws)
                    row["ref_triton_fused_ms"] = round(timeit(lambda: fused_dual_window_attn(q, k, v, wt, ws)), 3)
                    o_t = cuda.attn_forward(q, k, v, wt, ws, sc, True)[1]
                    row["max_abs_diff_vs_ref_teacher"] = round(float((o_t.float() - o_ref[0].float()).abs().max()), 5)
                except Exception as exc:
                    row["ref_triton_fused_error"] = f"{type(exc).__name__}: {exc}"[:160]
                try:
                    row["ref_lse_fa2_ms"] = round(timeit(lambda: lse_dual_window_attn(q, k, v, wt, ws)), 3)
                except Exception as exc:
                    row["ref_lse_fa2_error"] = f"{type(exc).__name__}: {exc}"[:160]
                if fa is not None:
                    ms_t = timeit(lambda: fa(q, k, v, causal=True, window_size=(wt - 1, 0)))
                    ms_s = timeit(lambda: fa(q, k, v, causal=True, window_size=(ws - 1, 0)))
                    row["ref_two_fa2_calls_ms"] = round(ms_t + ms_s, 3)
            best = min(v_ for k_, v_ in row.items() if k_.startswith("ref_") and k_.endswith("_ms"))
            row["speedup_vs_best_reference"] = round(best / ours, 2)
            emit(**row)
            del q, k, v
            torch.cuda.empty_cache()
    for K in (5, 4):
        for B in batches:
            x = torch.randn(B, 16, 4096, 3072, device="cuda", dtype=BF)
            conv = torch.nn.Conv1d(3072, 3072, K, groups=3072, bias=False, device="cuda", dtype=BF)
            w = conv.weight.detach().view(3072, K).contiguous()
            row = dict(bench="reference_dwconv_fwd", K=K, shape=list(x.shape))
            with torch.no_grad():
                row["ours_ms"] = round(timeit(lambda: cuda.dwconv_chunked(x, w, True)), 4)
                try:
                    y_ref = causal_dwconv_chunked(x, conv)
                    row["ref_triton_ms"] = round(timeit(lambda: causal_dwconv_chunked(x, conv)), 4)
                    row["max_abs_diff_vs_ref"] = round(float((cuda.dwconv_chunked(x, w, True).float() - y_ref.float()).abs().max()), 5)
                except Exception as exc:
                    row["ref_triton_error"] = f"{type(exc).__name__}: {exc}"[:160]

                def cudnn_path():                    # the reference's training path (modeling_ipttcdv9.py:203-211)
                    xf = x.view(B * 16, 4096, 3072).transpose(1, 2)
                    return conv(torch.nn.functional.pad(xf, (K - 1, 0))).transpose(1, 2)
                row["ref_cudnn_path_ms"] = round(timeit(cudnn_path), 4)
            emit(**row)
            del x
            torch.cuda.empty_cache()


def bench_reference_misc():
    """The reference's element-wise and loss kernels (fla Triton: add+RMSNorm, rotary, SwiGLU, fused linear
    cross-entropy), forward + backward on this GPU beside this library's, flagship shapes."""
    root = _reference_profiling()
    if root is None:
        emit(bench="reference_misc", error="reference checkout not found")
        return
    from ttcd_b200 import ops
    from ttcd_b200.ops import reference as ref
    try:
        from fla.modules import FusedLinearCrossEntropyLoss, RMSNorm, RotaryEmbedding
        from fla.modules.activations import swiglu as fla_swiglu
    except Exception as exc:
        emit(bench="reference_misc", error=f"{type(exc).__name__}: {exc}"[:200])
        return
    torch.manual_seed(0)
    T, d = 65536, 1024

    def guarded(row, key, fn, **kw):
        try:
            row[key] = round(timeit(fn, **kw), 4)
        except Exception as exc:
            row[key.replace("_ms", "_error")] = f"{type(exc).__name__}: {exc}"[:160]

    # --- add + RMSNorm (prenorm: returns the normalised rows and the new residual)
    x = torch.randn(1, T, d, device="cuda").to(BF).requires_grad_()
    res = torch.randn(1, T, d, device="cuda").to(BF).requires_grad_()
    w = torch.ones(d, device="cuda", dtype=BF).requires_grad_()
    g1, g2 = torch.randn(1, T, d, device="cuda").to(BF), torch.randn(1, T, d, device="cuda").to(BF)
    norm = RMSNorm(d, eps=1e-6).to("cuda", BF)
    row = dict(bench="reference_add_rmsnorm_fwd_bwd", shape=[T, d])
    guarded(row, "ours_ms", lambda: torch.autograd.grad(ops.rmsnorm(x, w, 1e-6, residual=res, prenorm=True), [x, res, w], [g1, g2]))
    guarded(row, "ref_triton_ms", lambda: torch.autograd.grad(norm(x, res, True), [x, res, norm.weight], [g1, g2]))
    emit(**row)
    # --- SwiGLU
    a = torch.randn(T, 3072, device="cuda").to(BF).requires_grad_()
    b = torch.randn(T, 3072, device="cuda").to(BF).requires_grad_()
    g = torch.randn(T, 3072, device="cuda").to(BF)
    row = dict(bench="reference_swiglu_fwd_bwd", shape=[T, 3072])
    guarded(row, "ours_ms", lambda: torch.autograd.grad(ops.swiglu(a, b), [a, b], g))
    guarded(row, "ref_triton_ms", lambda: torch.autograd.grad(fla_swiglu(a, b), [a, b], g))
    emit(**row)
    del a, b, g
    # --- rotary on q [1, T, 16, 128] and k [1, T, 8, 128] (this library fuses the per-head q/k RMSNorm into the same pass)
    q = torch.randn(1, T, 16, 128, device="cuda").to(BF).requires_grad_()
    k = torch.randn(1, T, 8, 128, device="cuda").to(BF).requires_grad_()
    gq, gk = torch.randn_like(q), torch.randn_like(k)
    cos, sin = ref.rope_tables(128, 1e6, T, device="cuda", dtype=BF)
    qw = torch.ones(128, device="cuda", dtype=BF).requires_grad_()
    kw = torch.ones(128, device="cuda", dtype=BF).requires_grad_()
    rot = RotaryEmbedding(128, base=1e6).to("cuda")
    qn, kn = RMSNorm(128, eps=1e-6).to("cuda", BF), RMSNorm(128, eps=1e-6).to("cuda", BF)
    row = dict(bench="reference_qknorm_rope_fwd_bwd", shape=[T, 16, 8, 128])
    guarded(row, "ours_fused_norm_rope_ms", lambda: torch.autograd.grad(ops.qkv_norm_rope(q, k, qw, kw, 1e-6, cos, sin), [q, k], [gq, gk]))
    guarded(row, "ref_triton_rope_only_ms", lambda: torch.autograd.grad(rot(q, k, seqlen_offset=0, max_seqlen=T), [q, k], [gq, gk]))
    guarded(row, "ref_triton_norm_then_rope_ms",
            lambda: torch.autograd.grad(rot(qn(q), kn(k), seqlen_offset=0, max_seqlen=T), [q, k], [gq, gk]))
    emit(**row)
    del q, k, gq, gk
    torch.cuda.empty_cache()
    # --- fused linear cross-entropy, 65536 x 1024 -> 151936
    vocab = 151936
    hid = (torch.randn(T, d, device="cuda") * 0.5).to(BF).requires_grad_()
    wl = (torch.randn(vocab, d, device="cuda") * 0.02).to(BF).requires_grad_()
    labels = torch.randint(0, vocab, (T,), device="cuda")
    crit = FusedLinearCrossEntropyLoss(num_chunks=8)
    row = dict(bench="reference_linear_cross_entropy_fwd_bwd", tokens=T, hidden=d, vocab=vocab)
    guarded(row, "ours_ms", lambda: torch.autograd.grad(ops.linear_cross_entropy(hid, labels, wl), [hid, wl]), iters=3)
    guarded(row, "ref_triton_ms", lambda: torch.autograd.grad(crit(hid.unsqueeze(0), labels.unsqueeze(0), wl, None), [hid, wl]),
            iters=3, warmup=1)
    emit(**row)


def bench_delta(batch: int, stages_only: bool = False):
    """Stages of the chunked (gated) delta rule at the 340M shapes of the two families, T = 4096 per sequence."""
    import os
    from ttcd_b200 import ops
    from ttcd_b200.ops import delta_chain as dc, delta_fused as df, reference as ref
    T = 4096
    for name, H, D, Dv, gated in (("delta_net_340M", 8, 128, 128, False), ("gated_deltanet_340M", 6, 256, 512, True)):
        torch.manual_seed(0)
        q, k = (torch.randn(batch, T, H, D, device="cuda").to(BF).requires_grad_() for _ in range(2))
        v = torch.randn(batch, T, H, Dv, device="cuda").to(BF).requires_grad_()
        beta = torch.rand(batch, T, H, device="cuda").requires_grad_()
        g = (-torch.rand(batch, T, H, device="cuda") * 0.1).requires_grad_() if gated else None
        leaves = [t for t in (q, k, v, g, beta) if t is not None]
        scale = D ** -0.5
        if not df.native_ok(q, v):
            emit(bench="delta", model=name, error="kernels do not take this shape")
            continue
        row = dict(bench="delta_rule", model=name, shape=[batch, T, H, D, Dv], gated=gated)
        with torch.no_grad():
            qd, kd, vd, bd = q.detach(), k.detach(), v.detach(), beta.detach()
            gd = None if g is None else g.detach()
            w, u, kt, q_in, qk, gamma = df._prep_fwd(qd, kd, vd, bd, gd, scale, True)
            s0 = torch.zeros(batch * H, D, Dv, device="cuda")
            vn, states, _ = dc._fwd(w, u, kt, gamma, s0)
            grads = [torch.randn_like(t) for t in (w, u, kt, q_in, qk, gamma)]
            d_states = torch.randn_like(states) * 0.01
            row["prep_fwd_ms"] = round(timeit(lambda: df._prep_fwd(qd, kd, vd, bd, gd, scale, True)), 4)
            row["chain_fwd_ms"] = round(timeit(lambda: dc._fwd(w, u, kt, gamma, s0)), 4)
            row["prep_bwd_ms"] = round(timeit(lambda: df._prep_bwd(qd, kd, vd, bd, gd, scale, True, *grads)), 4)
            row["chain_bwd_ms"] = round(timeit(lambda: dc._bwd(w, kt, gamma, grads[1], d_states, s0, states)), 4)
            del w, u, kt, q_in, qk, gamma, vn, states, grads, d_states
        if stages_only:
            emit(**row)
            continue
        go = torch.randn(batch, T, H, Dv, device="cuda").to(BF)

        def whole(fn):
            o = fn()
            torch.autograd.grad(o, leaves, go)

        row["op_fwd_bwd_ms"] = round(timeit(lambda: whole(lambda: ops.gated_delta_rule(q, k, v, g, beta)[0]), iters=5), 4)
        try:
            from torch.utils.checkpoint import checkpoint
            row["pytorch_statement_fwd_bwd_ms"] = round(timeit(lambda: whole(lambda: checkpoint(
                ref.gated_delta_rule_chunked, q, k, v, g, beta, None, True, 64, None, None, False, True, True,
                use_reentrant=False)[0]), iters=3, warmup=1), 4)
        except Exception as exc:
            row["pytorch_statement_error"] = f"{type(exc).__name__}: {exc}"[:160]
        torch.cuda.empty_cache()
        if _reference_profiling() is not None:
            try:
                if gated:
                    from fla.ops.gated_delta_rule import chunk_gated_delta_rule as fla_rule
                    call = lambda: fla_rule(q, k, v, g, beta.to(BF), use_qk_l2norm_in_kernel=True)[0]  # noqa: E731
                else:
                    from fla.ops.delta_rule import chunk_delta_rule as fla_rule
                    call = lambda: fla_rule(q, k, v, beta.to(BF), use_qk_l2norm_in_kernel=True)[0]  # noqa: E731
                row["ref_triton_fwd_bwd_ms"] = round(timeit(lambda: whole(call), iters=5), 4)
            except Exception as exc:
                row["ref_triton_error"] = f"{type(exc).__name__}: {exc}"[:160]
        emit(**row)
        del q, k, v, beta, g, go, leaves
        torch.cuda.empty_cache()


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
    if "misc" in what:
        bench_misc()
    if "delta" in what or "delta_stages" in what:
        bench_delta(batches[0], stages_only="delta" not in what)
    if "ref_misc" in what:
        bench_reference_misc()
    if "ref" in what:
        bench_reference(seqs, batches)
    st = _native.device_status()
    if st:
        emit(error=f"device status {st}")


if __name__ == "__main__":
    main()
