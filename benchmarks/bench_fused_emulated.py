"""The fused compute+collective kernels on ONE GPU with the peers emulated by local buffers, so that a
profiler can look at them (a multi-rank command is never run under a profiler).  "Peer" pointers address other
buffers of the same GPU; flags that a peer's kernel would raise are set beforehand; the kernels, their tile
schedules, copies, flag protocol and reductions are exactly those of the multi-GPU runs, only the bytes do not
cross NVLink.  Outputs are checked against a plain matmul.

    python benchmarks/bench_fused_emulated.py --what ag_gemm|gemm_rs|rs_norm [--world 2] [--tokens 16384]
"""
import argparse
import ctypes
import json
import statistics
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from ttcd_b200 import _native as nv  # noqa: E402


def ptrs(tensors):
    return (ctypes.c_longlong * len(tensors))(*[t.data_ptr() for t in tensors])


def timeit(fn, iters=10, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="ag_gemm")
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--lag", type=int, default=0, help="gemm_rs: rounds by which own row blocks trail the pushes (0: last)")
    args = ap.parse_args()
    nv.load(required=True)
    w_, m, k, n = args.world, args.tokens // args.world, args.k, args.n
    torch.manual_seed(0)
    epoch = [0]
    if args.what == "ag_gemm":
        xs = [(torch.randn(m, k, device="cuda") * 0.5).bfloat16() for _ in range(w_)]
        wt = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        out = torch.empty(m * w_, n, device="cuda", dtype=torch.bfloat16)
        gathered = torch.zeros(m * w_, k, device="cuda", dtype=torch.bfloat16)
        ready = torch.zeros(w_ * (m // 128), device="cuda", dtype=torch.int32)

        def run():
            epoch[0] += 1
            nv.call("ttcd_ag_gemm", ptrs(xs), nv.ptr(wt), nv.ptr(out), nv.ptr(gathered), nv.ptr(ready), nv.i32(0), nv.i32(w_),
                    nv.i64(m), nv.i64(n), nv.i64(k), nv.i64(k), nv.i64(n), nv.i32(0), nv.i32(epoch[0]), nv.i64(2_000_000_000),
                    nv.stream_ptr())
        ms = timeit(run)
        want = torch.cat(xs).float() @ wt.float().t()
        err = (out.float() - want).abs().max().item() / want.abs().max().item()
        flops = 2.0 * m * w_ * k * n
    elif args.what == "gemm_rs":
        x = (torch.randn(m * w_, k, device="cuda") * 0.5).bfloat16()
        wt = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        # receive buffers: ours holds the tiles that the peers "pushed" (given data, flags already raised); the peers'
        # buffers take what this rank pushes for their rows (local memory standing in for the other GPUs)
        parts = [(torch.randn(m * max(w_ - 1, 1), n, device="cuda") * 0.1).bfloat16() for _ in range(w_)]
        nflags = max(w_ - 1, 1) * (m // 128) * (n // 256)
        flags = [torch.zeros(nflags, device="cuda", dtype=torch.int32) for _ in range(w_)]
        flags[0].fill_(1 << 30)
        mine = parts[0].clone()

        def run():
            epoch[0] += 1
            nv.call("ttcd_gemm_rs", nv.ptr(x), nv.ptr(wt), nv.ptr(out), ptrs(parts), ptrs(flags), nv.i32(0), nv.i32(w_), nv.i64(m),
                    nv.i64(n), nv.i64(k), nv.i64(k), nv.i64(k), nv.i64(n), nv.i32(0), nv.i32(epoch[0]), nv.i64(2_000_000_000),
                    nv.i32(args.lag), nv.stream_ptr())
        ms = timeit(run)
        want = x[:m].float() @ wt.float().t() + sum(mine[d * m:(d + 1) * m].float() for d in range(w_ - 1))
        err = (out.float() - want).abs().max().item() / want.abs().max().item()
        # what this rank pushed for the next rank's rows (slot world - 2 of that rank's buffer)
        if w_ > 1:
            pushed = parts[1][(w_ - 2) * m:(w_ - 1) * m].float()
            want_p = x[m:2 * m].float() @ wt.float().t()
            err = max(err, (pushed - want_p).abs().max().item() / want_p.abs().max().item())
        flops = 2.0 * m * w_ * k * n
    elif args.what == "rs_norm":
        numel = m * k
        grads = [(torch.randn(numel * w_, device="cuda") * 0.1).bfloat16() for _ in range(w_)]
        out = torch.empty(numel, device="cuda")
        norm = torch.zeros(1, device="cuda")

        def run():
            nv.call("ttcd_rs_cast_scale_norm", ptrs(grads), nv.i32(w_), nv.i64(0), nv.i64(numel), nv.f32(1.0 / w_), nv.ptr(out),
                    nv.ptr(norm), nv.stream_ptr())
        ms = timeit(run)
        want = sum(g[:numel].float() for g in grads) / w_
        err = (out - want).abs().max().item()
        flops = 0.0
    elif args.what == "adamw_push":
        numel = m * k
        master = torch.randn(numel, device="cuda")
        grad = torch.randn(numel, device="cuda") * 0.01
        m1, m2 = torch.zeros(numel, device="cuda"), torch.zeros(numel, device="cuda")
        params = [torch.zeros(numel * w_, device="cuda", dtype=torch.bfloat16) for _ in range(w_)]    # every rank's flat buffer
        coef = torch.ones(1, device="cuda")
        want = master.clone()
        g32 = grad.clone()

        def run():
            nv.call("ttcd_adamw_push", nv.ptr(master), nv.ptr(grad), nv.ptr(m1), nv.ptr(m2), ptrs(params), nv.i32(w_), nv.i64(0),
                    nv.i64(numel), nv.f32(1e-3), nv.f32(0.9), nv.f32(0.95), nv.f32(1e-8), nv.f32(0.0), nv.f32(0.1),
                    nv.f32(0.05 ** 0.5), nv.ptr(coef), nv.ptr(None), nv.stream_ptr())
        run()
        torch.cuda.synchronize()
        # first step with these bias corrections: update = lr * (0.1 g / 0.1) / (sqrt(0.05 g^2 / 0.05) + eps) = lr * sign(g)
        want = want - 1e-3 * g32 / (g32.abs() + 1e-8)
        err = max((p_[:numel].float() - want).abs().max().item() for p_ in params)
        ms = timeit(run)
        flops = 0.0
    else:
        raise SystemExit(f"unknown --what {args.what}")
    torch.cuda.synchronize()
    print(json.dumps({"bench": "fused_emulated", "what": args.what, "world": w_, "m_shard": m, "n": n, "k": k, "ms": round(ms, 4),
                      "tflops": round(flops / ms / 1e9, 1), "max_rel_err": round(err, 5), "device_status": nv.device_status()}))


if __name__ == "__main__":
    main()
