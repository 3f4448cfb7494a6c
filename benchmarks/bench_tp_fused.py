"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels vs NCCL collective + cuBLAS, on the tensor-parallel
shapes of the Qwen3-0.6B IP-TTCD recipe at 64K tokens.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        benchmarks/bench_tp_fused.py [--tokens 65536]

Device-timed with CUDA events (median of 10 after 3 warm-ups, barrier before each timed call), maximum over
ranks.  Roofline: the slower of FLOPs / measured cuBLAS bf16 peak and NVLink bytes / 770 GB/s per direction.
"""
import argparse
import json
import os
import statistics
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    t = torch.tensor([statistics.median(ts)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--lags", default="0", help="comma list of gemm_rs lags to time (rounds; 0 = own row blocks last)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    from ttcd_b200.parallel.tensor import TensorParallel
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = peaks.get("bf16_tflops", 1590.0)
    m = args.tokens // world
    tp = TensorParallel(None, torch.device("cuda", local), max_rows_per_rank=m, max_features=4096)
    rows = []
    # (name, K, N_total): column-parallel shards N, row-parallel shards K
    for name, k, n in (("qkv", 1024, 4096), ("gate_up", 1024, 6144)):
        nl = n // world
        if nl % 256:
            continue
        x = torch.randn(m, k, device="cuda").bfloat16()
        w = (torch.randn(nl, k, device="cuda") * 0.02).bfloat16()
        full = torch.empty(m * world, k, device="cuda", dtype=torch.bfloat16)

        def base():
            dist.all_gather_into_tensor(full, x)
            return full @ w.t()

        t_f = timed(lambda: tp.ag_gemm(x, w))
        t_b = timed(base)
        flops = 2.0 * m * world * k * nl
        link = (world - 1) * m * k * 2 / 770e9 * 1e3
        roof = max(flops / (peak * 1e12) * 1e3, link)
        rows.append({"op": f"ag_gemm {name}", "M": m * world, "N": nl, "K": k, "fused_ms": round(t_f, 4), "nccl_cublas_ms": round(t_b, 4),
                     "speedup": round(t_b / t_f, 3), "roofline_ms": round(roof, 4), "of_roofline": round(roof / t_f, 3)})
    for name, k, n in (("o_proj", 2048, 1024), ("down", 3072, 1024)):
        kl = k // world
        if kl % 64:
            continue
        x = torch.randn(m * world, kl, device="cuda").bfloat16()
        w = (torch.randn(n, kl, device="cuda") * 0.02).bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

        def base():
            y = x @ w.t()
            dist.reduce_scatter_tensor(out, y)
            return out

        by_lag = {lag: timed(lambda: tp.gemm_rs(x, w, lag=lag)) for lag in [int(v) for v in args.lags.split(",")]}
        best_lag = min(by_lag, key=by_lag.get)
        t_f = by_lag[best_lag]
        t_b = timed(base)
        flops = 2.0 * m * world * kl * n
        link = (world - 1) * m * n * 2 / 770e9 * 1e3
        roof = max(flops / (peak * 1e12) * 1e3, link)
        rows.append({"op": f"gemm_rs {name}", "M": m * world, "N": n, "K": kl, "lag": best_lag,
                     "ms_by_lag": {str(k_): round(v_, 4) for k_, v_ in by_lag.items()},
                     "fused_ms": round(t_f, 4), "nccl_cublas_ms": round(t_b, 4),
                     "speedup": round(t_b / t_f, 3), "roofline_ms": round(roof, 4), "of_roofline": round(roof / t_f, 3)})
    tp.check()
    if rank == 0:
        for r in rows:
            print(json.dumps({"bench": "tp_fused", "world": world, **r}))
    tp.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
