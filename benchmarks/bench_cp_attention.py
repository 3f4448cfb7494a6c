"""Context-parallel dual-window attention: sequence sharded over the ranks, the K/V halo read from the previous
rank's memory inside the attention kernels (forward, and forward+backward).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29512 \
        benchmarks/bench_cp_attention.py [--seq 65536] [--batch 1] [--bwd]

Device-timed (CUDA events, median of 10 after 3 warm-ups, barrier before each), maximum over ranks.  Reported
against the single-GPU time of the whole sequence: ideal time = single / ranks.  Roofline of the halo:
2 (K, V) x halo x HK x D x 2 B over 770 GB/s per direction, fully overlappable with the local key blocks.
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
    ap.add_argument("--seq", type=int, default=65536)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--wt", type=int, default=8192)
    ap.add_argument("--ws", type=int, default=4096)
    ap.add_argument("--bwd", action="store_true")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    from ttcd_b200.ops import cuda
    from ttcd_b200.parallel import context as ctx
    H, HK, D = 16, 8, 128
    B, S = args.batch, args.seq
    s_l = S // world
    sc = D ** -0.5
    mk = lambda t, h: torch.randn(B, t, h, D, device="cuda", dtype=torch.bfloat16, requires_grad=args.bwd)  # noqa: E731
    # single-GPU reference time of the whole sequence (every rank measures the same thing)
    q, k, v = mk(S, H), mk(S, HK), mk(S, HK)
    if args.bwd:
        def whole():
            o_t, o_s, _, _ = cuda._Attention.apply(q, k, v, args.wt, args.ws, sc, True, None, None)
            torch.autograd.grad([o_t, o_s], [q, k, v], [o_t, o_s])
    else:
        def whole():
            with torch.no_grad():
                cuda.attn_forward(q, k, v, args.wt, args.ws, sc, True)
    t_single = timed(whole)
    del q, k, v
    cp = ctx.ContextParallel(None, args.wt)
    ctx._ACTIVE = cp
    ql, kl, vl = mk(s_l, H), mk(s_l, HK), mk(s_l, HK)
    if args.bwd:
        def shard():
            o_t, o_s = ctx.dual_window_attention(ql, kl, vl, args.wt, args.ws, sc, 0)
            torch.autograd.grad([o_t, o_s], [ql, kl, vl], [o_t, o_s])
    else:
        def shard():
            with torch.no_grad():
                ctx.dual_window_attention(ql, kl, vl, args.wt, args.ws, sc, 0)
    t_cp = timed(shard)
    torch.cuda.synchronize()
    from ttcd_b200 import _native
    status = _native.device_status()
    halo = (args.wt - 1 + 127) // 128 * 128 if world > 1 else 0       # what every rank but the first pulls
    halo_ms = 2 * halo * HK * D * 2 * B / 770e9 * 1e3
    if rank == 0:
        print(json.dumps({"bench": "cp_dual_attention", "pass": "fwd+bwd" if args.bwd else "fwd", "ranks": world, "B": B, "seq": S,
                          "w_t": args.wt, "w_s": args.ws, "single_gpu_ms": round(t_single, 3), "cp_ms": round(t_cp, 3),
                          "ideal_ms": round(t_single / world, 3), "efficiency": round(t_single / world / t_cp, 3),
                          "halo_keys": halo, "halo_link_ms": round(halo_ms, 4), "device_status": status}))
    ctx.shutdown()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
