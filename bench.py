"""Headline benchmark: IP-TTCD training throughput (tokens/s over the whole job).

Default config = the continued-training recipe on the Qwen3-0.6B shape: 28 layers, hidden 1024, 16 Q / 8 KV
heads, head_dim 128, SwiGLU 3072, vocab 151936, tied embeddings, window 8192, student window 4096, TTT layers
[0, 7, 14, 21]; bf16 compute, one 65536-token sequence per GPU, AdamW (eps 1e-15, clip 1.0), synthetic
uniform-random tokens, random-init weights.  Activation checkpointing: the headline ``value`` keeps the
activations of the step resident (``--ac none``: they fit in the 180 GB of a B200); the same line also carries
``ac_full`` (every block recomputed in backward, the recipe's setting for 80 GB GPUs) from a second timed
region.  The reference arm tries to run without checkpointing first and falls back to full checkpointing when
that does not fit; both arms name the setting they ran in ``config.activation_checkpointing``.

On more than one GPU the line also carries ``extra.cp``: the same model on ONE 65536-token sequence sharded over
all N ranks (context parallelism, strong scaling), measured in child processes so that a failure there cannot
take the headline with it.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 3 --warmup 3
    python bench.py --impl reference ...      # the unmodified upstream model from baseline/_ref under FSDP2

Two timed regions of K steps each, both bracketed by barrier + synchronize and timed with CUDA events
(max over ranks): (1) inputs already on the device -> ``value``; (2) end to end through the public API
(``Trainer.train_step`` on pinned host tensors: H2D copy of the step's tokens, step, D2H read of the loss)
-> ``e2e``.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
import warnings
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
warnings.filterwarnings("ignore")

METRIC = "train_tokens_per_second"
DEFAULT_CONFIG = ROOT / "configs" / "ipttcd" / "ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k.json"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=str(DEFAULT_CONFIG))
    ap.add_argument("--seq-len", type=int, default=65536)
    ap.add_argument("--batch-per-gpu", type=int, default=1)
    ap.add_argument("--layers", type=int, default=None, help="debug only: override num_hidden_layers (invalidates the number)")
    ap.add_argument("--ac", default="none", choices=["none", "full", "ttt", "op"],
                    help="activation checkpointing of this framework's arm; 'none' keeps the activations of one "
                         "64K-token step resident, which fits the 180 GB of a B200 (the reference recipe needs 'full')")
    ap.add_argument("--no-ac", action="store_true", help="same as --ac none (kept for older command lines)")
    ap.add_argument("--ref-ac", default="auto", choices=["auto", "none", "full"],
                    help="reference arm: 'auto' runs without activation checkpointing if that fits, else with full")
    ap.add_argument("--no-extra", action="store_true", help="skip the ac_full and context-parallel extras")
    ap.add_argument("--muon", action="store_true", help="Muon on the 2-D hidden weights, AdamW on the rest")
    ap.add_argument("--worker", default=None, choices=["cp", "zero3"], help=argparse.SUPPRESS)
    return ap.parse_args()


# ----------------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region (read-only)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1])); mx = float(parts[2])
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            out["sm_mhz"] = statistics.median(clocks)
            out["sm_max_mhz"] = mx
            out["reasons"] = sorted(reasons)
            out["samples"] = len(clocks)
        return out


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


def timed_region(torch, dist, world, fn, steps):
    """K calls of fn between barrier+sync brackets; device time via CUDA events, max over ranks."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([s.elapsed_time(e)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


# ----------------------------------------------------------------------------------------------------
# this framework
# ----------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from ttcd_b200 import _native
    from ttcd_b200.train.engine import EngineConfig, TrainEngine, load_model_config

    _native.load(required=True)
    overrides = {}
    if args.layers is not None:
        overrides["num_hidden_layers"] = args.layers
    cfg = load_model_config(args.config, **overrides)
    engine = TrainEngine(cfg, EngineConfig(activation_checkpoint="none" if args.no_ac else args.ac, enable_muon=args.muon),
                         device=f"cuda:{local}")
    B, S, V = args.batch_per_gpu, args.seq_len, cfg.vocab_size
    n_total = args.warmup + 2 * args.steps
    gen = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randint(0, V, (B, S), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_total)]
    dev = [t.cuda(non_blocking=True) for t in host[args.warmup:args.warmup + args.steps]]

    for i in range(args.warmup):
        engine.train_step(host[i], return_loss_on_host=False)
    torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = _native.launch_count
    ms_dev = timed_region(torch, dist, world, lambda i: engine.train_step(dev[i], return_loss_on_host=False), args.steps)
    launches = _native.launch_count - launches0
    losses = []
    e2e_host = host[args.warmup + args.steps:]
    ms_e2e = timed_region(torch, dist, world, lambda i: losses.append(engine.train_step(e2e_host[i])), args.steps)
    clocks = sampler.stop() if sampler else {}
    status = _native.device_status()
    peak_gib = round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)

    tokens = B * S * world * args.steps
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    ac_mode = "none" if args.no_ac else args.ac
    ac_full, extra = None, {}
    if not args.no_extra:
        if ac_mode != "full":
            # the recipe's setting (every block recomputed in backward): same engine, same inputs, second timed region
            try:
                engine.set_activation_checkpointing("full")
                engine.train_step(host[0], return_loss_on_host=False)
                ms_full = timed_region(torch, dist, world, lambda i: engine.train_step(dev[i], return_loss_on_host=False),
                                       args.steps)
                ac_full = {"ms_per_step": round(ms_full / args.steps, 2), "value": round(tokens / (ms_full / 1e3), 1),
                           "unit": "tokens/s"}
            except Exception as exc:  # pragma: no cover
                ac_full = {"error": f"{type(exc).__name__}: {exc}"[:200]}
            engine.set_activation_checkpointing(ac_mode)
        if world > 1:
            # the children build their own engines on the same GPUs: give this one's memory back first
            del dev, host, e2e_host
            engine.close()
            del engine
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            extra["cp"] = run_children(args, rank, world, "cp", 23)
            extra["zero3"] = run_children(args, rank, world, "zero3", 41)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "impl": "ours",
            "config": {"model": Path(args.config).stem, "global_batch": B * world, "seq_len": S,
                       "parallelism": f"sharded-dp{world}", "activation_checkpointing": ac_mode,
                       "optimizer": "Muon+AdamW" if args.muon else "AdamW", "l2": "per-step working set (several GB) exceeds the 126 MB L2",
                       "layers": cfg.num_hidden_layers},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e / args.steps, 2),
                    "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "final_loss": losses[-1] if losses else None, "device_status": status,
            "peak_mem_gib": peak_gib, "ac_full": ac_full, "extra": extra,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------------
# context-parallel extra (N > 1): one 64K sequence sharded over all ranks, measured in child processes
# ----------------------------------------------------------------------------------------------------
CP_STEPS, CP_WARMUP, CP_TIMEOUT_S = 5, 3, 420


def run_children(args, rank, world, what: str, port_offset: int) -> dict:
    """Every rank starts one child (``bench.py --worker <what>``) with the same rank / world size and its own
    rendezvous port; the children form their own process group, run the measurement and rank 0's child prints its
    JSON.  A child that fails or outlives its time limit is killed by PID and reported as an error."""
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(env.get("MASTER_PORT", "29500")) + port_offset)
    env["TORCHELASTIC_USE_AGENT_STORE"] = "False"          # rank 0's child hosts the store of the children's group
    for k in ("TORCHELASTIC_RUN_ID", "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS"):
        env.pop(k, None)
    cmd = [sys.executable, str(Path(__file__).resolve()), "--worker", what, "--gpus", str(world), "--config", args.config,
           "--seq-len", str(args.seq_len)]
    if args.layers is not None:
        cmd += ["--layers", str(args.layers)]
    try:
        proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        try:
            out, err = proc.communicate(timeout=CP_TIMEOUT_S)
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.communicate()
            return {"degree": world, "error": f"no result within {CP_TIMEOUT_S} s"}
        if rank != 0:
            return {}
        for line in reversed(out.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
        return {"degree": world, "error": f"child exit {proc.returncode}: {err.strip()[-300:]}"}
    except Exception as exc:  # pragma: no cover
        return {"degree": world, "error": f"{type(exc).__name__}: {exc}"[:300]}


def run_zero3_worker(args):
    """The headline configuration (one sequence per GPU, sharded data parallel) with the blocks' weights stored 1/N per
    rank and gathered inside each block's first GEMM (forward) / by the gather kernel (backward)."""
    import torch
    import torch.distributed as dist
    from datetime import timedelta

    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=timedelta(seconds=120))
    from ttcd_b200 import _native
    from ttcd_b200.train.engine import EngineConfig, TrainEngine, load_model_config

    _native.load(required=True)
    overrides = {} if args.layers is None else {"num_hidden_layers": args.layers}
    cfg = load_model_config(args.config, **overrides)
    engine = TrainEngine(cfg, EngineConfig(activation_checkpoint="none", shard_weights=True), device=f"cuda:{local}")
    S, V = args.seq_len, cfg.vocab_size
    gen = torch.Generator().manual_seed(77 + rank)
    ids = [torch.randint(0, V, (1, S), generator=gen, dtype=torch.int64).cuda() for _ in range(CP_WARMUP + CP_STEPS)]
    for i in range(CP_WARMUP):
        engine.train_step(ids[i], return_loss_on_host=False)
    ms = timed_region(torch, dist, world, lambda i: engine.train_step(ids[CP_WARMUP + i], return_loss_on_host=False), CP_STEPS)
    status = _native.device_status()
    peak = torch.cuda.max_memory_allocated() / 2 ** 30
    n_block = sum(g.numel for g in engine.sdp.groups if g.sharded)
    if rank == 0:
        print(json.dumps({"degree": world, "parallelism": f"sharded-dp{world}, block weights sharded 1/{world} (gather fused into the q|k|v GEMM)",
                          "steps": CP_STEPS, "warmup": CP_WARMUP, "ms_per_step": round(ms / CP_STEPS, 2),
                          "tokens_per_s": round(S * world * CP_STEPS / (ms / 1e3), 1), "scaling": "weak",
                          "final_loss": float(engine.last_loss), "device_status": status, "peak_mem_gib": round(peak, 1),
                          "block_params_per_rank_mib": round(n_block * 2 / world / 2 ** 20, 1)}), flush=True)
    dist.destroy_process_group()


def run_cp_worker(args):
    import torch
    import torch.distributed as dist
    from datetime import timedelta

    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=timedelta(seconds=120))
    from ttcd_b200 import _native
    from ttcd_b200.train.engine import EngineConfig, TrainEngine, load_model_config

    _native.load(required=True)
    overrides = {} if args.layers is None else {"num_hidden_layers": args.layers}
    cfg = load_model_config(args.config, **overrides)
    engine = TrainEngine(cfg, EngineConfig(activation_checkpoint="none", context_parallel=world), device=f"cuda:{local}")
    S, V = args.seq_len, cfg.vocab_size
    gen = torch.Generator().manual_seed(99)                 # every rank of the group sees the same sequence
    ids = [torch.randint(0, V, (1, S), generator=gen, dtype=torch.int64).cuda() for _ in range(CP_WARMUP + CP_STEPS)]
    for i in range(CP_WARMUP):
        engine.train_step(ids[i], return_loss_on_host=False)
    ms = timed_region(torch, dist, world, lambda i: engine.train_step(ids[CP_WARMUP + i], return_loss_on_host=False), CP_STEPS)
    loss = float(engine.last_loss)
    status = _native.device_status()
    peak = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        print(json.dumps({"degree": world, "parallelism": f"context-parallel {world} (one {S}-token sequence over {world} GPUs)",
                          "steps": CP_STEPS, "warmup": CP_WARMUP, "ms_per_step": round(ms / CP_STEPS, 2),
                          "tokens_per_s": round(S * CP_STEPS / (ms / 1e3), 1), "scaling": "strong", "final_loss": loss,
                          "device_status": status, "peak_mem_gib": round(peak, 1)}), flush=True)
    dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------------
# reference arm: the unmodified upstream model classes from baseline/_ref under PyTorch FSDP2
# ----------------------------------------------------------------------------------------------------
def run_reference(args):
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "custom_models").is_dir():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-deps --target baseline/_ref <reference checkout>)"}))
        return
    sys.path.insert(0, str(ref_root))
    for k in [k for k in sys.modules if k.split(".")[0] in ("custom_models", "flame", "fla")]:
        del sys.modules[k]
    try:
        from baseline.reference_arm import run
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"reference arm import failed: {type(exc).__name__}: {exc}"[:300]}))
        return
    run(args, METRIC, ClockSampler, timed_region, dist_env)


def main():
    args = parse_args()
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as exc:
            rank = int(os.environ.get("RANK", "0"))
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:400]}), flush=True)
        return
    if args.worker == "cp":
        run_cp_worker(args)
        return
    if args.worker == "zero3":
        run_zero3_worker(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
