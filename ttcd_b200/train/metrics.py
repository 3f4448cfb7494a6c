"""Logging and throughput metrics for the trainer.

Per log step the reference reports loss (global mean / max), tokens per second, TFLOPS, MFU, step and
data-loading time and memory statistics, to the console and optionally TensorBoard / W&B
(torchtitan components/metrics.py; flame/train.py:719-853).  This module provides the same quantities.
FLOPs per token follow flame/tools/utils.py:11-43: ``6 (N - N_emb) + 12 L H D_h T``.
"""
from __future__ import annotations

import logging
import os
import sys
import time
from dataclasses import dataclass

import torch

# dense bf16 peak used for MFU (NVIDIA's nominal figure, no sparsity)
PEAK_FLOPS = {"B200": 2.25e15, "H100": 989e12, "H200": 989e12, "A100": 312e12}


def get_peak_flops(device_name: str) -> float:
    for key, val in PEAK_FLOPS.items():
        if key in device_name:
            return val
    return 312e12


def init_logger(name: str = "ttcd_b200") -> logging.Logger:
    logger = logging.getLogger(name)
    if not logger.handlers:
        handler = logging.StreamHandler(sys.stdout)
        handler.setFormatter(logging.Formatter("[%(name)s] %(asctime)s - %(levelname)s - %(message)s"))
        logger.addHandler(handler)
        logger.setLevel(logging.INFO)
        logger.propagate = False
    return logger


def get_num_flop_per_token(num_params: int, model_config, seq_len: int) -> int:
    """6 * non-embedding params + attention term 12 * L * H * D_h * T."""
    layers = model_config.num_hidden_layers
    heads = model_config.num_heads
    head_dim = getattr(model_config, "head_dim", None) or model_config.hidden_size // heads
    return int(6 * num_params + 12 * layers * heads * head_dim * seq_len)


def count_params(model: torch.nn.Module, exclude_embedding: bool = True) -> int:
    total = sum(p.numel() for p in {id(p): p for p in model.parameters()}.values())
    if exclude_embedding:
        emb = getattr(getattr(model, "model", model), "embeddings", None)
        if emb is not None:
            total -= emb.weight.numel()
    return total


@dataclass
class DeviceMemStats:
    max_active_gib: float = 0.0
    max_active_pct: float = 0.0
    max_reserved_gib: float = 0.0
    max_reserved_pct: float = 0.0
    num_alloc_retries: int = 0
    num_ooms: int = 0


class DeviceMemoryMonitor:
    def __init__(self, device=None):
        self.enabled = torch.cuda.is_available()
        self.device = torch.device(device or (f"cuda:{torch.cuda.current_device()}" if self.enabled else "cpu"))
        self.capacity = torch.cuda.get_device_properties(self.device).total_memory if self.enabled else 1

    def peak(self) -> DeviceMemStats:
        if not self.enabled:
            return DeviceMemStats()
        s = torch.cuda.memory_stats(self.device)
        gib = 1 << 30
        act, res = s.get("active_bytes.all.peak", 0), s.get("reserved_bytes.all.peak", 0)
        return DeviceMemStats(act / gib, 100 * act / self.capacity, res / gib, 100 * res / self.capacity,
                              s.get("num_alloc_retries", 0), s.get("num_ooms", 0))

    def reset(self):
        if self.enabled:
            torch.cuda.reset_peak_memory_stats(self.device)


class MetricsLogger:
    """Fan-out of scalar metrics to TensorBoard and/or W&B (rank 0 unless ``save_for_all_ranks``)."""

    def __init__(self, job_config, rank: int = 0):
        m = job_config.metrics
        self.writers = []
        active = rank == 0 or m.save_for_all_ranks
        if active and m.enable_tensorboard:
            from torch.utils.tensorboard import SummaryWriter
            path = os.path.join(job_config.job.dump_folder, m.save_tb_folder, time.strftime("%Y%m%d-%H%M"))
            if m.save_for_all_ranks:
                path = os.path.join(path, f"rank_{rank}")
            tb = SummaryWriter(path, max_queue=1000)
            self.writers.append(lambda metrics, step: [tb.add_scalar(k, v, step) for k, v in metrics.items()])
            self._tb = tb
        if active and m.enable_wandb:
            try:
                import wandb
                os.makedirs(job_config.job.dump_folder, exist_ok=True)
                wandb.init(project=os.getenv("WANDB_PROJECT", "ttcd_b200"), dir=job_config.job.dump_folder,
                           config=job_config.to_dict(), mode=os.getenv("WANDB_MODE", "offline"))
                self.writers.append(lambda metrics, step: wandb.log(metrics, step=step))
            except Exception:  # pragma: no cover - optional sink
                pass

    def log(self, metrics: dict[str, float], step: int) -> None:
        for w in self.writers:
            w(metrics, step)

    def close(self) -> None:
        tb = getattr(self, "_tb", None)
        if tb is not None:
            tb.close()


class MetricsProcessor:
    """Accumulates per-step timing and turns it into tps / tflops / mfu at log time."""

    def __init__(self, job_config, num_flop_per_token: int, world_size: int, non_dp_size: int = 1, rank: int = 0,
                 logger: logging.Logger | None = None):
        self.job_config = job_config
        self.sink = MetricsLogger(job_config, rank)
        self.logger = logger or init_logger()
        self.num_flop_per_token = num_flop_per_token
        self.non_dp_size = non_dp_size
        self.memory = DeviceMemoryMonitor()
        name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
        self.peak_flops = get_peak_flops(name)
        self.ntokens_since_last_log = 0
        self.data_loading_times: list[float] = []
        self.time_last_log = time.perf_counter()
        self.memory.reset()

    def should_log(self, step: int) -> bool:
        return step == 1 or step % self.job_config.metrics.log_freq == 0

    def log(self, step: int, global_avg_loss: float, global_max_loss: float, extra: dict[str, float] | None = None):
        dt = time.perf_counter() - self.time_last_log
        tps = self.ntokens_since_last_log / (dt * self.non_dp_size) if dt > 0 else 0.0
        tflops = self.num_flop_per_token * tps / 1e12
        mfu = 100 * self.num_flop_per_token * tps / self.peak_flops
        freq = max(1, self.job_config.metrics.log_freq)
        t_step = dt / freq
        t_data = sum(self.data_loading_times) / max(1, len(self.data_loading_times))
        mem = self.memory.peak()
        metrics = {
            "loss_metrics/global_avg_loss": global_avg_loss, "loss_metrics/global_max_loss": global_max_loss,
            "throughput(tps)": tps, "tflops": tflops, "mfu(%)": mfu,
            "time_metrics/end_to_end(s)": t_step, "time_metrics/data_loading(s)": t_data,
            "time_metrics/data_loading(%)": 100 * t_data / t_step if t_step > 0 else 0.0,
            "memory/max_active(GiB)": mem.max_active_gib, "memory/max_active(%)": mem.max_active_pct,
            "memory/max_reserved(GiB)": mem.max_reserved_gib, "memory/max_reserved(%)": mem.max_reserved_pct,
            "memory/num_alloc_retries": mem.num_alloc_retries, "memory/num_ooms": mem.num_ooms,
        }
        if extra:
            metrics.update(extra)
        self.sink.log(metrics, step)
        self.logger.info(
            f"step: {step:5d}  loss: {global_avg_loss:7.4f}  memory: {mem.max_reserved_gib:5.2f}GiB({mem.max_reserved_pct:.1f}%)  "
            f"tps: {round(tps):,}  tflops: {tflops:,.1f}  mfu: {mfu:.2f}%" +
            "".join(f"  {k.split('/')[-1]}: {v:.4g}" for k, v in (extra or {}).items() if k.startswith("optimizer/")))
        self.ntokens_since_last_log = 0
        self.data_loading_times.clear()
        self.time_last_log = time.perf_counter()
        self.memory.reset()

    def close(self):
        self.sink.close()
