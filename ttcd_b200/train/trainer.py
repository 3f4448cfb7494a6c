"""Trainer entry point behind ``python -m flame.train``.

Sequence (flame/train.py:170-878 in the reference): parse flags, initialise the process group and device,
seed, tokenizer + dataset + dataloader, model config (vocab = max(tokenizer, config)), model build +
sharded runtime, LR schedule (with lr_min_absolute / anneal rewrites), checkpoint load (resume or initial
load), then the hot loop: gradient accumulation, forward/backward, clipping, optional NaN/Inf skip,
optimizer step, LR step, periodic logging (global mean/max loss, tps, MFU, ttt_norm/*), checkpoint save
on interval / last step / external trigger (SIGUSR1 or a trigger file), profiler and memory-snapshot
steps, periodic Python GC, and the process-group timeout tightened after the first step.
"""
from __future__ import annotations

import gc
import hashlib
import json
import os
import signal
import time
from datetime import timedelta

import torch
import torch.distributed as dist

from .checkpoint import CheckpointManager, TrainState
from .config_manager import JobConfig
from .data import build_dataloader, build_dataset
from .engine import EngineConfig, TrainEngine, load_model_config
from .lr_scheduler import build_lr_schedule
from .metrics import MetricsProcessor, count_params, get_num_flop_per_token, init_logger

SAVE_TRIGGER_FILE = "/tmp/flame_save_checkpoint"
_save_requested = False


def _on_sigusr1(signum, frame):  # noqa: ARG001
    global _save_requested
    _save_requested = True


def external_save_requested(rank: int) -> bool:
    """SIGUSR1 to rank 0 or touching the trigger file asks for a checkpoint at the next step boundary."""
    global _save_requested
    flag = False
    if rank == 0:
        flag = _save_requested or os.path.exists(SAVE_TRIGGER_FILE)
        if flag:
            _save_requested = False
            try:
                os.remove(SAVE_TRIGGER_FILE)
            except OSError:
                pass
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([1 if flag else 0], device="cuda" if torch.cuda.is_available() else "cpu")
        dist.broadcast(t, src=0)
        flag = bool(t.item())
    return flag


def snapshot_model_config(model_config, dump_folder: str, logger) -> None:
    """Write resolved_model_config.json (+ sha256) next to the run outputs."""
    os.makedirs(dump_folder, exist_ok=True)
    text = json.dumps(model_config.to_dict(), indent=2, sort_keys=True, default=str)
    digest = hashlib.sha256(text.encode()).hexdigest()
    with open(os.path.join(dump_folder, "resolved_model_config.json"), "w") as fh:
        fh.write(text)
    with open(os.path.join(dump_folder, "resolved_model_config.meta.json"), "w") as fh:
        json.dump({"sha256": digest, "model_type": model_config.model_type}, fh)
    logger.info(f"model config sha256 {digest[:16]} written to {dump_folder}/resolved_model_config.json")


def init_distributed(job_config, logger):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "3")
        if job_config.comm.trace_buf_size > 0:
            os.environ.setdefault("TORCH_NCCL_TRACE_BUFFER_SIZE", str(job_config.comm.trace_buf_size))
            os.environ.setdefault("TORCH_NCCL_DUMP_ON_TIMEOUT", "1")
        kwargs = dict(backend="nccl" if use_cuda else "gloo", timeout=timedelta(seconds=job_config.comm.init_timeout_seconds))
        if use_cuda:
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(**kwargs)
    rank = dist.get_rank() if dist.is_initialized() else 0
    return rank, local, world, torch.device("cuda", local) if use_cuda else torch.device("cpu")


def set_pg_timeouts(seconds: int) -> None:
    """Tighten the collective timeout once the first step (with its lazy initialisations) is done."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return
    dist.barrier()
    try:
        from torch.distributed.distributed_c10d import _get_default_group
        pg = _get_default_group()
        if hasattr(pg, "_set_default_timeout"):
            pg._set_default_timeout(timedelta(seconds=seconds))
        for backend_name in ("cuda", "cpu"):
            try:
                backend = pg._get_backend(torch.device(backend_name))
                if hasattr(backend, "_set_default_timeout"):
                    backend._set_default_timeout(timedelta(seconds=seconds))
            except Exception:
                pass
    except Exception:
        pass


def dist_mean_max(value: torch.Tensor) -> tuple[float, float]:
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        v = float(value)
        return v, v
    buf = torch.stack([value.detach().float(), value.detach().float()])
    mean, mx = buf[0:1].clone(), buf[1:2].clone()
    dist.all_reduce(mean, op=dist.ReduceOp.SUM)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    return float(mean) / dist.get_world_size(), float(mx)


def loss_by_position(logits, labels, buckets=((0, 2048), (2048, 4096), (4096, 8192), (8192, 16384))) -> dict[str, float]:
    """Mean next-token loss inside position buckets (only when logits exist, i.e. no fused linear-CE)."""
    out = {}
    if logits is None:
        return out
    with torch.no_grad():
        tgt = labels[:, 1:]
        nll = torch.nn.functional.cross_entropy(logits[:, :-1].float().transpose(1, 2), tgt, reduction="none", ignore_index=-100)
        for lo, hi in buckets:
            if lo >= nll.shape[1]:
                break
            seg = nll[:, lo:min(hi, nll.shape[1])]
            out[f"loss_by_pos/{lo // 1024}k_{hi // 1024}k"] = float(seg.mean())
    return out


def _ac_mode(job_config) -> str:
    ac = job_config.activation_checkpoint
    if ac.mode == "none":
        return "none"
    if ac.mode == "full":
        return "full"
    opt = str(ac.selective_ac_option)
    if opt.isdigit():
        return f"every{int(opt)}"
    if opt == "op":
        return "op"          # recompute the cheap ops, keep the GEMM / attention outputs (ops/selective.py)
    raise ValueError(f"--activation_checkpoint.selective_ac_option must be an integer or 'op', got {opt!r}")


def main(job_config: JobConfig) -> None:
    logger = init_logger("flame")
    signal.signal(signal.SIGUSR1, _on_sigusr1)
    gc.disable()
    gc.collect(1)
    rank, local, world, device = init_distributed(job_config, logger)
    tr = job_config.training
    if job_config.job.print_args and rank == 0:
        logger.info(json.dumps(job_config.to_dict(), indent=2, default=str))
    for note in job_config.equivalent_flag_notes():
        logger.info(f"accepted as equivalent: {note}")
    if job_config.experimental.pipeline_parallel_degree > 1:
        raise NotImplementedError("pipeline parallelism is not supported for these models")
    if job_config.experimental.custom_model_path:
        import importlib
        import sys
        sys.path.insert(0, job_config.experimental.custom_model_path)
        importlib.import_module(os.path.basename(job_config.experimental.custom_model_path.rstrip("/")))
    torch.manual_seed(tr.seed)
    if tr.deterministic:
        torch.use_deterministic_algorithms(True, warn_only=True)
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")

    tp = tr.tensor_parallel_degree
    cp = job_config.experimental.context_parallel_degree
    dp_world = world // (tp * cp)
    dp_rank = rank // (tp * cp)

    tokenizer = None
    if not tr.dataset.startswith("synthetic") and not tr.dataset.startswith("mds:"):
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(job_config.model.tokenizer_path, trust_remote_code=True)
    model_config = load_model_config(job_config.model.config)
    if tokenizer is not None:
        model_config.vocab_size = max(len(tokenizer), model_config.vocab_size)
    dataset = build_dataset(tr.dataset, tokenizer, tr.seq_len, dp_rank, dp_world, dataset_name=tr.dataset_name,
                            dataset_split=tr.dataset_split, data_dir=tr.data_dir, data_files=tr.data_files,
                            data_probs=tr.data_probs, streaming=tr.streaming, num_workers=tr.num_workers, seed=tr.seed,
                            shuffle_buffer_size=tr.shuffle_buffer_size, vocab_size=model_config.vocab_size)
    dataloader = build_dataloader(dataset, tokenizer, dp_rank, tr.batch_size, context_len=tr.context_len, varlen=tr.varlen,
                                  num_workers=tr.num_workers if not tr.dataset.startswith("synthetic") else 0,
                                  pin_memory=tr.pin_memory, persistent_workers=tr.persistent_workers,
                                  prefetch_factor=tr.prefetch_factor, bos_token_id=getattr(model_config, "bos_token_id", None),
                                  eos_token_id=getattr(model_config, "eos_token_id", None))
    if rank == 0:
        snapshot_model_config(model_config, job_config.job.dump_folder, logger)

    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[tr.mixed_precision_param]
    if device.type == "cpu":
        dtype = torch.float32
    opt = job_config.optimizer
    ecfg = EngineConfig(lr=opt.lr, betas=(opt.beta1, opt.beta2), eps=opt.eps, weight_decay=opt.weight_decay,
                        max_norm=tr.max_norm, activation_checkpoint=_ac_mode(job_config), dtype=dtype,
                        skip_nan_inf=tr.skip_nan_inf, seed=tr.seed, enable_muon=opt.enable_muon,
                        muon_momentum=opt.muon_momentum, tensor_parallel=tp, context_parallel=cp,
                        activation_offload=job_config.activation_offload.mode not in ("none", "", None),
                        replicate=(tr.data_parallel_shard_degree == 1 and tr.data_parallel_replicate_degree not in (0, 1)),
                        shard_weights=tr.fsdp_reshard_after_forward == "always",
                        replicate_degree=(tr.data_parallel_replicate_degree
                                          if tr.data_parallel_shard_degree != 1 and tr.data_parallel_replicate_degree > 1 else 1))
    engine = TrainEngine(model_config, ecfg, device=device)
    model = engine.model
    n_params = count_params(model, exclude_embedding=True)
    flop_per_token = get_num_flop_per_token(n_params, model_config, tr.seq_len)
    logger.info(f"model {model_config.model_type}: {count_params(model, False):,} parameters, "
                f"{flop_per_token / 1e9:.2f} GFLOP/token, dp={dp_world} tp={tp} cp={cp}")

    schedule = build_lr_schedule(job_config, logger if rank == 0 else None)
    train_state = TrainState()
    ckpt = CheckpointManager(engine, train_state, job_config, dataloader, lr_state=lambda: train_state.step, logger=logger if rank == 0 else None)
    if job_config.checkpoint.create_seed_checkpoint:
        assert world == 1, "seed checkpoints are created by a single process"
        ckpt.save_seed()
        logger.info("created seed checkpoint")
        return
    ckpt.load()
    metrics = MetricsProcessor(job_config, flop_per_token, world, non_dp_size=tp * cp, rank=rank, logger=logger)
    if rank == 0:
        for s, a, m in zip(train_state.log_steps, train_state.global_avg_losses, train_state.global_max_losses):
            metrics.sink.log({"loss_metrics/global_avg_loss": a, "loss_metrics/global_max_loss": m}, s)

    profiler = _maybe_profiler(job_config, rank)
    snapshotter = MemorySnapshotter(job_config, rank)
    data_iter = iter(dataloader)
    accum = tr.gradient_accumulation_steps
    t_start = time.perf_counter()
    logger.info(f"training starts at step {train_state.step + 1} of {tr.steps} "
                f"(batch {tr.batch_size} x seq {tr.seq_len} x accum {accum} per rank)")
    while train_state.step < tr.steps:
        train_state.step += 1
        step = train_state.step
        if step > 1 and step % tr.gc_freq == 0:
            gc.collect(1)
        engine.sdp.zero_grad()
        losses = []
        for micro in range(accum):
            engine.sdp.set_last_microbatch(micro == accum - 1)
            t0 = time.perf_counter()
            batch = next(data_iter)
            metrics.data_loading_times.append(time.perf_counter() - t0)
            kwargs = {}
            if "cu_seqlens" in batch:
                kwargs["cu_seqlens"] = batch["cu_seqlens"].to(device)
            if batch.get("attention_mask") is not None:
                kwargs["attention_mask"] = batch["attention_mask"].to(device)
            ids = batch["input_ids"]
            metrics.ntokens_since_last_log += ids.numel()
            train_state.token += ids.numel()
            losses.append(engine.forward_backward(ids, batch["labels"], scale=1.0 / accum, **kwargs))
        ckpt.maybe_wait_for_staging()
        grad_norm = engine.sdp.step(schedule.lr(step - 1))
        loss = torch.stack(losses).mean()
        if tr.skip_nan_inf and not bool(torch.isfinite(grad_norm)):
            train_state.skipped_step += 1
            logger.warning(f"step {step}: non-finite gradient norm, optimizer step skipped")
        if metrics.should_log(step):
            engine.sdp.check_health()          # a bounded device wait that ran out since the last log raises here
            avg, mx = dist_mean_max(loss)
            extra = {"optimizer/lr": schedule.lr(step - 1), "optimizer/grad_norm": float(grad_norm),
                     "optimizer/skipped_step": train_state.skipped_step}
            if hasattr(model, "get_ttt_norm_metrics"):
                extra.update(model.get_ttt_norm_metrics())
            if engine.last_logits is not None:     # only when the model materialises logits (no fused linear-CE)
                extra.update(loss_by_position(engine.last_logits, engine.last_labels))
            train_state.log_steps.append(step)
            train_state.global_avg_losses.append(avg)
            train_state.global_max_losses.append(mx)
            train_state.elapsed = time.perf_counter() - t_start
            metrics.log(step, avg, mx, extra)
        force_save = external_save_requested(rank)
        if ckpt.should_save(step, last=step == tr.steps, force=force_save):
            engine.sdp.check_health()          # never write weights of a run whose device-side waits ran out
        ckpt.save(step, last=step == tr.steps, force=force_save)
        if profiler is not None:
            profiler.step()
        snapshotter.step(step)
        if step == 1:
            set_pg_timeouts(job_config.comm.train_timeout_seconds)
    if profiler is not None:
        profiler.__exit__(None, None, None)
    metrics.close()
    logger.info("training completed")
    if dist.is_initialized():
        dist.destroy_process_group()


def _maybe_profiler(job_config, rank):
    p = job_config.profiling
    if not p.enable_profiling or not torch.cuda.is_available():
        return None
    folder = os.path.join(job_config.job.dump_folder, p.save_traces_folder)
    freq = max(5, p.profile_freq)

    def handler(prof):
        d = os.path.join(folder, f"iteration_{prof.step_num}")
        os.makedirs(d, exist_ok=True)
        prof.export_chrome_trace(os.path.join(d, f"rank{rank}_trace.json"))

    prof = torch.profiler.profile(
        activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
        schedule=torch.profiler.schedule(wait=freq - 4, warmup=3, active=1), on_trace_ready=handler)
    prof.__enter__()
    return prof


class MemorySnapshotter:
    """CUDA allocator history, dumped as a pickle per rank every ``profile_freq`` steps and on an out-of-memory
    error (``--profiling.enable_memory_snapshot``; the files open in pytorch.org/memory_viz)."""

    def __init__(self, job_config, rank: int):
        p = job_config.profiling
        self.enabled = bool(p.enable_memory_snapshot) and torch.cuda.is_available()
        self.folder = os.path.join(job_config.job.dump_folder, p.save_memory_snapshot_folder)
        self.freq, self.rank = max(1, p.profile_freq), rank
        if self.enabled:
            torch.cuda.memory._record_memory_history(max_entries=100000)

    def dump(self, name: str) -> None:
        d = os.path.join(self.folder, name)
        os.makedirs(d, exist_ok=True)
        torch.cuda.memory._dump_snapshot(os.path.join(d, f"rank{self.rank}_memory_snapshot.pickle"))

    def step(self, step: int, oom: bool = False) -> None:
        if self.enabled and (oom or step % self.freq == 0):
            self.dump(f"iteration_{step}" + ("_exit" if oom else ""))


def cli(argv=None):
    config = JobConfig().parse_args(argv)
    main(config)


if __name__ == "__main__":
    cli()
