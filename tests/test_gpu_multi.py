"""Multi-GPU checks (symmetric memory, flag barrier, fused reduce-scatter / AdamW-push vs the NCCL baseline).

Each test launches one process per GPU with torch.distributed.run and is skipped on machines with fewer
than two GPUs.  Host-side protocol logic is covered on CPU in tests/test_flag_protocol_model.py and
tests/test_sharded_runtime_cpu.py.
"""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(what: str, nproc: int, timeout: int = 600, **extra_env) -> str:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(ROOT / "tests" / "multi_gpu_worker.py"), what]
    env = dict(os.environ, PYTHONPATH=str(ROOT), **extra_env)
    for attempt in range(3):
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))
        out = res.stdout + res.stderr
        if "EADDRINUSE" not in out:
            break
        cmd[cmd.index("--master-port") + 1] = str(_free_port())      # somebody took the port between the probe and the bind
    assert res.returncode == 0 and "MULTI_GPU_OK" in out, out[-4000:]
    return out


def _ngpu() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_symmetric_memory_and_barrier():
    _launch("symmetric", min(_ngpu(), 8))


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_fused_sharded_step_matches_nccl_baseline():
    _launch("sharded", 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_muon_owner_pull_push_matches_nccl_baseline():
    _launch("muon", 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_fused_allgather_gemm_and_gemm_reducescatter():
    _launch("tp", 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_context_parallel_halo_attention_matches_single_gpu():
    _launch("cp", 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_late_rank_expires_the_peer_wait_and_every_rank_skips_the_step():
    # failure-detection runs keep NVLS off: a rank in trouble must not sit on an NVLink multicast object
    _launch("late_rank", 2, NCCL_NVLS_ENABLE="0")


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_gradient_accumulation_reduces_once_on_gpus():
    _launch("accum", 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_sharded_weights_gathered_inside_the_first_gemm():
    _launch("zero3", 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
@pytest.mark.timeout(900)
def test_replicated_pipeline_vocab_parallel_and_hybrid_layouts_on_gpus():
    """Replicated data parallelism, vocabulary-parallel cross-entropy and a two-stage pipeline on 2 GPUs; with 4 or
    more GPUs also hybrid sharding (2 replicas x 2 shards)."""
    _launch("layouts", 4 if _ngpu() >= 4 else 2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
@pytest.mark.timeout(900)
def test_trainer_entry_point_on_two_gpus_saves_and_resumes(tmp_path):
    """``python -m flame.train`` under torchrun on 2 GPUs (native kernels, fused peer-memory data parallelism, synthetic
    data): 4 steps with a checkpoint at 2 and 4, then a second launch that resumes at 4 and trains to 6."""
    import json
    cfg = dict(model_type="ipttcdv9", hidden_size=256, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
               intermediate_size=768, vocab_size=4096, window_size=256, max_position_embeddings=2048, ttt_mode=True,
               ttt_chunk=128, ttt_layers=[1], ttt_update_every=4, qk_norm=True, tie_word_embeddings=True,
               fuse_cross_entropy=False, fuse_linear_cross_entropy=True)
    (tmp_path / "model.json").write_text(json.dumps(cfg))

    def run(steps: int) -> str:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
               "--master-port", str(_free_port()), "-m", "flame.train", "--job.dump_folder", str(tmp_path / "run"),
               "--model.config", str(tmp_path / "model.json"), "--training.dataset", "synthetic", "--training.seq_len", "1024",
               "--training.batch_size", "1", "--training.steps", str(steps), "--optimizer.lr", "1e-3",
               "--lr_scheduler.warmup_steps", "2", "--checkpoint.enable_checkpoint", "--checkpoint.interval", "2",
               "--metrics.log_freq", "1", "--training.seed", "3"]
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, PYTHONPATH=str(ROOT)),
                             cwd=str(ROOT))
        out = res.stdout + res.stderr
        assert res.returncode == 0, out[-4000:]
        return out

    first = run(4)
    ckpt = tmp_path / "run" / "checkpoint"
    assert (ckpt / "step-2" / ".metadata").is_file() and (ckpt / "step-4" / ".metadata").is_file(), first[-2000:]
    second = run(6)
    assert (ckpt / "step-6" / ".metadata").is_file(), second[-2000:]
    assert "step-4" in second or "step 4" in second.lower() or "resum" in second.lower() or "load" in second.lower(), second[-2000:]
