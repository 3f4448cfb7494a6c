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
