"""Failure detection without faulting any device: failures are injected on the host (a rank that leaves
between steps, a corrupted checkpoint shard, a non-finite loss) and must turn into a clean error / skip /
resume, never a hang.  CPU ranks talk over gloo with short timeouts."""
import datetime
import json
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ttcd_b200.models import IPTTCDv9Config
from ttcd_b200.train.engine import EngineConfig, TrainEngine

KW = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=128,
          window_size=32, ttt_mode=True, ttt_chunk=8, ttt_layers=[1], fuse_cross_entropy=False, tie_word_embeddings=False)


def _leave(q):
    q.close()
    q.join_thread()          # flush the report before the abrupt exit
    os._exit(0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_leaves(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                     # step 1: everybody is there
    if rank == 1:
        q.put((rank, "left"))              # leaves between steps, nothing in flight
        _leave(q)
    try:
        dist.all_reduce(t)                 # step 2: the peer is gone -> error within the timeout, not a hang
        q.put((rank, "no error"))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, f"detected: {type(exc).__name__}"))
    _leave(q)


@pytest.mark.timeout(120)
def test_rank_leaving_between_steps_is_detected_by_timeout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_leaves, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=90) for _ in procs)
    for p in procs:
        p.join(30)
    assert got[1] == "left"
    assert got[0].startswith("detected"), got


def _rank_never_joins(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as exc:  # noqa: BLE001
        q.put(f"detected: {type(exc).__name__}")
    _leave(q)


@pytest.mark.timeout(120)
def test_rank_that_never_joins_fails_the_rendezvous():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_rank_never_joins, args=(0, 2, _free_port(), q))     # rank 1 is never started
    p.start()
    assert q.get(timeout=90).startswith("detected")
    p.join(30)


def test_non_finite_gradient_skips_the_step_and_keeps_weights():
    eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=1e-2, activation_checkpoint="none",
                                                         skip_nan_inf=True), device="cpu")
    ids = torch.randint(0, 128, (1, 32))
    eng.sdp.zero_grad()
    eng.forward_backward(ids)
    before = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    next(eng.model.parameters()).grad.view(-1)[0] = float("nan")          # injected on the host
    norm = eng.sdp.step(1e-2)
    assert not torch.isfinite(norm)
    for n, p in eng.model.named_parameters():
        assert torch.equal(p.detach(), before[n]), n
    eng.sdp.zero_grad()                                                      # the next clean step moves them again
    eng.forward_backward(ids)
    assert torch.isfinite(eng.sdp.step(1e-2))
    assert any(not torch.equal(p.detach(), before[n]) for n, p in eng.model.named_parameters())


def test_corrupted_newest_checkpoint_is_reported(tmp_path):
    from ttcd_b200.train.trainer import cli
    cfg = tmp_path / "model.json"
    cfg.write_text(json.dumps(dict(model_type="ipttcdv9", **KW)))
    args = ["--job.dump_folder", str(tmp_path / "run"), "--model.config", str(cfg), "--training.dataset", "synthetic",
            "--training.seq_len", "32", "--training.batch_size", "1", "--checkpoint.enable_checkpoint", "--checkpoint.interval", "1",
            "--lr_scheduler.warmup_steps", "1"]
    cli(args + ["--training.steps", "2"])
    shard = next((tmp_path / "run" / "checkpoint" / "step-2").glob("*.distcp"))
    shard.write_bytes(shard.read_bytes()[:128])                             # truncated shard
    with pytest.raises(Exception):
        cli(args + ["--training.steps", "3"])
    cli(args + ["--training.steps", "3", "--checkpoint.load_step", "1"])     # the operator falls back to the older step
    assert (tmp_path / "run" / "checkpoint" / "step-3" / ".metadata").is_file()
