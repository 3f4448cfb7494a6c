"""Resume is exact: N steps + save + load + M steps ends bit for bit where N + M uninterrupted steps end.

The runtime keeps bf16 compute weights and fp32 master weights; a checkpoint stores the masters, and a load must
put them back as they were (not their bf16 rounding), for AdamW-owned and Muon-owned parameters alike.  Runs on
CPU with bf16 parameters so that the master / compute split is real; world 1 and two gloo ranks.
"""
import os
import socket

import pytest
import torch

from ttcd_b200.models import IPTTCDv9Config
from ttcd_b200.train.checkpoint import CheckpointManager, TrainState
from ttcd_b200.train.config_manager import JobConfig
from ttcd_b200.train.engine import EngineConfig, TrainEngine

KW = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=128,
          window_size=32, ttt_mode=True, ttt_chunk=8, ttt_layers=[1], fuse_cross_entropy=False, tie_word_embeddings=False)
N_BEFORE, N_AFTER = 3, 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _engine(muon: bool):
    return TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.bfloat16, lr=3e-3, weight_decay=0.1, max_norm=1.0, seed=11,
                                                          activation_checkpoint="none", enable_muon=muon), device="cpu")


def _batch(step: int, rank: int):
    g = torch.Generator().manual_seed(1000 * rank + step)
    return torch.randint(0, 128, (1, 32), generator=g)


def _steps(eng, first: int, count: int, rank: int):
    for s in range(first, first + count):
        eng.sdp.zero_grad()
        eng.forward_backward(_batch(s, rank))
        eng.sdp.step(3e-3)


def _fingerprint(eng):
    out = {}
    for g in eng.sdp.groups:
        out[f"{g.name}.master"] = g.master.clone()
        out[f"{g.name}.exp_avg"] = g.exp_avg.clone()
        out[f"{g.name}.flat_param"] = g.flat_param.clone()
    for mp in eng.sdp.muon_params:
        if mp.master is not None:
            out[f"{mp.name}.master"] = mp.master.clone()
            out[f"{mp.name}.momentum"] = mp.momentum.clone()
    return out


def _job(folder):
    return JobConfig().parse_args(["--job.dump_folder", str(folder), "--checkpoint.enable_checkpoint", "--checkpoint.interval", "1"])


def _straight_vs_resumed(folder, muon: bool, rank: int = 0):
    straight = _engine(muon)
    _steps(straight, 0, N_BEFORE + N_AFTER, rank)
    first = _engine(muon)
    _steps(first, 0, N_BEFORE, rank)
    state = TrainState(step=N_BEFORE)
    CheckpointManager(first, state, _job(folder)).save(N_BEFORE, force=True)
    second = _engine(muon)
    with torch.no_grad():                      # a resumed process must not depend on its own initialisation
        for p in second.model.parameters():
            p.add_(0.25)
    state2 = TrainState()
    assert CheckpointManager(second, state2, _job(folder)).load()
    assert state2.step == N_BEFORE and second.sdp.step_count == N_BEFORE
    _steps(second, N_BEFORE, N_AFTER, rank)
    want, got = _fingerprint(straight), _fingerprint(second)
    assert want.keys() == got.keys()
    return [k for k in want if not torch.equal(want[k], got[k])]


@pytest.mark.timeout(600)
@pytest.mark.parametrize("muon", [False, True])
def test_resume_is_bitwise_single_process(tmp_path, muon):
    assert _straight_vs_resumed(tmp_path, muon) == []


def _worker(rank, world, port, folder, muon, q):
    import torch.distributed as dist
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        q.put((rank, _straight_vs_resumed(folder, muon, rank)))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error: " + traceback.format_exc()))


@pytest.mark.timeout(900)
@pytest.mark.parametrize("muon", [False, True])
def test_resume_is_bitwise_two_ranks(tmp_path, muon):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), muon, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, differing in results:
        assert differing == [], f"rank {rank}: {differing}"
