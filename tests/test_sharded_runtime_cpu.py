"""Host-side logic of the sharded runtime on gloo ranks: gradient accumulation reduces once and takes the right
norm, hybrid sharding (replicate x shard) equals one process, flags without machinery behind them are refused,
and the op-level recompute policy leaves gradients unchanged."""
import os
import socket

import pytest
import torch

from ttcd_b200.models import IPTTCDv9Config
from ttcd_b200.train.config_manager import JobConfig
from ttcd_b200.train.engine import EngineConfig, TrainEngine

KW = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=128,
          window_size=32, ttt_mode=True, ttt_chunk=8, ttt_layers=[1], fuse_cross_entropy=False, tie_word_embeddings=False)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(target, world, *args, timeout=300):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q, *args)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=timeout) for _ in procs]
    for p in procs:
        p.join(30)
    for res in results:
        assert res[1] != "error", res[2]
    return results


def _init(rank, world, port):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _engine(**over):
    cfg = dict(dtype=torch.float32, lr=0.02, weight_decay=0.1, max_norm=0.5, seed=5, activation_checkpoint="none")
    cfg.update(over)
    return TrainEngine(IPTTCDv9Config(**KW), EngineConfig(**cfg), device="cpu")


# ------------------------------------------------------------------------------------- gradient accumulation
def _accum_worker(rank, world, port, q, ids, replicate):
    try:
        import torch.distributed as dist
        _init(rank, world, port)
        mine = ids[rank * 2:(rank + 1) * 2]
        whole = _engine(replicate=replicate)
        whole.sdp.zero_grad()
        whole.forward_backward(mine)
        norm_a = float(whole.sdp.step(0.02))
        split = _engine(replicate=replicate)
        split.sdp.zero_grad()
        reductions = []
        orig = split.sdp._reduce_group
        split.sdp._reduce_group = lambda g: (reductions.append(g.name), orig(g))[1]
        for m in range(2):
            split.sdp.set_last_microbatch(m == 1)
            split.forward_backward(mine[m:m + 1], scale=0.5)
        norm_b = float(split.sdp.step(0.02))
        worst = max(((a - b).abs().max().item(), n) for (n, a), (_, b) in
                    zip(whole.model.named_parameters(), split.model.named_parameters()))
        q.put((rank, "ok", (norm_a, norm_b, worst, len(reductions), len(split.sdp.groups))))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.timeout(600)
@pytest.mark.parametrize("replicate", [False, True])
def test_accumulation_reduces_once_and_matches_one_batch(replicate):
    torch.manual_seed(3)
    ids = torch.randint(0, 128, (4, 48))
    for rank, _, (norm_a, norm_b, worst, n_red, n_groups) in _spawn(_accum_worker, 2, ids, replicate):
        assert n_red == n_groups, f"rank {rank}: {n_red} reductions for {n_groups} groups"
        assert norm_a > 0.5, "the clip must be active for the norm to matter"
        assert abs(norm_a - norm_b) < 1e-4 * norm_a, (norm_a, norm_b)
        assert worst[0] < 2e-5, worst


# ------------------------------------------------------------------------------------- hybrid sharding
def _hybrid_worker(rank, world, port, q, ids, want):
    try:
        import torch.distributed as dist
        _init(rank, world, port)
        eng = _engine(replicate_degree=2)
        assert eng.sdp.world == 2 and eng.sdp.replicate_world == 2
        for _ in range(2):
            eng.sdp.zero_grad()
            eng.forward_backward(ids[rank:rank + 1])
            eng.sdp.step(0.02)
        got = {n: p.detach() for n, p in eng.model.named_parameters()}
        q.put((rank, "ok", max(((got[n] - want[n]).abs().max().item(), n) for n in got)))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.timeout(600)
def test_hybrid_sharding_2x2_matches_one_process():
    torch.manual_seed(4)
    ids = torch.randint(0, 128, (4, 48))
    eng = _engine()
    for _ in range(2):
        eng.sdp.zero_grad()
        eng.forward_backward(ids)
        eng.sdp.step(0.02)
    want = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    for rank, _, worst in _spawn(_hybrid_worker, 4, ids, want):
        assert worst[0] < 1e-4, (rank, worst)


# ------------------------------------------------------------------------------------- flags
@pytest.mark.parametrize("flag", ["--training.enable_cpu_offload", "--optimizer.early_step_in_backward", "--training.compile",
                                  "--fault_tolerance.enable", "--float8.enable_fsdp_float8_all_gather",
                                  "--memory_estimation.enabled", "--experimental.enable_compiled_autograd"])
def test_flags_without_machinery_are_refused(flag):
    with pytest.raises(NotImplementedError):
        JobConfig().parse_args([flag])
    JobConfig().parse_args([])          # the defaults parse


def test_flag_for_another_schedule_of_the_same_update_is_accepted_with_a_note():
    cfg = JobConfig()
    cfg.parse_args(["--optimizer.use_distributed_muon"])
    notes = cfg.equivalent_flag_notes()
    assert len(notes) == 1 and "use_distributed_muon" in notes[0] and "owner" in notes[0]
    plain = JobConfig()
    plain.parse_args([])
    assert plain.equivalent_flag_notes() == []


# ------------------------------------------------------------------------------------- op-level recompute policy
def test_op_recompute_policy_keeps_gradients():
    torch.manual_seed(6)
    ids = torch.randint(0, 128, (2, 48))
    grads = {}
    for mode in ("none", "op", "full"):
        eng = _engine(activation_checkpoint=mode)
        eng.sdp.zero_grad()
        eng.forward_backward(ids)
        grads[mode] = {n: p.grad.detach().clone() for n, p in eng.model.named_parameters()}
    for mode in ("op", "full"):
        for n, g in grads["none"].items():
            torch.testing.assert_close(grads[mode][n], g, rtol=1e-5, atol=1e-6, msg=f"{mode}: {n}")


def test_keep_records_then_replays():
    from ttcd_b200.ops.selective import OpCache, keep
    cache, calls = OpCache(), []

    def launch(v):
        calls.append(v)
        return torch.full((2,), float(v)), None

    with cache.scope():
        a = keep(lambda: launch(1))
        b = keep(lambda: launch(2))
    with cache.scope():                       # the recomputation: nothing is launched again
        a2 = keep(lambda: launch(10))
        b2 = keep(lambda: launch(20))
    assert calls == [1, 2]
    assert torch.equal(a[0], a2[0]) and torch.equal(b[0], b2[0]) and a2[1] is None
    assert keep(lambda: launch(3))[0][0] == 3 and calls == [1, 2, 3]      # outside a scope: a plain call


# ------------------------------------------------------------------------------------- sharded weights (ZeRO-3)
def _zero3_worker(rank, world, port, q, ids, want, tmp):
    try:
        import torch.distributed as dist
        from ttcd_b200.train.checkpoint import CheckpointManager, TrainState
        _init(rank, world, port)
        for ac in ("none", "full"):
            eng = _engine(shard_weights=True, activation_checkpoint=ac)
            blocks = [g for g in eng.sdp.groups if g.sharded]
            assert len(blocks) == 2 and not eng.sdp.groups[-1].sharded
            assert all(g.shard_store.numel() * world == g.numel for g in blocks)
            for _ in range(2):
                eng.sdp.zero_grad()
                eng.forward_backward(ids[rank:rank + 1])
                eng.sdp.step(0.02)
            assert all(g.pool_slot < 0 for g in blocks), "a block kept its pooled buffer after the step"
            with eng.sdp.full_parameters():
                got = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
            worst = max(((got[n] - want[n]).abs().max().item(), n) for n in got)
            assert worst[0] < 1e-4, (ac, worst)
        # a checkpoint written from shards loads into a fresh engine and the run continues identically
        job = JobConfig().parse_args(["--job.dump_folder", tmp, "--checkpoint.enable_checkpoint"])
        CheckpointManager(eng, TrainState(step=2), job).save(2, force=True)
        other = _engine(shard_weights=True, seed=99)
        assert CheckpointManager(other, TrainState(), job).load()
        for e in (eng, other):
            e.sdp.zero_grad()
            e.forward_backward(ids[rank:rank + 1])
            e.sdp.step(0.02)
        for ga, gb in zip(eng.sdp.groups, other.sdp.groups):
            assert torch.equal(ga.master, gb.master), ga.name
        q.put((rank, "ok", worst))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.timeout(900)
def test_sharded_weights_match_resident_weights(tmp_path):
    """Block parameters stored 1/world per rank and gathered per block (forward, backward, recomputation) train like
    the resident layout, with and without activation checkpointing, and survive a checkpoint round trip."""
    torch.manual_seed(8)
    ids = torch.randint(0, 128, (2, 48))
    eng = _engine()
    for _ in range(2):
        eng.sdp.zero_grad()
        eng.forward_backward(ids)
        eng.sdp.step(0.02)
    want = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    _spawn(_zero3_worker, 2, ids, want, str(tmp_path))
