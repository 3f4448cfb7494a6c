"""Context-parallel logic on CPU (gloo, 2 ranks): sequence sharding, RoPE offsets, halo attention (all-gather
statement), fast-weight prefix over ranks, label shift across the shard boundary and loss weighting must
reproduce the single-process loss and gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ttcd_b200.models import IPTTCDv9Config

KW = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
          vocab_size=256, window_size=48, ttt_mode=True, ttt_chunk=16, ttt_visible_chunks=1, ttt_layers=[1], ttt_lr=0.05,
          ttt_update_every=2, fuse_cross_entropy=False, ttt_teacher_conv_init="identity", qk_norm=True,
          ttt_normalize_student_features=False, max_position_embeddings=256)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ids, ref_loss, ref_grads, q, window=48):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from ttcd_b200.train.engine import EngineConfig, TrainEngine
        cfg = IPTTCDv9Config(**dict(KW, window_size=window))
        eng = TrainEngine(cfg, EngineConfig(dtype=torch.float32, lr=0.0, seed=3, activation_checkpoint="none",
                                            context_parallel=world, max_norm=None), device="cpu")
        with torch.no_grad():
            for n, p in eng.model.named_parameters():
                if "conv" in n:
                    p.normal_(0, 0.3, generator=torch.Generator().manual_seed(11))
        eng.sdp.resync_master()
        eng.sdp.zero_grad()
        loss = eng.forward_backward(ids)
        grads = {n: p.grad.clone() for n, p in eng.model.named_parameters()}
        for g in grads.values():          # average over ranks == what the sharded runtime does
            dist.all_reduce(g)
            g /= world
        err = abs(float(loss) - ref_loss)
        worst = max(((grads[n] - ref_grads[n]).abs().max().item() / (ref_grads[n].abs().max().item() + 1e-6), n) for n in grads)
        q.put((rank, err, worst))
        dist.destroy_process_group()
    except Exception as exc:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.timeout(300)
@pytest.mark.parametrize("window", [48, None, 100])
def test_context_parallel_matches_single_process(window):
    """window 48: the K/V halo path.  None (full-attention teacher) and 100 (longer than the 64-token shard): the
    head-parallel path, where one all-to-all gives each rank all tokens of half the heads."""
    torch.manual_seed(0)
    ids = torch.randint(0, 256, (2, 128))
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(IPTTCDv9Config(**dict(KW, window_size=window)), EngineConfig(dtype=torch.float32, lr=0.0, seed=3, activation_checkpoint="none",
                                                         max_norm=None), device="cpu")
    with torch.no_grad():
        for n, p in eng.model.named_parameters():
            if "conv" in n:
                p.normal_(0, 0.3, generator=torch.Generator().manual_seed(11))
    eng.sdp.zero_grad()
    ref_loss = float(eng.forward_backward(ids))
    ref_grads = {n: p.grad.clone() for n, p in eng.model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ids, ref_loss, ref_grads, q, window)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err, worst in results:
        assert err != "error", worst
        assert err < 1e-4, f"rank {rank}: loss differs by {err}"
        assert worst[0] < 2e-3, f"rank {rank}: gradient of {worst[1]} differs by {worst[0]:.3g} (relative)"
