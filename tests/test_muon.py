"""Muon in the sharded runtime vs a direct statement of the reference update rule (CPU, fp32)."""
import math

import torch

from ttcd_b200.models import IPTTCDv9Config
from ttcd_b200.ops import reference as ref
from ttcd_b200.train.engine import EngineConfig, TrainEngine
from ttcd_b200.train.muon import assign_owners, default_is_muon, MuonParam, ns_cost

KW = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=128,
          window_size=32, ttt_mode=True, ttt_chunk=8, ttt_layers=[1], fuse_cross_entropy=False, tie_word_embeddings=False)


def test_param_split_and_owner_balance():
    assert default_is_muon("model.layers.0.attn.q_proj.weight", torch.empty(4, 4))
    assert not default_is_muon("model.embeddings.weight", torch.empty(4, 4))
    assert not default_is_muon("lm_head.weight", torch.empty(4, 4))
    assert not default_is_muon("model.layers.0.attn_norm.weight", torch.empty(4))
    ps = [MuonParam(f"p{i}", torch.nn.Parameter(torch.empty(s)), 0, 0) for i, s in enumerate([(64, 64), (128, 64), (64, 128), (32, 32)])]
    assign_owners(ps, 2)
    load = [sum(ns_cost(p.param.shape) for p in ps if p.owner == r) for r in range(2)]
    assert max(load) / sum(load) < 0.6


def test_muon_step_matches_reference_rule():
    torch.manual_seed(0)
    eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=0.02, weight_decay=0.1, max_norm=None,
                                                         activation_checkpoint="none", enable_muon=True, muon_momentum=0.95), device="cpu")
    w_before = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    ids = torch.randint(0, 128, (2, 64))
    eng.sdp.zero_grad()
    eng.forward_backward(ids)
    grads = {n: p.grad.detach().clone() for n, p in eng.model.named_parameters()}
    eng.sdp.step(0.02)
    name = "model.layers.0.mlp.gate_proj.weight"
    g = grads[name]                       # first step: buf = g, nesterov g + mu*buf
    gn = g + 0.95 * g
    u = ref.newton_schulz(gn, dtype=torch.float32)
    want = w_before[name] * (1 - 0.02 * 0.1) - 0.02 * 0.2 * math.sqrt(max(g.shape)) * u
    got = dict(eng.model.named_parameters())[name]
    torch.testing.assert_close(got, want, rtol=2e-2, atol=1e-3)   # the iteration itself runs in bf16
    # a non-Muon parameter follows AdamW: first step moves every element by ~lr in the gradient's sign
    emb = dict(eng.model.named_parameters())["model.embeddings.weight"]
    moved = (emb - w_before["model.embeddings.weight"] * (1 - 0.02 * 0.1)).abs()
    touched = grads["model.embeddings.weight"].abs() > 1e-8
    assert torch.allclose(moved[touched], torch.full_like(moved[touched], 0.02), rtol=1e-2, atol=1e-5)
    # q/k/v stay one contiguous slab so the fused projection still applies
    attn = eng.model.model.layers[0].attn
    assert attn.k_proj.weight.data_ptr() == attn.q_proj.weight.data_ptr() + attn.q_proj.weight.numel() * 4


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ids, want, q):
    import os
    import torch.distributed as dist
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=0.02, weight_decay=0.1, max_norm=1.0, seed=5,
                                                             activation_checkpoint="none", enable_muon=True), device="cpu")
        for _ in range(1):     # one step: Newton-Schulz amplifies rounding noise, so longer runs drift apart
            eng.sdp.zero_grad()
            eng.forward_backward(ids[rank:rank + 1])
            eng.sdp.step(0.02)
        got = {n: p.detach() for n, p in eng.model.named_parameters()}
        worst = max(((got[n] - want[n]).abs().max().item(), n) for n in got)
        sd = eng.sdp.full_optimizer_state()
        q.put((rank, worst, sorted(k for k in sd if k.endswith("momentum_buffer"))[:1]))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


def test_two_ranks_match_one():
    import torch.multiprocessing as mp
    torch.manual_seed(1)
    ids = torch.randint(0, 128, (2, 64))
    eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=0.02, weight_decay=0.1, max_norm=1.0, seed=5,
                                                         activation_checkpoint="none", enable_muon=True), device="cpu")
    for _ in range(1):
        eng.sdp.zero_grad()
        eng.forward_backward(ids)
        eng.sdp.step(0.02)
    want = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ids, want, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, worst, keys in results:
        assert worst != "error", keys
        assert worst[0] < 2e-3, worst
        assert keys, "Muon momentum missing from the optimizer state"


def _ddp_worker(rank, world, port, ids, want, q):
    import os
    import torch.distributed as dist
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=0.02, weight_decay=0.1, max_norm=1.0, seed=5,
                                                             activation_checkpoint="none", replicate=True), device="cpu")
        from ttcd_b200.parallel.replicated import ReplicatedDataParallel
        assert isinstance(eng.sdp, ReplicatedDataParallel)
        for _ in range(2):
            eng.sdp.zero_grad()
            eng.forward_backward(ids[rank:rank + 1])
            eng.sdp.step(0.02)
        got = {n: p.detach() for n, p in eng.model.named_parameters()}
        q.put((rank, max(((got[n] - want[n]).abs().max().item(), n) for n in got), []))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


def test_replicated_data_parallel_matches_single_process():
    """DDP fallback: all-reduced flat gradient buckets + full optimizer on every rank == one process on the whole batch."""
    import torch.multiprocessing as mp
    torch.manual_seed(2)
    ids = torch.randint(0, 128, (2, 64))
    eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=0.02, weight_decay=0.1, max_norm=1.0, seed=5,
                                                         activation_checkpoint="none"), device="cpu")
    for _ in range(2):
        eng.sdp.zero_grad()
        eng.forward_backward(ids)
        eng.sdp.step(0.02)
    want = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ddp_worker, args=(r, 2, port, ids, want, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, worst, extra in results:
        assert worst != "error", extra
        assert worst[0] < 1e-4, worst
