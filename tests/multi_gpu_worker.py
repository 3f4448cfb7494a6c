"""Worker run under torch.distributed.run by tests/test_gpu_multi.py (one rank per GPU, NCCL)."""
import os
import sys
import warnings
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
warnings.filterwarnings("ignore")


def check_symmetric():
    from ttcd_b200.comm.symmetric import PeerBarrier, SymmetricBuffer
    rank, world = dist.get_rank(), dist.get_world_size()
    buf = SymmetricBuffer(1 << 20)
    bar = PeerBarrier()
    from ttcd_b200 import _native as nv
    mine = buf.view(torch.bfloat16, 2048)
    mine.fill_(float(rank + 1))
    bar.sync()
    for r in range(world):
        got = torch.empty(2048, dtype=torch.bfloat16, device="cuda")
        # peers are only ever read by this library's own plain-load kernels
        nv.call("ttcd_peer_add", nv.ptr(got), nv.i64(buf.peer_ptrs[r]), nv.i64(2048), nv.i32(0), nv.stream_ptr())
        assert torch.all(got == float(r + 1)), f"rank {rank} read {got[:4]} from rank {r}"
    bar.sync()
    bar.check()
    buf.close()


def check_sharded_modes(muon: bool = False):
    """Optimizer steps with the fused peer-memory path and with the NCCL baseline must agree (AdamW, or
    Muon with the owner pulling whole-parameter gradients and pushing the new weights to every rank)."""
    from ttcd_b200.models import IPTTCDv9Config
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    rank = dist.get_rank()
    cfg = IPTTCDv9Config(hidden_size=256, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768,
                         vocab_size=4096, window_size=256, max_position_embeddings=2048, ttt_mode=True, ttt_chunk=128,
                         ttt_layers=[1], ttt_update_every=4, qk_norm=True, tie_word_embeddings=True, fuse_cross_entropy=False,
                         fuse_linear_cross_entropy=True, ttt_teacher_conv_init="identity")
    results = {}
    for mode in ("peer", "nccl"):
        os.environ["TTCD_COMM"] = mode
        engine = TrainEngine(cfg, EngineConfig(lr=1e-3, seed=7, enable_muon=muon), device=f"cuda:{torch.cuda.current_device()}")
        assert engine.sdp.peer == (mode == "peer")
        g = torch.Generator().manual_seed(100 + rank)
        losses = []
        for _ in range(1 if muon else 3):      # Newton-Schulz amplifies rounding noise: compare one step
            ids = torch.randint(0, cfg.vocab_size, (1, 512), generator=g).cuda()
            losses.append(engine.train_step(ids))
        flat = torch.cat([grp.flat_param.float() for grp in engine.sdp.groups])
        results[mode] = (losses, flat.clone(), float(engine.grad_norm))
        other = flat.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(other, flat), f"{mode}: parameters differ between ranks"
        del engine
        torch.cuda.synchronize()
    (lp, fp, gp), (ln, fn, gn) = results["peer"], results["nccl"]
    assert abs(lp[0] - ln[0]) < 1e-3, (lp, ln)
    assert abs(gp - gn) < 2e-2 * max(1.0, gn), (gp, gn)
    diff = (fp - fn).abs().max().item()
    assert diff < 2e-2, f"peer vs nccl parameter diff {diff}"
    assert lp[-1] < lp[0] + 0.5, lp


def _small_engine(**over):
    from ttcd_b200.models import IPTTCDv9Config
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    cfg = IPTTCDv9Config(hidden_size=256, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768,
                         vocab_size=4096, window_size=256, max_position_embeddings=2048, ttt_mode=True, ttt_chunk=128,
                         ttt_layers=[1], ttt_update_every=4, qk_norm=True, tie_word_embeddings=True, fuse_cross_entropy=False,
                         fuse_linear_cross_entropy=True, ttt_teacher_conv_init="identity")
    kw = dict(lr=1e-3, seed=7, activation_checkpoint="none")
    kw.update(over)
    return cfg, TrainEngine(cfg, EngineConfig(**kw), device=f"cuda:{torch.cuda.current_device()}")


def check_late_rank_is_detected_and_the_step_skipped():
    """A rank that is later than the peer-wait budget (a stalled data loader: it sleeps on the host between two
    steps, with nothing of its own in flight): its peers' flag wait runs out, every rank skips that optimizer step
    (agreed through the gradient-norm all-reduce), the weights stay identical, ``check_health`` raises on every
    rank, and training continues afterwards."""
    import time
    rank = dist.get_rank()
    os.environ["TTCD_COMM"] = "peer"
    os.environ["TTCD_PEER_WAIT_NS"] = "300000000"          # 0.3 s
    try:
        cfg, eng = _small_engine()
    finally:
        del os.environ["TTCD_PEER_WAIT_NS"]
    assert eng.sdp.peer and eng.sdp.peer_wait_ns == 300000000
    g = torch.Generator().manual_seed(100 + rank)
    batch = lambda: torch.randint(0, cfg.vocab_size, (1, 512), generator=g).cuda()      # noqa: E731
    eng.train_step(batch())
    eng.sdp.check_health()                                 # a healthy step raises nothing
    before = torch.cat([grp.flat_param.float() for grp in eng.sdp.groups]).clone()
    masters = [grp.master.clone() for grp in eng.sdp.groups]
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 1:
        time.sleep(1.5)                                    # late by five wait budgets
    eng.train_step(batch())
    torch.cuda.synchronize()
    after = torch.cat([grp.flat_param.float() for grp in eng.sdp.groups])
    assert torch.equal(before, after), "the step after an expired wait must leave the weights alone"
    for grp, m in zip(eng.sdp.groups, masters):
        assert torch.equal(grp.master, m)
    raised = False
    try:
        eng.sdp.check_health()
    except RuntimeError as exc:
        raised = True
        assert "wait ran out" in str(exc), exc
    assert raised, f"rank {rank}: the expired wait went unnoticed"
    dist.barrier()
    loss = eng.train_step(batch())                         # the run goes on
    eng.sdp.check_health()
    now = torch.cat([grp.flat_param.float() for grp in eng.sdp.groups])
    assert not torch.equal(now, before) and loss == loss
    other = now.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(other, now), "parameters differ between ranks after the recovery step"


def check_accumulation_on_gpus():
    """Two micro-batches with the reduction after the last one == one batch of both sequences (norm and weights)."""
    rank = dist.get_rank()
    os.environ["TTCD_COMM"] = "peer"
    g = torch.Generator().manual_seed(300 + rank)
    cfg, whole = _small_engine(max_norm=0.05)
    ids = torch.randint(0, cfg.vocab_size, (2, 512), generator=g).cuda()
    whole.sdp.zero_grad()
    whole.forward_backward(ids)
    norm_a = float(whole.sdp.step(1e-3))
    _, split = _small_engine(max_norm=0.05)
    split.sdp.zero_grad()
    for m in range(2):
        split.sdp.set_last_microbatch(m == 1)
        split.forward_backward(ids[m:m + 1], scale=0.5)
    norm_b = float(split.sdp.step(1e-3))
    assert norm_a > 0.05, norm_a                           # the clip is active, so a wrong norm would change the update
    assert abs(norm_a - norm_b) < 3e-2 * norm_a, (norm_a, norm_b)
    fa = torch.cat([grp.flat_param.float() for grp in whole.sdp.groups])
    fb = torch.cat([grp.flat_param.float() for grp in split.sdp.groups])
    assert (fa - fb).abs().max().item() < 1e-2, (fa - fb).abs().max().item()


def check_sharded_weights():
    """ZeRO-3 layout on GPUs: block parameters stored 1/world per rank, gathered INSIDE the fused q|k|v GEMM in the
    forward (and in the recomputation), by the stand-alone kernel for a backward without recomputation; three steps
    end where the resident layout ends."""
    from ttcd_b200.parallel import sharded as sharded_mod
    rank = dist.get_rank()
    os.environ["TTCD_COMM"] = "peer"
    results = {}
    for name, kw in (("resident", {}), ("sharded", {"shard_weights": True}), ("sharded_ac", {"shard_weights": True,
                                                                                            "activation_checkpoint": "full"})):
        calls = []
        orig = sharded_mod._native.call

        def counting(sym, *a, _orig=orig, _calls=calls):
            _calls.append(sym)
            return _orig(sym, *a)
        sharded_mod._native.call = counting
        try:
            cfg, eng = _small_engine(**kw)
            g = torch.Generator().manual_seed(100 + rank)
            losses = [eng.train_step(torch.randint(0, cfg.vocab_size, (1, 512), generator=g).cuda()) for _ in range(3)]
            torch.cuda.synchronize()
            eng.sdp.check_health()
        finally:
            sharded_mod._native.call = orig
        with eng.sdp.full_parameters():
            flat = torch.cat([p.detach().float().reshape(-1) for p in eng.model.parameters()]).clone()
        results[name] = (losses, flat)
        fused = calls.count("ttcd_wgather_gemm")
        plain = calls.count("ttcd_peer_gather")
        if name == "resident":
            assert fused == 0 and plain == 0
        elif name == "sharded":          # 2 blocks x 3 steps: fused in forward, stand-alone for backward (+ the final read)
            assert fused == 6 and plain >= 6, (fused, plain)
        else:                            # with recomputation the backward's gather is fused too
            assert fused == 12, (fused, plain)
        other = flat.clone()
        dist.broadcast(other, src=0)
        assert torch.equal(other, flat), f"{name}: parameters differ between ranks"
        del eng
        torch.cuda.synchronize()
    base_l, base_f = results["resident"]
    for name in ("sharded", "sharded_ac"):
        l, f = results[name]
        assert abs(l[0] - base_l[0]) < 1e-3 and abs(l[-1] - base_l[-1]) < 5e-2, (name, l, base_l)
        assert (f - base_f).abs().max().item() < 2e-2, (name, (f - base_f).abs().max().item())


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    from ttcd_b200 import _native
    _native.load(required=True)
    if what in ("all", "symmetric"):
        check_symmetric()
    if what in ("all", "sharded"):
        check_sharded_modes()
    if what in ("all", "muon"):
        check_sharded_modes(muon=True)
    if what in ("all", "tp"):
        from tests.multi_gpu_tp import check_tensor_parallel, check_tp_model
        check_tensor_parallel()
        check_tp_model()
        check_tp_model(muon=True)
    if what in ("all", "zero3"):
        check_sharded_weights()
    if what in ("all", "late_rank"):
        check_late_rank_is_detected_and_the_step_skipped()
    if what in ("all", "accum"):
        check_accumulation_on_gpus()
    if what in ("all", "cp"):
        from tests.multi_gpu_cp import check_context_parallel
        check_context_parallel()
        check_context_parallel(window=None)
    if what in ("all", "layouts"):
        from tests.multi_gpu_misc import check_all
        check_all()
    torch.cuda.synchronize()
    assert _native.device_status() == 0
    dist.barrier()
    if dist.get_rank() == 0:
        print("MULTI_GPU_OK", what)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
