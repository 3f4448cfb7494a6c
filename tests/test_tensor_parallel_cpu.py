"""Tensor + sequence parallel wiring on CPU (gloo, 2 ranks): head / row / column sharding, token-sharded
residual stream, the TP-legal fast-weight scan (all-reduced projection, reduce-scattered output), globally
shifted labels and replicated-gradient sums must reproduce the single-process loss and gradients."""
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
          ttt_normalize_student_features=False, max_position_embeddings=256, tie_word_embeddings=False)


def _prepare(eng):
    with torch.no_grad():
        for n, p in eng.model.named_parameters():
            if "conv" in n:
                p.normal_(0, 0.3, generator=torch.Generator().manual_seed(11))
    eng.sdp.resync_master()


def _update_error(before, after, ref_after, muon):
    """Worst deviation of the step from the single-process one.  AdamW: absolute, per element.  Muon: the update of a
    matrix as a whole, relative (five bf16 Newton-Schulz iterations amplify the last-bit differences that another
    summation order leaves in the gradient, most along the small singular directions, so single elements of the
    update move by several per cent while the update as a whole stays put)."""
    if not muon:
        return max(((after[n] - ref_after[n]).abs().max().item(), n) for n in ref_after)
    worst = (0.0, "")
    for n in ref_after:
        want = ref_after[n] - before[n]
        if float(want.norm()) == 0.0:
            continue
        worst = max(worst, (((after[n] - before[n]) - want).norm().item() / want.norm().item() * 1e-3, n))
    return worst


def _worker(rank, world, port, ids, ref_loss, ref_grads, ref_after, q, muon=False):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from ttcd_b200.train.engine import EngineConfig, TrainEngine
        # the full model is built first (same seed everywhere), conv weights set, then sharded by the engine
        import ttcd_b200.parallel.tensor as tpmod
        orig = tpmod.shard_model

        def shard_after_prepare(model, tp):
            with torch.no_grad():
                for n, p in model.named_parameters():
                    if "conv" in n:
                        p.normal_(0, 0.3, generator=torch.Generator().manual_seed(11))
            orig(model, tp)

        tpmod.shard_model = shard_after_prepare
        eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=1e-2, seed=3, activation_checkpoint="none",
                                                             tensor_parallel=world, max_norm=1.0, enable_muon=muon), device="cpu")
        assert bool(eng.sdp.muon_params) == muon
        eng.sdp.zero_grad()
        loss = eng.forward_backward(ids)
        worst = (0.0, "")
        for n, p in eng.model.named_parameters():
            want = ref_grads[n]
            shard = getattr(p, "_tp_shard", None)
            if shard is not None:
                per = want.shape[shard[0]] // world
                want = want.narrow(shard[0], rank * per, per)
            err = (p.grad - want).abs().max().item() / (want.abs().max().item() + 1e-6)
            worst = max(worst, (err, n))
        before = {n: t.clone() for n, t in tpmod.gather_full_state_dict(eng.model, eng.tp).items()}
        norm = float(eng.sdp.step(1e-2))
        full = tpmod.gather_full_state_dict(eng.model, eng.tp)
        after = _update_error(before, full, ref_after, muon)
        q.put((rank, abs(float(loss) - ref_loss), worst, norm, after))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), 0, 0))


@pytest.mark.timeout(300)
@pytest.mark.parametrize("muon", [False, True])
def test_tensor_parallel_matches_single_process(muon):
    """With ``muon``: the 2-D hidden weights are Muon-owned; the two ranks gather their weight slices into whole
    matrices for the Newton-Schulz step and must land on the single-process weights."""
    torch.manual_seed(0)
    ids = torch.randint(0, 256, (1, 128))
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=1e-2, seed=3, activation_checkpoint="none",
                                                         max_norm=1.0, enable_muon=muon), device="cpu")
    _prepare(eng)
    eng.sdp.zero_grad()
    loss = float(eng.forward_backward(ids))
    grads = {n: p.grad.clone() for n, p in eng.model.named_parameters()}
    ref_norm = float(eng.sdp.step(1e-2))
    after = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ids, loss, grads, after, q, muon)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, err, worst, norm, aft in results:
        assert err != "error", worst
        assert err < 1e-4, (rank, err)
        assert worst[0] < 2e-3, (rank, worst)
        assert abs(norm - ref_norm) < 1e-3 * max(1.0, ref_norm), (norm, ref_norm)
        assert aft[0] < 1e-4, aft


def _dp_tp_worker(rank, world, tp_degree, port, ids, ref_loss, ref_norm, ref_after, q, muon=False):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from ttcd_b200.train.engine import EngineConfig, TrainEngine
        import ttcd_b200.parallel.tensor as tpmod
        orig = tpmod.shard_model

        def shard_after_prepare(model, tp):
            with torch.no_grad():
                for n, p in model.named_parameters():
                    if "conv" in n:
                        p.normal_(0, 0.3, generator=torch.Generator().manual_seed(11))
            orig(model, tp)

        tpmod.shard_model = shard_after_prepare
        eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=1e-2, seed=3, activation_checkpoint="none",
                                                             tensor_parallel=tp_degree, max_norm=1.0, enable_muon=muon), device="cpu")
        assert eng.sdp.world == world // tp_degree and eng.tp.world == tp_degree and bool(eng.sdp.muon_params) == muon
        dp_rank = rank // tp_degree
        eng.sdp.zero_grad()
        loss = eng.forward_backward(ids[dp_rank:dp_rank + 1]).clone()
        dist.all_reduce(loss)                                   # every replica's loss, tp_degree times each
        before = {n: t.clone() for n, t in tpmod.gather_full_state_dict(eng.model, eng.tp).items()}
        norm = float(eng.sdp.step(1e-2))
        full = tpmod.gather_full_state_dict(eng.model, eng.tp)
        after = _update_error(before, full, ref_after, muon)
        q.put((rank, abs(float(loss) / world - ref_loss), abs(norm - ref_norm), after))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc(), 0))


@pytest.mark.timeout(400)
@pytest.mark.parametrize("muon", [False, True])
def test_data_parallel_times_tensor_parallel_matches_single_process(muon):
    """2 data-parallel replicas x 2 tensor-parallel ranks (4 gloo processes), one sequence per replica: loss,
    clipped gradient norm and the weights after one optimizer step (AdamW, or Muon + AdamW) equal the single-process
    batch of two."""
    torch.manual_seed(1)
    ids = torch.randint(0, 256, (2, 128))
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(IPTTCDv9Config(**KW), EngineConfig(dtype=torch.float32, lr=1e-2, seed=3, activation_checkpoint="none",
                                                         max_norm=1.0, enable_muon=muon), device="cpu")
    _prepare(eng)
    eng.sdp.zero_grad()
    loss = float(eng.forward_backward(ids))
    ref_norm = float(eng.sdp.step(1e-2))
    after = {n: p.detach().clone() for n, p in eng.model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_dp_tp_worker, args=(r, 4, 2, port, ids, loss, ref_norm, after, q, muon)) for r in range(4)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, dloss, dnorm, aft in results:
        assert dloss != "error", dnorm
        assert dloss < 1e-4, (rank, dloss)
        assert dnorm < 1e-3 * max(1.0, ref_norm), (rank, dnorm, ref_norm)
        assert aft[0] < 1e-4, (rank, aft)


def _trainer_rank(rank, world, port, folder, steps, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        import json
        from ttcd_b200.train.trainer import cli
        cfg = os.path.join(folder, "model.json")
        if rank == 0 and not os.path.exists(cfg):
            with open(cfg, "w") as f:
                json.dump(dict(model_type="ipttcdv9", **KW), f)
        import time
        while not os.path.exists(cfg):
            time.sleep(0.1)
        cli(["--job.dump_folder", os.path.join(folder, "run"), "--model.config", cfg, "--training.dataset", "synthetic",
             "--training.seq_len", "64", "--training.batch_size", "1", "--training.steps", str(steps),
             "--training.tensor_parallel_degree", "2", "--checkpoint.enable_checkpoint", "--checkpoint.interval", "1",
             "--lr_scheduler.warmup_steps", "1", "--metrics.log_freq", "1"])
        q.put((rank, "ok"))
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()))


@pytest.mark.timeout(600)
def test_trainer_with_tensor_parallel_saves_full_tensors_and_resumes(tmp_path):
    ctx = mp.get_context("spawn")
    for steps in (2, 3):                      # second launch resumes from step-2
        q = ctx.Queue()
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        procs = [ctx.Process(target=_trainer_rank, args=(r, 2, port, str(tmp_path), steps, q)) for r in range(2)]
        for p in procs:
            p.start()
        results = [q.get(timeout=280) for _ in procs]
        for p in procs:
            p.join(30)
        assert all(r[1] == "ok" for r in results), results
    import torch.distributed.checkpoint as dcp
    name = "model.model.layers.0.mlp.gate_proj.weight"
    full = {name: torch.empty(128, 64)}       # the checkpoint holds the un-sharded [intermediate, hidden] matrix
    dcp.load(full, checkpoint_id=str(tmp_path / "run" / "checkpoint" / "step-3"), no_dist=True)
    assert torch.isfinite(full[name]).all() and full[name].abs().sum() > 0


def _vp_worker(rank, world, port, logits, labels, want_loss, want_grad, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from ttcd_b200.parallel.tensor import TensorParallel, vocab_parallel_cross_entropy
        tp = TensorParallel(None, "cpu")
        vl = logits.shape[1] // world
        shard = logits[:, rank * vl:(rank + 1) * vl].clone().requires_grad_()
        loss = vocab_parallel_cross_entropy(shard, labels, tp)
        loss.backward()
        q.put((rank, abs(float(loss) - want_loss), float((shard.grad - want_grad[:, rank * vl:(rank + 1) * vl]).abs().max())))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.timeout(300)
def test_vocab_parallel_cross_entropy_matches_dense():
    torch.manual_seed(0)
    logits = (torch.randn(24, 64) * 3).requires_grad_()
    labels = torch.randint(0, 64, (24,))
    labels[::5] = -100
    loss = torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100)
    loss.backward()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_vp_worker, args=(r, 2, port, logits.detach(), labels, float(loss), logits.grad.clone(), q))
             for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=200) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, e_loss, e_grad in results:
        assert e_loss != "error", e_grad
        assert e_loss < 1e-5 and e_grad < 1e-6
