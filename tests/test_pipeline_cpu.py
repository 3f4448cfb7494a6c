"""Pipeline stage split + fill-drain schedule on 2 gloo ranks reproduce the single-process loss and gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ttcd_b200.models import TransformerConfig, TransformerForCausalLM
from ttcd_b200.parallel.pipeline import FillDrainSchedule, PipelineStageModule, stage_layer_ranges

KW = dict(hidden_size=32, num_hidden_layers=4, num_heads=4, num_kv_heads=2, intermediate_size=64, vocab_size=64, window_size=16,
          fuse_cross_entropy=False, fuse_linear_cross_entropy=False, tie_word_embeddings=False, max_position_embeddings=64)


def test_stage_ranges():
    assert [list(r) for r in stage_layer_ranges(7, 3)] == [[0, 1, 2], [3, 4], [5, 6]]
    assert [list(r) for r in stage_layer_ranges(8, 2, ["layers.3"])] == [[0, 1, 2], [3, 4, 5, 6, 7]]
    with pytest.raises(ValueError):
        stage_layer_ranges(8, 3, ["layers.3"])


def _worker(rank, world, port, ids, want_loss, want_grads, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        model = TransformerForCausalLM(TransformerConfig(**KW)).train()
        stage = PipelineStageModule(model, rank, world)
        sched = FillDrainSchedule(stage, rank, world, hidden_size=32)
        loss = sched.step(ids, ids, n_microbatches=2)
        names = {id(p): n for n, p in model.named_parameters()}
        worst = max(((p.grad - want_grads[names[id(p)]]).abs().max().item(), names[id(p)]) for p in stage.parameters())
        q.put((rank, None if loss is None else abs(float(loss) - want_loss), worst))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        import traceback
        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.timeout(300)
def test_two_stage_pipeline_matches_single_process():
    torch.manual_seed(0)
    model = TransformerForCausalLM(TransformerConfig(**KW)).train()
    ids = torch.randint(0, 64, (4, 24), generator=torch.Generator().manual_seed(1))
    whole = PipelineStageModule(model, 0, 1)
    loss = sum(whole(c, c) for c in ids.chunk(2)) / 2
    loss.backward()
    want = {n: p.grad.clone() for n, p in model.named_parameters()}
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ids, float(loss), want, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(30)
    for rank, err, worst in results:
        assert err != "error", worst
        assert worst[0] < 1e-5, worst
        if rank == 1:
            assert err < 1e-5
