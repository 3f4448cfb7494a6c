"""The layouts that the main multi-GPU checks do not cover, on real GPUs (NCCL, native bf16 kernels): replicated data
parallelism (the DDP role), vocabulary-parallel cross-entropy, a two-stage pipeline, and on 4 GPUs hybrid sharding
(2 replicas x 2 shards).  Each is compared with the same computation in one process on this rank's GPU."""
import torch
import torch.distributed as dist


def _engine(**over):
    from tests.multi_gpu_worker import _small_engine
    return _small_engine(**over)[1]


def check_replicated_matches_sharded():
    """Same data, same seed: replicated data parallelism (whole optimizer state on every rank, bucketed all-reduce) and
    the sharded runtime end on the same weights."""
    rank, world = dist.get_rank(), dist.get_world_size()
    gen = torch.Generator().manual_seed(21)
    ids = torch.randint(0, 4096, (world, 1024), generator=gen).cuda()
    finals = {}
    for name, kw in (("sharded", {}), ("replicated", dict(replicate=True))):
        eng = _engine(**kw)
        losses = [eng.train_step(ids[rank:rank + 1]) for _ in range(3)]
        finals[name] = (losses, torch.cat([p.detach().float().flatten() for p in eng.model.parameters()]))
        del eng
        torch.cuda.empty_cache()
    (ls, fs), (lr, fr) = finals["sharded"], finals["replicated"]
    assert abs(ls[0] - lr[0]) < 1e-3 and abs(ls[-1] - lr[-1]) < 5e-2, (ls, lr)
    assert (fs - fr).abs().max().item() < 2e-2, (fs - fr).abs().max().item()


def check_vocab_parallel_cross_entropy():
    from ttcd_b200.parallel.tensor import TensorParallel, vocab_parallel_cross_entropy
    rank, world = dist.get_rank(), dist.get_world_size()
    gen = torch.Generator().manual_seed(22)
    rows, vocab = 512, 4096 * world
    logits = (torch.randn(rows, vocab, generator=gen) * 2).cuda()
    labels = torch.randint(0, vocab, (rows,), generator=gen).cuda()
    labels[::9] = -100
    dense = logits.clone().requires_grad_()
    want = torch.nn.functional.cross_entropy(dense, labels, ignore_index=-100)
    want.backward()
    tp = TensorParallel(None, "cuda", fused=False)
    vl = vocab // world
    shard = logits[:, rank * vl:(rank + 1) * vl].clone().requires_grad_()
    loss = vocab_parallel_cross_entropy(shard, labels, tp)
    loss.backward()
    assert abs(float(loss) - float(want)) < 1e-4 * max(1.0, float(want)), (float(loss), float(want))
    assert (shard.grad - dense.grad[:, rank * vl:(rank + 1) * vl]).abs().max().item() < 1e-6
    tp.close()


def check_two_stage_pipeline():
    """Fill-drain schedule over the first two ranks (activations and their gradients travel by NCCL send/recv, the
    blocks run the native bf16 kernels) against the whole model on one GPU."""
    from ttcd_b200.models import TransformerConfig, TransformerForCausalLM
    from ttcd_b200.parallel.pipeline import FillDrainSchedule, PipelineStageModule
    rank = dist.get_rank()
    group = dist.new_group([0, 1])
    if rank > 1:
        return
    cfg = TransformerConfig(hidden_size=256, num_hidden_layers=4, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768,
                            vocab_size=4096, window_size=256, max_position_embeddings=1024, fuse_cross_entropy=False,
                            fuse_linear_cross_entropy=False, tie_word_embeddings=False)
    gen = torch.Generator().manual_seed(23)
    ids = torch.randint(0, 4096, (4, 512), generator=gen).cuda()

    def build():
        torch.manual_seed(5)
        return TransformerForCausalLM(cfg).to("cuda", torch.bfloat16).train()

    whole_model = build()
    whole = PipelineStageModule(whole_model, 0, 1)
    loss = sum(whole(c, c) for c in ids.chunk(2)) / 2
    loss.backward()
    want = {n: p.grad.float().clone() for n, p in whole_model.named_parameters()}
    model = build()
    stage = PipelineStageModule(model, rank, 2)
    sched = FillDrainSchedule(stage, rank, 2, group=group, hidden_size=256, dtype=torch.bfloat16, device="cuda")
    got = sched.step(ids, ids, n_microbatches=2)
    if rank == 1:
        assert abs(float(got) - float(loss)) < 2e-2, (float(got), float(loss))
    names = {id(p): n for n, p in model.named_parameters()}
    for p in stage.parameters():
        w = want[names[id(p)]]
        err = (p.grad.float() - w).norm().item() / max(w.norm().item(), 1e-9)
        assert err < 3e-2, (names[id(p)], err)


def check_hybrid_sharding():
    """4 GPUs as 2 replicas x 2 shards against plain sharding over all 4: same data, same weights afterwards."""
    rank, world = dist.get_rank(), dist.get_world_size()
    if world != 4:
        return
    gen = torch.Generator().manual_seed(24)
    ids = torch.randint(0, 4096, (world, 1024), generator=gen).cuda()
    finals = {}
    for name, kw in (("flat", {}), ("hybrid", dict(replicate_degree=2))):
        eng = _engine(**kw)
        if name == "hybrid":
            assert eng.sdp.world == 2 and eng.sdp.replicate_world == 2
        losses = [eng.train_step(ids[rank:rank + 1]) for _ in range(3)]
        finals[name] = (losses, torch.cat([p.detach().float().flatten() for p in eng.model.parameters()]))
        del eng
        torch.cuda.empty_cache()
    (la, fa), (lb, fb) = finals["flat"], finals["hybrid"]
    assert abs(la[-1] - lb[-1]) < 5e-2, (la, lb)
    assert (fa - fb).abs().max().item() < 2e-2, (fa - fb).abs().max().item()


def check_all():
    check_vocab_parallel_cross_entropy()
    check_two_stage_pipeline()
    check_replicated_matches_sharded()
    check_hybrid_sharding()
