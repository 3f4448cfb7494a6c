"""Context-parallel numerics on GPUs: sharded sequence + fused K/V halo vs the same model on one GPU."""
import torch
import torch.distributed as dist


def check_context_parallel(window=512):
    """``window`` 512: the K/V halo path.  None: a full-attention teacher, which takes the head-parallel path (one
    all-to-all gives every rank all tokens of its share of the heads)."""
    from ttcd_b200.models import IPTTCDv9Config
    from ttcd_b200.parallel import context
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg = IPTTCDv9Config(hidden_size=256, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768,
                         vocab_size=4096, window_size=window, max_position_embeddings=8192, ttt_mode=True, ttt_chunk=256,
                         ttt_layers=[1], ttt_update_every=2, qk_norm=True, tie_word_embeddings=True, fuse_cross_entropy=False,
                         fuse_linear_cross_entropy=True, ttt_teacher_conv_init="identity", ttt_normalize_student_features=False)
    S = 1024 * world
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (1, S), generator=g).cuda()
    dev = f"cuda:{torch.cuda.current_device()}"

    # single-GPU statement, computed redundantly on every rank without any communication
    import os
    os.environ["TTCD_COMM"] = "nccl"
    ref = TrainEngine(cfg, EngineConfig(lr=0.0, seed=9, activation_checkpoint="none", max_norm=None), device=dev)
    ref.model.zero_grad(set_to_none=True)
    out = ref.model(input_ids=ids, labels=ids)
    out.loss.backward()
    ref_loss = float(out.loss)
    ref_grads = {n: p.grad.detach().float().clone() for n, p in ref.model.named_parameters()}
    del ref, out
    torch.cuda.empty_cache()

    os.environ["TTCD_COMM"] = "peer"
    eng = TrainEngine(cfg, EngineConfig(lr=0.0, seed=9, activation_checkpoint="none", max_norm=None, context_parallel=world),
                      device=dev)
    eng.sdp.zero_grad()
    loss = eng.forward_backward(ids)
    torch.cuda.synchronize()
    assert abs(float(loss) - ref_loss) < 2e-2, (float(loss), ref_loss)
    worst = (0.0, "")
    for n, p in eng.model.named_parameters():
        gsum = p.grad.detach().float().clone()
        dist.all_reduce(gsum)
        gsum /= world
        denom = ref_grads[n].norm().item() + 1e-6
        rel = (gsum - ref_grads[n]).norm().item() / denom
        worst = max(worst, (rel, n))
    assert worst[0] < 6e-2, f"context-parallel gradient mismatch: {worst}"
    context.shutdown()
    if rank == 0:
        print(f"context parallel (window {window}) ok: loss {float(loss):.4f} vs {ref_loss:.4f}, worst relative grad error {worst[0]:.3g} ({worst[1]})")
