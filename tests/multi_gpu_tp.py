"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels against NCCL collectives + fp32 matmul."""
import torch
import torch.distributed as dist


def check_tensor_parallel():
    from ttcd_b200.parallel.tensor import TensorParallel, column_parallel_linear, row_parallel_linear
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    tp = TensorParallel(None, dev, max_rows_per_rank=1024, max_features=1024)
    assert tp.fused
    g = torch.Generator(device=dev).manual_seed(10 + rank)
    m, k, n = 512, 512, 768
    # ---- column parallel: x sharded over tokens, W sharded over outputs -------------------------------
    x = (torch.randn(m, k, device=dev, generator=g) * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(n, k, device=dev, generator=g) * 0.05).bfloat16().requires_grad_()
    for rep in range(3):                      # repeated calls exercise the double buffering and the epochs
        y = column_parallel_linear(x, w, tp)
    xs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(xs, x.detach())
    full = torch.cat(xs).float()
    want = full @ w.detach().float().t()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=2e-2)
    dy = (torch.randn(m * world, n, device=dev, generator=g) * 0.1).bfloat16()
    y.backward(dy)
    dx_all = dy.float() @ w.detach().float()                    # partial over this rank's output columns
    dist.all_reduce(dx_all)
    torch.testing.assert_close(x.grad.float(), dx_all[rank * m:(rank + 1) * m], rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w.grad.float(), dy.float().t() @ full, rtol=3e-2, atol=6e-2)
    # ---- row parallel: x holds all tokens and this rank's input columns -------------------------------
    x2 = (torch.randn(m * world, k, device=dev, generator=g) * 0.5).bfloat16().requires_grad_()
    w2 = (torch.randn(n + 256, k, device=dev, generator=g) * 0.05).bfloat16().requires_grad_()
    for rep in range(2):
        y2 = row_parallel_linear(x2, w2, tp)
    want2 = x2.detach().float() @ w2.detach().float().t()
    dist.all_reduce(want2)
    torch.testing.assert_close(y2.float(), want2[rank * m:(rank + 1) * m], rtol=3e-2, atol=3e-2)
    dy2 = (torch.randn(m, n + 256, device=dev, generator=g) * 0.1).bfloat16()
    y2.backward(dy2)
    dys = [torch.empty_like(dy2) for _ in range(world)]
    dist.all_gather(dys, dy2)
    dyf = torch.cat(dys).float()
    torch.testing.assert_close(x2.grad.float(), dyf @ w2.detach().float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w2.grad.float(), dyf.t() @ x2.detach().float(), rtol=3e-2, atol=6e-2)
    tp.check()
    tp.close()


def check_tp_model(muon: bool = False):
    """IP-TTCD under tensor+sequence parallelism (fused kernels where the shapes allow) vs the same model on
    one GPU: loss, gradient norm and weights after one optimizer step (AdamW, or with ``muon`` Muon on the hidden
    matrices: the ranks gather their weight slices into whole matrices for the Newton-Schulz step)."""
    from ttcd_b200.models import IPTTCDv9Config
    from ttcd_b200.parallel import tensor as tpmod
    from ttcd_b200.train.engine import EngineConfig, TrainEngine
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = f"cuda:{torch.cuda.current_device()}"
    cfg = IPTTCDv9Config(hidden_size=256, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=1024,
                         vocab_size=4096, window_size=256, max_position_embeddings=2048, ttt_mode=True, ttt_chunk=128,
                         ttt_layers=[1], ttt_update_every=4, qk_norm=True, tie_word_embeddings=False, fuse_cross_entropy=False,
                         fuse_linear_cross_entropy=True, ttt_teacher_conv_init="identity", ttt_normalize_student_features=False)
    ids = torch.randint(0, cfg.vocab_size, (1, 1024), generator=torch.Generator().manual_seed(5)).cuda()
    ref = TrainEngine(cfg, EngineConfig(lr=1e-3, seed=7, activation_checkpoint="none", enable_muon=muon), device=dev,
                      process_group=False)
    ref.sdp.zero_grad()
    ref_loss = float(ref.forward_backward(ids))
    ref_norm = float(ref.sdp.step(1e-3))
    ref_after = {n: p.detach().float().clone() for n, p in ref.model.named_parameters()}
    del ref
    eng = TrainEngine(cfg, EngineConfig(lr=1e-3, seed=7, activation_checkpoint="none", tensor_parallel=world,
                                        enable_muon=muon), device=dev)
    assert eng.tp is not None and eng.tp.fused and bool(eng.sdp.muon_params) == muon
    eng.sdp.zero_grad()
    loss = float(eng.forward_backward(ids))
    norm = float(eng.sdp.step(1e-3))
    assert eng.tp.calls > 0, "no fused tensor-parallel kernel ran"
    assert abs(loss - ref_loss) < 2e-2, (loss, ref_loss)
    assert abs(norm - ref_norm) < 5e-2 * max(1.0, ref_norm), (norm, ref_norm)
    full = tpmod.gather_full_state_dict(eng.model, eng.tp)
    worst = max(((full[n].float() - ref_after[n]).abs().max().item(), n) for n in ref_after)
    assert worst[0] < 2e-2, worst
    eng.tp.check()
    eng.tp.close()
