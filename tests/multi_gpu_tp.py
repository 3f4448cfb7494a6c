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
