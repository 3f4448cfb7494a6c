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
    if what in ("all", "cp"):
        from tests.multi_gpu_cp import check_context_parallel
        check_context_parallel()
    torch.cuda.synchronize()
    assert _native.device_status() == 0
    dist.barrier()
    if dist.get_rank() == 0:
        print("MULTI_GPU_OK", what)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
