"""Reference arm of bench.py: the UNMODIFIED upstream model classes (installed under baseline/_ref) trained
the way the upstream trainer trains them.

The upstream entry point ``python -m flame.train`` cannot be imported on this image (it needs
``torchtitan.components.ft.FTParallelDims`` and other symbols absent from the installed torchtitan), so this
file performs the same sequence the upstream trainer does with stock PyTorch pieces and nothing from
ttcd_b200: HF ``AutoModelForCausalLM.from_config`` of the upstream-registered ``ipttcdv9`` class, its
``FusedLinearCrossEntropyLoss(num_chunks=8)`` criterion (flame/train.py:331-337), full activation
checkpointing per block, FSDP2 ``fully_shard`` per block + root with bf16 parameters and fp32 gradient
reduction (flame/models/parallelize_fla.py:436-497), fused AdamW (eps 1e-15, betas 0.9/0.95, wd 0.1) and
``clip_grad_norm_(1.0)``.

Activation checkpointing (``--ref-ac``): ``full`` wraps every block in ``checkpoint_wrapper`` as the recipe does;
``none`` does not; ``auto`` (default) builds the model without checkpointing, runs one step, and rebuilds it with
full checkpointing if that step runs out of memory on any rank (the ranks agree through an all-reduce).  The
printed line names the setting that the timed steps ran with.
"""
from __future__ import annotations

import json
import os
from pathlib import Path


def run(args, metric, ClockSampler, timed_region, dist_env):
    import torch
    import torch.distributed as dist
    from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import checkpoint_wrapper
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import custom_models  # noqa: F401  upstream package: registers ipttcdv9 / ipttt
    import fla  # noqa: F401
    from fla.modules import FusedLinearCrossEntropyLoss
    from transformers import AutoConfig, AutoModelForCausalLM

    data = json.loads(Path(args.config).read_text())
    if args.layers is not None:
        data["num_hidden_layers"] = args.layers
        data["ttt_layers"] = [l for l in data.get("ttt_layers", []) if l < args.layers]
    model_type = data.pop("model_type")
    cfg = AutoConfig.for_model(model_type, **data)
    # transformers >= 5 wants `_tied_weights_keys` as a {target: source} dict; upstream (pinned to 4.57)
    # declares the same tie as a list.  Setting the attribute changes no computation and is needed
    # to construct the tied-embedding recipe config at all on this image.
    compat = []
    # transformers >= 5 fills `rope_scaling` with {"rope_type": "default", ...} for plain RoPE; upstream's attention
    # layer (written against 4.57, where the field stays None) refuses every type but "yarn".  Plain RoPE is what the
    # config asks for either way, so the field is put back to None (no computation changes).
    scaling = getattr(cfg, "rope_scaling", None)
    if isinstance(scaling, dict) and (scaling.get("rope_type") or scaling.get("type")) == "default":
        cfg.rope_scaling = None
        compat.append("config.rope_scaling {'rope_type': 'default'} -> None (transformers 5.x)")
    if getattr(cfg, "tie_word_embeddings", False):
        cls = AutoModelForCausalLM._model_mapping[type(cfg)]
        for klass in cls.__mro__:
            if isinstance(klass.__dict__.get("_tied_weights_keys"), (list, tuple)):
                klass._tied_weights_keys = {"lm_head.weight": "model.embeddings.weight"}
                compat.append(f"{klass.__name__}._tied_weights_keys list->dict (transformers 5.x)")
    mesh = init_device_mesh("cuda", (world,))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)

    def build(use_ac: bool):
        torch.manual_seed(42)
        with torch.device("cuda"):
            model = AutoModelForCausalLM.from_config(cfg)
        model.train()
        if cfg.fuse_linear_cross_entropy:
            model.criterion = FusedLinearCrossEntropyLoss(num_chunks=8)
        layers = model.model.layers
        if use_ac:
            for i in range(len(layers)):
                layers[i] = checkpoint_wrapper(layers[i], preserve_rng_state=False)
        for i, blk in enumerate(layers):
            fully_shard(blk, mesh=mesh, mp_policy=mp, reshard_after_forward=i < len(layers) - 1)
        fully_shard(model, mesh=mesh, mp_policy=mp)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), eps=1e-15, weight_decay=0.1, fused=True)
        return model, opt

    ref_ac = "none" if args.no_ac else getattr(args, "ref_ac", "full")
    use_ac = ref_ac == "full"
    model, opt = build(use_ac)

    B, S, V = args.batch_per_gpu, args.seq_len, cfg.vocab_size
    n_total = args.warmup + 2 * args.steps
    gen = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randint(0, V, (B, S), generator=gen, dtype=torch.int64).pin_memory() for _ in range(n_total)]
    dev = [t.cuda(non_blocking=True) for t in host[args.warmup:args.warmup + args.steps]]

    def step(ids, read_loss):
        ids = ids.cuda(non_blocking=True)
        opt.zero_grad(set_to_none=True)
        out = model(input_ids=ids, labels=ids)
        out.loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0, foreach=True)
        opt.step()
        return float(out.loss.item()) if read_loss else None

    if ref_ac == "auto":
        # does one step fit without activation checkpointing?  every rank must come to the same answer
        failed = torch.zeros(1, device="cuda")
        try:
            step(host[0], False)
            torch.cuda.synchronize()
        except torch.OutOfMemoryError:
            failed.fill_(1.0)
        if world > 1:
            dist.all_reduce(failed, op=dist.ReduceOp.MAX)
        if float(failed) > 0:
            del model, opt
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            use_ac = True
            model, opt = build(True)
    for i in range(args.warmup):
        step(host[i], False)
    torch.cuda.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms_dev = timed_region(torch, dist, world, lambda i: step(dev[i], False), args.steps)
    losses = []
    e2e_host = host[args.warmup + args.steps:]
    ms_e2e = timed_region(torch, dist, world, lambda i: losses.append(step(e2e_host[i], True)), args.steps)
    clocks = sampler.stop() if sampler else {}
    tokens = B * S * world * args.steps
    if rank == 0:
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": round(tokens / (ms_dev / 1e3), 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": Path(args.config).stem, "global_batch": B * world, "seq_len": S,
                       "parallelism": f"fsdp2-dp{world}", "activation_checkpointing": "full" if use_ac else "none",
                       "activation_checkpointing_requested": ref_ac,
                       "optimizer": "AdamW(fused)", "layers": cfg.num_hidden_layers,
                       "stack": "upstream model classes + Triton/flash-attn 2/cuBLAS/cuDNN + FSDP2"},
            "clocks": clocks,
            "e2e": {"value": round(tokens / (ms_e2e / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e / args.steps, 2),
                    "h2d_bytes_per_step": B * S * 8, "d2h_bytes_per_step": 4},
            "final_loss": losses[-1] if losses else None, "compat": compat,
        }), flush=True)
    dist.destroy_process_group()
