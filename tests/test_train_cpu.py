"""Host-side training stack on CPU: flag/TOML configuration, LR schedule, data pipeline (collator, MDS shards,
resumable state), and the trainer end to end with checkpoint + resume (the reference tests none of this; the
behaviours checked are those of flame/config_manager.py, flame/train.py:413-452, flame/data.py and
flame/data_mds.py)."""
import json
import math
import os

import numpy as np
import pytest
import torch

from ttcd_b200.train.config_manager import JobConfig
from ttcd_b200.train.data import (BufferShuffledIterableDataset, DataCollatorForLanguageModeling, SyntheticTokenDataset,
                                  build_dataloader, build_dataset)
from ttcd_b200.train.data_mds import MDSPretokenizedDataset, build_mds_dataset, parse_mds_uri, write_mds
from ttcd_b200.train.lr_scheduler import LRSchedule, build_lr_schedule

TINY = dict(model_type="ipttcdv9", hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
            intermediate_size=128, vocab_size=128, window_size=32, ttt_mode=True, ttt_chunk=8, ttt_layers=[1],
            fuse_cross_entropy=False, tie_word_embeddings=False, max_position_embeddings=256)


# ------------------------------------------------------------------------------------------- config
def test_flags_toml_overlay_and_cmdline_precedence(tmp_path):
    toml = tmp_path / "job.toml"
    toml.write_text('[training]\nsteps = 77\nseq_len = 512\n[optimizer]\nlr = 1e-3\n')
    cfg = JobConfig().parse_args(["--job.config_file", str(toml), "--training.seq_len", "1024", "--optimizer.enable_muon"])
    assert cfg.training.steps == 77                 # from the file
    assert cfg.training.seq_len == 1024             # the command line wins over the file
    assert cfg.optimizer.lr == 1e-3 and cfg.optimizer.enable_muon is True
    assert cfg.optimizer.beta2 == 0.95              # default
    assert cfg.to_dict()["training"]["steps"] == 77


def test_string_list_flags():
    cfg = JobConfig().parse_args(["--checkpoint.exclude_from_loading", "optimizer,lr_scheduler"])
    assert cfg.checkpoint.exclude_from_loading == ["optimizer", "lr_scheduler"]


# ------------------------------------------------------------------------------------------- LR
def test_lr_schedule_shapes():
    s = LRSchedule(peak_lr=1.0, training_steps=100, warmup_steps=10, decay_ratio=0.2, decay_type="linear", lr_min=0.1)
    assert s.factor(0) == pytest.approx(1 / 11)
    assert s.factor(9) == pytest.approx(10 / 11)
    assert all(s.factor(i) == 1.0 for i in range(10, 80))
    assert s.factor(80) < 1.0 and s.factor(99) > 0.1          # the virtual extra step keeps the last rate above the floor
    c = LRSchedule(peak_lr=2.0, training_steps=50, warmup_steps=0, decay_type="cosine", lr_min=0.0)
    assert c.lr(24) == pytest.approx(2.0 * 0.5 * (1 + math.cos(math.pi * 25 / 51)))
    vals = [c.lr(i) for i in range(50)]
    assert vals == sorted(vals, reverse=True)


def test_lr_min_absolute_and_anneal_rewrite():
    cfg = JobConfig().parse_args(["--training.steps", "1000", "--optimizer.lr", "1e-3", "--lr_scheduler.lr_min_absolute", "1e-4",
                                  "--lr_scheduler.warmup_steps", "10"])
    s = build_lr_schedule(cfg)
    assert s.lr_min == pytest.approx(0.1)
    # a floor at or above the peak rate means "no decay" (ratio clamped to 1), never a rising rate
    cfg = JobConfig().parse_args(["--training.steps", "100", "--optimizer.lr", "1e-4", "--lr_scheduler.lr_min_absolute", "3e-4",
                                  "--lr_scheduler.warmup_steps", "0"])
    s = build_lr_schedule(cfg)
    assert s.lr_min == 1.0 and s.lr(99) == pytest.approx(1e-4)


def test_anneal_begin_step_rewrites_the_run_length():
    """steps 10000, begin 4000, ratio 0.1: the run ends at 4400 and decays linearly over its last 400 steps
    (values worked out by hand from the reference's rewrite, flame/train.py:430-452)."""
    cfg = JobConfig().parse_args(["--training.steps", "10000", "--optimizer.lr", "1.0", "--lr_scheduler.warmup_steps", "200",
                                  "--lr_scheduler.decay_ratio", "0.1", "--lr_scheduler.anneal_begin_step", "4000",
                                  "--lr_scheduler.decay_type", "linear"])
    s = build_lr_schedule(cfg)
    assert cfg.training.steps == 4400 and s.training_steps == 4400
    assert cfg.lr_scheduler.decay_ratio == pytest.approx(400 / 4400)
    assert s.decay_steps == 400 and s.stable_steps == 3800
    assert s.lr(3999) == 1.0                                   # last stable step
    assert s.lr(4000) == pytest.approx(1.0 - 1 / 401)          # first decay step
    assert s.lr(4199) == pytest.approx(1.0 - 200 / 401)        # half way
    assert s.lr(4399) == pytest.approx(1.0 - 400 / 401)        # last step stays above the floor
    with pytest.raises(ValueError):
        build_lr_schedule(JobConfig().parse_args(["--training.steps", "100", "--lr_scheduler.anneal_begin_step", "40"]))


# ------------------------------------------------------------------------------------------- data
def test_collator_stack_pad_and_varlen():
    col = DataCollatorForLanguageModeling(pad_token_id=0)
    b = col([{"input_ids": torch.arange(1, 9)}, {"input_ids": torch.arange(11, 19)}])
    assert b["input_ids"].shape == (2, 8) and torch.equal(b["labels"], b["input_ids"])      # the shift happens in the model
    b = col([{"input_ids": torch.arange(1, 9)}, {"input_ids": torch.arange(1, 5)}])
    assert b["attention_mask"][1].tolist() == [0, 0, 0, 0, 1, 1, 1, 1] and (b["labels"][1, :4] == -100).all()
    packed = DataCollatorForLanguageModeling(varlen=True, bos_token_id=1, context_len=4)
    b = packed([{"input_ids": torch.tensor([1, 5, 6, 1, 7, 8, 9, 9, 9, 9, 1, 3])}])
    assert b["input_ids"].shape == (1, 12)
    assert b["cu_seqlens"].tolist() == [0, 3, 7, 10, 12]       # documents at BOS, the 7-token one split at context_len


def test_synthetic_dataset_rank_distinct_and_resumable():
    a = SyntheticTokenDataset(100, 16, rank=0, world_size=2, seed=1)
    b = SyntheticTokenDataset(100, 16, rank=1, world_size=2, seed=1)
    ia, ib = iter(a), iter(b)
    xa = [next(ia)["input_ids"] for _ in range(3)]
    assert not torch.equal(xa[0], next(ib)["input_ids"])
    c = SyntheticTokenDataset(100, 16, rank=0, world_size=2, seed=1)
    c.load_state_dict({"index": 2})
    assert torch.equal(next(iter(c))["input_ids"], xa[2])


def test_shuffle_buffer_emits_every_item_once():
    ds = BufferShuffledIterableDataset(list(range(50)), buffer_size=8, seed=3)
    out = list(ds)
    assert sorted(out) == list(range(50)) and out != list(range(50))


def _make_mds(root, n_per=6, seq=32):
    rng = np.random.default_rng(0)
    all_rows = []
    for domain, proc in (("books", "proc00-64"), ("books", "proc11-64"), ("code", "proc01-64")):
        rows = [rng.integers(0, 1000, seq + 4, dtype=np.int32) for _ in range(n_per)]
        write_mds(os.path.join(root, domain, proc), [{"input_ids": r, "domain": domain} for r in rows],
                  {"input_ids": "ndarray:int32", "domain": "str"}, shard_samples=4)
        all_rows.append((domain, proc, rows))
    return all_rows


def test_mds_uri_discovery_roundtrip_sharding_and_resume(tmp_path):
    root = str(tmp_path / "mds")
    rows = _make_mds(root)
    assert parse_mds_uri("mds:/x/y?proc=proc0*-64&domain=a,b") == ("/x/y", {"proc": "proc0*-64", "domain": "a,b"})
    ds = build_mds_dataset(f"mds:{root}?seq_len=32", shuffle=False)
    assert len(ds) == 12                         # default glob proc0[0-9]-64 leaves proc11 out
    first = next(iter(ds))["input_ids"]
    assert first.dtype == torch.long and first.numel() == 32 and torch.equal(first, torch.from_numpy(rows[0][2][0][:32]).long())
    only_code = build_mds_dataset(f"mds:{root}?domain=code&seq_len=32", shuffle=False)
    assert len(only_code) == 6
    every = build_mds_dataset(f"mds:{root}?proc=proc*-64&seq_len=32")
    assert len(every) == 18
    # two ranks see disjoint halves of one epoch's permutation
    seen = []
    for r in range(2):
        d = MDSPretokenizedDataset(root, 32, "proc*-64", shuffle=True, seed=7, rank=r, world_size=2)
        it = iter(d)
        seen.append({tuple(next(it)["input_ids"].tolist()) for _ in range(9)})
    assert len(seen[0] | seen[1]) == 18
    # resume mid-epoch
    d = MDSPretokenizedDataset(root, 32, "proc*-64", shuffle=True, seed=7)
    it = iter(d)
    for _ in range(5):
        next(it)
    state = d.state_dict()
    want = next(it)["input_ids"]
    d2 = MDSPretokenizedDataset(root, 32, "proc*-64", shuffle=True, seed=7)
    d2.load_state_dict(state)
    assert torch.equal(next(iter(d2))["input_ids"], want)


def test_dataloader_state_is_keyed_by_rank():
    ds = build_dataset("synthetic", None, 16, rank=1, world_size=2, vocab_size=50)
    dl = build_dataloader(ds, None, 1, 2)
    it = iter(dl)
    next(it)
    state = dl.state_dict()
    assert list(state) == ["rank_1"]
    nxt = next(it)["input_ids"]
    ds2 = build_dataset("synthetic", None, 16, rank=1, world_size=2, vocab_size=50)
    dl2 = build_dataloader(ds2, None, 1, 2)
    dl2.load_state_dict(state)
    assert torch.equal(next(iter(dl2))["input_ids"], nxt)


# ------------------------------------------------------------------------------------------- trainer
def _train(tmp_path, steps, extra=()):
    from ttcd_b200.train.trainer import cli
    cfg = tmp_path / "model.json"
    cfg.write_text(json.dumps(TINY))
    cli(["--job.dump_folder", str(tmp_path / "run"), "--model.config", str(cfg), "--training.dataset", "synthetic",
         "--training.seq_len", "64", "--training.batch_size", "2", "--training.steps", str(steps), "--optimizer.lr", "1e-2",
         "--lr_scheduler.warmup_steps", "2", "--checkpoint.enable_checkpoint", "--checkpoint.interval", "2",
         "--metrics.log_freq", "1", "--training.seed", "3", *extra])


@pytest.mark.timeout(600)
def test_trainer_runs_checkpoints_and_resumes(tmp_path):
    _train(tmp_path, 2)
    run = tmp_path / "run"
    assert (run / "checkpoint" / "step-2" / ".metadata").is_file()
    assert (run / "resolved_model_config.json").is_file()
    _train(tmp_path, 4)                                  # picks up step-2 and continues to 4
    assert (run / "checkpoint" / "step-4" / ".metadata").is_file()
    from ttcd_b200.train.checkpoint import checkpoint_keys
    keys = checkpoint_keys(str(run / "checkpoint" / "step-4"))
    assert any(k.startswith("model.") for k in keys) and any("train_state" in k for k in keys)
    # an uninterrupted 4-step run ends with the same weights as 2 + resume + 2
    other = tmp_path / "straight"
    other.mkdir()
    _train(other, 4)
    import torch.distributed.checkpoint as dcp
    name = "model.model.layers.0.mlp.gate_proj.weight"
    a, b = {name: torch.empty(128, 64)}, {name: torch.empty(128, 64)}
    dcp.load(a, checkpoint_id=str(run / "checkpoint" / "step-4"), no_dist=True)
    dcp.load(b, checkpoint_id=str(other / "run" / "checkpoint" / "step-4"), no_dist=True)
    torch.testing.assert_close(a[name], b[name], rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------------------------------- IP-TTT inference
def test_ipttt_fast_weights_persist_across_incremental_calls():
    """Feeding a prompt in pieces (and token by token) through the fast-weight cache gives the logits of one
    full forward: the adapted down_proj weight and the unfinished chunk survive between calls
    (custom_models/ipttt/inference.py:505-538)."""
    from ttcd_b200.models import IPTTTConfig, IPTTTForCausalLM
    from ttcd_b200.models.modeling_ipttt import FastWeightCache
    torch.manual_seed(0)
    cfg = IPTTTConfig(hidden_size=32, num_hidden_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=64, vocab_size=64,
                      window_size=64, ttt_mode=True, ttt_chunk=8, ttt_layers=[0, 1], ttt_lr=0.5, ttt_proj=True, ttt_conv=True,
                      fuse_cross_entropy=False, max_position_embeddings=128, tie_word_embeddings=False)
    model = IPTTTForCausalLM(cfg).eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "ttt_conv" in n or "ttt_proj" in n:
                p.normal_(0, 0.3)
    ids = torch.randint(0, 64, (1, 29))
    with torch.no_grad():
        full = model(input_ids=ids, use_cache=True).logits
        cache = FastWeightCache()
        pieces = [model(input_ids=ids[:, a:b], past_key_values=cache, use_cache=True).logits
                  for a, b in ((0, 11), (11, 12), (12, 13), (13, 24), (24, 29))]
    assert cache.ttt_get(0)[2] is not None and cache.ttt_get(0)[0].shape[1] == 29 % 8
    torch.testing.assert_close(torch.cat(pieces, dim=1), full, rtol=1e-4, atol=1e-4)
    # the fast weight did move away from the slow weight
    assert (cache.ttt_get(0)[2][0] - model.model.layers[0].mlp.down_proj.weight).abs().max() > 1e-4
    out = model.generate(ids, max_new_tokens=4)
    assert out.shape == (1, 33)


# ------------------------------------------------------------------------------------------- checkpoint policy / metrics
def test_checkpoint_policies_keep_k_weights_only_export_and_trigger(tmp_path):
    import time as _time
    import torch.distributed.checkpoint as dcp
    from ttcd_b200.train import trainer
    from ttcd_b200.train.checkpoint import checkpoint_keys
    # keep_latest_k purges older steps; the last save is weights-only in the export dtype with raw keys
    _train(tmp_path, 4, ["--checkpoint.interval", "1", "--checkpoint.keep_latest_k", "2", "--checkpoint.last_save_model_weights_only",
                         "--checkpoint.export_dtype", "bfloat16"])
    folder = tmp_path / "run" / "checkpoint"
    for _ in range(50):                       # the purge runs on a background thread
        if sorted(p.name for p in folder.iterdir()) == ["step-3", "step-4"]:
            break
        _time.sleep(0.1)
    assert sorted(p.name for p in folder.iterdir()) == ["step-3", "step-4"]
    last = checkpoint_keys(str(folder / "step-4"))
    assert "model.layers.0.mlp.gate_proj.weight" in last and not any(k.startswith("optimizer") for k in last)
    t = {"model.layers.0.mlp.gate_proj.weight": torch.empty(128, 64, dtype=torch.bfloat16)}
    dcp.load(t, checkpoint_id=str(folder / "step-4"), no_dist=True)
    full = checkpoint_keys(str(folder / "step-3"))
    assert any(k.startswith("optimizer.") for k in full) and any(k.startswith("model.model.") for k in full)
    # external trigger: SIGUSR1 (or the trigger file) asks for one save at the next step boundary
    trainer._on_sigusr1(None, None)
    assert trainer.external_save_requested(0) is True
    assert trainer.external_save_requested(0) is False
    open(trainer.SAVE_TRIGGER_FILE, "w").close()
    assert trainer.external_save_requested(0) is True and not os.path.exists(trainer.SAVE_TRIGGER_FILE)


def test_seed_checkpoint_and_initial_load(tmp_path):
    from ttcd_b200.train.checkpoint import checkpoint_keys
    seed_dir = tmp_path / "seed"
    seed_dir.mkdir()
    _train(seed_dir, 1, ["--checkpoint.create_seed_checkpoint"])
    step0 = seed_dir / "run" / "checkpoint" / "step-0"
    keys = checkpoint_keys(str(step0))
    assert "model.embeddings.weight" in keys and not any(k.startswith("optimizer") for k in keys)     # raw keys, weights only
    # a fresh run that starts from it trains normally
    run2 = tmp_path / "ft"
    run2.mkdir()
    _train(run2, 2, ["--checkpoint.initial_load_path", str(step0)])
    assert (run2 / "run" / "checkpoint" / "step-2" / ".metadata").is_file()


def test_flop_and_param_counts():
    from ttcd_b200.models import TransformerConfig, TransformerForCausalLM
    from ttcd_b200.train.metrics import count_params, get_num_flop_per_token, get_peak_flops
    cfg = TransformerConfig(hidden_size=32, num_hidden_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=64, vocab_size=64,
                            tie_word_embeddings=False, fuse_cross_entropy=False)
    model = TransformerForCausalLM(cfg)
    total = sum(p.numel() for p in model.parameters())
    assert count_params(model, exclude_embedding=False) == total
    assert count_params(model, exclude_embedding=True) == total - 64 * 32
    n = count_params(model)
    assert get_num_flop_per_token(n, cfg, 128) == 6 * n + 12 * 2 * 4 * 8 * 128
    assert get_peak_flops("NVIDIA B200") == 2.25e15
