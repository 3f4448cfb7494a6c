"""Whole-model checks on the GPU: the bf16 model on the native kernels against the same weights in fp32 through the
PyTorch statements of the ops (loss and gradients), the op-level recompute policy, and the cached decode path."""
import pytest
import torch

from ttcd_b200 import _native
from ttcd_b200.models import IPTTCDv9Config, IPTTCDv9ForCausalLM
from ttcd_b200.train.engine import EngineConfig, TrainEngine

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(autouse=True)
def _status():
    _native.load(required=True)
    yield
    torch.cuda.synchronize()
    assert _native.device_status() == 0, "a bounded device wait expired"


def _config(**over):
    kw = dict(hidden_size=512, num_hidden_layers=4, num_heads=4, num_kv_heads=2, head_dim=128, intermediate_size=1536,
              vocab_size=4096, window_size=1024, max_position_embeddings=4096, ttt_mode=True, ttt_chunk=512,
              ttt_visible_chunks=1, ttt_layers=[2], ttt_update_every=8, qk_norm=True, tie_word_embeddings=True,
              fuse_cross_entropy=False, fuse_linear_cross_entropy=True, ttt_teacher_conv_init="identity",
              ttt_proj_init="diagonal_gaussian", ttt_normalize_student_features=False, ttt_output_use_teacher_conv=False)
    kw.update(over)
    return IPTTCDv9Config(**kw)


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    if float(a.norm()) == 0.0 and float(b.norm()) == 0.0:
        return 1.0                                   # e.g. a gate whose input features are zero at initialisation
    return float(torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-30))


def test_bf16_native_model_matches_fp32_statement():
    """4 layers (one fast-weight layer), 4096 tokens, hidden 512: loss within 2e-2 and gradient cosine >= 0.99 on every
    kind of parameter."""
    torch.manual_seed(0)
    cfg = _config()
    ref_model = IPTTCDv9ForCausalLM(cfg).to(DEV, torch.float32).train()
    with torch.no_grad():                      # give the fast-weight path something to do
        for n, p in ref_model.named_parameters():
            if "ttt_student_conv" in n or "b_proj" in n:
                p.normal_(0, 0.1)
    model = IPTTCDv9ForCausalLM(cfg).to(DEV, torch.bfloat16).train()
    model.load_state_dict(ref_model.state_dict())
    ref_model.load_state_dict(model.state_dict())          # both see the bf16-rounded weights
    ids = torch.randint(0, cfg.vocab_size, (1, 4096), device=DEV)
    before = _native.launch_count
    loss = model(input_ids=ids, labels=ids).loss
    loss.backward()
    assert _native.launch_count - before > 100, "the native kernels did not run"
    ref_loss = ref_model(input_ids=ids, labels=ids).loss
    ref_loss.backward()
    assert abs(float(loss) - float(ref_loss)) < 2e-2, (float(loss), float(ref_loss))
    want = dict(ref_model.named_parameters())
    kinds = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "ttt_proj", "ttt_student_conv",
             "ttt_teacher_conv", "b_proj", "embeddings", "attn_norm", "mlp_norm", "q_norm", "k_norm")
    seen = set()
    for n, p in model.named_parameters():
        kind = next((k for k in kinds if k in n), None)
        if kind is None or p.grad is None:
            continue
        seen.add(kind)
        c = _cos(p.grad, want[n].grad)
        floor = 0.98 if kind in ("ttt_teacher_conv", "b_proj", "q_norm", "k_norm") else 0.99     # tiny tensors: noisier
        assert c >= floor, f"{n}: gradient cosine {c:.4f}"
    assert {"q_proj", "down_proj", "ttt_proj", "ttt_student_conv", "b_proj", "embeddings"} <= seen, seen


def test_op_recompute_policy_matches_resident_activations_with_fewer_launches():
    cfg = _config()
    ids = torch.randint(0, cfg.vocab_size, (1, 2048), device=DEV)
    grads, launches, peak = {}, {}, {}
    for mode in ("none", "op", "full"):
        eng = TrainEngine(cfg, EngineConfig(lr=1e-3, activation_checkpoint=mode, seed=3), device=DEV)
        eng.sdp.zero_grad()
        eng.forward_backward(ids)                # warm-up (lazy initialisation of the kernels)
        eng.sdp.zero_grad()
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        before = _native.launch_count
        eng.forward_backward(ids)
        torch.cuda.synchronize()
        launches[mode] = _native.launch_count - before
        peak[mode] = torch.cuda.max_memory_allocated() - base
        grads[mode] = {n: p.grad.detach().float().clone() for n, p in eng.model.named_parameters()}
        del eng
    for n, g in grads["none"].items():
        assert _cos(grads["op"][n], g) > 0.9999, n          # the same kernels on the same inputs
        torch.testing.assert_close(grads["op"][n], g, rtol=2e-2, atol=2e-3, msg=n)
    assert launches["none"] < launches["op"] < launches["full"], launches
    assert peak["full"] < peak["op"] < peak["none"], peak


def test_decode_steps_match_one_forward():
    """Prefill then token-by-token steps through the window cache (the small-query attention kernel) give the logits
    of one forward over the whole sequence."""
    torch.manual_seed(1)
    cfg = _config(ttt_layers=[], ttt_mode=False, num_hidden_layers=2, window_size=384)
    model = IPTTCDv9ForCausalLM(cfg).to(DEV, torch.bfloat16).eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 700), device=DEV)
    with torch.no_grad():
        full = model(input_ids=ids).logits.float()
        out = model(input_ids=ids[:, :640], use_cache=True)
        cache, steps = out.past_key_values, [out.logits.float()]
        before = _native.launch_count
        for t in range(640, 700, 20):                     # 20-token continuations, then single tokens
            out = model(input_ids=ids[:, t:t + 19], past_key_values=cache, use_cache=True)
            steps.append(out.logits.float())
            out = model(input_ids=ids[:, t + 19:t + 20], past_key_values=cache, use_cache=True)
            steps.append(out.logits.float())
        assert _native.launch_count > before
    got = torch.cat(steps, dim=1)
    err = (got - full).abs()
    assert err.max() < 0.25 and err.mean() < 2e-2, (float(err.max()), float(err.mean()))
    agree = (got.argmax(-1) == full.argmax(-1)).float().mean()
    assert agree > 0.97, float(agree)


@pytest.mark.parametrize("Tq,Tk,H,HK,D,W", [(1, 8192, 16, 8, 128, 8192), (1, 300, 4, 2, 64, None), (19, 1000, 4, 2, 128, 512),
                                             (127, 127, 3, 1, 64, 50), (5, 70000, 2, 1, 128, None)])
def test_small_query_attention_kernel(Tq, Tk, H, HK, D, W):
    from ttcd_b200.ops import cuda, reference as ref
    q = torch.randn(2, Tq, H, D, device=DEV).bfloat16()
    k = torch.randn(2, Tk, HK, D, device=DEV).bfloat16()
    v = torch.randn(2, Tk, HK, D, device=DEV).bfloat16()
    assert cuda.attn_small_q_supported(q, k)
    got = cuda.attn_small_q(q, k, v, W)
    want = ref.attention(q.float(), k.float(), v.float(), W)
    err = (got.float() - want).abs()
    assert err.max() < 2e-2, float(err.max())


def _distinct_shapes():
    import glob
    import json
    from pathlib import Path
    root = Path(__file__).resolve().parents[1] / "configs"
    seen = {}
    for f in sorted(glob.glob(str(root / "*" / "*.json"))):
        d = json.loads(Path(f).read_text())
        hs, nh = d.get("hidden_size"), d.get("num_heads")
        key = (d["model_type"], hs, nh, d.get("num_kv_heads"), d.get("head_dim"), d.get("intermediate_size"), d.get("hidden_ratio"),
               bool(d.get("qk_norm")), d.get("window_size") is None)
        seen.setdefault(key, f)
    return sorted(seen.values())


@pytest.mark.parametrize("path", _distinct_shapes(), ids=lambda p: p.split("/")[-1][:-5])
def test_every_shipped_shape_runs_one_layer(path):
    """One block of every distinct (model type, widths, heads) among the shipped configs: forward, backward and an
    optimizer step on the native path (hidden 4096 takes the wide-row norm kernels, head_dim 80 / 96 the PyTorch
    attention, 15 / 5 heads the masked tile edges)."""
    from ttcd_b200.train.engine import load_model_config
    cfg = load_model_config(path, num_hidden_layers=1, vocab_size=4096, max_position_embeddings=2048)
    if getattr(cfg, "ttt_layers", None):
        cfg.ttt_layers = [0]
        cfg.ttt_chunk = 256
    if getattr(cfg, "window_size", None):
        cfg.window_size = min(cfg.window_size, 384)
    eng = TrainEngine(cfg, EngineConfig(lr=1e-3, activation_checkpoint="none"), device=DEV)
    ids = torch.randint(0, 4096, (1, 1024), device=DEV)
    l0 = eng.train_step(ids)
    l1 = eng.train_step(ids)
    assert l0 == l0 and l1 == l1 and l1 < l0 + 0.5, (l0, l1)


@pytest.mark.parametrize("family", ["delta_net", "gated_deltanet"])
def test_recurrent_family_decodes_from_its_state(family):
    """bf16 on the native path (convolution, norm and GEMM kernels): prefill + token-by-token decoding from the state
    cache against one forward over the whole row."""
    from ttcd_b200.models import (DeltaNetConfig, DeltaNetForCausalLM, GatedDeltaNetConfig, GatedDeltaNetForCausalLM,
                                  RecurrentCache)
    torch.manual_seed(0)
    if family == "delta_net":
        model = DeltaNetForCausalLM(DeltaNetConfig(hidden_size=256, num_hidden_layers=2, num_heads=4, vocab_size=512))
    else:
        model = GatedDeltaNetForCausalLM(GatedDeltaNetConfig(hidden_size=256, num_hidden_layers=2, num_heads=2, head_dim=64,
                                                             vocab_size=512))
    model = model.to(DEV, torch.bfloat16).eval()
    ids = torch.randint(0, 512, (2, 300), device=DEV)
    with torch.no_grad():
        full = model(input_ids=ids, use_cache=False).logits.float()
        cache = RecurrentCache()
        first = model(input_ids=ids[:, :290], past_key_values=cache, use_cache=True).logits
        steps = [model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits for t in range(290, 300)]
    got = torch.cat([first, *steps], dim=1).float()
    assert _cos(got, full) > 0.999, _cos(got, full)


def test_graph_decoding_follows_eager_decoding():
    """The captured decode step (fixed-address ring cache, positions and fill count on the device) against the eager
    loop, teacher-forced so that one near-tie cannot send the two down different continuations: per-step logits agree;
    then ``generate`` end to end, and a second prompt through the same capture."""
    from ttcd_b200.models import decoding
    from ttcd_b200.models.layers import WindowKVCache
    torch.manual_seed(0)
    model = IPTTCDv9ForCausalLM(_config(window_size=256, max_position_embeddings=4096)).to(DEV, torch.bfloat16).eval()
    prompt, new = 700, 300                                     # the 256-row rings wrap
    ids = torch.randint(0, 1024, (2, prompt + new), device=DEV)
    with torch.no_grad():
        grow, source = WindowKVCache(), WindowKVCache()
        model(input_ids=ids[:, :prompt], past_key_values=grow, use_cache=True, logits_to_keep=1)
        model(input_ids=ids[:, :prompt], past_key_values=source, use_cache=True, logits_to_keep=1)
        dec = decoding.GraphDecoder(model, source, new)
        worst = 1.0
        for t in range(prompt, prompt + new):
            want = model(input_ids=ids[:, t:t + 1], past_key_values=grow, use_cache=True, logits_to_keep=1).logits[:, -1]
            dec.token.copy_(ids[:, t:t + 1])
            dec.graph.replay()
            worst = min(worst, _cos(dec.last_logits, want))
        assert worst > 0.999, worst
        launches = _native.launch_count
        a = model.generate(ids[:, :prompt], max_new_tokens=24)
        b = model.generate(ids[:, :prompt], max_new_tokens=24, use_graph=False)
        assert a.shape == b.shape == (2, prompt + 24)
        assert torch.equal(a[:, :prompt + 2], b[:, :prompt + 2])
        first = model._graph_decoder
        c = model.generate(ids[:, 100:100 + prompt], max_new_tokens=24)       # another prompt: the capture is reused
        assert model._graph_decoder is first and c.shape == (2, prompt + 24)
        d = model.generate(ids[:, 100:100 + prompt], max_new_tokens=24, use_graph=False)
        assert torch.equal(c[:, :prompt + 2], d[:, :prompt + 2])
        assert _native.launch_count > launches


@pytest.mark.parametrize("gated", [False, True])
def test_delta_rule_on_the_gpu_matches_the_token_by_token_statement(gated):
    """The chunked rule on CUDA (the one-op form: chunk-local kernels, chain kernels, batched products; bf16 / TF32
    operands with fp32 sums) against the fp32 recurrence evaluated on the CPU: outputs, final state and gradients, on a
    length that is not a multiple of the chunk."""
    from ttcd_b200 import ops
    from ttcd_b200.ops import reference as ref
    gen = torch.Generator().manual_seed(3)
    B, T, H, D, Dv = 2, 1300, 3, 64, 128
    q, k = torch.randn(B, T, H, D, generator=gen), torch.randn(B, T, H, D, generator=gen)
    v = torch.randn(B, T, H, Dv, generator=gen)
    beta = torch.rand(B, T, H, generator=gen)
    g = -torch.rand(B, T, H, generator=gen) * 0.2 if gated else None
    cpu = [t.clone().requires_grad_() for t in (q, k, v, beta)]
    o_ref, s_ref = ref.gated_delta_rule_recurrent(cpu[0], cpu[1], cpu[2], g, cpu[3], output_final_state=True)
    (o_ref.square().sum() + s_ref.sum()).backward()
    dev = [t.clone().to(DEV).requires_grad_() for t in (q, k, v, beta)]
    o, s = ops.gated_delta_rule(dev[0], dev[1], dev[2], None if g is None else g.to(DEV), dev[3], output_final_state=True)
    (o.square().sum() + s.sum()).backward()
    assert _cos(o.cpu(), o_ref) > 0.9999 and _cos(s.cpu(), s_ref) > 0.9999
    for a, b, name in zip(dev, cpu, ("q", "k", "v", "beta")):
        assert _cos(a.grad.cpu(), b.grad) > 0.999, (name, _cos(a.grad.cpu(), b.grad))
