"""The ``delta_net`` and ``gated_deltanet`` families on CPU: the chunked rule against the token-by-token statement
(values and gradients), against the upstream tree's own naive recurrence, decoding from the state cache against one
full forward, padded batches, and the parameter names of the upstream classes."""
import sys

import pytest
import torch

from tests import reference_oracle
from ttcd_b200.models import (DeltaNetConfig, DeltaNetForCausalLM, GatedDeltaNetConfig, GatedDeltaNetForCausalLM,
                              RecurrentCache)
from ttcd_b200.ops import reference as R

DN = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, vocab_size=128, fuse_cross_entropy=False)
GDN = dict(hidden_size=64, num_hidden_layers=2, num_heads=2, head_dim=16, expand_v=2, vocab_size=128, fuse_cross_entropy=False)


def _rule_inputs(B=2, T=150, H=3, D=16, Dv=24, seed=0):
    gen = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, D, generator=gen), torch.randn(B, T, H, D, generator=gen)
    v = torch.randn(B, T, H, Dv, generator=gen)
    beta = torch.rand(B, T, H, generator=gen) * 2
    g = -torch.rand(B, T, H, generator=gen) * 0.4
    return q, k, v, g, beta


@pytest.mark.parametrize("gated", [False, True])
def test_chunked_rule_matches_recurrent_values_state_and_gradients(gated):
    q, k, v, g, beta = _rule_inputs()
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
    twins = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
    init = torch.randn(2, 3, 16, 24) * 0.1

    def run(fn, ts):
        o, s = fn(ts[0], ts[1], ts[2], ts[3] if gated else None, ts[4], initial_state=init, output_final_state=True)
        (o.square().sum() + s.sum()).backward()
        return o, s

    o_r, s_r = run(R.gated_delta_rule_recurrent, leaves)
    o_c, s_c = run(R.gated_delta_rule_chunked, twins)
    torch.testing.assert_close(o_c, o_r, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s_c, s_r, rtol=1e-4, atol=1e-5)
    for a, b, name in zip(twins, leaves, "qkvgb"):
        if name == "g" and not gated:
            continue
        torch.testing.assert_close(a.grad, b.grad, rtol=2e-3, atol=2e-4, msg=lambda m, n=name: f"d{n}: {m}")


def test_packed_sequences_restart_the_state():
    q, k, v, g, beta = _rule_inputs(B=1, T=200)
    cu = torch.tensor([0, 70, 71, 200], dtype=torch.int32)
    o, s = R.gated_delta_rule_chunked(q, k, v, g, beta, cu_seqlens=cu, output_final_state=True)
    for i, (a, b) in enumerate(((0, 70), (70, 71), (71, 200))):
        o_i, s_i = R.gated_delta_rule_recurrent(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], beta[:, a:b], output_final_state=True)
        torch.testing.assert_close(o[:, a:b], o_i, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(s[i:i + 1], s_i, rtol=1e-4, atol=1e-5)


@pytest.mark.skipif(not reference_oracle.available(), reason="reference tree not mounted")
def test_plain_rule_matches_the_upstream_naive_recurrence():
    import importlib.util
    path = reference_oracle.REFERENCE_ROOT / "fla" / "ops" / "delta_rule" / "naive.py"
    spec = importlib.util.spec_from_file_location("_upstream_delta_naive", path)
    naive = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(naive)
    q, k, v, _, beta = _rule_inputs(T=96)
    qn, kn = torch.nn.functional.normalize(q, dim=-1), torch.nn.functional.normalize(k, dim=-1)
    want, s_want = naive.delta_rule_recurrence(*(t.transpose(1, 2) for t in (qn, kn, v)), beta.transpose(1, 2))
    got, s_got = R.gated_delta_rule_chunked(q, k, v, None, beta, output_final_state=True)
    torch.testing.assert_close(got, want.transpose(1, 2), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s_got, s_want, rtol=1e-4, atol=1e-5)


def _models():
    torch.manual_seed(0)
    yield "delta_net", DeltaNetForCausalLM(DeltaNetConfig(**DN)).float()
    yield "delta_net_gate", DeltaNetForCausalLM(DeltaNetConfig(**DN, use_gate=True, qk_activation="elu", qk_norm="sum")).float()
    yield "gated_deltanet", GatedDeltaNetForCausalLM(GatedDeltaNetConfig(**GDN)).float()
    yield "gated_deltanet_vheads", GatedDeltaNetForCausalLM(GatedDeltaNetConfig(**GDN, num_v_heads=4, allow_neg_eigval=True)).float()
    yield "hybrid", GatedDeltaNetForCausalLM(GatedDeltaNetConfig(**GDN, attn=dict(layers=[1], num_heads=4, window_size=32))).float()


@pytest.mark.parametrize("name,model", list(_models()), ids=[n for n, _ in _models()])
def test_model_trains_and_decodes_from_its_state(name, model):
    ids = torch.randint(0, 128, (2, 100), generator=torch.Generator().manual_seed(1))
    model.train()
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    assert torch.isfinite(out.loss)
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert not missing, missing
    model.eval()
    with torch.no_grad():
        full = model(input_ids=ids, use_cache=False).logits
        cache = RecurrentCache()
        first = model(input_ids=ids[:, :77], past_key_values=cache, use_cache=True).logits
        steps = [model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits for t in range(77, 90)]
        tail = model(input_ids=ids[:, 90:], past_key_values=cache, use_cache=True).logits      # a multi-token continuation
    got = torch.cat([first, *steps, tail], dim=1)
    torch.testing.assert_close(got, full, rtol=2e-3, atol=2e-4)
    tokens = model.generate(ids[:, :20], max_new_tokens=4)
    assert tokens.shape == (2, 24)


def test_left_padded_batch_equals_the_samples_alone():
    torch.manual_seed(2)
    model = GatedDeltaNetForCausalLM(GatedDeltaNetConfig(**GDN)).float().eval()
    a, b = torch.randint(0, 128, (1, 40)), torch.randint(0, 128, (1, 25))
    ids = torch.cat([a, torch.cat([torch.zeros(1, 15, dtype=torch.long), b], dim=1)])
    mask = torch.ones(2, 40, dtype=torch.long)
    mask[1, :15] = 0
    with torch.no_grad():
        cache = RecurrentCache()
        both = model(input_ids=ids, attention_mask=mask, past_key_values=cache, use_cache=True).logits
        nxt = torch.randint(0, 128, (2, 1))
        step = model(input_ids=nxt, attention_mask=torch.cat([mask, mask.new_ones(2, 1)], 1), past_key_values=cache,
                     use_cache=True).logits
        want_a = model(input_ids=torch.cat([a, nxt[:1]], 1)).logits
        want_b = model(input_ids=torch.cat([b, nxt[1:]], 1)).logits
    torch.testing.assert_close(both[0], want_a[0, :40], rtol=2e-3, atol=2e-4)
    torch.testing.assert_close(both[1, 15:], want_b[0, :25], rtol=2e-3, atol=2e-4)
    torch.testing.assert_close(step[0, 0], want_a[0, 40], rtol=2e-3, atol=2e-4)
    torch.testing.assert_close(step[1, 0], want_b[0, 25], rtol=2e-3, atol=2e-4)


def test_decay_parameters_are_initialised_in_range_and_exempt_from_weight_decay():
    torch.manual_seed(3)
    model = GatedDeltaNetForCausalLM(GatedDeltaNetConfig(**dict(GDN, num_heads=8, hidden_size=128)))
    mixer = model.model.layers[0].attn
    a = mixer.A_log.exp()
    assert (a > 0).all() and (a <= 16).all() and a.std() > 0
    dt = torch.nn.functional.softplus(mixer.dt_bias)
    assert (dt >= 1e-4 - 1e-7).all() and (dt <= 0.1 + 1e-6).all()
    assert mixer.A_log._no_weight_decay and mixer.dt_bias._no_weight_decay


@pytest.mark.skipif(not reference_oracle.available(), reason="reference tree not mounted")
@pytest.mark.parametrize("family", ["delta_net", "gated_deltanet"])
def test_parameter_names_and_shapes_match_the_upstream_classes(family):
    root = str(reference_oracle.REFERENCE_ROOT)
    sys.path.insert(0, root)
    try:
        if family == "delta_net":
            from fla.models.delta_net import DeltaNetConfig as C, DeltaNetForCausalLM as M
            kw, mine = dict(DN, use_gate=True), DeltaNetForCausalLM(DeltaNetConfig(**DN, use_gate=True))
        else:
            from fla.models.gated_deltanet import GatedDeltaNetConfig as C, GatedDeltaNetForCausalLM as M
            kw, mine = dict(GDN, num_v_heads=4), GatedDeltaNetForCausalLM(GatedDeltaNetConfig(**GDN, num_v_heads=4))
        theirs = M(C(**kw))
    finally:
        sys.path.remove(root)
    want = {n: tuple(p.shape) for n, p in theirs.state_dict().items()}
    got = {n: tuple(p.shape) for n, p in mine.state_dict().items()}
    assert got == want, (set(got) ^ set(want), {n for n in set(got) & set(want) if got[n] != want[n]})
    mine.load_state_dict(theirs.state_dict())


def test_shipped_configs_build_on_the_meta_device():
    import json
    from pathlib import Path
    from ttcd_b200.models import MODEL_CLASSES
    files = sorted((Path(__file__).resolve().parents[1] / "configs").glob("*delta*net/*.json"))
    assert len(files) == 7, files
    for f in files:
        raw = json.loads(f.read_text())
        cfg_cls, model_cls = MODEL_CLASSES[raw["model_type"]]
        with torch.device("meta"):
            model = model_cls(cfg_cls(**raw))
        assert sum(p.numel() for p in model.parameters()) > 1e8, f


def test_chain_op_backward_matches_autograd():
    """The hand-written backward of the chunk-to-chunk chain (a reverse chain plus batched products) against autograd
    through the same recurrence, in float64."""
    from ttcd_b200.ops import delta_chain as dc
    torch.manual_seed(0)
    BH, n, C, D, Dv = 3, 5, 8, 16, 24
    mk = lambda *s: (torch.randn(*s, dtype=torch.float64) * 0.3).requires_grad_()  # noqa: E731
    w, u, kt, s0 = mk(BH, n, C, D), mk(BH, n, C, Dv), mk(BH, n, C, D), mk(BH, D, Dv)
    gamma = torch.rand(BH, n, dtype=torch.float64).requires_grad_()

    def loop(w, u, kt, gamma, s0):
        S, vns, sts = s0, [], []
        for i in range(n):
            sts.append(S)
            vn = u[:, i] - w[:, i] @ S
            vns.append(vn)
            S = gamma[:, i, None, None] * S + kt[:, i].transpose(-1, -2) @ vn
        return torch.stack(vns, 1), torch.stack(sts, 1), S

    want = loop(w, u, kt, gamma, s0)
    got = dc.delta_chain(w, u, kt, gamma, s0)
    gs = [torch.randn_like(o) for o in want]
    g_want = torch.autograd.grad(want, [w, u, kt, gamma, s0], gs)
    g_got = torch.autograd.grad(got, [w, u, kt, gamma, s0], gs)
    for a, b in zip(got + g_got, want + g_want):
        torch.testing.assert_close(a, b, rtol=1e-10, atol=1e-10)


@pytest.mark.parametrize("gated,l2norm", [(False, True), (True, True), (True, False)])
def test_fused_op_statement_matches_the_recurrence(gated, l2norm):
    """The one-op form of the chunked rule (hand-written backward through the chunk-local part, the chain and the output
    products; its PyTorch statement, which is also the oracle of the CUDA kernels) against the token-by-token rule:
    outputs, final state and the gradients of q, k, v, g, beta and the initial state, on a ragged length."""
    from ttcd_b200.ops.delta_fused import gated_delta_rule_fused
    q, k, v, g, beta = (t.double() for t in _rule_inputs())
    if not l2norm:
        k = torch.nn.functional.normalize(k, dim=-1)
    if not gated:
        g = None
    s0 = torch.randn(2, 3, 16, 24, dtype=torch.float64) * 0.1
    leaves = [None if t is None else t.clone().requires_grad_() for t in (q, k, v, g, beta, s0)]
    twins = [None if t is None else t.clone().requires_grad_() for t in (q, k, v, g, beta, s0)]
    o_r, s_r = R.gated_delta_rule_recurrent(*leaves[:5], None, l2norm, leaves[5], True)
    o_f, s_f = gated_delta_rule_fused(*twins[:5], None, l2norm, twins[5], True)
    go, gs = torch.randn_like(o_r), torch.randn_like(s_r)
    ((o_r * go).sum() + (s_r * gs).sum()).backward()
    ((o_f * go).sum() + (s_f * gs).sum()).backward()
    torch.testing.assert_close(o_f, o_r.double(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(s_f, s_r.double(), rtol=1e-4, atol=1e-5)
    for a, b, name in zip(twins, leaves, ("q", "k", "v", "g", "beta", "s0")):
        if a is not None:
            torch.testing.assert_close(a.grad, b.grad.double(), rtol=1e-3, atol=1e-4, msg=lambda m, name=name: f"d{name}: {m}")


def test_kept_intermediates_stay_within_their_share_of_memory(monkeypatch):
    """The keep-or-rebuild decision of the fused op: sets are kept while the ones still waiting for their backward fit
    the allowed share of the device memory, the count falls when a call's graph goes away, and a process that has
    already peaked near the device's capacity keeps nothing."""
    import gc
    from ttcd_b200.ops import delta_fused as df

    class Ctx:
        needs_input_grad = (True,)

    class FakeQ:
        is_cuda, device = True, "cuda:0"

    class Props:
        total_memory = 1000

    peak = {"v": 0}
    monkeypatch.setattr(df.torch.cuda, "get_device_properties", lambda d: Props)
    monkeypatch.setattr(df.torch.cuda, "max_memory_allocated", lambda d: peak["v"])
    monkeypatch.setattr(df.torch.cuda, "memory_allocated", lambda d: 0)
    monkeypatch.setattr(df, "_kept_bytes", 0)
    monkeypatch.delenv("TTCD_DELTA_KEEP", raising=False)
    a, b, c = Ctx(), Ctx(), Ctx()
    assert df._keep_intermediates(a, FakeQ, 90) and df._keep_intermediates(b, FakeQ, 90)
    assert not df._keep_intermediates(c, FakeQ, 90)            # 270 > a fifth of 1000
    del a
    gc.collect()
    assert df._kept_bytes == 90 and df._keep_intermediates(c, FakeQ, 90)
    peak["v"] = 750
    assert not df._keep_intermediates(Ctx(), FakeQ, 60)         # 750 + 60 > 80 % of 1000
    no_grad = Ctx()
    no_grad.needs_input_grad = (False,)
    peak["v"] = 0
    assert not df._keep_intermediates(no_grad, FakeQ, 1)
    monkeypatch.setenv("TTCD_DELTA_KEEP", "1")
    assert df._keep_intermediates(Ctx(), FakeQ, 10_000)
