"""Delta-rule op (chunked WY form vs the token-by-token recurrence, values and gradients) and the DeltaNet
baseline model: starts identical to the plain transformer (zero-initialised output projection), runs the
sub-layer in training only."""
import torch

from ttcd_b200.models import DeltaNetBaselineConfig, DeltaNetBaselineForCausalLM
from ttcd_b200.ops import reference as ref


def test_chunked_delta_rule_matches_recurrence():
    torch.manual_seed(0)
    B, T, H, D = 2, 50, 3, 16
    q, k, v = (torch.randn(B, T, H, D, dtype=torch.float64, requires_grad=True) for _ in range(3))
    beta = torch.rand(B, T, H, dtype=torch.float64, requires_grad=True)
    a = ref.delta_rule_recurrent(q, k, v, beta)
    b = ref.delta_rule_chunked(q, k, v, beta, chunk=16)
    torch.testing.assert_close(a.float(), b.float(), rtol=1e-4, atol=1e-5)
    ga = torch.autograd.grad(a.float().square().sum(), (q, k, v, beta))
    gb = torch.autograd.grad(b.float().square().sum(), (q, k, v, beta))
    for x, y in zip(ga, gb):
        torch.testing.assert_close(x.float(), y.float(), rtol=1e-3, atol=1e-4)
    # packed sequences restart the state at every boundary
    cu = torch.tensor([0, 20, 50])
    c = ref.delta_rule_chunked(q, k, v, beta, chunk=16, cu_seqlens=cu)
    torch.testing.assert_close(c[:, 20:].float(), ref.delta_rule_recurrent(q[:, 20:], k[:, 20:], v[:, 20:], beta[:, 20:]).float(),
                               rtol=1e-4, atol=1e-5)


def test_model_trains_sublayer_only_in_training_mode():
    torch.manual_seed(0)
    cfg = DeltaNetBaselineConfig(hidden_size=32, num_hidden_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=64,
                                 vocab_size=64, window_size=16, ttt_mode=True, ttt_layers=[1], fuse_cross_entropy=False,
                                 max_position_embeddings=64, tie_word_embeddings=False)
    model = DeltaNetBaselineForCausalLM(cfg)
    blk = model.model.layers[1]
    assert blk.is_deltanet_layer and not model.model.layers[0].is_deltanet_layer
    assert float(blk.dn_o_proj.weight.abs().max()) == 0.0
    ids = torch.randint(0, 64, (2, 24))
    model.train()
    loss_train = model(input_ids=ids, labels=ids).loss
    model.eval()
    loss_eval = model(input_ids=ids, labels=ids).loss
    torch.testing.assert_close(loss_train, loss_eval)         # zero output projection: same function at init
    model.train()
    model(input_ids=ids, labels=ids).loss.backward()
    assert blk.dn_o_proj.weight.grad.abs().max() > 0          # the sub-layer is in the graph and learns
    with torch.no_grad():
        blk.dn_o_proj.weight.normal_(0, 0.1)
    a = model(input_ids=ids, labels=ids).loss
    model.eval()
    b = model(input_ids=ids, labels=ids).loss
    assert abs(float(a) - float(b)) > 1e-6                    # training-only path


def test_lse_combination_equals_dual_window_attention():
    """The LSE-merge formulation (student pass + shifted far-band pass) gives the fused op's outputs."""
    from ttcd_b200 import ops
    torch.manual_seed(0)
    B, T, H, HK, D = 2, 96, 4, 2, 16
    q, k, v = torch.randn(B, T, H, D), torch.randn(B, T, HK, D), torch.randn(B, T, HK, D)
    for wt, ws in ((48, 16), (64, 32), (200, 24)):
        t_ref, s_ref = ref.dual_window_attention(q, k, v, wt, ws)
        t, s = ops.lse_dual_window_attention(q, k, v, wt, ws)
        torch.testing.assert_close(s, s_ref, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(t, t_ref, rtol=1e-4, atol=1e-5)


def test_dual_window_backward_through_one_softmax():
    """The per-row ratio identity behind the combined backward kernels equals autograd of the two-softmax op."""
    torch.manual_seed(1)
    B, T, H, HK, D = 2, 80, 4, 2, 8
    q = torch.randn(B, T, H, D, dtype=torch.float64, requires_grad=True)
    k = torch.randn(B, T, HK, D, dtype=torch.float64, requires_grad=True)
    v = torch.randn(B, T, HK, D, dtype=torch.float64, requires_grad=True)
    for wt, ws in ((48, 16), (64, 24)):
        o_t, o_s = ref.dual_window_attention(q, k, v, wt, ws)
        g_t, g_s = torch.randn_like(o_t), torch.randn_like(o_s)
        want = torch.autograd.grad([o_t, o_s], [q, k, v], [g_t, g_s])
        got = ref.dual_window_attention_backward_combined(q.detach(), k.detach(), v.detach(), g_t, g_s, wt, ws)
        for a, b in zip(got, want):
            torch.testing.assert_close(a, b.float(), rtol=1e-4, atol=1e-4)
