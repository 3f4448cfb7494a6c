"""The fixed-address decoding cache against the growing one, step by step on CPU (the captured-graph path itself
needs a GPU: tests/test_gpu_model.py)."""
import pytest
import torch

from ttcd_b200.models import IPTTCDv9Config, IPTTCDv9ForCausalLM, TransformerConfig, TransformerForCausalLM
from ttcd_b200.models.decoding import _windows, pack_projection_weights
from ttcd_b200.models.layers import StaticWindowCache, WindowKVCache

KW = dict(hidden_size=64, num_hidden_layers=3, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=128,
          fuse_cross_entropy=False, qk_norm=True)


def _models():
    torch.manual_seed(0)
    yield "windowed_ttcd", IPTTCDv9ForCausalLM(IPTTCDv9Config(**KW, window_size=32, ttt_mode=True, ttt_chunk=8, ttt_layers=[1, 2]))
    yield "full_attention", TransformerForCausalLM(TransformerConfig(**KW))
    yield "short_prompt", TransformerForCausalLM(TransformerConfig(**KW, window_size=64))


@pytest.mark.parametrize("name,model", list(_models()), ids=[n for n, _ in _models()])
def test_static_cache_steps_equal_the_growing_cache(name, model):
    model = model.float().eval()
    prompt_len, new = (50, 45) if name != "short_prompt" else (10, 30)          # the windowed ring wraps more than once
    ids = torch.randint(0, 128, (2, prompt_len + new), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        grow = WindowKVCache()
        model(input_ids=ids[:, :prompt_len], past_key_values=grow, use_cache=True)
        source = WindowKVCache()
        model(input_ids=ids[:, :prompt_len], past_key_values=source, use_cache=True)
        static = StaticWindowCache(source, _windows(model), new)
        assert static.get_seq_length() == prompt_len
        want0 = None
        for t in range(prompt_len, prompt_len + new):
            want = model(input_ids=ids[:, t:t + 1], past_key_values=grow, use_cache=True).logits
            got = model(input_ids=ids[:, t:t + 1], past_key_values=static, use_cache=True).logits
            static.advance()
            static.host_advance()
            want0 = want if want0 is None else want0
            torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5, msg=lambda m, t=t: f"token {t}: {m}")
        assert static.get_seq_length() == prompt_len + new == grow.get_seq_length()
        # rewinding and replaying the same tokens gives the same logits again (what a reused capture does)
        static2 = StaticWindowCache(source, _windows(model), new)
        first = model(input_ids=ids[:, prompt_len:prompt_len + 1], past_key_values=static2, use_cache=True).logits
        torch.testing.assert_close(first, want0, rtol=1e-4, atol=1e-5)


def test_packing_projection_weights_changes_no_output():
    torch.manual_seed(2)
    model = TransformerForCausalLM(TransformerConfig(**KW)).float().eval()
    ids = torch.randint(0, 128, (1, 20))
    with torch.no_grad():
        before = model(input_ids=ids).logits
        assert pack_projection_weights(model) == 6          # q|k|v and gate|up of three blocks
        assert pack_projection_weights(model) == 0          # already adjacent
        after = model(input_ids=ids).logits
    assert torch.equal(before, after)
    attn = model.model.layers[0].attn
    assert attn.q_proj.weight.data_ptr() + attn.q_proj.weight.numel() * 4 == attn.k_proj.weight.data_ptr()
    sd = model.state_dict()
    assert sd["model.layers.0.attn.k_proj.weight"].shape == attn.k_proj.weight.shape


def test_l2_softmax_attention_statement_and_model_path():
    """Weights exp(s - m) / ||exp(s - m)||_2 over the causal prefix, against a per-row loop; a model with the flag
    set runs through it (forward, backward) and differs from the softmax model."""
    from ttcd_b200.ops import reference as R
    torch.manual_seed(3)
    q, k, v = torch.randn(2, 9, 4, 8), torch.randn(2, 12, 2, 8), torch.randn(2, 12, 2, 8)
    got = R.l2_softmax_attention(q, k, v, block=4)
    for b in range(2):
        for h in range(4):
            for i in range(9):
                hi = 12 - 9 + i + 1
                s = (k[b, :hi, h // 2] @ q[b, i, h]) * 8 ** -0.5
                e = torch.exp(s - s.max())
                want = (e / e.square().sum().sqrt()) @ v[b, :hi, h // 2]
                torch.testing.assert_close(got[b, i, h], want, rtol=1e-5, atol=1e-6)
    plain = TransformerForCausalLM(TransformerConfig(**KW)).float()
    l2 = TransformerForCausalLM(TransformerConfig(**KW, use_l2_softmax=True)).float()
    l2.load_state_dict(plain.state_dict())
    ids = torch.randint(0, 128, (2, 24))
    out = l2(input_ids=ids, labels=ids)
    out.loss.backward()
    assert all(p.grad is not None for p in l2.parameters())
    assert not torch.allclose(out.logits, plain(input_ids=ids).logits, atol=1e-3)
