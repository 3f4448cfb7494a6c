"""IP-TTT behind the HF-Llama interface against a plain-PyTorch statement of the reference's inference port
(custom_models/ipttt/inference.py: Llama block, fast-weight MLP updated chunk by chunk from the residual stream that
enters the block, state carried across calls), written here with Llama parameter names and nothing from the package."""
import pytest
import torch
import torch.nn.functional as F

from ttcd_b200.models import IPTTTLlamaForCausalLM, TTTDynamicCache, ipttt_config_from_llama

LLAMA = dict(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
             vocab_size=96, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False,
             ttt_mode=True, ttt_layers=[1, 2], ttt_chunk=16, ttt_lr=0.2, ttt_proj=True)


def _llama_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    d, di, hd = cfg["hidden_size"], cfg["intermediate_size"], cfg["hidden_size"] // cfg["num_attention_heads"]
    kv = cfg["num_key_value_heads"] * hd
    sd = {"model.embed_tokens.weight": torch.randn(cfg["vocab_size"], d, generator=g) * 0.5,
          "model.norm.weight": 1 + 0.1 * torch.randn(d, generator=g),
          "lm_head.weight": torch.randn(cfg["vocab_size"], d, generator=g) * 0.2}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = 1 + 0.1 * torch.randn(d, generator=g)
        sd[p + "post_attention_layernorm.weight"] = 1 + 0.1 * torch.randn(d, generator=g)
        for name, rows in (("q_proj", d), ("k_proj", kv), ("v_proj", kv), ("o_proj", d)):
            sd[p + f"self_attn.{name}.weight"] = torch.randn(rows, d if name != "o_proj" else d, generator=g) * 0.15
        sd[p + "mlp.gate_proj.weight"] = torch.randn(di, d, generator=g) * 0.15
        sd[p + "mlp.up_proj.weight"] = torch.randn(di, d, generator=g) * 0.15
        sd[p + "mlp.down_proj.weight"] = torch.randn(d, di, generator=g) * 0.15
        if i in cfg["ttt_layers"]:
            sd[p + "mlp.ttt_proj.weight"] = torch.randn(d, d, generator=g) * 0.1
            sd[p + "mlp.ttt_conv.weight"] = torch.randn(d, 1, 5, generator=g) * 0.3
    return sd


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rot(x, pos, theta):
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2).float() / hd))
    ang = pos[:, None].float() * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return x * cos[None, :, None, :] + torch.cat([-x2, x1], -1) * sin[None, :, None, :]


def _port_forward(sd, cfg, ids):
    """Whole-sequence statement: every complete chunk updates down_proj after producing its outputs."""
    d, H, HK = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, C, eps = d // H, cfg["ttt_chunk"], cfg["rms_norm_eps"]
    T = ids.shape[1]
    pos = torch.arange(T)
    x = sd["model.embed_tokens.weight"][ids]
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        layer_in = x
        h = _rms(x, sd[p + "input_layernorm.weight"], eps)
        q = _rot((h @ sd[p + "self_attn.q_proj.weight"].t()).view(1, T, H, hd), pos, cfg["rope_theta"])
        k = _rot((h @ sd[p + "self_attn.k_proj.weight"].t()).view(1, T, HK, hd), pos, cfg["rope_theta"])
        v = (h @ sd[p + "self_attn.v_proj.weight"].t()).view(1, T, HK, hd)
        k, v = k.repeat_interleave(H // HK, 2), v.repeat_interleave(H // HK, 2)
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) * hd ** -0.5
        a = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s.masked_fill(~causal, float("-inf")), -1), v).reshape(1, T, d)
        x = x + a @ sd[p + "self_attn.o_proj.weight"].t()
        h = _rms(x, sd[p + "post_attention_layernorm.weight"], eps)
        feats = F.silu(h @ sd[p + "mlp.gate_proj.weight"].t()) * (h @ sd[p + "mlp.up_proj.weight"].t())
        w = sd[p + "mlp.down_proj.weight"]
        if i not in cfg["ttt_layers"] or T < C:
            x = x + feats @ w.t()
            continue
        outs = []
        for c0 in range(0, T, C):
            f_c, t_c = feats[0, c0:c0 + C], layer_in[0, c0:c0 + C]
            outs.append(f_c @ w.t())
            if f_c.shape[0] == C:                                            # complete chunk: update
                t_conv = F.conv1d(t_c.t()[None], sd[p + "mlp.ttt_conv.weight"], padding=2, groups=d)[0].t()
                w = w + cfg["ttt_lr"] * (t_conv @ sd[p + "mlp.ttt_proj.weight"]).t() @ f_c
        x = x + torch.cat(outs)[None]
    return _rms(x, sd["model.norm.weight"], eps) @ sd["lm_head.weight"].t()


@pytest.fixture(scope="module")
def pair():
    sd = _llama_weights(LLAMA)
    model = IPTTTLlamaForCausalLM.from_llama_config(LLAMA).float().eval()
    model.load_llama_state_dict(sd)
    return sd, model


def test_config_translation_and_names(pair):
    sd, model = pair
    cfg = model.config
    assert (cfg.num_heads, cfg.num_kv_heads, cfg.ttt_target, cfg.ttt_conv_kernel_size, cfg.window_size) == (4, 2, "layer_input", 5, None)
    back = model.llama_state_dict()
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k], sd[k]), k
    from transformers import LlamaConfig
    hf = LlamaConfig(**{k: v for k, v in LLAMA.items() if not k.startswith("ttt_")})
    again = ipttt_config_from_llama(hf, ttt_mode=True, ttt_layers=[1], ttt_chunk=16)
    assert again.hidden_size == 64 and again.rope_theta == 10000.0 and again.ttt_layers == [1]
    with pytest.raises(KeyError):
        model.load_llama_state_dict({**sd, "model.layers.0.mlp.unknown.weight": torch.zeros(1)})


def test_incremental_calls_equal_the_whole_sequence_statement(pair):
    sd, model = pair
    ids = torch.randint(0, 96, (1, 75), generator=torch.Generator().manual_seed(1))
    want = _port_forward(sd, LLAMA, ids)
    with torch.no_grad():
        cache = TTTDynamicCache()
        got = [model(input_ids=ids[:, :40], past_key_values=cache, use_cache=True).logits]      # 2 chunks + 8 left over
        got += [model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits for t in range(40, 60)]
        got.append(model(input_ids=ids[:, 60:], past_key_values=cache, use_cache=True).logits)
    torch.testing.assert_close(torch.cat(got, dim=1), want, rtol=2e-4, atol=2e-4)
    # the adapted weight really differs from the base one by now, and the unfinished chunk is carried
    tail_h, tail_t, w = cache.ttt_get(2)
    assert tail_h.shape[1] == 75 % 16 and not torch.allclose(w[0], sd["model.layers.2.mlp.down_proj.weight"])


def test_generate_carries_fast_weights_and_checks_its_arguments(pair):
    sd, model = pair
    ids = torch.randint(0, 96, (1, 30), generator=torch.Generator().manual_seed(2))
    out = model.generate(input_ids=ids, max_new_tokens=12, past_key_values=TTTDynamicCache())
    assert out.shape == (1, 42)
    # greedy continuation equals arg-max decoding of the whole-sequence statement, token by token
    seq = ids
    for _ in range(12):
        nxt = _port_forward(sd, LLAMA, seq)[:, -1].argmax(-1, keepdim=True)
        seq = torch.cat([seq, nxt], dim=1)
    assert torch.equal(out, seq)
    with pytest.raises(ValueError):
        model.generate(input_ids=ids.repeat(2, 1), max_new_tokens=2)
    from ttcd_b200.models.layers import WindowKVCache
    with pytest.raises(TypeError):
        model.generate(input_ids=ids, max_new_tokens=2, past_key_values=WindowKVCache())
