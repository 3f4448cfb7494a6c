"""HF-key mapping, DCP round trips in both key conventions and checkpoint averaging (CPU)."""
import json

import torch

from ttcd_b200.models import IPTTCDForCausalLM, IPTTCDv9Config, TransformerConfig, TransformerForCausalLM
from ttcd_b200.train.checkpoint import checkpoint_keys, load_model_weights
from ttcd_b200.utils import convert

KW = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128, vocab_size=128,
          window_size=32, fuse_cross_entropy=False, qk_norm=True)


def _hf_like_state(vocab=100):
    g = torch.Generator().manual_seed(0)
    sd = {"model.embed_tokens.weight": torch.randn(vocab, 64, generator=g), "model.norm.weight": torch.randn(64, generator=g),
          "lm_head.weight": torch.randn(vocab, 64, generator=g)}
    for i in range(2):
        p = f"model.layers.{i}."
        sd.update({p + "self_attn.q_proj.weight": torch.randn(64, 64, generator=g), p + "self_attn.k_proj.weight": torch.randn(32, 64, generator=g),
                   p + "self_attn.v_proj.weight": torch.randn(32, 64, generator=g), p + "self_attn.o_proj.weight": torch.randn(64, 64, generator=g),
                   p + "self_attn.q_norm.weight": torch.randn(16, generator=g), p + "self_attn.k_norm.weight": torch.randn(16, generator=g),
                   p + "input_layernorm.weight": torch.randn(64, generator=g), p + "post_attention_layernorm.weight": torch.randn(64, generator=g),
                   p + "mlp.gate_proj.weight": torch.randn(128, 64, generator=g), p + "mlp.up_proj.weight": torch.randn(128, 64, generator=g),
                   p + "mlp.down_proj.weight": torch.randn(64, 128, generator=g), p + "self_attn.rotary_emb.inv_freq": torch.randn(8, generator=g)})
    return sd


def test_key_mapping():
    assert convert.map_hf_key("model.layers.3.self_attn.q_proj.weight") == "model.layers.3.attn.q_proj.weight"
    assert convert.map_hf_key("model.layers.0.input_layernorm.weight") == "model.layers.0.attn_norm.weight"
    assert convert.map_hf_key("model.layers.0.post_attention_layernorm.weight") == "model.layers.0.mlp_norm.weight"
    assert convert.map_hf_key("model.embed_tokens.weight") == "model.embeddings.weight"
    assert convert.map_hf_key("model.layers.0.self_attn.rotary_emb.inv_freq") is None


def test_hf_to_ipttcd_dcp_and_load(tmp_path):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(dict(model_type="ipttcdv9", ttt_mode=True, ttt_layers=[1], ttt_chunk=8, tie_word_embeddings=False, **KW)))
    src = _hf_like_state(vocab=100)
    report = convert.convert_hf_causal_lm_to_dcp("unused", str(cfg_path), str(tmp_path / "seed"), source_state_dict=src)
    assert report["copied"] == len(src) - 2 and report["skipped_source_keys"] == [f"model.layers.{i}.self_attn.rotary_emb.inv_freq" for i in range(2)]
    keys = checkpoint_keys(str(tmp_path / "seed"))
    assert "model.layers.1.mlp.ttt_proj.weight" in keys and "lm_head.weight" in keys and not any(k.startswith("model.model.") for k in keys)
    model = IPTTCDForCausalLM(IPTTCDv9Config(ttt_mode=True, ttt_layers=[1], ttt_chunk=8, tie_word_embeddings=False, **KW))
    load_model_weights(model, str(tmp_path / "seed"))
    torch.testing.assert_close(model.model.layers[0].attn.q_proj.weight, src["model.layers.0.self_attn.q_proj.weight"])
    torch.testing.assert_close(model.model.embeddings.weight[:100], src["model.embed_tokens.weight"])   # vocab 128 > 100: prefix copy
    torch.testing.assert_close(model.model.layers[1].mlp_norm.weight, src["model.layers.1.post_attention_layernorm.weight"])


def test_transformer_to_ipttcd_and_merge(tmp_path):
    tcfg = TransformerConfig(**KW)
    tf = TransformerForCausalLM(tcfg)
    tf.save_pretrained(tmp_path / "tf", safe_serialization=True)
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(dict(model_type="ipttcdv9", ttt_mode=True, ttt_layers=[0], ttt_chunk=8, **KW)))
    rep = convert.convert_transformer_to_ipttcd_dcp(str(tmp_path / "tf"), str(cfg_path), str(tmp_path / "dcp"))
    assert any("ttt_proj" in k for k in rep["target_only_keys"]) and rep["copied"] > 10
    m = IPTTCDForCausalLM(IPTTCDv9Config(ttt_mode=True, ttt_layers=[0], ttt_chunk=8, **KW))
    load_model_weights(m, str(tmp_path / "dcp"))
    torch.testing.assert_close(m.model.layers[1].mlp.down_proj.weight, tf.model.layers[1].mlp.down_proj.weight)
    assert convert.merge_weights([10, 20], "sma") == [0.5, 0.5]
    w = convert.merge_weights([10, 20, 30], "wma", alpha=0.5)
    assert abs(sum(w) - 1.0) < 1e-9
