"""Tiny-config parity of loss, gradients and one AdamW step against the upstream model on CPU."""
import copy

import pytest
import torch

from tests import reference_oracle
from ttcd_b200.models import IPTTCDForCausalLM, IPTTCDv9Config, IPTTTConfig, IPTTTForCausalLM

pytestmark = pytest.mark.skipif(not reference_oracle.available(), reason="reference tree not mounted")


def _step(model, ids):
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-15, weight_decay=0.1)
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    opt.step()
    return out.loss.detach(), grads, {n: p.detach().clone() for n, p in model.named_parameters()}


def test_ipttcdv9_matches_reference(tiny_v9_kwargs):
    ref = reference_oracle.load()
    from transformers import AutoConfig  # noqa: F401
    ref_cfg_cls = ref["v9"].IPTTCDv9Config
    torch.manual_seed(0)
    ref_model = ref["v9"].IPTTCDForCausalLM(ref_cfg_cls(**tiny_v9_kwargs)).float()
    # make every special-init tensor non-trivial so the comparison exercises all paths
    with torch.no_grad():
        for n, p in ref_model.named_parameters():
            if "ttt_student_conv" in n or "ttt_teacher_conv" in n:
                p.normal_(0, 0.3)
    mine = IPTTCDForCausalLM(IPTTCDv9Config(**tiny_v9_kwargs)).float()
    missing, unexpected = mine.load_state_dict(ref_model.state_dict(), strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m or "inv_freq" in m for m in missing), missing
    ref_model.train(); mine.train()
    ids = torch.randint(0, 1024, (2, 256), generator=torch.Generator().manual_seed(0))
    l_ref, g_ref, p_ref = _step(ref_model, ids)
    l_mine, g_mine, p_mine = _step(mine, ids)
    assert abs(float(l_ref) - float(l_mine)) < 1e-4, (l_ref, l_mine)
    assert set(g_ref) == set(g_mine)
    for n in g_ref:
        torch.testing.assert_close(g_mine[n], g_ref[n], rtol=2e-3, atol=2e-5, msg=lambda m, n=n: f"{n}: {m}")
        torch.testing.assert_close(p_mine[n], p_ref[n], rtol=1e-4, atol=2e-5, msg=lambda m, n=n: f"{n}: {m}")


def test_ipttt_matches_reference():
    ref = reference_oracle.load()
    kw = dict(hidden_size=128, num_hidden_layers=2, num_heads=4, num_kv_heads=2, intermediate_size=384,
              vocab_size=1024, window_size=64, ttt_mode=True, ttt_chunk=16, ttt_layers=[0, 1], ttt_lr=0.05,
              ttt_conv_causal=True, fuse_norm=False, fuse_swiglu=False, fuse_cross_entropy=False)
    torch.manual_seed(1)
    ref_model = ref["ipttt"].IPTTTForCausalLM(ref["ipttt"].IPTTTConfig(**kw)).float()
    with torch.no_grad():
        for n, p in ref_model.named_parameters():
            if "ttt_conv" in n:
                p.normal_(0, 0.3)
    mine = IPTTTForCausalLM(IPTTTConfig(**kw)).float()
    mine.load_state_dict(ref_model.state_dict(), strict=False)
    ref_model.train(); mine.train()
    ids = torch.randint(0, 1024, (2, 100), generator=torch.Generator().manual_seed(3))
    l_ref, g_ref, _ = _step(ref_model, ids)
    l_mine, g_mine, _ = _step(mine, ids)
    assert abs(float(l_ref) - float(l_mine)) < 1e-4
    for n in g_ref:
        torch.testing.assert_close(g_mine[n], g_ref[n], rtol=2e-3, atol=2e-5, msg=lambda m, n=n: f"{n}: {m}")
