"""The attention kernels at the training recipe's shape: T = 65536, windows 8192 / 4096, 16 query / 8 key-value heads,
head_dim 128 (hundreds of key blocks per tile, several waves of CTAs), forward and backward.

A dense oracle of that size does not fit, so the comparison runs on samples: a few hundred query rows (outputs, LSE
and dQ) and a few blocks of key rows (dK, dV), each against an fp32 statement restricted to those rows.  The oracle
uses nothing from the kernels: the softmax statistics of every query row that a sampled key needs are recomputed in
fp32 here.  (The reference gates its own 64K case behind IPTTCD_RUN_LARGE_KERNEL_TESTS,
test/test_fused_dual_attn.py:382-402; here it always runs.)
"""
import pytest
import torch

from ttcd_b200 import _native, ops

pytestmark = pytest.mark.gpu
DEV, BF = "cuda", torch.bfloat16
T, H, HK, D, WT, WS = 65536, 16, 8, 128, 8192, 4096
G = H // HK


@pytest.fixture(autouse=True)
def _status():
    _native.load(required=True)
    yield
    torch.cuda.synchronize()
    assert _native.device_status() == 0, "a bounded device wait expired"


def _rel(got, want):
    got, want = got.float(), want.float()
    return ((got - want).norm() / want.norm().clamp_min(1e-12)).item()


def _window_rows(rows, W):
    """Key indices [n, W] of the windows ending at ``rows`` and their validity (index >= 0)."""
    idx = rows[:, None] - torch.arange(W - 1, -1, -1, device=rows.device)[None, :]
    return idx.clamp_min(0), idx >= 0


@pytest.fixture(scope="module")
def problem():
    torch.manual_seed(7)
    q = torch.randn(1, T, H, D, device=DEV).to(BF).requires_grad_()
    k = torch.randn(1, T, HK, D, device=DEV).to(BF).requires_grad_()
    v = torch.randn(1, T, HK, D, device=DEV).to(BF).requires_grad_()
    o_t, o_s = ops.dual_window_attention(q, k, v, WT, WS)
    g_t = torch.randn_like(o_t)
    g_s = torch.randn_like(o_s)
    torch.autograd.backward([o_t, o_s], [g_t, g_s])
    torch.cuda.synchronize()
    return dict(q=q.detach(), k=k.detach(), v=v.detach(), o_t=o_t.detach(), o_s=o_s.detach(), g_t=g_t, g_s=g_s,
                dq=q.grad, dk=k.grad, dv=v.grad)


def test_forward_and_dq_on_sampled_query_rows(problem):
    p = problem
    scale = D ** -0.5
    gen = torch.Generator(device="cpu").manual_seed(1)
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 4095, 4096, 8191, 8192, 12287, T - 1]),
                      torch.randint(0, T, (246,), generator=gen)]).unique().to(DEV)
    worst = {"o_t": 0.0, "o_s": 0.0, "dq": 0.0}
    for h in range(0, H, 3):                   # heads 0, 3, ..., 15 cover both heads of several GQA groups
        kvh = h // G
        kf, vf = p["k"][0, :, kvh].float(), p["v"][0, :, kvh].float()
        for chunk in rows.split(64):
            qf = p["q"][0, chunk, h].float()                                   # [n, D]
            dq = torch.zeros_like(qf)
            for W, o_name, g_name in ((WT, "o_t", "g_t"), (WS, "o_s", "g_s")):
                idx, ok = _window_rows(chunk, W)
                s = torch.einsum("nd,nwd->nw", qf, kf[idx]) * scale
                s = s.masked_fill(~ok, float("-inf"))
                prob = torch.softmax(s, dim=-1)
                o = torch.einsum("nw,nwd->nd", prob, vf[idx])
                worst[o_name] = max(worst[o_name], _rel(p[o_name][0, chunk, h], o))
                do = p[g_name][0, chunk, h].float()
                dp = torch.einsum("nd,nwd->nw", do, vf[idx])
                ds = prob * (dp - (do * o).sum(-1, keepdim=True))
                dq += torch.einsum("nw,nwd->nd", ds, kf[idx]) * scale
            worst["dq"] = max(worst["dq"], _rel(p["dq"][0, chunk, h], dq))
    assert worst["o_t"] < 1e-2 and worst["o_s"] < 1e-2, worst
    assert worst["dq"] < 2e-2, worst


def test_dk_dv_on_sampled_key_blocks(problem):
    p = problem
    scale = D ** -0.5
    worst = {"dk": 0.0, "dv": 0.0}
    nkeys = 32
    for j0, kvh in ((0, 0), (8192 - 16, 3), (30000, 5), (T - 4096 - 16, 7), (T - 32, 1)):
        keys = torch.arange(j0, j0 + nkeys, device=DEV)
        q_lo, q_hi = j0, min(T, j0 + nkeys + WT - 1)                   # query rows that can see these keys
        rows = torch.arange(q_lo, q_hi, device=DEV)
        k_lo = max(0, q_lo - WT + 1)                                  # every key that those queries can see
        kf, vf = p["k"][0, k_lo:q_hi, kvh].float(), p["v"][0, k_lo:q_hi, kvh].float()
        jj = torch.arange(k_lo, q_hi, device=DEV)
        dk = torch.zeros(nkeys, D, device=DEV)
        dv = torch.zeros(nkeys, D, device=DEV)
        for h in range(kvh * G, (kvh + 1) * G):
            qf = p["q"][0, q_lo:q_hi, h].float()
            s = (qf @ kf.t()) * scale                                  # [rows, keys]
            causal = jj[None, :] <= rows[:, None]
            for W, o_name, g_name in ((WT, "o_t", "g_t"), (WS, "o_s", "g_s")):
                vis = causal & (jj[None, :] > rows[:, None] - W)
                prob = torch.softmax(s.masked_fill(~vis, float("-inf")), dim=-1)
                do = p[g_name][0, q_lo:q_hi, h].float()
                o = prob @ vf
                ds = prob * (do @ vf.t() - (do * o).sum(-1, keepdim=True))
                sel = slice(j0 - k_lo, j0 - k_lo + nkeys)
                dv += prob[:, sel].t() @ do
                dk += ds[:, sel].t() @ qf * scale
        worst["dk"] = max(worst["dk"], _rel(p["dk"][0, keys, kvh], dk))
        worst["dv"] = max(worst["dv"], _rel(p["dv"][0, keys, kvh], dv))
    assert worst["dk"] < 2e-2 and worst["dv"] < 2e-2, worst
