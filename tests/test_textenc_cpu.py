"""Text-encoder ops against explicit per-token float64 loops."""

import torch
import torch.nn.functional as F

from kohakumosstrainer_b200.ops import textenc as T


def _cu(lengths):
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    return cu


def test_causal_conv_and_gated_norm():
    torch.manual_seed(0)
    lengths = (5, 1, 9)
    n, c, w = sum(lengths), 6, 4
    x, weight = torch.randn(n, c), torch.randn(c, w)
    out = T.causal_conv_varlen(x, weight, _cu(lengths))
    ref = torch.zeros(n, c, dtype=torch.float64)
    start = 0
    for length in lengths:
        for t in range(length):
            for j in range(w):
                if t - j >= 0:
                    ref[start + t] += weight[:, w - 1 - j].double() * x[start + t - j].double()
        start += length
    assert torch.allclose(out.double(), F.silu(ref), atol=1e-5)
    z, g = torch.randn(n, c), torch.rand(c) + 0.5
    y = T.rms_norm_gated(x, z, g, 1e-6)
    ref = x / x.square().mean(-1, keepdim=True).add(1e-6).sqrt() * g * F.silu(z)
    assert torch.allclose(y, ref, atol=1e-5)


def test_causal_gqa_attention():
    torch.manual_seed(1)
    lengths = (7, 3)
    n = sum(lengths)
    q, k, v = torch.randn(n, 4, 8), torch.randn(n, 2, 8), torch.randn(n, 2, 8)
    out = T.attention_varlen_causal(q, k, v, _cu(lengths), max(lengths), 8**-0.5)
    start = 0
    for length in lengths:
        for h in range(4):
            qs, ks, vs = q[start : start + length, h], k[start : start + length, h // 2], v[start : start + length, h // 2]
            s = (qs @ ks.t()) * 8**-0.5
            s = s.masked_fill(torch.ones(length, length).triu(1).bool(), float("-inf"))
            assert torch.allclose(out[start : start + length, h], s.softmax(-1) @ vs, atol=1e-5)
        start += length


def test_gated_delta_rule_matches_token_loop():
    torch.manual_seed(2)
    lengths = (6, 11, 1)
    n, hk, hv, dk, dv = sum(lengths), 2, 4, 8, 6
    q, k, v = torch.randn(n, hk, dk), torch.randn(n, hk, dk), torch.randn(n, hv, dv)
    a, b = torch.randn(n, hv), torch.randn(n, hv)
    a_log, dt_bias = torch.randn(hv) * 0.3, torch.randn(hv) * 0.3
    out = T.gated_delta_rule_varlen(q, k, v, a, b, a_log, dt_bias, _cu(lengths), max(lengths))
    g = (-a_log.double().exp() * F.softplus(a.double() + dt_bias.double()))
    beta = torch.sigmoid(b.double())
    start = 0
    for length in lengths:
        for h in range(hv):
            S = torch.zeros(dk, dv, dtype=torch.float64)
            for t in range(length):
                i = start + t
                kk = k[i, h // 2].double()
                kk = kk / (kk.square().sum() + T.L2_EPS).sqrt()
                qq = q[i, h // 2].double()
                qq = qq / (qq.square().sum() + T.L2_EPS).sqrt() * dk**-0.5
                S = S * g[i, h].exp()
                S = S + torch.outer(kk, beta[i, h] * (v[i, h].double() - S.t() @ kk))
                assert torch.allclose(out[i, h].double(), S.t() @ qq, atol=1e-4), (i, h)
        start += length
