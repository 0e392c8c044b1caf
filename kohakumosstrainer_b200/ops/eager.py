"""Reference semantics of every op in plain PyTorch (fp32 accumulation, one rounding).

These functions are the numerical contract of the CUDA kernels and the CPU execution path.
Signatures follow the reference op table (`src/kohakumoss_kernels/ops.py:5-81`) and its
eager backend (`src/kohakumoss_kernels/backends/eager/{norm,rope,ffn,loss,attention}.py`).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


def _acc(*tensors: Tensor | None) -> torch.dtype:
    dt = torch.float32
    for t in tensors:
        if t is not None:
            dt = torch.promote_types(dt, t.dtype)
    return dt


def _rms(xf: Tensor, eps: float) -> Tensor:
    return xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)


def rms_norm(x: Tensor, weight: Tensor | None, eps: float) -> Tensor:
    dt = _acc(x)
    y = _rms(x.to(dt), eps)
    if weight is not None:
        y = y * weight.to(dt)
    return y.to(x.dtype)


def rms_norm_mod(x, weight, shift, scale, seg, eps: float) -> Tensor:
    """`rms_norm(x) * w * (1 + scale[seg]) + shift[seg]`; shift/scale are per-sample [B, D]
    (possibly strided views of a [B, 6, D] modulation tensor)."""
    dt = _acc(x)
    y = _rms(x.to(dt), eps)
    if weight is not None:
        y = y * weight.to(dt)
    if scale is not None:
        y = y * (1.0 + scale.to(dt).index_select(0, seg.long()))
    if shift is not None:
        y = y + shift.to(dt).index_select(0, seg.long())
    return y.to(x.dtype)


def gated_residual(x, o, gate, seg, r: float = 1.0) -> Tensor:
    """`x * r + o * gate[seg]`; gate None means a plain residual add."""
    dt = _acc(x, o)
    of = o.to(dt)
    if gate is not None:
        of = of * gate.to(dt).index_select(0, seg.long())
    xf = x.to(dt)
    if r != 1.0:
        xf = xf * r
    return (xf + of).to(x.dtype)


def rope_sin_cos(pos: Tensor, bands: Tensor, dtype=torch.float32) -> tuple[Tensor, Tensor]:
    """[N, Dh/2] sin, cos: half-dim j uses axis j // n_bands, band j % n_bands."""
    phase = (pos.to(dtype).unsqueeze(-1) * bands.to(dtype)).flatten(-2)
    return phase.sin(), phase.cos()


def _norm_rotate(x, weight, sin, cos, eps):
    dt = sin.dtype
    xf = _rms(x.to(dt), eps) * weight.to(dt)
    a, b = xf.chunk(2, -1)
    s, c = sin.unsqueeze(1), cos.unsqueeze(1)
    return torch.cat((a * c - b * s, b * c + a * s), -1).to(x.dtype)


def qk_norm_rope(q, k, q_weight, k_weight, pos, bands, eps: float):
    """q, k [N, H, Dh]: per-head RMSNorm then split-half rotation of pairs (j, j + Dh/2)."""
    sin, cos = rope_sin_cos(pos, bands, _acc(q, k))
    return _norm_rotate(q, q_weight, sin, cos, eps), _norm_rotate(k, k_weight, sin, cos, eps)


def situ_glu(x: Tensor) -> Tensor:
    """x [N, 2F] = [up | gate] -> (4 tanh(g/4) sigmoid(g)) * (25 tanh(u/25))."""
    u, g = x.to(_acc(x)).chunk(2, -1)
    a = (4.0 * torch.tanh(g / 4.0) * torch.sigmoid(g)) * (25.0 * torch.tanh(u / 25.0))
    return a.to(x.dtype)


def situ_pair(u: Tensor, g: Tensor) -> Tensor:
    dt = _acc(u, g)
    uf, gf = u.to(dt), g.to(dt)
    a = (4.0 * torch.tanh(gf / 4.0) * torch.sigmoid(gf)) * (25.0 * torch.tanh(uf / 25.0))
    return a.to(u.dtype)


def token_mse(pred, target, seg, weight, mask=None) -> Tensor:
    """sum_tokens weight[seg] * mask * mean_c (pred - target)^2 in fp32."""
    dt = _acc(pred, target)
    err = (pred.to(dt) - target.to(dt)).square().mean(-1)
    w = weight.to(dt).index_select(0, seg.long())
    if mask is not None:
        w = w * mask.to(dt)
    return (err * w).sum()


def attention_varlen(q, k, v, cu_seqlens, max_seqlen: int, scale: float, lengths=None) -> Tensor:
    """q, k, v [N, H, Dh] packed by `cu_seqlens`; full (non-causal) attention inside each
    segment. `lengths` (host tuple) avoids a device read-back of `cu_seqlens`."""
    if lengths is None:
        bounds = cu_seqlens.tolist()
        lengths = [b - a for a, b in zip(bounds[:-1], bounds[1:])]
    outs = []
    start = 0
    for n in lengths:
        if n == 0:
            continue
        qs, ks, vs = (t[start : start + n].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
        o = F.scaled_dot_product_attention(qs, ks, vs, scale=scale)
        outs.append(o.squeeze(0).transpose(0, 1))
        start += n
    if start < q.shape[0]:
        outs.append(torch.zeros_like(q[start:]))
    return torch.cat(outs) if outs else torch.zeros_like(q)


def attention_varlen_math(q, k, v, lengths, scale: float, dtype=torch.float64) -> Tensor:
    """Explicit softmax(QK^T)V per segment in `dtype`: the fp64 oracle of the tests."""
    outs, start = [], 0
    for n in lengths:
        qs, ks, vs = (t[start : start + n].to(dtype).transpose(0, 1) for t in (q, k, v))
        p = torch.softmax(qs @ ks.transpose(1, 2) * scale, -1)
        outs.append((p @ vs).transpose(0, 1))
        start += n
    return torch.cat(outs)


def linear(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    return F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))


def linear_qk_rope(y, wq, wk, q_weight, k_weight, pos, bands, eps, heads):
    q = linear(y, wq).unflatten(-1, (heads, -1))
    k = linear(y, wk).unflatten(-1, (heads, -1))
    return qk_norm_rope(q, k, q_weight, k_weight, pos, bands, eps)


def linear_situ(y, w, bias=None):
    return situ_glu(linear(y, w, bias))


def linear_gated_residual(a, w, bias, x, gate, seg, r: float = 1.0):
    return gated_residual(x, linear(a, w, bias), gate, seg, r)


def timestep_embedding(t: Tensor, freq_dim: int) -> Tensor:
    """t [B] in 0..1000 -> fp32 [B, freq_dim] = [cos | sin](t * 10000^(-k/half))."""
    half = freq_dim // 2
    freq = 10000 ** (-torch.arange(half, device=t.device, dtype=torch.float32) / half)
    phase = t.float()[:, None] * freq
    return torch.cat((phase.cos(), phase.sin()), -1)
