"""Text-encoder ops (Qwen3.5: gated-DeltaNet layers + causal GQA attention), forward only.

Op names and semantics follow the reference table (`src/kohakumoss_kernels/ops.py:37-49`, eager
forms in `backends/eager/textenc.py:34-191`):

* `causal_conv_varlen(x[N, C], weight[C, W], cu)`: `silu(sum_j weight[:, W-1-j] * x[t-j])` over
  the taps inside the token's own segment;
* `rms_norm_gated(x, z, weight, eps)`: `x / rms(x) * weight * silu(z)`;
* `attention_varlen_causal(q[N, H, Dh], k[N, Hkv, Dh], v, cu, max_len, scale)`: causal attention
  inside each segment, query head h reading kv head `h // (H / Hkv)`;
* `gated_delta_rule_varlen(q[N, Hk, Dk], k, v[N, Hv, Dv], a[N, Hv], b[N, Hv], a_log[Hv],
  dt_bias[Hv], cu, max_len)`: per segment and value head, with `g = -exp(a_log) softplus(a +
  dt_bias)`, `beta = sigmoid(b)`, L2-normalised q / k and q scaled by Dk^-0.5:
  `S_t = e^g S_(t-1) + k_t (beta (v_t - e^g S_(t-1)^T k_t))^T`, `o_t = S_t^T q_t`.

The text encoder runs once per caption and its outputs are cached by the data layer, so these
stay PyTorch ops (the scan is vectorised over segments and heads: one step per token position,
not per token); attention uses the library kernel.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

L2_EPS = 1e-6


def segment_positions(cu: Tensor, n: int) -> tuple[Tensor, Tensor]:
    """(segment id, position inside the segment) per token."""
    idx = torch.arange(n, device=cu.device)
    seg = torch.searchsorted(cu[1:].to(torch.int64), idx, right=True)
    return seg, idx - cu.to(torch.int64).index_select(0, seg)


def causal_conv_varlen(x: Tensor, weight: Tensor, cu_seqlens: Tensor) -> Tensor:
    n, width = x.shape[0], weight.shape[1]
    xf, w = x.float(), weight.float()
    _, pos = segment_positions(cu_seqlens, n)
    out = xf * w[:, width - 1]
    for j in range(1, width):
        shifted = F.pad(xf, (0, 0, j, 0))[:n]
        out = out + torch.where((pos >= j).unsqueeze(1), shifted, torch.zeros_like(shifted)) * w[:, width - 1 - j]
    return F.silu(out).to(x.dtype)


def rms_norm_gated(x: Tensor, z: Tensor, weight: Tensor, eps: float) -> Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    return (y * weight.float() * F.silu(z.float())).to(x.dtype)


def attention_varlen_causal(q: Tensor, k: Tensor, v: Tensor, cu_seqlens: Tensor, max_seqlen: int, scale: float) -> Tensor:
    groups = q.shape[1] // k.shape[1]
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        try:
            from flash_attn import flash_attn_varlen_func

            cu = cu_seqlens.to(torch.int32)
            return flash_attn_varlen_func(q.contiguous(), k.contiguous(), v.contiguous(), cu, cu, int(max_seqlen), int(max_seqlen),
                                          softmax_scale=scale, causal=True)
        except ImportError:
            pass
    out = torch.empty_like(q)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e == s:
            continue
        qs, ks, vs = (t[s:e].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
        o = F.scaled_dot_product_attention(qs, ks.repeat_interleave(groups, 1), vs.repeat_interleave(groups, 1), is_causal=True, scale=scale)
        out[s:e] = o.squeeze(0).transpose(0, 1)
    return out


def gated_delta_rule_varlen(q: Tensor, k: Tensor, v: Tensor, a: Tensor, b: Tensor, a_log: Tensor, dt_bias: Tensor, cu_seqlens: Tensor,
                            max_seqlen: int) -> Tensor:
    n, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    groups = hv // hk
    g = -a_log.float().exp() * F.softplus(a.float() + dt_bias.float())          # [N, Hv] log decay
    beta = torch.sigmoid(b.float())
    qf = q.float().repeat_interleave(groups, 1)
    kf = k.float().repeat_interleave(groups, 1)
    qf = qf * torch.rsqrt(qf.square().sum(-1, keepdim=True) + L2_EPS) * dk**-0.5
    kf = kf * torch.rsqrt(kf.square().sum(-1, keepdim=True) + L2_EPS)
    seg, pos = segment_positions(cu_seqlens, n)
    nseg = cu_seqlens.shape[0] - 1
    length = int(max_seqlen)

    def pad(t: Tensor) -> Tensor:      # [N, ...] -> [B, L, ...], zeros past each segment
        out = t.new_zeros((nseg, length) + tuple(t.shape[1:]))
        out[seg, pos] = t
        return out

    qp, kp, vp, gp, bp = pad(qf), pad(kf), pad(v.float()), pad(g), pad(beta)
    state = qf.new_zeros(nseg, hv, dk, dv)
    outs = []
    for t in range(length):            # one step per position, all segments and heads at once
        decay = gp[:, t].exp()[..., None, None]
        state = state * decay
        kt, vt = kp[:, t], vp[:, t]                                             # [B, Hv, Dk], [B, Hv, Dv]
        pred = torch.einsum("bhkv,bhk->bhv", state, kt)
        delta = bp[:, t][..., None] * (vt - pred)
        state = state + torch.einsum("bhk,bhv->bhkv", kt, delta)
        outs.append(torch.einsum("bhkv,bhk->bhv", state, qp[:, t]))
    out = torch.stack(outs, 1)                                                  # [B, L, Hv, Dv]
    return out[seg, pos].to(v.dtype)
