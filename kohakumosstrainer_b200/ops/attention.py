"""Packed variable-length attention on CUDA.

`attention_varlen(q, k, v, cu_seqlens, max_seqlen, scale, lengths)` with q, k, v `[N, H, Dh]`
bf16: full (non-causal) attention inside each segment. The sm_100a kernel
(`csrc/attention_sm100.cu`) covers head_dim 128; other shapes use the per-segment library
path, which is also the timed baseline (`src/kohakumoss_kernels/backends/varlen_choice.py`
in the reference picks between its Triton kernel, torch varlen and an SDPA loop the same way).
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import eager, native

_STATE = {"native": None}


def _native_ready() -> bool:
    if _STATE["native"] is None:
        try:
            _STATE["native"] = hasattr(native.load()._ops, "attention_fwd")
        except Exception:
            _STATE["native"] = False
    return _STATE["native"]


class AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu, max_len, scale):
        ops = native.load()
        o = torch.empty_like(q)
        lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
        ops.attention_fwd(q, k, v, cu, max_len, scale, o, lse)
        ctx.save_for_backward(q, k, v, o, lse, cu)
        ctx.max_len, ctx.scale = max_len, scale
        return o

    @staticmethod
    def backward(ctx, do):
        ops = native.load()
        q, k, v, o, lse, cu = ctx.saved_tensors
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ops.attention_bwd(do.contiguous(), q, k, v, o, lse, cu, ctx.max_len, ctx.scale, dq, dk, dv)
        return dq, dk, dv, None, None, None


def _dense(t: Tensor) -> Tensor:
    """[N, H, Dh] with unit inner stride and Dh-contiguous heads (views of a fused qkv
    projection qualify: row stride 3*H*Dh)."""
    return t if t.stride(2) == 1 and t.stride(1) == t.shape[2] else t.contiguous()


def attention_varlen(q, k, v, cu_seqlens, max_seqlen, scale, lengths=None) -> Tensor:
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and _native_ready():
        return AttentionFn.apply(_dense(q), _dense(k), _dense(v), cu_seqlens, int(max_seqlen), float(scale))
    return library_attention(q, k, v, cu_seqlens, max_seqlen, scale, lengths)


def library_attention(q, k, v, cu_seqlens, max_seqlen, scale, lengths=None) -> Tensor:
    """Baseline path: flash-attn varlen when importable, else one SDPA call per segment."""
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        try:
            from flash_attn import flash_attn_varlen_func

            return flash_attn_varlen_func(
                q.contiguous(), k.contiguous(), v.contiguous(), cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                softmax_scale=scale, causal=False,
            )
        except ImportError:
            pass
    return eager.attention_varlen(q, k, v, cu_seqlens, max_seqlen, scale, lengths)
