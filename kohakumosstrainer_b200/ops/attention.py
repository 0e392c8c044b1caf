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


def tile_table(lengths, device, block: int = 128) -> Tensor:
    """int32 [T, 4] = (first row of the tile, segment start, segment end, 0) for every
    `block`-row tile of every segment; built on the host from the plan's lengths."""
    rows, start = [], 0
    for n in lengths:
        for t0 in range(0, n, block):
            rows.append((start + t0, start, start + n, 0))
        start += n
    table = torch.tensor(rows or [(0, 0, 0, 0)], dtype=torch.int32).reshape(-1, 4)[: len(rows)]
    if torch.device(device).type == "cuda":
        return table.pin_memory().to(device, non_blocking=True)
    return table


_TILES: dict[tuple, Tensor] = {}


def _tiles_for(lengths, device) -> Tensor:
    key = (tuple(lengths), str(device))
    t = _TILES.get(key)
    if t is None:
        if len(_TILES) > 256:
            _TILES.clear()
        t = _TILES[key] = tile_table(lengths, device)
    return t


class AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, tiles, scale, plan):
        ops = native.load()
        o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
        ops.attention_fwd(q, k, v, tiles, scale, o, lse)
        ctx.save_for_backward(q, k, v, o, lse, tiles)
        ctx.scale, ctx.plan = scale, plan
        return o

    @staticmethod
    def backward(ctx, do):
        ops = native.load()
        q, k, v, o, lse, tiles = ctx.saved_tensors
        if hasattr(ops._ops, "attention_bwd"):
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            ops.attention_bwd(_dense(do), q, k, v, o, lse, tiles, ctx.scale, dq, dk, dv)
            return dq, dk, dv, None, None, None
        cu, max_len, lengths = ctx.plan
        with torch.enable_grad():
            qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
            out = library_attention(qq, kk, vv, cu, max_len, ctx.scale, lengths)
            dq, dk, dv = torch.autograd.grad(out, (qq, kk, vv), do)
        return dq, dk, dv, None, None, None


class AttentionQkvFn(torch.autograd.Function):
    """Attention on the fused projection output `qkv` [N, 3, H, 128]: forward reads q / k / v as strided views,
    backward lets the dQ and dK/dV kernels write straight into one `d qkv` buffer (no concatenation of three
    gradients afterwards)."""

    @staticmethod
    def forward(ctx, qkv, tiles, scale):
        ops = native.load()
        q, k, v = qkv.unbind(1)
        o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        lse = torch.empty(q.shape[1], q.shape[0], dtype=torch.float32, device=q.device)
        ops.attention_fwd(q, k, v, tiles, scale, o, lse)
        ctx.save_for_backward(qkv, o, lse, tiles)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        ops = native.load()
        qkv, o, lse, tiles = ctx.saved_tensors
        q, k, v = qkv.unbind(1)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv.unbind(1)
        ops.attention_bwd(_dense(do), q, k, v, o, lse, tiles, ctx.scale, dq, dk, dv)
        return dqkv, None, None


def attention_qkv(qkv: Tensor, lengths, scale: float) -> Tensor:
    """`qkv` [N, 3, H, 128] bf16 (contiguous) -> o [N, H, 128]."""
    return AttentionQkvFn.apply(qkv, _tiles_for(tuple(lengths), qkv.device), float(scale))


def _dense(t: Tensor) -> Tensor:
    """[N, H, Dh] with unit inner stride and Dh-contiguous heads (views of a fused qkv
    projection qualify: row stride 3*H*Dh)."""
    ok = t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def attention_varlen(q, k, v, cu_seqlens, max_seqlen, scale, lengths=None) -> Tensor:
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and _native_ready():
        if lengths is None:
            bounds = cu_seqlens.tolist()
            lengths = tuple(b - a for a, b in zip(bounds[:-1], bounds[1:]))
        tiles = _tiles_for(lengths, q.device)
        return AttentionFn.apply(_dense(q), _dense(k), _dense(v), tiles, float(scale), (cu_seqlens, int(max_seqlen), lengths))
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
