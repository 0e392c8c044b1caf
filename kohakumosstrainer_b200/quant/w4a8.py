"""W4A8 base weights (ComfyUI `asym_w4a8_int8`): 4- or 6-bit codes over an int8 grid.

Stored per layer (`src/kohakumoss/quant/w4a8.py:1-75` describes the layout): `weight` int8
`[N, K * bits / 8]` packed codes (the K/2-byte nibble plane, even column = low nibble; at 6 bits
a K/4-byte plane of each code's top two bits follows), `weight_s_rel` e4m3 `[N, K / group]`
group scales, `weight_s_channel` fp32 `[N]`, optionally `weight_codebook` (2^bits levels; the
uniform grid `code - 2^(bits-1)` without it) and `weight_correction` `[K / group, N]`. The int8
grid is `round(level * s_rel)` clamped to +-127, the weight is `grid * s_channel (+ correction)`,
stored rotated by the ConvRot group when the record says so.

On a 180 GB card nothing is gained by decoding per call: a layer is decoded ONCE at load into the
int8 weight-only format (`Int8Weight`, 1 byte per weight, the int8 tcgen05 GEMM or the exact
int8 -> bf16 widening), or into a dense weight when it carries a correction term.
`quantize_w4a8` writes the format (uniform grid) for files that must stay small on disk.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .formats import Int8Weight, hadamard_matrix

BITS = (4, 6)
E4M3 = torch.float8_e4m3fn


def geometry(q: Tensor, s_rel: Tensor, group: int) -> tuple[int, int, int]:
    n, cols = q.shape
    k = s_rel.shape[1] * group
    bits = (cols * 8) // k if k else 0
    if bits not in BITS or k * bits != cols * 8 or tuple(s_rel.shape) != (n, k // group):
        raise ValueError(f"W4A8 codes {tuple(q.shape)} with group scales {tuple(s_rel.shape)} and group {group} are not a 4- or 6-bit layout")
    return n, k, bits


def unpack_codes(q: Tensor, k: int, bits: int) -> Tensor:
    n = q.shape[0]
    packed = q.view(torch.uint8).to(torch.int32)
    low = packed[:, : k // 2]
    codes = torch.stack((low & 0xF, (low >> 4) & 0xF), dim=-1).reshape(n, k)
    if bits == 6:
        shifts = torch.arange(0, 8, 2, device=q.device, dtype=torch.int32)
        high = (packed[:, k // 2:].unsqueeze(-1) >> shifts) & 0x3
        codes = codes | (high.reshape(n, k) << 4)
    return codes


def pack_codes(codes: Tensor, bits: int) -> Tensor:
    n, k = codes.shape
    c = codes.to(torch.int32)
    low = (c[:, 0::2] & 0xF) | ((c[:, 1::2] & 0xF) << 4)
    planes = [low]
    if bits == 6:
        top = (c >> 4) & 0x3
        planes.append(top[:, 0::4] | (top[:, 1::4] << 2) | (top[:, 2::4] << 4) | (top[:, 3::4] << 6))
    return torch.cat(planes, 1).to(torch.uint8).view(torch.int8)


def decode_codes(q: Tensor, s_rel: Tensor, codebook: Tensor | None, group: int, bits: int) -> Tensor:
    """The int8 grid [N, K]."""
    n = q.shape[0]
    k = s_rel.shape[1] * group
    codes = unpack_codes(q, k, bits)
    levels = codebook.float()[codes.long()] if codebook is not None else (codes - (1 << (bits - 1))).float()
    values = levels.view(n, k // group, group) * s_rel.float().unsqueeze(-1)
    return values.view(n, k).round().clamp_(-127, 127).to(torch.int8)


def load_layer(path: str, sd: dict[str, Tensor], group: int, rotation: int = 0, int8_compute: bool = False, dtype=torch.bfloat16):
    """One stored layer -> `Int8Weight` (decoded once), or a dense `dtype` weight when the layer has a correction term."""
    q, s_rel, s_ch = sd[f"{path}.weight"], sd[f"{path}.weight_s_rel"], sd[f"{path}.weight_s_channel"].float().reshape(-1)
    codebook, correction = sd.get(f"{path}.weight_codebook"), sd.get(f"{path}.weight_correction")
    n, k, bits = geometry(q, s_rel, group)
    grid = decode_codes(q, s_rel, codebook, group, bits)
    if correction is None:
        return Int8Weight(grid.contiguous(), s_ch, rotation, int8_compute)
    if tuple(correction.shape) != (k // group, n):
        raise ValueError(f"{path}: W4A8 correction {tuple(correction.shape)} is not {(k // group, n)}")
    w = grid.float().view(n, k // group, group) * s_ch.view(-1, 1, 1) + correction.t().float().unsqueeze(-1)
    w = w.view(n, k)
    if rotation > 1:
        w = (w.reshape(-1, rotation) @ hadamard_matrix(rotation, torch.float32, w.device)).reshape(n, k)
    return w.to(dtype)


def quantize_w4a8(w: Tensor, group: int = 64, bits: int = 4, rotation: int = 0) -> dict[str, Tensor]:
    """Dense weight -> the stored tensors (uniform grid, no codebook, no correction)."""
    if bits not in BITS or w.shape[1] % group or (rotation and w.shape[1] % rotation):
        raise ValueError("W4A8 needs bits in (4, 6) and K a multiple of the group (and of the rotation group)")
    n, k = w.shape
    wf = w.float()
    if rotation > 1:
        wf = (wf.reshape(-1, rotation) @ hadamard_matrix(rotation, torch.float32, w.device)).reshape(n, k)
    s_ch = (wf.abs().amax(1).clamp_min(1e-12) / 127.0)
    grid = wf / s_ch[:, None]                                     # the int8-range target
    half = 1 << (bits - 1)
    g = grid.view(n, k // group, group)
    s_rel = (g.abs().amax(-1).clamp_min(1e-6) / (half - 1)).to(E4M3)   # level * s_rel spans the group
    levels = (g / s_rel.float().clamp_min(2.0**-9).unsqueeze(-1)).round().clamp_(-half, half - 1)
    codes = (levels + half).to(torch.int32).view(n, k)
    return {"weight": pack_codes(codes, bits), "weight_s_rel": s_rel, "weight_s_channel": s_ch}
