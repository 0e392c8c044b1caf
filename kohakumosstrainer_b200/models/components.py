"""Small building blocks: RMSNorm weight holder, timestep MLP, RoPE frequency bands.

Key names (`0.*`, `2.*`, `bands`) follow the official state dict
(`src/kohakumoss/model/components/embed.py:9-60`, `components/norm.py`).
"""

from __future__ import annotations

import torch
from torch import Tensor, nn

from .linear import MossLinear


class RMSNorm(nn.Module):
    """Learned per-channel weight plus `eps`; the math runs in the op set."""

    def __init__(self, dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.eps = eps

    def init_weights(self) -> None:
        nn.init.ones_(self.weight)

    def extra_repr(self) -> str:
        return f"{self.weight.shape[0]}, eps={self.eps:g}"


class TimeEmbedding(nn.Sequential):
    """Linear(freq_dim, dim) -> SiLU -> Linear(dim, dim)."""

    def __init__(self, freq_dim: int, dim: int, device=None, dtype=None):
        super().__init__(
            MossLinear(freq_dim, dim, device=device, dtype=dtype),
            nn.SiLU(),
            MossLinear(dim, dim, device=device, dtype=dtype),
        )


def default_bands(n_bands: int, base: float, device=None) -> Tensor:
    exponent = torch.arange(n_bands, dtype=torch.float32) / n_bands
    return (1 / (base**exponent)).to(device)


class RopeBands(nn.Module):
    """fp32 `bands` buffer; dtype casts of the module never touch it."""

    def __init__(self, n_bands: int, base: float, device=None):
        super().__init__()
        self.n_bands, self.base = n_bands, base
        device = None if str(device) == "meta" else device
        self.register_buffer("bands", default_bands(n_bands, base, device))

    def _apply(self, fn, recurse=True):
        super()._apply(fn, recurse=recurse)
        device = self.bands.device
        self.bands = default_bands(self.n_bands, self.base, None if device.type == "meta" else device)
        return self

    def _load_from_state_dict(self, state_dict, prefix, *_args, **_kwargs):
        # `bands` is derived: files may or may not carry it, and it is never read from one.
        state_dict.pop(prefix + "bands", None)
        self.bands = default_bands(self.n_bands, self.base, self.bands.device)
