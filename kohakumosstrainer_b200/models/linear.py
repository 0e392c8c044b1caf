"""MossLinear: an `nn.Linear` whose base-weight storage and adapter are swappable.

State-dict names stay `weight` / `bias`, so HF and ComfyUI checkpoints load unchanged
(reference: `src/kohakumoss/model/linear.py:15-126`). Three things can be attached, each
resolved once by `rebind()` instead of per call:

* `base`   - a stored (frozen) weight in another format: fp8 per-tensor / row scaled,
             MXFP8 block-scaled, int8 / fp8 weight-only (`quant.weights`);
* `compute`- an fp8 / MXFP8 compute cache of the *trainable* dense weight (`quant.compute`);
* `adapter`- a LyCORIS-style adapter module (`adapters.modules`) applied as a bypass
             (`y = base(x) + adapter(x)`) or merged (`y = x (W + dW)^T`).

On CUDA the forward is one fused op (`ops.native.fused_linear`) that runs the base GEMM,
the adapter bypass and the epilogue in a single tcgen05 kernel where the shapes allow.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor, nn


class MossLinear(nn.Linear):
    def __init__(self, in_features, out_features, bias=True, device=None, dtype=None):
        super().__init__(in_features, out_features, bias, device=device, dtype=dtype)
        self.__dict__["base"] = None
        self.__dict__["compute"] = None
        self.__dict__["adapter"] = None
        self.__dict__["adapter_mode"] = "bypass"
        self.__dict__["native"] = True

    def reset_parameters(self) -> None:  # weights come from the builder or a checkpoint
        pass

    def init_weights(self, std: float = 0.02) -> None:
        nn.init.normal_(self.weight, std=std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    # -- structural changes -------------------------------------------------------------
    def set_base(self, base) -> None:
        """Attach stored weight storage (or None for the dense parameter)."""
        self.__dict__["base"] = base

    def set_compute(self, cache) -> None:
        self.__dict__["compute"] = cache

    def set_adapter(self, adapter, mode: str = "bypass") -> None:
        if mode not in ("bypass", "merge"):
            raise ValueError(f"adapter mode must be bypass|merge, got {mode}")
        self.__dict__["adapter"] = adapter
        self.__dict__["adapter_mode"] = mode

    def drop_weight(self) -> None:
        """Free the dense parameter after a stored base took over (keeps dtype/device)."""
        w = self._parameters.get("weight")
        if w is not None:
            self.__dict__["_held"] = torch.empty(0, dtype=w.dtype, device=w.device)
            del self._parameters["weight"]

    @property
    def weight_like(self) -> Tensor:
        w = self._parameters.get("weight")
        return w if w is not None else self.__dict__["_held"]

    @property
    def is_plain(self) -> bool:
        return self.base is None and self.compute is None and self.adapter is None

    def _apply(self, fn, recurse=True):
        held = self.__dict__.get("_held")
        if held is not None:
            self.__dict__["_held"] = fn(held)
        base = self.__dict__.get("base")
        if base is not None and hasattr(base, "_apply"):
            base._apply(fn)
        return super()._apply(fn, recurse)

    # -- math -----------------------------------------------------------------------------
    def base_weight(self, dtype: torch.dtype) -> Tensor:
        """The (dequantised) base weight in `dtype`."""
        if self.base is not None:
            return self.base.weight(dtype)
        return self.weight.to(dtype)

    def effective_weight(self, dtype: torch.dtype) -> Tensor:
        """Base weight plus the merged adapter delta."""
        w = self.base_weight(dtype)
        if self.adapter is not None:
            w = self.adapter.merged(w)
        return w

    def forward(self, x: Tensor) -> Tensor:
        if x.is_cuda and self.native:
            from ..ops import native_ops

            return native_ops.fused_linear(self, x)
        return self.forward_eager(x)

    def forward_eager(self, x: Tensor) -> Tensor:
        bias = None if self.bias is None else self.bias.to(x.dtype)
        adapter = self.adapter
        if adapter is not None and self.adapter_mode == "merge":
            return F.linear(x, adapter.merged(self.base_weight(x.dtype)).to(x.dtype), bias)
        if self.base is not None:
            y = self.base.linear(x, bias)
        elif self.compute is not None:
            y = self.compute.linear(x, self.weight, bias)
        else:
            y = F.linear(x, self.weight.to(x.dtype), bias)
        if adapter is not None:
            y = adapter.bypass(x, y, self)
        return y
