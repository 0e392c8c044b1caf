"""AdamW as one multi-tensor CUDA launch (fp32 states, optional fp32 masters, fused EMA).

Semantics of the reference AdamW (`src/kohakumoss_kernels/optim/reference.py:13-131`,
defaults `scripts/train/moss.py:137-151`): decoupled weight decay, bias-corrected moments,
decay-to-one for the norm weights the `moss` rule marks. On CUDA the step is
`csrc/optim.cu::adamw_multi`: the descriptor table is built once (addresses are stable), the
clip coefficient and the skip flag stay on the device, so `step()` never synchronises. On CPU
the same math runs in plain torch (the test oracle).
"""

from __future__ import annotations

import struct

import torch
from torch import Tensor

_DT = {torch.float32: 0, torch.bfloat16: 1}


class ParamTable:
    """Device table of `OptTensor` records plus the chunk map for a list of tensors."""

    def __init__(self, entries: list[dict], device):
        from ..ops import native

        ops = native.load()
        chunk = ops.opt_chunk_elems()
        rec = bytearray()
        chunks = []
        for ti, e in enumerate(entries):
            p, g = e["param"], e["grad"]
            rec += struct.pack(
                "<7q2f4i", p.data_ptr(), g.data_ptr(), e["m"].data_ptr() if e.get("m") is not None else 0,
                e["v"].data_ptr() if e.get("v") is not None else 0,
                e["master"].data_ptr() if e.get("master") is not None else 0,
                e["ema"].data_ptr() if e.get("ema") is not None else 0,
                p.numel(), float(e.get("lr_mul", 1.0)), float(e.get("wd", 0.0)), _DT[p.dtype], _DT[g.dtype],
                int(bool(e.get("decay_to_one", False))), 0,
            )
            for c in range((p.numel() + chunk - 1) // chunk):
                chunks.append((ti, c))
        assert len(rec) == ops.opt_record_bytes() * len(entries)
        self.table = torch.frombuffer(bytes(rec) or b"\0", dtype=torch.uint8).clone().to(device)
        self.chunks = torch.tensor(chunks or [(0, 0)], dtype=torch.int32).reshape(-1, 2)[: len(chunks)].to(device)
        self.keys = tuple((e["param"].data_ptr(), e["grad"].data_ptr()) for e in entries)


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, master_weights: bool = False):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, lr_mul=1.0, decay_to_one=False)
        super().__init__(params, defaults)
        self.master_weights = master_weights
        self.ema_buffers: dict[int, Tensor] = {}
        self.ema_decay = 1.0
        self._tables: dict[int, ParamTable] = {}
        self._steps = 0

    # -- EMA fused into the step -----------------------------------------------------------
    def attach_ema(self, buffers: dict[int, Tensor]) -> None:
        """`buffers[id(param)]` fp32 EMA copies updated inside the step kernel."""
        self.ema_buffers = buffers
        self._tables.clear()

    def _state(self, p: Tensor) -> dict:
        st = self.state[p]
        if not st:
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
            if self.master_weights and p.dtype != torch.float32:
                st["master"] = p.detach().float().clone()
        return st

    def _entries(self, group) -> list[dict]:
        out = []
        for p in group["params"]:
            if p.grad is None:
                continue
            st = self._state(p)
            out.append(dict(param=p.data, grad=p.grad, m=st["exp_avg"], v=st["exp_avg_sq"], master=st.get("master"),
                            ema=self.ema_buffers.get(id(p)), lr_mul=group.get("lr_mul", 1.0), wd=group["weight_decay"],
                            decay_to_one=group.get("decay_to_one", False)))
        return out

    @torch.no_grad()
    def step(self, closure=None, grad_scale: Tensor | None = None, skip: Tensor | None = None):
        self._steps += 1
        for gi, group in enumerate(self.param_groups):
            entries = self._entries(group)
            if not entries:
                continue
            b1, b2 = group["betas"]
            if entries[0]["param"].is_cuda:
                from ..ops import native

                keys = tuple((e["param"].data_ptr(), e["grad"].data_ptr()) for e in entries)
                table = self._tables.get(gi)
                if table is None or table.keys != keys:
                    table = ParamTable(entries, entries[0]["param"].device)
                    self._tables[gi] = table
                native.load().adamw_multi(table.table, table.chunks, group["lr"], b1, b2, group["eps"], self._steps,
                                          self.ema_decay, grad_scale, skip)
            else:
                self._reference_step(entries, group, grad_scale, skip)

    def _reference_step(self, entries, group, grad_scale, skip) -> None:
        if skip is not None and int(skip) != 0:
            return
        b1, b2 = group["betas"]
        bc1 = 1 - b1**self._steps
        bc2 = 1 - b2**self._steps
        gs = 1.0 if grad_scale is None else float(grad_scale)
        for e in entries:
            g = e["grad"].float() * gs
            p = e["master"] if e["master"] is not None else e["param"].float()
            lr = group["lr"] * e["lr_mul"]
            e["m"].mul_(b1).add_(g, alpha=1 - b1)
            e["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
            denom = e["v"].sqrt() / bc2**0.5 + group["eps"]
            decay = 1 - lr * e["wd"]
            p = 1 + (p - 1) * decay if e["decay_to_one"] else p * decay
            p = p - lr / bc1 * e["m"] / denom
            if e["master"] is not None:
                e["master"].copy_(p)
            e["param"].copy_(p.to(e["param"].dtype))
            if e["ema"] is not None:
                e["ema"].add_((p - e["ema"]) * (1 - self.ema_decay))

    def state_dict(self):
        sd = super().state_dict()
        sd["kmoss_steps"] = self._steps
        return sd

    def load_state_dict(self, sd):
        sd = dict(sd)
        self._steps = sd.pop("kmoss_steps", 0)
        super().load_state_dict(sd)
        self._tables.clear()
