"""Host memory shared by the ranks of one node, and the AdamW that steps out of it.

Under DDP every rank of a node holds the same weights, so host-resident fp32 masters need to
exist once per node, not once per rank. `SharedHostRegion` is one `/dev/shm` file that the
first rank of the group creates and every rank maps (then it is unlinked, so it disappears with
the last process); `take(shape, dtype)` hands out aligned views in call order, which is the same
on every rank. With a GPU the mapping is page-locked (`cudaHostRegister`) so copies from it are
asynchronous. Role of `src/kohakumoss/offload/weights/shared.py:18-87`.

`SharedHostAdamW` puts the fp32 masters and the compute-dtype staging copy in the region and
splits the optimiser work ZeRO-1 style: rank r owns the r-th contiguous slice of the flat
parameter space, keeps the two moments of that slice only (private host memory), fetches only
that slice of the (already all-reduced) gradients from its device, updates its slice of the
shared masters, and after one barrier every rank uploads the whole staging copy to its own
device. Per node this is 4 + 2 shared bytes and 8 split bytes per parameter instead of 14 per rank,
and each rank moves 1 / world of the gradient bytes over PCIe.
"""

from __future__ import annotations

import math
import os
import uuid

import torch
import torch.distributed as dist
from torch import Tensor

ALIGN = 64
SHM_DIR = "/dev/shm"


def aligned(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def slice_bounds(total: int, world: int, rank: int, grain: int = 1024) -> tuple[int, int]:
    """The contiguous slice of `total` elements rank `rank` owns; multiples of `grain` except at the end."""
    per = aligned_up(math.ceil(total / world), grain)
    lo = min(total, rank * per)
    return lo, min(total, lo + per)


def aligned_up(n: int, grain: int) -> int:
    return (n + grain - 1) // grain * grain


class SharedHostRegion:
    def __init__(self, nbytes: int, pin: bool = False, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nbytes = max(int(nbytes), ALIGN)
        first = self.rank == 0
        name = [f"kmoss-{uuid.uuid4().hex}" if first else None]
        if self.world > 1:
            dist.broadcast_object_list(name, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        path = os.path.join(SHM_DIR if os.path.isdir(SHM_DIR) else "/tmp", name[0])
        if first:
            with open(path, "wb") as f:
                f.truncate(self.nbytes)
        self._barrier()
        self.buf = torch.from_file(path, shared=True, size=self.nbytes, dtype=torch.uint8)
        self._barrier()
        if first:
            os.unlink(path)      # the mapping keeps the memory alive; nothing is left behind when the ranks exit
        self.pinned = bool(pin) and self._register()
        self.offset = 0

    def _barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)

    def _register(self) -> bool:
        if not torch.cuda.is_available():
            return False
        rt = torch.cuda.cudart()
        return rt.cudaHostRegister(self.buf.data_ptr(), self.nbytes, 0) == rt.cudaError.success

    def take(self, shape, dtype: torch.dtype) -> Tensor:
        n = math.prod(shape) * dtype.itemsize
        start = self.offset
        if start + n > self.nbytes:
            raise ValueError(f"shared host region of {self.nbytes} B is full")
        self.offset = aligned(start + n)
        return self.buf[start : start + n].view(dtype).view(shape)

    def ready(self) -> None:
        """Every rank: what the others wrote into the region is in place."""
        self._barrier()

    def close(self) -> None:
        if self.pinned:
            torch.cuda.cudart().cudaHostUnregister(self.buf.data_ptr())
            self.pinned = False


class SharedHostAdamW(torch.optim.Optimizer):
    """AdamW over node-shared host masters; call `step` on every rank with equal (reduced) gradients."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01, group=None, pinned: bool = True):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, lr_mul=1.0))
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.flat_params = [[p for p in g["params"] if p.requires_grad] for g in self.param_groups]
        sizes = [sum(p.numel() for p in ps) for ps in self.flat_params]
        dtypes = [ps[0].dtype if ps else torch.float32 for ps in self.flat_params]
        need = sum(aligned(n * 4) + aligned(n * dt.itemsize) for n, dt in zip(sizes, dtypes))
        self.region = SharedHostRegion(need, pin=pinned, group=group)
        self.master, self.out, self.m, self.v, self.grad, self.bounds, self.spans = [], [], [], [], [], [], []
        for ps, n, dt in zip(self.flat_params, sizes, dtypes):
            master, out = self.region.take((n,), torch.float32), self.region.take((n,), dt)
            lo, hi = slice_bounds(n, self.world, self.rank)
            spans, off = [], 0
            for p in ps:
                spans.append((off, p.numel()))
                off += p.numel()
            if self.rank == 0:
                for p, (o, k) in zip(ps, spans):
                    master[o : o + k].copy_(p.detach().reshape(-1).float())
            pin = pinned and torch.cuda.is_available()
            mk = lambda: torch.zeros(hi - lo, dtype=torch.float32, pin_memory=pin)  # noqa: E731
            self.master.append(master)
            self.out.append(out)
            self.m.append(mk())
            self.v.append(mk())
            self.grad.append(mk())
            self.bounds.append((lo, hi))
            self.spans.append(spans)
        self.region.ready()
        self.steps = 0
        self.bytes_d2h = self.bytes_h2d = 0

    @torch.no_grad()
    def step(self, closure=None, grad_scale: Tensor | float | None = None, skip=None):
        if skip is not None and bool(skip):
            return None
        scale = float(grad_scale) if grad_scale is not None else 1.0
        self.steps += 1
        for gi, group in enumerate(self.param_groups):
            lo, hi = self.bounds[gi]
            g = self.grad[gi]
            for p, (off, n) in zip(self.flat_params[gi], self.spans[gi]):  # only the owned slice leaves the device
                a, b = max(lo, off), min(hi, off + n)
                if a >= b:
                    continue
                dst = g[a - lo : b - lo]
                if p.grad is None:
                    dst.zero_()
                else:
                    dst.copy_(p.grad.reshape(-1)[a - off : b - off], non_blocking=True)
                    self.bytes_d2h += (b - a) * p.grad.element_size()
            if torch.cuda.is_available():
                torch.cuda.current_stream().synchronize()
            if hi > lo:
                b1, b2 = group["betas"]
                lr = group["lr"] * group.get("lr_mul", 1.0)
                if scale != 1.0:
                    g.mul_(scale)
                m, v, master = self.m[gi], self.v[gi], self.master[gi][lo:hi]
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                c1, c2 = 1 - b1**self.steps, 1 - b2**self.steps
                denom = v.sqrt().div_(math.sqrt(c2)).add_(group["eps"])
                if group["weight_decay"]:
                    master.mul_(1 - lr * group["weight_decay"])
                master.addcdiv_(m, denom, value=-lr / c1)
                self.out[gi][lo:hi].copy_(master)
        self.region.ready()   # every slice of the staging copy is written
        for gi in range(len(self.param_groups)):
            for p, (off, n) in zip(self.flat_params[gi], self.spans[gi]):
                p.copy_(self.out[gi][off : off + n].view_as(p), non_blocking=True)
                self.bytes_h2d += n * p.element_size()
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        self.region.ready()   # nobody overwrites the staging copy while a rank still uploads it
        return None

    def state_dict(self):
        return {"steps": self.steps, "bounds": list(self.bounds), "m": [t.clone() for t in self.m], "v": [t.clone() for t in self.v],
                "master": [t.clone() for t in self.master] if self.rank == 0 else None,
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, state):
        self.steps = int(state["steps"])
        for gi in range(len(self.param_groups)):
            if tuple(state["bounds"][gi]) != tuple(self.bounds[gi]):
                raise ValueError("shared host optimiser state was saved with another world size")
            self.m[gi].copy_(state["m"][gi])
            self.v[gi].copy_(state["v"][gi])
            if self.rank == 0 and state.get("master") is not None:
                self.master[gi].copy_(state["master"][gi])
        for g, saved in zip(self.param_groups, state["param_groups"]):
            g.update(saved)
        self.region.ready()
