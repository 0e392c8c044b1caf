"""Where device memory went: parameters by dtype, gradients, optimiser state, allocator totals,
and the step's peak windows (`src/kohakumoss/memory/device_use.py`, `kernels/hardware/memory.py`
in the reference)."""

from __future__ import annotations

import torch


def tensor_bytes(tensors) -> int:
    seen, total = set(), 0
    for t in tensors:
        if t is None or not t.is_cuda:
            continue
        key = (t.untyped_storage().data_ptr(), t.untyped_storage().nbytes())
        if key not in seen:
            seen.add(key)
            total += key[1]
    return total


def breakdown(model=None, optimizer=None, device=None) -> dict:
    out = {}
    if model is not None:
        by: dict[str, list] = {}
        for p in list(model.parameters()) + list(model.buffers()):
            by.setdefault(str(p.dtype).replace("torch.", ""), []).append(p)
        out["params"] = {k: tensor_bytes(v) for k, v in by.items()}
        out["grads"] = tensor_bytes(p.grad for p in model.parameters())
    if optimizer is not None:
        out["optim_state"] = tensor_bytes(v for st in optimizer.state.values() for v in st.values() if isinstance(v, torch.Tensor))
    if torch.cuda.is_available():
        out["allocated"] = torch.cuda.memory_allocated(device)
        out["reserved"] = torch.cuda.memory_reserved(device)
        out["peak_allocated"] = torch.cuda.max_memory_allocated(device)
        free, total = torch.cuda.mem_get_info(device)
        out["device_free"], out["device_total"] = free, total
    return out


class PeakWindow:
    """`with PeakWindow() as w: ...; w.peak` = the window's own peak above its start."""

    def __init__(self, device=None):
        self.device, self.peak, self.start = device, 0, 0

    def __enter__(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
            torch.cuda.reset_peak_memory_stats(self.device)
            self.start = torch.cuda.memory_allocated(self.device)
        return self

    def __exit__(self, *exc):
        if torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
            self.peak = torch.cuda.max_memory_allocated(self.device) - self.start
        return False
