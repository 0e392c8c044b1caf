"""Device facts and measured rates.

`arch_of` names the device class; `device_rates` measures what rooflines divide by (a
STREAM-style copy and a bf16 GEMM, CUDA events, best of several) and caches the result per
card in `~/.cache/kmoss_b200/rates-<name>.json`; `time_block_ops` times the block's kernels
at one token count. Role of the reference's `kernels/hardware/{arch,device}.py`.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path


@dataclass(frozen=True)
class Arch:
    name: str
    sm: int
    has_bf16: bool
    has_fp8: bool
    has_tcgen05: bool
    sms: int
    smem_per_block: int
    l2_bytes: int


def arch_of(device="cuda:0") -> Arch:
    import torch

    if not torch.cuda.is_available():
        return Arch("cpu", 0, False, False, False, 0, 0, 0)
    p = torch.cuda.get_device_properties(device)
    sm = p.major * 10 + p.minor
    return Arch(p.name, sm, sm >= 80, sm >= 89, sm == 100, p.multi_processor_count, getattr(p, "shared_memory_per_block_optin", 0),
                getattr(p, "L2_cache_size", 0))


def cache_dir() -> Path:
    root = Path(os.environ.get("KMOSS_CACHE", Path.home() / ".cache" / "kmoss_b200"))
    root.mkdir(parents=True, exist_ok=True)
    return root


def _time(fn, iters: int = 10) -> float:
    import torch

    for _ in range(3):
        fn()
    best = float("inf")
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        best = min(best, s.elapsed_time(e))
    return best


def device_rates(device="cuda:0", refresh: bool = False) -> dict:
    """{"hbm_gbs", "bf16_tflops"} of this card (measured once, cached by device name)."""
    import torch

    name = torch.cuda.get_device_name(device).replace(" ", "_")
    path = cache_dir() / f"rates-{name}.json"
    if path.exists() and not refresh:
        return json.loads(path.read_text())
    n = 1 << 28
    a = torch.empty(n, dtype=torch.bfloat16, device=device)
    b = torch.empty_like(a)
    copy_ms = _time(lambda: b.copy_(a))
    x = torch.randn(8192, 8192, device=device).bfloat16()
    y = torch.randn(8192, 8192, device=device).bfloat16()
    mm_ms = _time(lambda: torch.matmul(x, y))
    out = {"device": name, "hbm_gbs": round(2 * n * 2 / copy_ms / 1e6, 1), "bf16_tflops": round(2 * 8192**3 / mm_ms / 1e9, 1)}
    path.write_text(json.dumps(out))
    return out


def time_block_ops(tokens: int, device="cuda:0", dim: int = 3072, ffn: int = 8192) -> dict:
    """Milliseconds of the joint block's GEMMs at `tokens` rows (bf16 and fp8)."""
    import torch

    from ..ops import native

    out = {"tokens": tokens}
    x = torch.randn(tokens, dim, device=device).bfloat16()
    xq, xs = native.quantize_fp8(x)
    for label, n, k in (("qkv", 3 * dim, dim), ("o", dim, dim), ("up_gate", 2 * ffn, dim), ("down", dim, ffn)):
        a = x if k == dim else torch.randn(tokens, k, device=device).bfloat16()
        w = (torch.randn(n, k, device=device) * 0.02).bfloat16()
        y = torch.empty(tokens, n, device=device, dtype=torch.bfloat16)
        out[f"{label}_bf16_ms"] = round(_time(lambda: native.gemm(a, w, out=y), 5), 4)
        aq, as_ = (xq, xs) if k == dim else native.quantize_fp8(a)
        wq, ws = native.quantize_fp8(w)
        out[f"{label}_fp8_ms"] = round(_time(lambda: native.gemm(aq, wq, out=y, scale_a=as_[:1], scale_b=ws[:1]), 5), 4)
    native.check_status()
    return out
