"""Error statistics of an op against a float64 reference (`src/kohakumoss_kernels/error_stats.py:15-62`
there): what numerics tests and probes report instead of a bare allclose."""

from __future__ import annotations

import torch
from torch import Tensor


def error_stats(got: Tensor, ref: Tensor) -> dict:
    """max / mean absolute error, relative L2 error, max error in units of the reference's RMS, and the worst ulp
    distance in `got`'s dtype."""
    g, r = got.detach().double().flatten(), ref.detach().double().flatten()
    diff = (g - r).abs()
    rms = r.square().mean().sqrt().clamp_min(1e-300)
    eps = torch.finfo(got.dtype).eps if got.dtype.is_floating_point else 1.0
    ulp = diff / (r.abs().clamp_min(float(rms) * 1e-3) * eps)
    return {"max_abs": float(diff.max()), "mean_abs": float(diff.mean()), "rel_l2": float(diff.norm() / r.norm().clamp_min(1e-300)),
            "max_over_rms": float(diff.max() / rms), "max_ulp": float(ulp.max()), "nonfinite": int((~torch.isfinite(g)).sum())}


def compare(fn, ref_fn, *inputs) -> dict:
    """`fn(*inputs)` against `ref_fn` run on float64 CPU copies of the inputs."""
    ref_in = [t.detach().double().cpu() if isinstance(t, Tensor) and t.is_floating_point() else (t.cpu() if isinstance(t, Tensor) else t) for t in inputs]
    return error_stats(fn(*inputs).cpu(), ref_fn(*ref_in))
