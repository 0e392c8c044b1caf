"""Python face of the sm_100a kernels: library loading, functional wrappers, autograd.

The extension is built in-tree (`csrc/build.py`) and loaded once. On a CUDA machine a
missing or stale library is an error (never a silent eager fallback): the op set of a CUDA
model is the native one or nothing.
"""

from __future__ import annotations

import threading
from pathlib import Path

import torch
from torch import Tensor

_LOCK = threading.Lock()
_OPS = None

EPI_LINEAR, EPI_SITU, EPI_QK_ROPE = 0, 1, 2
FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


def library_path() -> Path:
    return Path(__file__).resolve().parent.parent / "_C.so"


def load(build_if_missing: bool = True):
    """`torch.ops.kmoss_b200`, loading (and if needed building) the in-tree library."""
    global _OPS
    if _OPS is not None:
        return _OPS
    with _LOCK:
        if _OPS is not None:
            return _OPS
        path = library_path()
        if build_if_missing:
            from ..csrc import build as _build

            if not _build.is_fresh():
                _build.build()
        if not path.exists():
            raise RuntimeError(f"native library {path} is missing; run python -m kohakumosstrainer_b200.csrc.build")
        torch.ops.load_library(str(path))
        _OPS = _CountingOps(torch.ops.kmoss_b200)
    return _OPS


# Kernel launches behind each op (own kernels only), for the launch counter benchmarks report.
_LAUNCHES_PER_OP = {
    "gemm": 1, "rms_norm_mod_fwd": 1, "rms_norm_mod_bwd": 1, "norm_weight_grad": 1, "seg_sum": 2, "rope_table": 1,
    "qk_norm_rope_fwd": 1, "qk_norm_rope_bwd": 1, "situ_fwd": 1, "situ_bwd": 1, "gated_residual": 1, "seg_scale": 1,
    "situ_bwd_quant": 1, "seg_scale_quant": 1,
    "token_mse_fwd": 2, "token_mse_bwd": 1, "quantize_fp8_tensor": 3, "cast_fp8": 1, "quantize_fp8_rows": 1,
    "adamw_multi": 1, "grad_norm_multi": 2, "ema_multi": 1, "attention_fwd": 1, "attention_bwd": 3,
    "allreduce": 1, "reduce_scatter_adamw": 1, "allgather": 1,
}
LAUNCHES = {"count": 0}


class _CountingOps:
    """`torch.ops.kmoss_b200` with a launch counter: `LAUNCHES["count"]` grows by the number
    of this library's kernels each call enqueues (a split-K GEMM counts its reduction too)."""

    def __init__(self, ops):
        self._ops = ops
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._ops, name)
            n = _LAUNCHES_PER_OP.get(name, 0)
            if n == 0:
                fn = raw
            elif name == "gemm":
                def fn(*args, _raw=raw, **kw):
                    LAUNCHES["count"] += 2 if args[28] > 1 else 1  # split-K adds the reduction launch
                    return _raw(*args, **kw)
            else:
                def fn(*args, _raw=raw, _n=n, **kw):
                    LAUNCHES["count"] += _n
                    return _raw(*args, **kw)
            self._cache[name] = fn
        return fn


def available() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10


def check_status() -> None:
    """Raise if any kernel recorded a bounded-wait timeout (synchronises)."""
    st = load().kernel_status().tolist()
    if st[0] != 0:
        raise RuntimeError(f"kernel status: code={st[0]} where={st[1]} block={st[2]} extra={st[3]}")


class _Workspace:
    """Per-device scratch buffers reused across calls (split-K partials and the like)."""

    def __init__(self):
        self.buffers: dict[tuple, Tensor] = {}

    def get(self, device, nbytes: int, tag: str = "ws") -> Tensor:
        key = (device, tag)
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            self.buffers[key] = buf
        return buf


WORKSPACE = _Workspace()


def gemm(
    a: Tensor,
    b: Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    alpha: float = 1.0,
    scale_a: Tensor | None = None,
    scale_b: Tensor | None = None,
    row_scale: Tensor | None = None,
    col_scale: Tensor | None = None,
    bias: Tensor | None = None,
    res: Tensor | None = None,
    beta: float = 1.0,
    gate: Tensor | None = None,
    seg: Tensor | None = None,
    t: Tensor | None = None,
    u: Tensor | None = None,
    epilogue: int = EPI_LINEAR,
    aux: Tensor | None = None,
    q_norm_w: Tensor | None = None,
    k_norm_w: Tensor | None = None,
    rope: Tensor | None = None,
    rope_cols: int = 0,
    eps: float = 1e-6,
    head_rstd: Tensor | None = None,
    splits: int | None = 1,
    gather: dict | None = None,
) -> Tensor:
    """`out = epilogue(A . B^T)` on the tcgen05 GEMM.

    `a` is `[M, K]` (or `[K, M]` with `a_mn`), `b` is `[N, K]` (or `[K, N]` with `b_mn`); with
    `EPI_SITU` `b` holds `2N` rows (up | gate) and `out` is `[M, N]`. `splits=None` picks a
    split-K factor for skinny problems.
    """
    ops = load()
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    if b_mn:
        N = b.shape[1]
    else:
        N = b.shape[0] // 2 if epilogue == EPI_SITU else b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if splits is None:
        splits = ops.gemm_pick_splits(M, N, K, a.element_size()) if epilogue == EPI_LINEAR else 1
    ws = None
    if splits > 1:
        ws = WORKSPACE.get(a.device, splits * M * N * 4, "splitk")
    ops.gemm(
        a, b, M, N, K, a_mn, b_mn, out, alpha, scale_a, scale_b, row_scale, col_scale, bias, res, beta,
        gate, seg, t, u, epilogue, aux, q_norm_w, k_norm_w, rope, rope_cols, eps, head_rstd, splits, ws,
        None, **(gather or {}),
    )
    return out


def quantize_fp8(x: Tensor, dtype: torch.dtype = torch.float8_e4m3fn) -> tuple[Tensor, Tensor]:
    """Per-tensor dynamic quantisation of a bf16 tensor -> (q, scale[2] = {dequant, quant})."""
    return load().quantize_fp8_tensor(x.contiguous(), dtype == torch.float8_e5m2)


def quantize_fp8_rows(x: Tensor, dtype: torch.dtype = torch.float8_e4m3fn, both: bool = False) -> tuple[Tensor, Tensor]:
    """Per-row dynamic quantisation in one pass -> (q, scales): fp32 `[rows]` dequant scales, or
    `[2, rows]` = {dequant, quant} with `both`."""
    return load().quantize_fp8_rows(x, dtype == torch.float8_e5m2, both)


def rope_table(pos: Tensor, bands: Tensor) -> Tensor:
    """[N, 128] fp32 = cos | sin of pos[n, axis] * bands[band]; built once per batch and
    shared by every block (positions do not change across the 42 blocks)."""
    return load().rope_table(pos.contiguous(), bands.contiguous())
