"""Bench the LoRA bypass accumulated into the base GEMM's tensor-memory accumulator against the
separate product and add (`base + (x A^T) B^T * s` as three launches), forward and forward +
backward, at a MOSS layer shape (role of `scripts/bench/adapters/fold_base.py`). Needs a GPU.

    python scripts/bench/adapters/fold_base.py [--tokens 20480] [--inp 3072] [--out-features 9216] [--rank 8]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "kernel"))
from case import run  # noqa: E402

from kohakumosstrainer_b200.ops import native  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=20480)
    ap.add_argument("--inp", type=int, default=3072)
    ap.add_argument("--out-features", type=int, default=9216)
    ap.add_argument("--rank", type=int, default=8)
    ap.add_argument("--iters", type=int, default=7)
    args = ap.parse_args()
    M, K, N, R = args.tokens, args.inp, args.out_features, args.rank
    g = torch.Generator("cuda").manual_seed(0)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).bfloat16()
    down = (torch.randn(R, K, device="cuda", generator=g) * 0.02).bfloat16()
    up = (torch.randn(N, R, device="cuda", generator=g) * 0.02).bfloat16()
    d = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    scale = torch.full((R,), 1.0, device="cuda")

    def fused_fwd():
        t = native.gemm(x, down, col_scale=scale, splits=None)
        return native.gemm(x, w, t=t, u=up)

    def split_fwd():
        t = native.gemm(x, down, col_scale=scale, splits=None)
        return native.gemm(x, w) + native.gemm(t, up)

    def fused_bwd():
        t2 = native.gemm(d, up, b_mn=True, col_scale=scale, splits=None)
        return native.gemm(d, w, b_mn=True, t=t2, u=down.t().contiguous())

    def split_bwd():
        t2 = native.gemm(d, up, b_mn=True, col_scale=scale, splits=None)
        return native.gemm(d, w, b_mn=True) + native.gemm(t2, down, b_mn=True)

    err = float((fused_fwd().float() - split_fwd().float()).abs().max())
    rows = {"shape": [M, K, N, R], "max_abs_diff_fused_vs_split": err}
    for name, fn in (("fused_fwd", fused_fwd), ("split_fwd", split_fwd), ("fused_dgrad", fused_bwd), ("split_dgrad", split_bwd)):
        rows[f"{name}_ms"] = round(run(fn, args.iters), 4)
    native.check_status()
    rows["fwd_speedup"] = round(rows["split_fwd_ms"] / rows["fused_fwd_ms"], 3)
    rows["dgrad_speedup"] = round(rows["split_dgrad_ms"] / rows["fused_dgrad_ms"], 3)
    print(json.dumps(rows))


if __name__ == "__main__":
    main()
