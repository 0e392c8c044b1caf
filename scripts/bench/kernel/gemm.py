"""GEMM bench at MOSS shapes: the tcgen05 family against the library products.

    python scripts/bench/kernel/gemm.py [--tokens 17408] [--json out.json]

Prints, per problem, device time (CUDA events, L2 flushed between runs), TFLOP/s and the
fraction of the measured cuBLAS bf16 peak (`MEASURED_PEAKS.json` when present).
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
from kohakumosstrainer_b200.ops import native  # noqa: E402


def timeit(fn, iters=10, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=17408)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    peaks = {}
    for cand in (Path("MEASURED_PEAKS.json"), Path(__file__).resolve().parents[3] / "MEASURED_PEAKS.json"):
        if cand.exists():
            peaks = json.loads(cand.read_text())
            break
    peak = peaks.get("bf16_tflops", 1590.0)
    M = args.tokens
    rows = []
    for name, N, K in (("q/k/v/o", 3072, 3072), ("qkv fused", 9216, 3072), ("up_gate", 16384, 3072), ("down", 3072, 8192)):
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        xq, xs = native.quantize_fp8(x)
        wq, ws = native.quantize_fp8(w)
        flops = 2.0 * M * N * K
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        col = ws[0].expand(N).contiguous()
        one = torch.ones((), device="cuda")
        cases = {
            "ours bf16": lambda: native.gemm(x, w, out=out),
            "cublas bf16": lambda: torch.matmul(x, w.t(), out=out),
            "ours fp8 (scalar scales)": lambda: native.gemm(xq, wq, out=out, scale_a=xs[:1], scale_b=ws[:1]),
            "ours fp8 (col scale)": lambda: native.gemm(xq, wq, out=out, scale_a=xs[:1], col_scale=col),
            "ours fp8 dgrad (B MN-major)": lambda: native.gemm(xq[:, : min(K, N)].contiguous() if False else xq, wq, out=out) if False else None,
            "library fp8 (_scaled_mm)": lambda: torch._scaled_mm(xq, wq.t(), scale_a=xs[0].reshape(()), scale_b=ws[0].reshape(()), out_dtype=torch.bfloat16),
        }
        dy = torch.randn(M, N, device="cuda").bfloat16()
        dyq, dys = native.quantize_fp8(dy, torch.float8_e5m2)
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        cases["ours fp8 dgrad (B MN-major)"] = lambda: native.gemm(dyq, wq, b_mn=True, out=dx, scale_a=dys[:1], scale_b=ws[:1])
        cases["ours bf16 dgrad (B MN-major)"] = lambda: native.gemm(dy, w, b_mn=True, out=dx)
        for label, fn in cases.items():
            try:
                ms = timeit(fn)
            except Exception as err:  # a library path may be missing on some builds
                rows.append({"problem": name, "case": label, "error": str(err)[:80]})
                continue
            tf = flops / ms / 1e9
            rows.append({"problem": f"{name} {M}x{N}x{K}", "case": label, "ms": round(ms, 4), "tflops": round(tf, 1),
                         "of_measured_bf16_peak": round(tf / peak, 3)})
            print(rows[-1], flush=True)
    native.check_status()
    if args.json:
        Path(args.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
