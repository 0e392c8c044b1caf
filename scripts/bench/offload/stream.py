"""Host <-> device copy bandwidth and the cost of weight-ring streaming: pinned H2D / D2H at several sizes, then
a ring of block-sized buffers streamed behind a GEMM of one block's FLOPs (role of `scripts/bench/offload/stream.py`).

    python scripts/bench/offload/stream.py [--sizes-mb 16 64 256 1024]
"""

from __future__ import annotations

import argparse
import json

import torch


def timed(fn, iters=5):
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=int, nargs="+", default=[16, 64, 256, 1024])
    args = ap.parse_args()
    for mb in args.sizes_mb:
        host = torch.empty(mb << 20, dtype=torch.uint8, pin_memory=True)
        dev = torch.empty(mb << 20, dtype=torch.uint8, device="cuda")
        h2d = timed(lambda: dev.copy_(host, non_blocking=True))
        d2h = timed(lambda: host.copy_(dev, non_blocking=True))
        print(json.dumps({"mb": mb, "h2d_gbs": round(mb / 1024 / h2d * 1e3, 1), "d2h_gbs": round(mb / 1024 / d2h * 1e3, 1)}), flush=True)
    # one block of the base model in fp8 is ~122 MB; its forward at 20k tokens is ~2.4 ms of GEMMs
    block = torch.empty(122 << 20, dtype=torch.uint8, pin_memory=True)
    slots = [torch.empty_like(block, device="cuda") for _ in range(2)]
    x = torch.randn(20480, 3072, device="cuda").bfloat16()
    w = torch.randn(3072, 3072, device="cuda").bfloat16()
    copy = torch.cuda.Stream()

    def compute_only():
        for _ in range(8):
            torch.matmul(x, w)

    def with_stream():
        with torch.cuda.stream(copy):
            slots[0].copy_(block, non_blocking=True)
        compute_only()
        torch.cuda.current_stream().wait_stream(copy)

    a, b = timed(compute_only), timed(with_stream)
    print(json.dumps({"block_mb": 122, "compute_ms": round(a, 3), "compute_plus_stream_ms": round(b, 3), "exposed_ms": round(max(b - a, 0), 3)}), flush=True)


if __name__ == "__main__":
    main()
