"""Text-encoder op timing table: per shape (segments x length) the time of
`gated_delta_rule_varlen` and `attention_varlen_causal` on this device and their error against
an fp64 evaluation of the same op (role of `scripts/bench/textenc/ops.py`). Shapes use the
Qwen3.5-9B head layout (delta: 16 key / 32 value heads of 128; attention: 16 query / 4 kv heads
of 256). Writes `<out>/<device>_ops_<dtype>.json`.

    python scripts/bench/textenc/ops.py --shapes 1x300,16x300,64x150 --dtype bf16 --out runs/bench/textenc
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
from kohakumosstrainer_b200.ops import textenc  # noqa: E402
from kohakumosstrainer_b200.ops.error_stats import error_stats  # noqa: E402


def timed(fn, iters, cuda):
    fn()
    if cuda:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    if cuda:
        torch.cuda.synchronize()
    return (time.perf_counter() - t0) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="1x300,16x300,64x150")
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "fp16", "fp32"))
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--out", default="runs/bench/textenc")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--heads-scale", type=float, default=1.0, help="shrink the head counts for a host dry run")
    args = ap.parse_args()
    dev = torch.device(args.device)
    cuda = dev.type == "cuda"
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    if not cuda:
        dt = torch.float32
    hk, hv = max(1, int(16 * args.heads_scale)), max(2, int(32 * args.heads_scale))
    hq, hkv = max(4, int(16 * args.heads_scale)), max(1, int(4 * args.heads_scale))
    rows = []
    for shape in args.shapes.split(","):
        segs, length = (int(v) for v in shape.split("x"))
        n = segs * length
        cu = torch.arange(0, n + 1, length, device=dev, dtype=torch.int32)
        g = torch.Generator().manual_seed(n)
        r = lambda *s: torch.randn(*s, generator=g).to(dev)  # noqa: E731
        q, k, v = r(n, hk, 128), r(n, hk, 128), r(n, hv, 128)
        a, b, a_log, dt_bias = r(n, hv), r(n, hv), r(hv) * 0.1, r(hv) * 0.1
        delta = lambda c=dt: textenc.gated_delta_rule_varlen(q.to(c), k.to(c), v.to(c), a.to(c), b.to(c), a_log, dt_bias, cu, length)  # noqa: E731
        qa, ka, va = r(n, hq, 256), r(n, hkv, 256), r(n, hkv, 256)
        attn = lambda c=dt: textenc.attention_varlen_causal(qa.to(c), ka.to(c), va.to(c), cu, length, 256**-0.5)  # noqa: E731
        row = {"shape": shape, "tokens": n}
        for name, fn in (("gated_delta_rule_varlen", delta), ("attention_varlen_causal", attn)):
            ms = timed(fn, args.iters, cuda)
            ref = fn(torch.float64).double() if not cuda or n <= 8192 else None
            row[name] = {"ms": round(ms, 3), "tokens_per_s": round(n / ms * 1e3)}
            if ref is not None:
                row[name]["error"] = error_stats(fn().double(), ref)
        rows.append(row)
        print(json.dumps(row), flush=True)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    tag = torch.cuda.get_device_name(dev).replace(" ", "_") if cuda else "cpu"
    (out / f"{tag}_ops_{args.dtype}.json").write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
