"""Per-op parity: every native op against the eager reference on the same inputs, relative error per op as a table
(role of `scripts/probe/parity.py`). Needs a GPU.

    python scripts/probe/parity.py [--tokens 4096]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from kohakumosstrainer_b200.ops import eager  # noqa: E402
from kohakumosstrainer_b200.ops.native_ops import NativeOps  # noqa: E402


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    args = ap.parse_args()
    n, d, f = args.tokens, 3072, 8192
    ops = NativeOps()
    g = torch.Generator("cuda").manual_seed(0)
    x = torch.randn(n, d, device="cuda", generator=g).bfloat16()
    seg = (torch.arange(n, device="cuda") // 1024).int()
    b = int(seg.max()) + 1
    w = torch.randn(d, device="cuda", generator=g) * 0.1 + 1
    shift, scale = torch.randn(b, d, device="cuda", generator=g) * 0.1, torch.randn(b, d, device="cuda", generator=g) * 0.1
    rows = {"rms_norm_mod": rel(ops.rms_norm_mod(x, w, shift, scale, seg, 1e-6), eager.rms_norm_mod(x.float(), w, shift, scale, seg, 1e-6))}
    ug = torch.randn(n, 2 * f, device="cuda", generator=g).bfloat16()
    rows["situ_glu"] = rel(ops.situ_glu(ug), eager.situ_glu(ug.float()))
    o = torch.randn(n, d, device="cuda", generator=g).bfloat16()
    gate = torch.randn(b, d, device="cuda", generator=g)
    rows["gated_residual"] = rel(ops.gated_residual(x, o, gate, seg, 0.7), eager.gated_residual(x.float(), o.float(), gate, seg, 0.7))
    pred, target = torch.randn(n, 128, device="cuda", generator=g).bfloat16(), torch.randn(n, 128, device="cuda", generator=g)
    wt = torch.rand(b, device="cuda", generator=g)
    rows["token_mse"] = rel(ops.token_mse(pred, target, seg, wt, None), eager.token_mse(pred.float(), target, seg, wt, None))
    print(json.dumps({k: f"{v:.2e}" for k, v in rows.items()}, indent=1))


if __name__ == "__main__":
    main()
