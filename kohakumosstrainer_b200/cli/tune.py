"""`python -m kohakumosstrainer_b200.cli.tune`: measure this card and the block ops once.

The reference tunes Triton / TileLang tile choices per card and shape and stores them in a
table (`src/kohakumoss/cli/tune.py`, `kernels/tuning/*`). This framework has one architecture
and fixed kernel configurations, so there is nothing to choose; what remains useful is the
measurement: device rates (copy bandwidth, bf16 GEMM throughput) and the time of every block
op at the shapes of the requested image sizes, written to a per-card JSON that `doctor` and
the throughput callback read for roofline fractions.

    python -m kohakumosstrainer_b200.cli.tune --sizes 1024x1024 832x1216 --batch 4 [--out card.json]
"""

from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kmoss-tune", description=__doc__)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--sizes", nargs="+", default=["1024x1024"])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--text", type=int, default=256)
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    import torch

    if not torch.cuda.is_available():
        print("no CUDA device: nothing to measure")
        return 1
    from ..utils.hardware import device_rates, time_block_ops

    torch.cuda.set_device(torch.device(args.device))
    report = {"rates": device_rates(args.device), "shapes": {}}
    for size in args.sizes:
        w, h = (int(v) for v in size.lower().split("x"))
        tokens = args.batch * ((w // 16) * (h // 16) + args.text)
        report["shapes"][size] = time_block_ops(tokens, args.device)
    text = json.dumps(report, indent=1)
    print(text)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as f:
            f.write(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
