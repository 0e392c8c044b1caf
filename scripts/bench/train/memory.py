"""Per-phase device memory of the trainer's startup and first steps: allocated, peak allocated
and reserved GiB after the model build (or load), the base-precision and plan apply, the
trainable set and optimiser, and every one of the first steps, next to the plan's analytic
estimate (role of `scripts/bench/train/memory.py`). One profile per process. Needs a GPU.

    python scripts/bench/train/memory.py [--weights <root>/base] --profile none --algo lora --tokens 20480 \
        [--depth 6] --out runs/bench/train
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))


def snapshot(tag, rows, device):
    torch.cuda.synchronize(device)
    gib = 2**30
    rows.append({"phase": tag, "allocated_gib": round(torch.cuda.memory_allocated(device) / gib, 3),
                 "peak_gib": round(torch.cuda.max_memory_allocated(device) / gib, 3),
                 "reserved_gib": round(torch.cuda.memory_reserved(device) / gib, 3)})
    torch.cuda.reset_peak_memory_stats(device)
    print(json.dumps(rows[-1]), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default="")
    ap.add_argument("--profile", default="none")
    ap.add_argument("--algo", default="lora")
    ap.add_argument("--precision", default="bf16")
    ap.add_argument("--base-precision", default="fp8_compute")
    ap.add_argument("--tokens", type=int, default=20480)
    ap.add_argument("--depth", type=int, default=0, help="override the depth (0 = the variant's)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--out", default="runs/bench/train")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args()
    from kohakumosstrainer_b200.data import SyntheticConfig, SyntheticDataset
    from kohakumosstrainer_b200.memory import Workload, estimate, resolve_profile
    from kohakumosstrainer_b200.training import Trainer, TrainerConfig

    dev = torch.device(args.device)
    rows: list[dict] = []
    plan = resolve_profile({"MEMORY_PROFILE": args.profile})
    over = {"depth": args.depth} if args.depth else {}
    cfg = TrainerConfig(variant="base", arch_overrides=over, algo=args.algo, dim=8, alpha=8.0, precision=args.precision,
                        base_precision=args.base_precision, schedule={"mode": "constant"}, memory=plan if args.profile != "none" else None)
    snapshot("start", rows, dev)
    tr = Trainer(cfg, device=args.device)
    if args.weights:
        from kohakumosstrainer_b200.models.io import load_backbone

        load_backbone(tr.model, args.weights)
    snapshot("trainer built (model, base precision, plan, adapters, optimiser)", rows, dev)
    data = SyntheticDataset(SyntheticConfig(max_tokens=args.tokens, seed=1))
    for i in range(args.steps):
        tr.train_step(data.materialize(i))
        snapshot(f"step {i + 1}", rows, dev)
    arch = tr.model.cfg
    hb = data.materialize(0)
    trainable = sum(p.numel() for p in tr.params)
    work = Workload(arch, hb.image_tokens, hb.text_tokens if hasattr(hb, "text_tokens") else args.tokens - hb.image_tokens,
                    trainable_params=trainable, full_ft=args.algo == "full")
    est = estimate(work, plan)
    report = {"profile": args.profile, "algo": args.algo, "tokens": args.tokens, "depth": arch.depth, "phases": rows,
              "estimate_gib": {k: round(v / 2**30, 3) for k, v in est.items() if isinstance(v, (int, float))},
              "measured_peak_gib": max(r["peak_gib"] for r in rows)}
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    (out / f"memory_{args.profile}_{args.algo}.json").write_text(json.dumps(report, indent=1))
    print(json.dumps({k: report[k] for k in ("measured_peak_gib", "estimate_gib")}))


if __name__ == "__main__":
    main()
