"""Training-step bench through the public entry, one line per memory profile / checkpoint mode: ms per step,
tokens/s and peak device memory (role of `scripts/bench/step/step.py` and `bench/train/memory.py`).

    python scripts/bench/step/step.py --profiles speed balanced --tokens 20480 --steps 6 [--depth 42]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
from kohakumosstrainer_b200.data import SyntheticConfig, SyntheticDataset  # noqa: E402
from kohakumosstrainer_b200.memory import Workload, estimate, resolve_profile  # noqa: E402
from kohakumosstrainer_b200.training.trainer import Trainer, TrainerConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profiles", nargs="+", default=["speed", "balanced"])
    ap.add_argument("--tokens", type=int, default=20480)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--depth", type=int, default=42)
    ap.add_argument("--algo", default="lora")
    ap.add_argument("--base", default="fp8_compute")
    args = ap.parse_args()
    data = SyntheticDataset(SyntheticConfig(max_tokens=args.tokens, seed=1234))
    batches = [data.materialize(i) for i in range(args.steps + args.warmup)]
    for name in args.profiles:
        plan = resolve_profile({"MEMORY_PROFILE": name})
        cfg = TrainerConfig(variant="base", arch_overrides={"depth": args.depth}, algo=args.algo, dim=8, alpha=8.0,
                            base_precision=args.base if args.algo != "full" else "auto", memory=plan, schedule={"mode": "constant"})
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        tr = Trainer(cfg, device="cuda:0")
        for hb in batches[: args.warmup]:
            tr.train_step(hb)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        tokens = 0
        for hb in batches[args.warmup :]:
            tr.train_step(hb)
            tokens += hb.image_tokens
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / args.steps
        arch = tr.model.cfg
        est = estimate(Workload(arch, args.tokens, 0, trainable_params=sum(p.numel() for p in tr.params), full_ft=args.algo == "full",
                                stored_precision=args.base if args.algo != "full" else "compute"), plan)
        print(json.dumps({"profile": name, "ms_per_step": round(ms, 2), "latent_tokens_per_s": round(tokens / args.steps / ms * 1e3, 1),
                          "peak_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2), "estimate_gib": round(est["total"] / 2**30, 2)}), flush=True)
        del tr


if __name__ == "__main__":
    main()
