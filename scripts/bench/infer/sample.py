"""Sampling bench: fp8 MOSS-Image-Base DiT (random init), rectified-flow Euler steps with packed
CFG, 1024^2 images with 256-token N(0, 1) text embeddings, data-parallel over the ranks.

    python scripts/bench/infer/sample.py --images 8 --steps 32 --cfg 3 [--batch 4]
    torchrun --nproc-per-node 8 scripts/bench/infer/sample.py --images 64

Metric: seconds per image = max over ranks of the device time of the rank's sampling loops,
divided by the total number of images.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
from kohakumosstrainer_b200.inference.pipeline import MossPipeline, synthetic_requests  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--images", type=int, default=8)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--cfg", type=float, default=3.0)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--variant", default="base")
    ap.add_argument("--base", default="fp8_compute")
    ap.add_argument("--recipe", default="tensor")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--size", type=int, default=1024)
    args = ap.parse_args()
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    pipe = MossPipeline.from_pretrained(variant=args.variant, device=f"cuda:{local}", base_precision=args.base, fp8_recipe=args.recipe)
    text_dim = pipe.backbone.cfg.text_dim
    reqs = synthetic_requests(args.images, text_dim, (args.size, args.size))
    warm = synthetic_requests(min(args.batch, args.images), text_dim, (args.size, args.size), seed=99)
    pipe.generate(warm, steps=3, cfg=args.cfg, batch=args.batch, graph=not args.no_graph, decode=False)
    torch.cuda.synchronize()
    out = pipe.generate_distributed(reqs, rank, world, steps=args.steps, cfg=args.cfg, batch=args.batch,
                                    graph=not args.no_graph, decode=False)
    ms = torch.tensor([out["device_ms"]], device=f"cuda:{local}")
    if world > 1:
        torch.distributed.all_reduce(ms, op=torch.distributed.ReduceOp.MAX)
    finite = all(torch.isfinite(z).all().item() for z in out["latents"])
    if rank == 0:
        print(json.dumps({"metric": "sampling_seconds_per_image", "value": ms.item() / 1e3 / args.images, "unit": "s/image",
                          "n_gpus": world, "images": args.images, "steps": args.steps, "cfg": args.cfg, "batch": args.batch,
                          "size": args.size, "base": args.base, "graph": not args.no_graph, "finite": finite,
                          "s_per_step_per_rank": ms.item() / 1e3 / (args.steps * max(1, -(-len(out["latents"]) // args.batch)))}))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
