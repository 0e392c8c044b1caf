"""Base-precision study of the DiT for inference: velocity of every base precision against an
fp64 host forward of the same weights, next to bf16; weight bytes, forward time, and a short
generate compared on the final latents (role of `scripts/probe/fp8_inference.py`; its text-encoder
stage needs the encoder weights and is skipped without `--text-weights`). One JSON report.

    python scripts/probe/fp8_inference.py [--weights <root>] [--size 512] [--steps 8] --out runs/probe/fp8
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from kohakumosstrainer_b200.inference.pipeline import MossPipeline, synthetic_requests  # noqa: E402
from kohakumosstrainer_b200.types import build_seqinfo  # noqa: E402

SMALL = {"dim": 256, "depth": 4, "heads": 2, "ffn_dim": 512, "text_dim": 64, "text_blocks": 1}
PRECISIONS = ("compute", "fp8", "fp8_compute", "int8", "mxfp8")


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


def weight_bytes(model) -> int:
    seen, total = set(), 0
    for t in list(model.parameters()) + list(model.buffers()):
        if t.data_ptr() not in seen and t.numel():
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
    for m in model.modules():
        for name in ("base", "compute"):
            holder = getattr(m, name, None)
            for v in vars(holder).values() if holder is not None and hasattr(holder, "__dict__") else ():
                if torch.is_tensor(v) and v.data_ptr() not in seen and v.numel():
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
    return total


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default="")
    ap.add_argument("--size", type=int, default=512)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--out", default="runs/probe/fp8")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--precisions", default=",".join(PRECISIONS))
    args = ap.parse_args()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    over = None if args.weights else SMALL
    cuda = torch.device(args.device).type == "cuda"

    def load(base, precision="bf16", device=args.device):
        return MossPipeline.from_pretrained(args.weights, arch_overrides=over, device=device, precision=precision, base_precision=base)

    # the oracle: the same weights in fp64 on the host
    oracle = load("compute", "fp32", "cpu")
    ref_model = oracle.backbone.double()
    cfg = ref_model.cfg
    side = args.size // 16
    g = torch.Generator().manual_seed(3)
    seq_cpu = build_seqinfo(torch.tensor([[side, side]]), torch.tensor([24]))
    x = torch.randn(seq_cpu.n_img, cfg.latent_channels, generator=g)
    text = torch.randn(seq_cpu.n_txt, cfg.text_dim, generator=g)
    sigma = torch.tensor([0.6])
    with torch.no_grad():
        want = ref_model(x.double(), text.double(), sigma.double(), seq_cpu)
    del oracle, ref_model
    report = {"size": args.size, "weights": args.weights or "random-init small", "dit": {}, "generate": {}}
    reqs = synthetic_requests(args.batch, cfg.text_dim, (args.size, args.size), 24, seed=5)
    final_bf16 = None
    for base in [p for p in args.precisions.split(",") if p]:
        try:
            pipe = load(base)
        except Exception as e:  # a precision this device cannot run is reported, not fatal
            report["dit"][base] = {"error": f"{type(e).__name__}: {e}"[:200]}
            continue
        dev, dt = pipe.device, pipe.dtype
        seq = seq_cpu.to(dev)
        args_dev = (x.to(dev, dt), text.to(dev, dt), sigma.to(dev), seq)
        with torch.no_grad():
            got = pipe.backbone(*args_dev)
            if cuda:
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(3):
                pipe.backbone(*args_dev)
            if cuda:
                torch.cuda.synchronize()
            fwd_ms = (time.perf_counter() - t0) / 3 * 1e3
        row = {"rel_err_vs_fp64": rel(got.cpu(), want), "weight_mb": round(weight_bytes(pipe.backbone) / 2**20, 1), "forward_ms": round(fwd_ms, 3)}
        report["dit"][base] = row
        if cuda:
            torch.cuda.reset_peak_memory_stats()
        t0 = time.perf_counter()
        res = pipe.generate(reqs, steps=args.steps, cfg=3.0, decode=False, skip_layers="none" if over else "default")
        lat = torch.cat([z.float().cpu().flatten() for z in res["latents"]])
        if base == "compute":
            final_bf16 = lat
        report["generate"][base] = {"seconds": round(time.perf_counter() - t0, 3), "per_image_s": round(res["per_image_s"], 4),
                                    "peak_mb": round(torch.cuda.max_memory_allocated() / 2**20, 1) if cuda else None,
                                    "final_latent_rel_vs_bf16": None if final_bf16 is None else rel(lat, final_bf16)}
        del pipe
    (out / "fp8_inference.json").write_text(json.dumps(report, indent=1))
    print(json.dumps(report))


if __name__ == "__main__":
    main()
