"""Adapter round trip: a random adapter on the live model against the same adapter exported
(comfy / lycoris) and loaded by `MossPipeline` (merge / bypass), in fp32; one JSON report of
relative errors (role of `scripts/probe/adapter_e2e.py`). Runs on random-init weights of a small
architecture when WEIGHTS is empty, on CPU or GPU.

    python scripts/probe/adapter_e2e.py [--weights <root>] [--algo lora] [--out runs/e2e]
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from kohakumosstrainer_b200 import adapters as A  # noqa: E402
from kohakumosstrainer_b200.adapters.export import export  # noqa: E402
from kohakumosstrainer_b200.inference.pipeline import MossPipeline  # noqa: E402
from kohakumosstrainer_b200.types import build_seqinfo  # noqa: E402

SMALL = {"dim": 128, "depth": 3, "heads": 2, "ffn_dim": 256, "text_dim": 64, "text_blocks": 1}


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default="")
    ap.add_argument("--algo", default="lora")
    ap.add_argument("--dim", type=int, default=8)
    ap.add_argument("--out", default="runs/probe/adapter_e2e")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    over = None if args.weights else SMALL
    live = MossPipeline.from_pretrained(args.weights, arch_overrides=over, device=args.device, precision="fp32", base_precision="compute")
    model = live.backbone
    aset = A.apply(model, A.AdapterConfig(algo=args.algo, preset="attn-mlp", dim=args.dim, alpha=float(args.dim), mode="bypass"))
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in aset.parameters():
            p.copy_(torch.randn(p.shape, generator=g).to(p) * 0.05)
    cfg = model.cfg
    hw = torch.tensor([[8, 8], [4, 12]])
    seq = build_seqinfo(hw, torch.tensor([9, 5])).to(args.device)
    x = torch.randn(seq.n_img, cfg.latent_channels, generator=g).to(args.device)
    text = torch.randn(seq.n_txt, cfg.text_dim, generator=g).to(args.device)
    sigma = torch.tensor([0.3, 0.8], device=args.device)
    with torch.no_grad():
        want = model(x, text, sigma, seq)
    report = {"algo": args.algo, "dim": args.dim, "cases": {}}
    for fmt in ("lycoris", "comfy"):
        path = export(aset, model, out / f"probe-{fmt}.safetensors", fmt)
        for mode in ("merge", "bypass"):
            pipe = MossPipeline.from_pretrained(args.weights, arch_overrides=over, device=args.device, precision="fp32",
                                                base_precision="compute", adapters=[(str(path), 1.0)], adapter_mode=mode)
            with torch.no_grad():
                got = pipe.backbone(x, text, sigma, seq)
            report["cases"][f"{fmt}/{mode}"] = rel(got, want)
    report["worst"] = max(report["cases"].values())
    (out / "adapter_e2e.json").write_text(json.dumps(report, indent=1))
    print(json.dumps(report))
    return 0 if report["worst"] < 1e-4 else 1


if __name__ == "__main__":
    raise SystemExit(main())
