"""Encode the probe prompts (and the empty prompt) once; later probes load the file
(role of `scripts/probe/embed.py`). Without `--weights` the deterministic synthetic text encoder
stands in, so the downstream probes run on a box without the checkpoints.

    python scripts/probe/embed.py [--weights <root>/text_encoder] --out runs/probe/embeds.pt
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from kohakumosstrainer_b200 import encoders  # noqa: E402

PROMPTS = (
    "a photograph of a red fox standing in fresh snow at dawn, shallow depth of field",
    "an isometric illustration of a tiny workshop full of tools, warm lamp light",
    "a watercolor painting of a harbour town with sailing boats, loose brush strokes",
    "portrait of an elderly clockmaker, dramatic side lighting, 85mm",
)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", default="")
    ap.add_argument("--out", default="runs/probe/embeds.pt")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--text-dim", type=int, default=4096)
    args = ap.parse_args()
    enc = encoders.text_encoder(args.weights, args.device) if args.weights else encoders.synthetic_text_encoder(args.text_dim)
    texts = list(PROMPTS) + [""]
    emb = enc.encode(texts) if hasattr(enc, "encode") else enc(texts)
    out = Path(args.out)
    out.parent.mkdir(parents=True, exist_ok=True)
    torch.save({"prompts": texts, "positive": [e.cpu() for e in emb[:-1]], "negative": emb[-1].cpu(),
                "encoder": args.weights or "synthetic"}, out)
    print(f"{len(texts)} prompts -> {out}")


if __name__ == "__main__":
    main()
