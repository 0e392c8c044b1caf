"""VAE dtype bench: precision of encode (latents) and decode (pixels) in bf16 / fp16 against the
fp32 VAE (error statistics; non-finite = overflow) and ms per image / peak allocated GiB per
dtype x {encode, decode} x area x batch, eager and channels_last (role of
`scripts/bench/vae/vae.py`). Needs the VAE weights and `diffusers`; images are read from
`--images` or drawn as smooth synthetic pictures. Writes `<out>/<gpu>.json`.

    python scripts/bench/vae/vae.py --weights <root>/vae [--images <dir>] --device cuda:0
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[3]))
from kohakumosstrainer_b200.ops.error_stats import error_stats  # noqa: E402


def pictures(folder: str, area: int, count: int, device):
    side = int(area**0.5) // 16 * 16
    if folder:
        import numpy as np
        from PIL import Image

        files = sorted(p for p in Path(folder).iterdir() if p.suffix.lower() in (".png", ".jpg", ".jpeg", ".webp"))[:count]
        imgs = [torch.as_tensor(np.array(Image.open(f).convert("RGB").resize((side, side), Image.Resampling.LANCZOS))) for f in files]
        return torch.stack(imgs).permute(0, 3, 1, 2).float().div(127.5).sub(1.0).to(device)
    g = torch.Generator().manual_seed(area)
    low = torch.randn(count, 3, side // 32, side // 32, generator=g)
    return torch.nn.functional.interpolate(low, size=(side, side), mode="bicubic").clamp(-1, 1).to(device)


def timed(fn, cuda):
    fn()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
    t0 = time.perf_counter()
    out = fn()
    if cuda:
        torch.cuda.synchronize()
    return out, (time.perf_counter() - t0) * 1e3, (torch.cuda.max_memory_allocated() / 2**30 if cuda else 0.0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--weights", required=True)
    ap.add_argument("--images", default="")
    ap.add_argument("--areas", default="512x512,1024x1024")
    ap.add_argument("--batches", default="1,4")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--out", default="runs/bench/vae")
    args = ap.parse_args()
    from kohakumosstrainer_b200.encoders import FluxVae

    dev = torch.device(args.device)
    cuda = dev.type == "cuda"
    ref = FluxVae(args.weights, dev, torch.float32)
    rows = []
    for area_s in args.areas.split(","):
        w, h = (int(v) for v in area_s.split("x"))
        for batch in (int(b) for b in args.batches.split(",")):
            imgs = pictures(args.images, w * h, batch, dev)
            z32 = ref.encode(imgs)
            px32 = ref.decode(z32)
            for dtype in (torch.bfloat16, torch.float16):
                for layout in ("eager", "channels_last"):
                    vae = FluxVae(args.weights, dev, dtype)
                    x = imgs.to(dtype)
                    if layout == "channels_last":
                        vae.vae = vae.vae.to(memory_format=torch.channels_last)
                        x = x.contiguous(memory_format=torch.channels_last)
                    z, enc_ms, enc_gb = timed(lambda: vae.encode(x), cuda)
                    px, dec_ms, dec_gb = timed(lambda: vae.decode(z32.to(dtype)), cuda)
                    row = {"area": area_s, "batch": batch, "dtype": str(dtype).replace("torch.", ""), "layout": layout,
                           "encode_ms_per_image": round(enc_ms / batch, 3), "decode_ms_per_image": round(dec_ms / batch, 3),
                           "encode_peak_gib": round(enc_gb, 3), "decode_peak_gib": round(dec_gb, 3),
                           "encode_error": error_stats(z.float(), z32), "decode_error": error_stats(px.float(), px32)}
                    rows.append(row)
                    print(json.dumps(row), flush=True)
                    del vae
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    tag = torch.cuda.get_device_name(dev).replace(" ", "_") if cuda else "cpu"
    (out / f"{tag}.json").write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
