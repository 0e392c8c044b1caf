"""Generate images (or latents) with a MOSS-Image DiT: UPPER_CASE globals are the knobs
(`scripts/sample/sample.py:43-98` in the reference).

    python -m kohakumosstrainer_b200.cli.run scripts/sample/sample.py --set PROMPT="a cat" --set STEPS=32

Without a text encoder / VAE (this repository ships none) prompts cannot be encoded: pass
`TEXT_EMBEDDINGS` (a `.safetensors` with `positive.<i>` / `negative.<i>` tensors) or
`SYNTHETIC=True` for N(0, 1) embeddings, and the outputs are latents (`<index>_<seed>.pt`).
"""

WEIGHTS = ""
VARIANT = "base"
TRANSFORMER = ""
TEXT_ENCODER = ""
VAE = ""
ADAPTERS = []                # [(path, multiplier)]
ADAPTER_MODE = "merge"
PRECISION = "bf16"
FP16_FIX = "none"
FP16_FIX_KWARGS = {}
TUNE = "off"
DEVICE = "cuda"
TEXT_DEVICE = ""
TEXT_ENCODE = {}
VAE_ENCODE = {}
VAE_DTYPE = "bf16"
MEMORY_PROFILE = "speed"
MEMORY_OVERRIDES = {}
STREAM = "off"
STREAM_RESIDENT = 0
PINNED = True
BASE_PRECISION = "auto"
FP8_RECIPE = "row"
INT8_COMPUTE = False
PROMPT = ""
PROMPTS = []
PROMPTS_FILE = ""
NEGATIVE = ""
TEXT_EMBEDDINGS = ""
SYNTHETIC = False
SIZE = (1024, 1024)
SEEDS = (0,)
SEED_BASE = 0
STEPS = 50
CFG = 3.0
SHIFT = 5.0
SKIP_LAYERS = "default"
CFG_MODE = "packed"
BATCH = 4
OUT = "outputs"
PROGRESS = True
ARCH_OVERRIDES = {}

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json
    from pathlib import Path

    import torch

    from kohakumosstrainer_b200.config import check, collect, script_knobs
    from kohakumosstrainer_b200.inference.pipeline import MossPipeline, SampleRequest, synthetic_requests
    from kohakumosstrainer_b200.training.knobs import CHOICES

    k = check(collect(globals()), script_knobs(__file__), {n: CHOICES[n] for n in ("VARIANT", "ADAPTER_MODE", "PRECISION", "CFG_MODE", "BASE_PRECISION")})
    device = k["DEVICE"] if torch.cuda.is_available() else "cpu"
    pipe = MossPipeline.from_pretrained(k["TRANSFORMER"] or k["WEIGHTS"], k["VARIANT"], dict(k["ARCH_OVERRIDES"]), device, k["PRECISION"],
                                        k["BASE_PRECISION"], k["FP8_RECIPE"], list(k["ADAPTERS"]), k["ADAPTER_MODE"])
    prompts = list(k["PROMPTS"]) or ([k["PROMPT"]] if k["PROMPT"] else [])
    if k["PROMPTS_FILE"]:
        prompts += [line.strip() for line in Path(k["PROMPTS_FILE"]).read_text().splitlines() if line.strip()]
    seeds = list(k["SEEDS"])
    text_dim = pipe.backbone.cfg.text_dim
    if k["TEXT_EMBEDDINGS"]:
        from safetensors.torch import load_file

        emb = load_file(k["TEXT_EMBEDDINGS"])
        n = len([e for e in emb if e.startswith("positive.")])
        reqs = [SampleRequest(emb[f"positive.{i}"], emb.get(f"negative.{i}"), tuple(k["SIZE"]), k["SEED_BASE"] + s, meta={"index": i})
                for i in range(n) for s in seeds]
    elif k["SYNTHETIC"] or not prompts:
        reqs = synthetic_requests(max(1, len(prompts)) * len(seeds), text_dim, tuple(k["SIZE"]), seed=k["SEED_BASE"],
                                  dtype=torch.bfloat16 if device != "cpu" else torch.float32)
    else:
        pos = pipe.encode(prompts)
        neg = pipe.encode([k["NEGATIVE"]] * len(prompts))
        reqs = [SampleRequest(p, n, tuple(k["SIZE"]), k["SEED_BASE"] + s, prompt=t) for p, n, t in zip(pos, neg, prompts) for s in seeds]
    out = pipe.generate(reqs, k["STEPS"], k["CFG"], k["SHIFT"], k["SKIP_LAYERS"], k["CFG_MODE"], k["BATCH"])
    folder = Path(k["OUT"])
    folder.mkdir(parents=True, exist_ok=True)
    meta = []
    for i, (req, z) in enumerate(zip(reqs, out["latents"])):
        name = f"{i:05d}_{req.seed}"
        if out["images"] is not None:
            out["images"][i].save(folder / f"{name}.png")
        else:
            torch.save(z.cpu(), folder / f"{name}.pt")
        meta.append({"file": name, "seed": req.seed, "size": list(req.size), "prompt": req.prompt})
    (folder / "metadata-00000.json").write_text(json.dumps({"steps": k["STEPS"], "cfg": k["CFG"], "shift": k["SHIFT"],
                                                           "seconds_per_image": out["per_image_s"], "items": meta}, indent=1))
    return out


if __name__ == "__main__":
    main()
