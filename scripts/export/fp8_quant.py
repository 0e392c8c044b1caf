"""Write a pre-quantised fp8 transformer: every block linear as e4m3 `<n>.weight` + `<n>.weight_scale`
+ `comfy_quant` record, the rest as SAVE_DTYPE; loading attaches the stored bases without building a
16-bit copy (role of `scripts/export/fp8_quant.py`).

    ... scripts/export/fp8_quant.py --set WEIGHTS=<root>/base --set FP8_RECIPE=row --set OUT=moss_fp8.safetensors
"""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
PRECISION = "fp8_compute"   # fp8_compute (mxfp8 payloads are written by the same tool once a loader needs them)
FP8_RECIPE = "row"          # tensor | row
SAVE_DTYPE = "bf16"
MIN_FEATURES = 256
LAYERS = r"layers\.\d+\.proj\.[a-z_]+"
OUT = ""
DEVICE = "cpu"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import json

    import torch
    from safetensors.torch import save_file

    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import resolve_arch
    from kohakumosstrainer_b200.models.io import export_state, load_backbone
    from kohakumosstrainer_b200.quant.comfy import fp8_state

    if not OUT:
        raise SystemExit("set OUT")
    model = build_backbone(resolve_arch(VARIANT, ARCH_OVERRIDES), device=DEVICE, dtype=torch.float32, seed=0, init=not WEIGHTS)
    if WEIGHTS:
        load_backbone(model, WEIGHTS)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[SAVE_DTYPE]
    state = fp8_state(export_state(model, torch.float32), LAYERS, FP8_RECIPE, dtype, int(MIN_FEATURES))
    meta = {"kohakumoss_format": "transformer", "kohakumoss_fp8": json.dumps({"precision": PRECISION, "recipe": FP8_RECIPE})}
    save_file({k: v.contiguous() for k, v in state.items()}, OUT, metadata=meta)
    n = sum(k.endswith(".comfy_quant") for k in state)
    print(f"wrote {OUT}: {n} fp8 layers")
    return n


if __name__ == "__main__":
    main()
