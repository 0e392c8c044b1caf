"""Write a ComfyUI int8 ConvRot transformer: block linears as int8 codes of W R + per-row scales + a
`comfy_quant` record, joint q / k / v fused, the rest as SAVE_DTYPE (role of `scripts/export/comfy_int8.py`).

    ... scripts/export/comfy_int8.py --set WEIGHTS=merged.safetensors --set OUT=moss_int8_convrot.safetensors
"""

WEIGHTS = ""
VARIANT = "base"
ARCH_OVERRIDES = {}
LAYERS = r"layers\.\d+\.proj\.[a-z_]+"
GROUP = 256
SAVE_DTYPE = "bf16"
ATTENTION_HINT = "comfy_kitchen_int8"
OUT = ""
DEVICE = "cpu"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import torch
    from safetensors.torch import save_file

    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import resolve_arch
    from kohakumosstrainer_b200.models.io import export_state, load_backbone
    from kohakumosstrainer_b200.models.numerics import unfold_stream_scale
    from kohakumosstrainer_b200.quant.comfy import int8_convrot_state

    if not OUT:
        raise SystemExit("set OUT")
    model = build_backbone(resolve_arch(VARIANT, ARCH_OVERRIDES), device=DEVICE, dtype=torch.float32, seed=0, init=not WEIGHTS)
    if WEIGHTS:
        load_backbone(model, WEIGHTS)
    unfold_stream_scale(model)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[SAVE_DTYPE]
    state = int8_convrot_state(export_state(model, torch.float32), LAYERS, int(GROUP), dtype, True, ATTENTION_HINT)
    save_file({k: v.contiguous() for k, v in state.items()}, OUT, metadata={"kohakumoss_format": "transformer", "kohakumoss_int8": f"convrot{GROUP}"})
    n = sum(k.endswith(".comfy_quant") for k in state)
    print(f"wrote {OUT}: {n} int8 ConvRot layers")
    return n


if __name__ == "__main__":
    main()
