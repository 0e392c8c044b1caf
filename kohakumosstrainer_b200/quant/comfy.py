"""ComfyUI quantised checkpoints, read and written.

A quantised layer `<n>` stores its codes as `<n>.weight`, its scales as `<n>.weight_scale` (or
`scale_weight`) and `<n>.comfy_quant`, a uint8 tensor holding a JSON record of the format
(`src/kohakumoss/quant/comfy_format.py:1-60`, `quant/comfy_write.py` in the reference):

| format | tensors | becomes |
|---|---|---|
| `int8_tensorwise` | weight int8 [N, K], weight_scale fp32 [N, 1] or scalar; `convrot` + `convrot_groupsize` for a rotated file | `Int8Weight` |
| `float8_e4m3fn` | weight e4m3 [N, K], weight_scale | `Fp8Weight` (row or tensor scaled) |

A record-less int8 / fp8 `<n>.weight` next to a scale key is read the same way (no rotation).
| `asym_w4a8_int8` | packed 4- / 6-bit codes, weight_s_rel e4m3, weight_s_channel, optional codebook / correction; `group_size` | decoded once at load into `Int8Weight` (`quant/w4a8.py`) |

Joint q / k / v stored fused (`proj.qkv`) are split on load and fused on save.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass

import torch
from torch import Tensor

from .formats import Int8Weight, quantize_weight_int8
from .weights import Fp8Weight, _quantize

RECORD = "comfy_quant"
FORMATS = {"int8_tensorwise": "int8", "float8_e4m3fn": "fp8", "asym_w4a8_int8": "w4a8"}
SCALE_KEYS = ("weight_scale", "scale_weight")
IGNORED = ("scale_input", "input_scale")


@dataclass(frozen=True)
class ComfyLayer:
    path: str
    fmt: str            # int8 | fp8 | w4a8
    rotation: int       # ConvRot group (0 = none)
    keys: tuple
    group: int = 0      # w4a8: input columns per group scale


def write_record(fmt: str, rotation: int = 0) -> Tensor:
    rec = {"format": fmt}
    if rotation:
        rec.update(convrot=True, convrot_groupsize=int(rotation))
    return torch.tensor(list(json.dumps(rec).encode("utf-8")), dtype=torch.uint8)


def read_record(t: Tensor) -> dict:
    return json.loads(bytes(t.to(torch.uint8).tolist()).decode("utf-8"))


def scan_layers(sd: dict[str, Tensor]) -> dict[str, ComfyLayer]:
    """Every quantised layer of a state dict by module path."""
    out = {}
    for key, t in sd.items():
        if not key.endswith(".weight"):
            continue
        path = key[: -len(".weight")]
        rec_key = f"{path}.{RECORD}"
        scale_key = next((f"{path}.{s}" for s in SCALE_KEYS if f"{path}.{s}" in sd), None)
        if rec_key in sd:
            rec = read_record(sd[rec_key])
            fmt = FORMATS.get(rec.get("format"))
            if fmt is None:
                raise ValueError(f"{path}: unknown comfy_quant format {rec.get('format')!r}")
            rot = int(rec.get("convrot_groupsize", 0)) if rec.get("convrot") else 0
            if fmt == "w4a8":
                extra = tuple(k for k in (f"{path}.weight_{n}" for n in ("s_rel", "s_channel", "codebook", "correction")) if k in sd)
                out[path] = ComfyLayer(path, fmt, rot, (key, rec_key) + extra, int(rec.get("group_size", 0)))
                continue
        elif scale_key is not None and t.dtype in (torch.int8, torch.float8_e4m3fn):
            fmt, rot = ("int8" if t.dtype == torch.int8 else "fp8"), 0
        else:
            continue
        keys = tuple(k for k in (key, rec_key, scale_key, *(f"{path}.{i}" for i in IGNORED)) if k and k in sd)
        out[path] = ComfyLayer(path, fmt, rot, keys)
    return out


def base_of(layer: ComfyLayer, sd: dict[str, Tensor], int8_compute: bool = False):
    """The stored-weight object of one quantised layer."""
    if layer.fmt == "w4a8":
        from .w4a8 import load_layer

        return load_layer(layer.path, sd, layer.group, layer.rotation, int8_compute)
    w = sd[f"{layer.path}.weight"]
    scale = next(sd[f"{layer.path}.{s}"] for s in SCALE_KEYS if f"{layer.path}.{s}" in sd).float().reshape(-1)
    if scale.numel() == 1:
        scale = scale.expand(w.shape[0]).contiguous()
    if layer.fmt == "int8":
        return Int8Weight(w.contiguous(), scale, layer.rotation, int8_compute)
    per_tensor = bool((scale == scale[0]).all())
    stacked = torch.stack((scale[0], 1.0 / scale[0])) if per_tensor else torch.ones(2)
    return Fp8Weight(w.contiguous(), stacked.float(), scale, per_tensor)


def split_fused(sd: dict[str, Tensor]) -> dict[str, Tensor]:
    """`proj.qkv.{weight, weight_scale, comfy_quant, bias}` -> separate q / k / v entries."""
    out = dict(sd)
    for key in list(sd):
        m = re.match(r"(.*\.proj)\.qkv\.weight$", key)
        if not m:
            continue
        stem = m.group(1)
        n = sd[key].shape[0] // 3
        for i, name in enumerate("qkv"):
            out[f"{stem}.{name}.weight"] = sd[key][i * n : (i + 1) * n]
            for extra in (*SCALE_KEYS, "bias"):
                src = f"{stem}.qkv.{extra}"
                if src in sd:
                    t = sd[src]
                    out[f"{stem}.{name}.{extra}"] = t[i * n : (i + 1) * n] if t.dim() and t.shape[0] == 3 * n else t
            if f"{stem}.qkv.{RECORD}" in sd:
                out[f"{stem}.{name}.{RECORD}"] = sd[f"{stem}.qkv.{RECORD}"]
        for extra in ("weight", *SCALE_KEYS, "bias", RECORD):
            out.pop(f"{stem}.qkv.{extra}", None)
    return out


def attach_quantized(model, sd: dict[str, Tensor], int8_compute: bool = False) -> tuple[dict[str, Tensor], int]:
    """Attach every quantised layer of `sd` to `model` as a stored base (no 16-bit copy is
    built); returns the remaining (dense) entries and the number of layers attached."""
    sd = split_fused(sd)
    layers = scan_layers(sd)
    modules = dict(model.named_modules())
    rest = dict(sd)
    count = 0
    for path, layer in layers.items():
        mod = modules.get(path)
        if mod is None or not hasattr(mod, "set_base"):
            continue
        base = base_of(layer, sd, int8_compute)
        if torch.is_tensor(base):      # a W4A8 layer with a correction term decodes to a dense weight
            with torch.no_grad():
                mod.weight.copy_(base.to(mod.weight))
        else:
            mod.set_base(base)
            mod.drop_weight()
        for k in layer.keys:
            rest.pop(k, None)
        count += 1
    if count:
        from ..ops import native_ops

        native_ops.invalidate_packs(model)
    return rest, count


def int8_convrot_state(state: dict[str, Tensor], layers: str = r"layers\.\d+\.proj\.[a-z_]+", group: int = 256, save_dtype=torch.bfloat16,
                       fuse_qkv: bool = True, attention_hint: str = "") -> dict[str, Tensor]:
    """A dense state dict -> the ComfyUI int8 ConvRot layout: matching linears as int8 codes of
    W R + per-row scales + record, joint q / k / v fused, the rest as `save_dtype`."""
    pat = re.compile(layers)
    out: dict[str, Tensor] = {}
    for key, t in state.items():
        path = key[: -len(".weight")] if key.endswith(".weight") else None
        if path is not None and pat.fullmatch(path) and t.dim() == 2:
            g = group if group and t.shape[1] % group == 0 else 0
            q, s = quantize_weight_int8(t, g)
            out[key] = q
            out[f"{path}.weight_scale"] = s.reshape(-1, 1)
            out[f"{path}.{RECORD}"] = write_record("int8_tensorwise", g)
        else:
            out[key] = t.to(save_dtype) if t.is_floating_point() else t
    if fuse_qkv:
        out = fuse_quantized_qkv(out)
    if attention_hint:
        for i in sorted({int(m.group(1)) for k in out if (m := re.match(r"layers\.(\d+)\.", k))}):
            out[f"layers.{i}.comfy_attention.config"] = torch.tensor(list(attention_hint.encode("utf-8")), dtype=torch.uint8)
    return out


def fp8_state(state: dict[str, Tensor], layers: str = r"layers\.\d+\.proj\.[a-z_]+", recipe: str = "row", save_dtype=torch.bfloat16,
              min_features: int = 256) -> dict[str, Tensor]:
    pat = re.compile(layers)
    out: dict[str, Tensor] = {}
    for key, t in state.items():
        path = key[: -len(".weight")] if key.endswith(".weight") else None
        if path is not None and pat.fullmatch(path) and t.dim() == 2 and min(t.shape) >= min_features:
            q, scale, col = _quantize(t, recipe)
            out[key] = q
            out[f"{path}.weight_scale"] = (scale[:1] if recipe == "tensor" else col.reshape(-1, 1)).float()
            out[f"{path}.{RECORD}"] = write_record("float8_e4m3fn")
        else:
            out[key] = t.to(save_dtype) if t.is_floating_point() else t
    return out


def fuse_quantized_qkv(sd: dict[str, Tensor]) -> dict[str, Tensor]:
    out = dict(sd)
    for key in list(sd):
        m = re.match(r"(.*\.proj)\.q\.weight$", key)
        if not m:
            continue
        stem = m.group(1)
        names = [f"{stem}.{n}" for n in "qkv"]
        if not all(f"{n}.weight" in sd for n in names):
            continue
        out[f"{stem}.qkv.weight"] = torch.cat([sd[f"{n}.weight"] for n in names], 0)
        for extra in (*SCALE_KEYS, "bias"):
            if all(f"{n}.{extra}" in sd for n in names):
                out[f"{stem}.qkv.{extra}"] = torch.cat([sd[f"{n}.{extra}"].reshape(sd[f"{n}.weight"].shape[0], -1) if extra != "bias" else sd[f"{n}.{extra}"]
                                                       for n in names], 0)
        if f"{names[0]}.{RECORD}" in sd:
            out[f"{stem}.qkv.{RECORD}"] = sd[f"{names[0]}.{RECORD}"]
        for n in names:
            for extra in ("weight", *SCALE_KEYS, "bias", RECORD):
                out.pop(f"{n}.{extra}", None)
    return out
