"""`python -m kohakumosstrainer_b200.cli.config_cmd {list,new,wizard,check}`: compose starter
configs from the layered presets under `configs/` and validate any config through the knob
checks of the script it drives (role of `src/kohakumoss/cli/config/*` in the reference).

    ... config_cmd list                                    # layers and their configs
    ... config_cmd new my.py --algo lora --data kohya --parallel ddp --precision fp8 --set DIM=16
    ... config_cmd wizard my.py                            # the same, asked interactively
    ... config_cmd check my.py [--script scripts/train/moss.py] [--set KEY=VALUE]
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

from ..config import ConfigError, apply_sets, check, load_config, script_knobs

ROOT = Path(__file__).resolve().parents[2]
LAYERS = ("_base", "algo", "data", "parallel", "precision", "vram", "weights", "recipes", "scale", "quality")


def layers(root: Path = ROOT) -> dict[str, list[str]]:
    out = {}
    base = root / "configs" / "moss"
    for layer in LAYERS:
        folder = base / layer
        if folder.is_dir():
            out[layer] = sorted(p.stem.split("_", 1)[1] if "_" in p.stem else p.stem for p in folder.glob("*.py"))
    return out


def layer_path(layer: str, name: str, root: Path = ROOT) -> str:
    stem = layer.lstrip("_")
    path = root / "configs" / "moss" / layer / f"{stem}_{name}.py"
    if not path.exists():
        have = ", ".join(layers(root).get(layer, []))
        raise SystemExit(f"no config {layer}/{stem}_{name}.py (have: {have})")
    return f"moss/{layer}/{stem}_{name}"


def compose(choices: dict[str, str], sets: list[str], root: Path = ROOT) -> str:
    """Text of a config that `use_config`s the chosen layers and then sets the overrides."""
    lines = ['"""Composed by the config command: edit freely."""', ""]
    for layer in LAYERS:
        name = choices.get(layer.lstrip("_"))
        if name:
            lines.append(f'use_config("{layer_path(layer, name, root)}")')
    lines.append("")
    for item in sets:
        key, _, value = item.partition("=")
        lines.append(f"{key.strip()} = {value.strip()}")
    return "\n".join(lines) + "\n"


def validate(path: str, script: str, sets: list[str], root: Path = ROOT) -> dict:
    defaults = script_knobs(root / script)
    knobs = {**defaults, **load_config(path, [root / "configs", root])}
    knobs = apply_sets(knobs, sets)
    if Path(script).name == "moss.py":
        from ..training.knobs import CHOICES, cross_checks

        return check(knobs, defaults, CHOICES, (cross_checks,))
    return check(knobs, defaults)


def _ask(prompt: str, options: list[str], default: str, read=input) -> str:
    text = read(f"{prompt} [{'/'.join(options)}] ({default}): ").strip()
    if not text:
        return default
    if text not in options:
        raise SystemExit(f"{text!r} is not one of {options}")
    return text


def wizard(read=input, root: Path = ROOT) -> tuple[dict, list[str]]:
    have = layers(root)
    choices = {"base": _ask("what do you train", have.get("_base", ["lora"]), "lora", read)}
    for layer, default in (("algo", "lora"), ("data", "synthetic"), ("parallel", ""), ("precision", "fp8")):
        options = have.get(layer, [])
        if options:
            pick = _ask(layer, options + [""], default if default in options else "", read)
            if pick:
                choices[layer] = pick
    sets = []
    tokens = read("MAX_TOKENS per packed batch (20480): ").strip()
    if tokens:
        sets.append(f"MAX_TOKENS={int(tokens)}")
    return choices, sets


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kmoss-config", description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    new = sub.add_parser("new")
    new.add_argument("out")
    for layer in LAYERS:
        new.add_argument(f"--{layer.lstrip('_')}", default="")
    new.add_argument("--set", dest="sets", action="append", default=[])
    wiz = sub.add_parser("wizard")
    wiz.add_argument("out")
    chk = sub.add_parser("check")
    chk.add_argument("config")
    chk.add_argument("--script", default="scripts/train/moss.py")
    chk.add_argument("--set", dest="sets", action="append", default=[])
    args = ap.parse_args(argv)
    if args.cmd == "list":
        for layer, names in layers().items():
            print(f"{layer}: {', '.join(names)}")
        return 0
    if args.cmd in ("new", "wizard"):
        if args.cmd == "new":
            choices = {layer.lstrip("_"): getattr(args, layer.lstrip("_")) for layer in LAYERS}
            sets = args.sets
        else:
            choices, sets = wizard()
        text = compose(choices, sets)
        Path(args.out).write_text(text, encoding="utf-8")
        try:
            validate(args.out, "scripts/train/moss.py", [])
        except ConfigError as err:
            print(f"wrote {args.out}, but it does not validate:\n{err}")
            return 1
        print(f"wrote {args.out} (validates against scripts/train/moss.py)")
        return 0
    try:
        knobs = validate(args.config, args.script, args.sets)
    except ConfigError as err:
        print(err)
        return 1
    print(f"{args.config}: ok ({len(knobs)} knobs)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
