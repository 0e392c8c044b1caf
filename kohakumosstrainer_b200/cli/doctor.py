"""Environment report: OS, Python, torch, GPUs, toolchain, the native extension and its ops,
peer-access / symmetric-memory availability, and what the install lacks for this machine.

    python -m kohakumosstrainer_b200.cli.doctor [--json report.json] [--memory] [--smoke]

The report holds no paths, host or user names (role of `src/kohakumoss/cli/doctor.py` in the
reference). `--smoke` runs one tiny tcgen05 GEMM against a PyTorch product on the first GPU.
"""

from __future__ import annotations

import argparse
import importlib.metadata as metadata
import json
import platform
import re
import shutil
import subprocess
import sys

import torch

PACKAGES = ("torch", "numpy", "safetensors", "transformers", "diffusers", "pillow", "pyarrow", "tqdm", "wandb")
PATH_RE = re.compile(r"[A-Za-z]:[\\/][^\s'\",;]*|(?<![\w.])/[\w.-]+/[^\s'\",;]*")


def versions() -> dict:
    out = {}
    for name in PACKAGES:
        try:
            out[name] = metadata.version(name)
        except metadata.PackageNotFoundError:
            out[name] = None
    return out


def devices() -> list[dict]:
    out = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out.append({"index": i, "name": p.name, "capability": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                        "memory_gib": round(p.total_memory / 2**30, 2), "native_target": (p.major, p.minor) == (10, 0)})
    return out


def toolchain() -> dict:
    out = {}
    for tool in ("nvcc", "g++", "ninja", "ncu"):
        path = shutil.which(tool)
        ver = None
        if path and tool in ("nvcc", "g++"):
            try:
                text = subprocess.run([tool, "--version"], capture_output=True, text=True, timeout=20).stdout
                m = re.search(r"release ([\d.]+)|\) ([\d.]+)", text)
                ver = next((g for g in (m.groups() if m else ()) if g), None)
            except (OSError, subprocess.SubprocessError):
                pass
        out[tool] = {"found": bool(path), "version": ver}
    return out


def extension() -> dict:
    from ..csrc import build as build_mod

    info = {"built": build_mod.is_current() if hasattr(build_mod, "is_current") else None, "ops": []}
    try:
        from ..ops import native

        ops = native.load()
        info["loaded"] = True
        known = ("gemm", "attention_fwd", "attention_bwd", "rms_norm_mod_fwd", "adamw_multi", "allreduce", "reduce_scatter_adamw",
                 "allgather", "group_hadamard", "quantize_int8_rows", "quantize_mxfp8", "quantize_fp8_tensor")
        info["ops"] = [n for n in known if hasattr(ops, n)]
    except Exception as exc:  # report, never raise: the doctor runs on broken installs
        info["loaded"] = False
        info["error"] = PATH_RE.sub("<path>", f"{type(exc).__name__}: {exc}")[:300]
    return info


def peer_matrix() -> list[list[bool]] | None:
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        return None
    n = torch.cuda.device_count()
    return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]


def missing(report: dict) -> list[str]:
    """One line per thing this machine lacks, with what fixes it."""
    out = []
    if not report["devices"]:
        out.append("no CUDA device: only the CPU reference paths (tests, config checks, data tools) run here")
    for d in report["devices"]:
        if not d["native_target"]:
            out.append(f"GPU {d['index']} ({d['name']}, sm_{d['capability'].replace('.', '')}) is not sm_100: the native kernels target B200 only")
    if not report["toolchain"]["nvcc"]["found"]:
        out.append("nvcc not found: the extension cannot be rebuilt (a built _C.so in the tree still loads)")
    if not report["extension"].get("loaded") and report["devices"]:
        out.append("the native extension did not load: run `python -c 'import __graft_entry__ as g; g.build()'` at the repository root")
    for pkg, why in (("safetensors", "model and adapter files"), ("pillow", "image datasets"), ("transformers", "the text encoder")):
        if report["packages"].get(pkg) is None:
            out.append(f"package {pkg} is missing: needed for {why}")
    if report["packages"].get("diffusers") is None:
        out.append("package diffusers is missing: the VAE wrapper cannot load (training from latent caches and latent sampling still work)")
    return out


def smoke() -> dict:
    from ..ops import native

    a = torch.randn(256, 512, device="cuda").bfloat16()
    b = torch.randn(384, 512, device="cuda").bfloat16()
    got = native.gemm(a, b).float()
    ref = a.float() @ b.float().t()
    native.check_status()
    return {"gemm_rel_error": float((got - ref).abs().max() / ref.abs().max())}


def collect(memory: bool = False, run_smoke: bool = False) -> dict:
    report = {"os": platform.system(), "os_release": platform.release(), "python": platform.python_version(), "torch": torch.__version__,
              "cuda_runtime": torch.version.cuda, "packages": versions(), "devices": devices(), "toolchain": toolchain(),
              "extension": extension(), "peer_access": peer_matrix(),
              "symmetric_memory": bool(torch.cuda.is_available() and hasattr(torch.distributed, "_symmetric_memory"))}
    if memory:
        from ..memory import ORDER, MemoryPlan, Workload, estimate, resolve_profile
        from ..types.arch import PRESETS

        work = Workload(PRESETS["base"], 18000, 2000, trainable_params=60_000_000, stored_precision="fp8_compute")
        report["memory_profiles_gib"] = {n: round(estimate(work, resolve_profile({"MEMORY_PROFILE": n}))["total"] / 2**30, 1) for n in ORDER}
        del MemoryPlan
    if run_smoke and report["devices"]:
        report["smoke"] = smoke()
    report["missing"] = missing(report)
    return report


def render(report: dict) -> str:
    lines = [f"python {report['python']}  torch {report['torch']}  cuda {report['cuda_runtime']}  {report['os']} {report['os_release']}"]
    for d in report["devices"]:
        lines.append(f"gpu{d['index']}: {d['name']} sm_{d['capability'].replace('.', '')} {d['sms']} SMs {d['memory_gib']} GiB"
                     + ("" if d["native_target"] else "  (not a native target)"))
    lines.append("toolchain: " + ", ".join(f"{k}={'yes' if v['found'] else 'no'}{' ' + v['version'] if v['version'] else ''}" for k, v in report["toolchain"].items()))
    ext = report["extension"]
    lines.append(f"extension: loaded={ext.get('loaded')} ops={len(ext.get('ops', []))}" + (f" error={ext['error']}" if ext.get("error") else ""))
    lines.append("packages: " + ", ".join(f"{k}={v or '-'}" for k, v in report["packages"].items()))
    if report.get("peer_access"):
        lines.append("peer access: " + ("all pairs" if all(all(r) for r in report["peer_access"]) else "partial"))
    if "memory_profiles_gib" in report:
        lines.append("memory profiles (LoRA r8, fp8 base, 20k tokens): " + ", ".join(f"{k}={v} GiB" for k, v in report["memory_profiles_gib"].items()))
    if "smoke" in report:
        lines.append(f"smoke: gemm relative error {report['smoke']['gemm_rel_error']:.2e}")
    lines += ["missing:"] + [f"  - {m}" for m in report["missing"]] if report["missing"] else ["missing: nothing"]
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kmoss-doctor", description=__doc__)
    ap.add_argument("--json", default="")
    ap.add_argument("--memory", action="store_true")
    ap.add_argument("--smoke", action="store_true")
    args = ap.parse_args(argv)
    report = collect(args.memory, args.smoke)
    print(render(report))
    if args.json:
        with open(args.json, "w", encoding="utf-8") as f:
            json.dump(report, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
