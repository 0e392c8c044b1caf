"""Per-step callbacks of the training loop: throughput / MFU, VRAM, the step line and metric
rows, the non-finite guard with its repro dump, trace / profile windows.

Counterparts of `src/kohakumoss/training/callbacks/{monitor,finite,repro,progress}.py` and the
trace windows of `parallel/telemetry/trace.py:22-110`.
"""

from __future__ import annotations

import time
from pathlib import Path

import torch

from ..models.flops import PEAK_TFLOPS, step_flops
from ..utils.log import get_logger

log = get_logger("train")


class Throughput:
    """samples/s, tokens/s, model TFLOP/s and MFU over the window since the last row."""

    def __init__(self, cfg, trainable_base: bool, checkpointing: bool, world: int = 1, peak_tflops: float | None = None,
                 reduce=None):
        self.cfg, self.trainable_base, self.checkpointing, self.world = cfg, trainable_base, checkpointing, world
        self.peak = peak_tflops or PEAK_TFLOPS["B200"]["bf16"]
        self.reduce = reduce
        self.reset()

    def reset(self):
        self.t0, self.tokens, self.joint, self.samples, self.flops = time.perf_counter(), 0, 0, 0, 0.0

    def observe(self, host_batches) -> None:
        for hb in host_batches:
            self.tokens += hb.image_tokens
            self.joint += hb.joint_tokens
            self.samples += hb.samples
            self.flops += step_flops(self.cfg, hb.seq.attn_joint.lengths, self.trainable_base, self.checkpointing,
                                     n_img=hb.seq.n_img, n_txt=hb.seq.n_txt)

    def row(self) -> dict:
        dt = max(1e-9, time.perf_counter() - self.t0)
        tokens, samples = self.tokens, self.samples
        if self.reduce is not None and self.world > 1:
            t = self.reduce(torch.tensor([float(tokens), float(samples)], device=self.reduce_device))
            tokens, samples = t.tolist()
        tf = self.flops / dt / 1e12
        out = {"speed/tokens_per_s": tokens / dt, "speed/joint_tokens_per_s": self.joint / dt * (self.world if self.reduce is None else 1),
               "speed/samples_per_s": samples / dt, "speed/tflops_per_gpu": tf, "speed/mfu": tf / self.peak}
        self.reset()
        return out


class FiniteGuard:
    """Counts consecutive skipped (non-finite) steps; past `patience` it dumps a repro file and
    stops the run (`NONFINITE_PATIENCE`)."""

    def __init__(self, patience: int, run_dir: Path):
        self.patience, self.run_dir, self.bad = patience, Path(run_dir), 0

    def observe(self, ok: bool, step: int, trainer=None, host_batches=None) -> None:
        self.bad = 0 if ok else self.bad + 1
        if self.patience and self.bad >= self.patience:
            path = self.run_dir / "instability" / "repro_step.pt"
            path.parent.mkdir(parents=True, exist_ok=True)
            payload = {"step": step, "loss": trainer.bundle.last_loss if trainer else None,
                       "batches": [{"hw": hb.hw, "text_len": hb.text_len, "index": hb.index} for hb in (host_batches or [])],
                       "rng": trainer.step_fn.rng_state() if trainer else None}
            torch.save(payload, path)
            raise RuntimeError(f"{self.bad} consecutive non-finite steps; repro written to {path}")


class StepTrace:
    """`TRACE_STEPS=(a, b)`: torch.profiler over steps a+1..b, one trace per rank;
    `PROFILE_STEPS=(a, b)`: cudaProfilerStart / Stop window for external profilers."""

    def __init__(self, trace_steps, profile_steps, run_dir: Path, rank: int):
        self.trace, self.profile = tuple(trace_steps or ()), tuple(profile_steps or ())
        self.run_dir, self.rank, self.prof = Path(run_dir), rank, None

    def before(self, step: int) -> None:
        if self.trace and step == self.trace[0]:
            from torch.profiler import ProfilerActivity, profile

            self.prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA])
            self.prof.__enter__()
        if self.profile and step == self.profile[0] and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStart()

    def after(self, step: int) -> None:
        if self.prof is not None and step + 1 == self.trace[1]:
            self.prof.__exit__(None, None, None)
            out = self.run_dir / "ranks"
            out.mkdir(parents=True, exist_ok=True)
            self.prof.export_chrome_trace(str(out / f"trace.rank{self.rank}.json.gz"))
            self.prof = None
        if self.profile and step + 1 == self.profile[1] and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStop()


def vram_row(device) -> dict:
    if torch.device(device).type != "cuda":
        return {}
    return {"mem/peak_gb": torch.cuda.max_memory_allocated(device) / 2**30, "mem/reserved_gb": torch.cuda.memory_reserved(device) / 2**30}
