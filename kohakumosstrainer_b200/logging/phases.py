"""Profiler phase ranges `kohakumoss.{data,forward,backward,recompute,optimizer}`: visible in
torch.profiler traces and Nsight timelines (`src/kohakumoss/logging/phases.py:5-18`)."""

from contextlib import contextmanager

import torch

PHASES = ("data", "forward", "backward", "recompute", "optimizer")


@contextmanager
def phase(name: str):
    with torch.profiler.record_function(f"kohakumoss.{name}"):
        yield
