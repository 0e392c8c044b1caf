"""Parallel engines: launcher + store gates, symmetric memory, DDP, FSDP, pipelines."""

from .launch import ParallelPlan, default_backend, spawn

__all__ = ["ParallelPlan", "default_backend", "spawn"]
