"""Metric sinks (console + metrics.jsonl, optional wandb), metric key groups, profiler phases."""

from .sinks import ConsoleSink, JsonlSink, MetricWriter, WandbSink, build_writer
from .keys import GROUPS, level_allows
from .phases import PHASES, phase

__all__ = ["ConsoleSink", "JsonlSink", "MetricWriter", "WandbSink", "build_writer", "GROUPS", "level_allows", "PHASES", "phase"]
