"""Where metric rows go: the console step line, `metrics.jsonl`, optionally wandb
(`src/kohakumoss/logging/sinks.py:64-177`)."""

from __future__ import annotations

import json
import time
from pathlib import Path

from ..utils.log import get_logger
from .keys import level_allows

log = get_logger("train")


class ConsoleSink:
    def write(self, step: int, row: dict) -> None:
        parts = [f"step {step}"]
        for k, v in row.items():
            name = k.split("/", 1)[-1]
            parts.append(f"{name}={v:.5g}" if isinstance(v, float) else f"{name}={v}")
        log.info(" ".join(parts))

    def close(self) -> None:
        pass


class JsonlSink:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.file = open(self.path, "a")

    def write(self, step: int, row: dict) -> None:
        self.file.write(json.dumps({"step": step, "time": time.time(), **row}) + "\n")
        self.file.flush()

    def close(self) -> None:
        self.file.close()


class WandbSink:
    """Optional: imported lazily; resumes the run id stored in the run directory."""

    def __init__(self, project: str, run_dir: Path, name: str = "", config: dict | None = None):
        import wandb  # noqa: PLC0415

        id_file = Path(run_dir) / "wandb_id.txt"
        run_id = id_file.read_text().strip() if id_file.exists() else wandb.util.generate_id()
        id_file.write_text(run_id)
        self.run = wandb.init(project=project, name=name or None, id=run_id, resume="allow", config=config or {})

    def write(self, step: int, row: dict) -> None:
        self.run.log(row, step=step)

    def close(self) -> None:
        self.run.finish()


class MetricWriter:
    def __init__(self, sinks: list, level: str = "train"):
        self.sinks, self.level = sinks, level

    def write(self, step: int, row: dict) -> None:
        row = {k: v for k, v in row.items() if v is not None and level_allows(self.level, k)}
        for s in self.sinks:
            s.write(step, row)

    def close(self) -> None:
        for s in self.sinks:
            s.close()


def build_writer(logger: str, run_dir: Path, level: str = "train", project: str = "kohakumoss", name: str = "",
                 config: dict | None = None, rank: int = 0) -> MetricWriter:
    if rank != 0:
        return MetricWriter([], level)
    sinks = [ConsoleSink(), JsonlSink(Path(run_dir) / "metrics.jsonl")]
    if logger == "wandb":
        try:
            sinks.append(WandbSink(project, run_dir, name, config))
        except ImportError:
            log.warning("LOGGER='wandb' but wandb is not installed; console + metrics.jsonl only")
    return MetricWriter(sinks, level)
