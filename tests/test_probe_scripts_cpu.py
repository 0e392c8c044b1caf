"""The probe scripts run end to end on random-init small models on the host (what they report on real weights
is a study, what is checked here is that the tooling works and its invariants hold)."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def run(script, *args, timeout=300):
    proc = subprocess.run([sys.executable, str(ROOT / script), *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout


@pytest.mark.parametrize("algo", ["lokr", "boft"])
def test_adapter_round_trip_probe(tmp_path, algo):
    out = run("scripts/probe/adapter_e2e.py", "--device", "cpu", "--algo", algo, "--out", str(tmp_path))
    report = json.loads(out.strip().splitlines()[-1])
    assert set(report["cases"]) == {"lycoris/merge", "lycoris/bypass", "comfy/merge", "comfy/bypass"}
    assert report["worst"] < 1e-5


def test_embed_and_fp16_study_probes(tmp_path):
    run("scripts/probe/embed.py", "--out", str(tmp_path / "embeds.pt"), "--text-dim", "64")
    import torch

    saved = torch.load(tmp_path / "embeds.pt")
    assert len(saved["positive"]) == len(saved["prompts"]) - 1 and saved["negative"].shape[1] == 64
    run("scripts/probe/fp16_study.py", "--device", "cpu", "--factors", "1,16", "--seeds", "0", "--out", str(tmp_path / "study"))
    report = json.loads((tmp_path / "study" / "fp16_study.json").read_text())
    assert [r["c"] for r in report["sweep"]] == [1.0, 16.0]
    assert report["sweep"][1]["stream_peak"] < report["sweep"][0]["stream_peak"]     # the fold shrinks the stream
    assert report["sweep"][0]["fp32_fold_error"] == 0.0
