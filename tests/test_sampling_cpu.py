"""Sampler: schedule parity with the upstream module, packed CFG = two-pass CFG, pipeline API."""

import importlib.util

import torch

from kohakumosstrainer_b200.diffusion import MossTimestep, moss_sigmas
from kohakumosstrainer_b200.inference.pipeline import MossPipeline, synthetic_requests


def test_schedule_and_timestep_match_reference(reference):
    spec = importlib.util.spec_from_file_location("ref_sched", reference / "kohakumoss/diffusion/sampling/schedule.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for steps, shift in ((50, 5.0), (32, 5.0), (20, 3.0)):
        assert torch.equal(moss_sigmas(steps, shift), mod.moss_sigmas(steps, shift))
    import kohakumoss.diffusion.timestep.moss as ref_t

    g1, g2 = torch.Generator().manual_seed(3), torch.Generator().manual_seed(3)
    assert torch.equal(MossTimestep().sample(64, g1, 0), ref_t.MossTimestep().sample(64, g2, 0))
    assert torch.equal(MossTimestep(schedule="tech_report").sample(64, g1, 150000),
                       ref_t.MossTimestep(schedule="tech_report").sample(64, g2, 150000))


def test_packed_cfg_equals_two_pass_and_is_seed_deterministic():
    pipe = MossPipeline.from_pretrained(variant="tiny", device="cpu", arch_overrides={"text_dim": 64})
    reqs = synthetic_requests(3, 64, (128, 192), text_tokens=7, dtype=torch.float32)
    a = pipe.generate(reqs, steps=4, batch=2)
    b = pipe.generate(reqs, steps=4, batch=2, cfg_mode="two_pass")
    c = pipe.generate(reqs[::-1], steps=4, batch=3)
    assert [tuple(z.shape) for z in a["latents"]] == [(1, 128, 8, 12)] * 3
    for x, y in zip(a["latents"], b["latents"]):
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-5)
    # a sample depends only on its own seed, size and text, not on its batch neighbours
    torch.testing.assert_close(a["latents"][0], c["latents"][2], rtol=1e-4, atol=1e-5)


def test_skip_layers_outside_depth_raise():
    import pytest

    pipe = MossPipeline.from_pretrained(variant="tiny", device="cpu", arch_overrides={"text_dim": 64})
    reqs = synthetic_requests(1, 64, (64, 64), text_tokens=3, dtype=torch.float32)
    with pytest.raises(ValueError, match="outside"):
        pipe.generate(reqs, steps=2, skip_layers="22")
