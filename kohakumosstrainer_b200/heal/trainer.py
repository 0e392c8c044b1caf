"""Heal trainer: the shrunk student is distilled from the original model while the channel
weights of its norms anneal to 1, so it ends as a plain DiT without massive channels.

Loss = rel_sq(v_student, v_teacher) + hard_weight * rel_sq(v_student, target) + conc_weight *
top-k energy share of the block outputs (`src/kohakumoss/heal/losses.py:12-60`). Only the stream
writers train (AdamW); data parallel ranks average gradients with a plain all-reduce
(`src/kohakumoss/heal/trainer.py:188`). `merge_student` writes the healed weights as an
ordinary transformer file; `rescale_stream` is the exact uniform rescale of the stream.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor

from ..diffusion.objective import noise_latents
from ..training.extras import top_share
from .channels import apply_shrink, channel_mean_square, peak_ratio, reader_norms, shrink_scales, top_channels, writer_params
from .wnorm import WeightedOps, anneal_lam, anneal_t


@dataclass
class HealConfig:
    tau: float = 8.0                 # channels above tau x the median RMS are shrunk to it
    steps: int = 1000
    anneal_steps: int = 600
    warmup: int = 20
    lr: float = 1e-5
    hard_weight: float = 0.0
    conc_weight: float = 0.0
    conc_k: int = 8
    calib_batches: int = 4
    seed: int = 0


def rel_sq(a: Tensor, b: Tensor) -> Tensor:
    a, b = a.float(), b.float()
    return (a - b).square().sum() / b.square().sum().clamp_min(torch.finfo(torch.float32).tiny)


def lr_scale(step: int, total: int, warmup: int) -> float:
    import math

    if step < warmup:
        return (step + 1) / max(1, warmup)
    return 0.5 * (1 + math.cos(math.pi * (step - warmup) / max(1, total - warmup)))


class Heal:
    def __init__(self, model, cfg: HealConfig, dataset, device="cpu", dtype=torch.float32):
        self.cfg, self.dataset, self.device, self.dtype = cfg, dataset, torch.device(device), dtype
        self.teacher = model.eval().requires_grad_(False)
        self.student = copy.deepcopy(model).train()
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.step_index = 0
        self.sigma_gen = torch.Generator().manual_seed(cfg.seed + 17 * self.rank)
        self.noise_gen = torch.Generator(self.device).manual_seed(cfg.seed + 31 * self.rank)
        self.report = self.calibrate()
        self.d = self.report["d"].to(self.device)
        apply_shrink(self.student, self.d)                     # writers x D, reader gains / D
        self.wops = WeightedOps(self.student.ops, self.student.cfg.dim, self.device)
        self.wops.lam = anneal_lam(self.d, 0.0)                # exact at t = 0
        self.student.bind_ops(self.wops)
        for p in self.student.parameters():
            p.requires_grad_(False)
        self.named = writer_params(self.student)
        for _, p in self.named:
            p.requires_grad_(True)
        self.opt = torch.optim.AdamW([p for _, p in self.named], lr=cfg.lr, betas=(0.9, 0.95), weight_decay=0.0)
        self.blocks: list[Tensor] = []
        if cfg.conc_weight > 0:
            for layer in self.student.layers:
                layer.register_forward_hook(lambda m, a, out: self.blocks.append(out))

    # -- calibration ------------------------------------------------------------------------------
    def _inputs(self, index: int, sigma_value: float | None = None):
        hb = self.dataset.materialize(index, self.rank, self.world)
        b = hb.to_device(self.device, torch.float32, self.dtype)
        seq = b.seq
        if sigma_value is None:
            sigma = torch.rand(seq.batch, generator=self.sigma_gen).to(self.device)
        else:
            sigma = torch.full((seq.batch,), sigma_value, device=self.device)
        eps = torch.randn(b.latents.shape, generator=self.noise_gen, device=self.device, dtype=torch.float32)
        z, target = noise_latents(b.latents.float(), eps, sigma, seq.seg_img)
        return z.to(self.dtype), b.text.to(self.dtype), sigma, seq, target

    def calibrate(self) -> dict:
        batches = [self._inputs(1_000_000 + i, 0.5) for i in range(self.cfg.calib_batches)]
        ms = channel_mean_square(self.teacher, batches, lambda b: self.teacher(b[0], b[1], b[2], b[3]))
        peak = peak_ratio(ms)
        d = shrink_scales(peak, self.cfg.tau)
        return {"peak": peak, "d": d, "top": top_channels(peak, 8), "shrunk": int((d < 1).sum())}

    # -- training -----------------------------------------------------------------------------------
    def train_step(self) -> dict:
        cfg = self.cfg
        t = anneal_t(self.step_index, cfg.anneal_steps)
        self.wops.lam = anneal_lam(self.d, t)
        for g in self.opt.param_groups:
            g["lr"] = cfg.lr * lr_scale(self.step_index, cfg.steps, cfg.warmup)
        z, text, sigma, seq, target = self._inputs(self.step_index)
        with torch.no_grad():
            v_t = self.teacher(z, text, sigma, seq)
        self.blocks.clear()
        v_s = self.student(z, text, sigma, seq)
        loss = soft = rel_sq(v_s, v_t)
        parts = {"soft": float(soft.detach())}
        if cfg.hard_weight > 0:
            hard = rel_sq(v_s, target)
            loss = loss + cfg.hard_weight * hard
            parts["hard"] = float(hard)
        if cfg.conc_weight > 0:
            conc = torch.stack([top_share(h, cfg.conc_k) for h in self.blocks]).mean()
            loss = loss + cfg.conc_weight * conc
            parts["conc"] = float(conc)
        self.opt.zero_grad(set_to_none=True)
        loss.backward()
        if self.world > 1:
            for _, p in self.named:
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad.div_(self.world)
        self.opt.step()
        self.step_index += 1
        return {"loss": float(loss.detach()), "t": t, **parts}

    @torch.no_grad()
    def evaluate(self, n: int = 2) -> dict:
        """rel_sq against the teacher at the CURRENT anneal point and as a plain model (lam = 1)."""
        out = {}
        for name, lam in (("current", self.wops.lam), ("plain", torch.ones_like(self.d))):
            keep, self.wops.lam = self.wops.lam, lam
            errs = []
            for i in range(n):
                z, text, sigma, seq, _ = self._inputs(2_000_000 + i, 0.5)
                errs.append(float(rel_sq(self.student(z, text, sigma, seq), self.teacher(z, text, sigma, seq))))
            self.wops.lam = keep
            out[name] = sum(errs) / len(errs)
        return out


def merge_student(heal: Heal):
    """The healed weights as a plain model (op set restored, lam = 1 assumed reached)."""
    student = heal.student
    student.bind_ops(heal.wops._ops)
    student.eval().requires_grad_(False)
    return student


@torch.no_grad()
def rescale_stream(model, c: float) -> dict:
    """Exact uniform rescale of the residual stream by 1 / c: writers / c and every reader norm's
    eps / c^2, so the function is unchanged to rounding (`src/kohakumoss/heal/rescale.py:13-40`)."""
    from ..models.numerics import fold_stream_scale

    before = {site: norm.eps for site, norm in reader_norms(model).items()}
    fold_stream_scale(model, c)
    for norm in reader_norms(model).values():
        norm.eps = norm.eps / (c * c)
    return before
