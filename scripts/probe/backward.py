"""Backward parity of one joint block: gradients of the native path against the eager fp32 path on the same inputs,
relative error per input / parameter (role of `scripts/probe/backward.py`). Needs a GPU."""

TOKENS = 2048
ALGO = "lora"
DEVICE = "cuda"

globals().update(globals().pop("__kmoss_overrides__", {}))


def main():
    import torch

    from kohakumosstrainer_b200.data import SyntheticConfig, SyntheticDataset
    from kohakumosstrainer_b200.training.trainer import Trainer, TrainerConfig

    if not torch.cuda.is_available():
        raise SystemExit("needs a GPU")
    data = SyntheticDataset(SyntheticConfig(max_tokens=int(TOKENS), min_area=256 * 256, max_area=512 * 512, seed=3))
    hb = data.materialize(0)
    out = {}
    grads = {}
    for kernels in ({}, {"all": "eager"}):
        cfg = TrainerConfig(variant="base", arch_overrides={"depth": 2}, algo=ALGO, dim=8, alpha=8.0, base_precision="auto", kernels=kernels,
                            schedule={"mode": "constant"}, grad_clip=0.0)
        tr = Trainer(cfg, device=DEVICE)
        batch = hb.to_device(tr.device, torch.float32, tr.dtype)
        loss = tr.step_fn(batch, float(hb.image_tokens))
        loss.backward()
        grads["eager" if kernels else "native"] = {n: p.grad.detach().float().clone() for n, p in tr.named_trainable if p.grad is not None}
        out["eager" if kernels else "native"] = float(loss)
    worst = sorted(((float((grads["native"][n] - g).norm() / g.norm().clamp_min(1e-12)), n) for n, g in grads["eager"].items()), reverse=True)[:8]
    print(f"loss native {out['native']:.6f} eager {out['eager']:.6f}")
    for err, name in worst:
        print(f"{err:.3e}  {name}")
    return worst


if __name__ == "__main__":
    main()
