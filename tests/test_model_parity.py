"""CPU fp32 parity of the tiny DiT against the upstream implementation.

Tiny MOSS-style DiT (4 blocks, hidden 256, 4 heads, head_dim 64), packed batch of three
samples with latent grids 16x16, 12x20, 8x8 and text lengths 32, 17, 50, logit-normal
sigmas, rectified-flow velocity target: one forward + backward, outputs and every
parameter gradient compared.
"""

import pytest
import torch

from kohakumosstrainer_b200.models import build_backbone
from kohakumosstrainer_b200.types import MossArchConfig, build_seqinfo

CFG = dict(dim=256, depth=4, heads=4, ffn_dim=512, text_dim=256, text_blocks=2)


def _batch(seed=0):
    g = torch.Generator().manual_seed(seed)
    hw = torch.tensor([[16, 16], [12, 20], [8, 8]])
    tl = torch.tensor([32, 17, 50])
    n_img = int((hw[:, 0] * hw[:, 1]).sum())
    z0 = torch.randn(n_img, 128, generator=g)
    eps = torch.randn(n_img, 128, generator=g)
    text = torch.randn(int(tl.sum()), 256, generator=g)
    sigma = torch.sigmoid(torch.randn(3, generator=g))
    return hw, tl, z0, eps, text, sigma


def test_forward_backward_matches_reference(reference):
    from kohakumoss.model.backbone import MossBackbone as RefBackbone
    from kohakumoss.model.opset import OpSet as RefOpSet
    from kohakumoss.types.arch import MossArchConfig as RefCfg
    from kohakumoss.types.seqinfo import build_seqinfo as ref_seqinfo

    ours = build_backbone(MossArchConfig(**CFG), seed=0)
    ref = RefBackbone(RefCfg(**CFG))
    ref.load_state_dict(ours.state_dict(), strict=True)
    ref.bind_ops(RefOpSet.resolve("cpu", torch.float32, {n: "eager" for n in (
        "rms_norm", "rms_norm_mod", "qk_norm_rope", "attention_varlen", "situ_glu",
        "gated_residual", "token_mse", "linear_qk_rope", "linear_situ", "linear_gated_residual")}))

    hw, tl, z0, eps, text, sigma = _batch()
    seq, rseq = build_seqinfo(hw, tl), ref_seqinfo(hw, tl)
    for name in ("seg_img", "seg_txt", "seg_joint", "pos_txt", "pos_joint", "img_in_joint",
                 "txt_in_joint", "cu_img", "cu_txt"):
        assert torch.equal(getattr(seq, name), getattr(rseq, name)), name
    assert torch.equal(seq.attn_joint.cu_seqlens, rseq.attn_joint.cu_seqlens)

    s = sigma.index_select(0, seq.seg_img.long()).unsqueeze(-1)
    z = z0 + s * (eps - z0)
    target = eps - z0
    v = ours(z, text, sigma, seq)
    rv = ref(z, text, sigma, rseq)
    assert v.shape == (560, 128)
    torch.testing.assert_close(v, rv, rtol=1e-5, atol=1e-5)

    (v - target).square().mean().backward()
    (rv - target).square().mean().backward()
    rgrads = dict(ref.named_parameters())
    checked = 0
    for name, p in ours.named_parameters():
        assert p.grad is not None, name
        torch.testing.assert_close(p.grad, rgrads[name].grad, rtol=2e-4, atol=1e-6, msg=name)
        checked += 1
    assert checked > 50


def test_state_dict_keys_match_reference(reference):
    from kohakumoss.model.backbone import MossBackbone as RefBackbone
    from kohakumoss.types.arch import MossArchConfig as RefCfg

    ours = build_backbone(MossArchConfig(**CFG), seed=0)
    ref = RefBackbone(RefCfg(**CFG))
    ok, rk = dict(ours.state_dict()), dict(ref.state_dict())
    assert set(ok) == set(rk)
    for k in ok:
        assert ok[k].shape == rk[k].shape, k


def test_segment_skip_masks_only_flagged_samples():
    model = build_backbone(MossArchConfig(**CFG), seed=1)
    hw, tl, z0, eps, text, sigma = _batch(1)
    seq = build_seqinfo(hw, tl)
    full = model(z0, text, sigma, seq)
    skipped = model.bind_forward(skip_layers=(2,))(z0, text, sigma, seq)
    mask = torch.tensor([False, True, False])
    mixed = model.bind_forward(segment_skip_layers=(2,))(z0, text, sigma, seq, mask)
    seg = seq.seg_img.long()
    torch.testing.assert_close(mixed[seg != 1], full[seg != 1])
    torch.testing.assert_close(mixed[seg == 1], skipped[seg == 1])
    assert not torch.allclose(full[seg == 1], skipped[seg == 1])


def test_seqinfo_img_keep_positions():
    hw = torch.tensor([[4, 4], [2, 3]])
    tl = torch.tensor([3, 2])
    keep = [torch.tensor([0, 5, 15]), None]
    seq = build_seqinfo(hw, tl, img_keep=keep)
    assert seq.n_img == 3 + 6 and seq.n_joint == 3 + 3 + 6 + 2
    full = build_seqinfo(hw, tl)
    torch.testing.assert_close(seq.pos_joint[:3], full.pos_joint[[0, 5, 15]])
    assert seq.attn_joint.lengths == (6, 8)
