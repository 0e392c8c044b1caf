"""Varlen tcgen05 attention against an explicit fp32 softmax(QK^T)V per segment."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(x, y):
    return ((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-12)).item()


def _make(lengths, heads, seed, fused=False, scale_q=1.0):
    n = sum(lengths)
    g = torch.Generator(device="cuda").manual_seed(seed)
    if fused:  # views of one [N, 3, H, 128] projection, like the fused qkv GEMM output
        qkv = torch.randn(n, 3, heads, 128, device="cuda", generator=g).bfloat16()
        q, k, v = qkv.unbind(1)
    else:
        q, k, v = (torch.randn(n, heads, 128, device="cuda", generator=g).bfloat16() for _ in range(3))
    return (q * scale_q).bfloat16() if scale_q != 1.0 else q, k, v


def _cu(lengths):
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    return cu.cuda()


@pytest.mark.parametrize("lengths", [(128,), (64,), (200, 77, 1), (4352, 1300), (333, 129, 640, 17)])
@pytest.mark.parametrize("fused", [False, True])
def test_forward_matches_fp32_reference(lengths, fused):
    from kohakumosstrainer_b200.ops import attention, eager, native

    q, k, v = _make(lengths, 3, sum(lengths), fused)
    scale = 128 ** -0.5
    o = attention.attention_varlen(q, k, v, _cu(lengths), max(lengths), scale, lengths)
    native.check_status()
    ref = eager.attention_varlen_math(q, k, v, lengths, scale, torch.float32)
    assert o.shape == q.shape
    assert _rel(o, ref) < 8e-3


def test_forward_large_logits_need_rescale():
    """Scores spread over hundreds of log2 units force the lazy O rescale path."""
    from kohakumosstrainer_b200.ops import attention, eager, native

    lengths = (700, 300)
    q, k, v = _make(lengths, 2, 5, scale_q=6.0)
    scale = 128 ** -0.5
    o = attention.attention_varlen(q, k, v, _cu(lengths), max(lengths), scale, lengths)
    native.check_status()
    ref = eager.attention_varlen_math(q, k, v, lengths, scale, torch.float32)
    assert torch.isfinite(o.float()).all()
    assert _rel(o, ref) < 1.5e-2


def test_backward_matches_fp32_reference():
    from kohakumosstrainer_b200.ops import attention, eager, native

    lengths = (300, 140, 64)
    q, k, v = _make(lengths, 2, 9)
    scale = 128 ** -0.5
    qs, ks, vs = (t.clone().requires_grad_() for t in (q, k, v))
    o = attention.attention_varlen(qs, ks, vs, _cu(lengths), max(lengths), scale, lengths)
    do = torch.randn_like(o)
    o.backward(do)
    native.check_status()
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = eager.attention_varlen_math(qr, kr, vr, lengths, scale, torch.float32)
    ref.backward(do.float())
    assert _rel(qs.grad, qr.grad) < 2e-2
    assert _rel(ks.grad, kr.grad) < 2e-2
    assert _rel(vs.grad, vr.grad) < 2e-2
