"""Rotation, int8 and MXFP8 kernels against plain PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from kohakumosstrainer_b200.quant import formats as F  # noqa: E402


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from kohakumosstrainer_b200.ops import native

    native.load()
    return native


@pytest.mark.parametrize("group", [4, 16, 64, 256, 1024])
def test_group_hadamard_matches_matrix(group):
    _dev()
    torch.manual_seed(group)
    x = torch.randn(300, 3072, device="cuda").bfloat16()
    y = F.group_hadamard(x, group)
    h = F.hadamard_matrix(group, torch.float32, "cuda")
    ref = (x.float().reshape(-1, group) @ h).reshape(x.shape)
    assert (y.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    back = F.group_hadamard(y, group)
    assert (back.float() - x.float()).abs().max() <= 3e-2 * x.float().abs().max()
    xg = x.clone().requires_grad_(True)
    F.group_hadamard(xg, group).backward(y)
    assert (xg.grad.float() - back.float()).abs().max() == 0       # self-adjoint: backward is the same kernel


@pytest.mark.parametrize("group", [0, 64])
def test_int8_row_quantiser(group):
    native = _dev()
    x = torch.randn(257, 8192, device="cuda").bfloat16() * torch.rand(257, 1, device="cuda").bfloat16() * 4
    q, s = native.load().quantize_int8_rows(x, group)
    v = x.float()
    if group:
        v = (v.reshape(-1, group) @ F.hadamard_matrix(group, torch.float32, "cuda")).reshape(v.shape)
    amax = v.abs().amax(1)
    assert torch.allclose(s, amax / 127, rtol=1e-5)
    ref = torch.clamp(torch.round(v / s[:, None]), -127, 127)
    assert (q.float() - ref).abs().max() <= 1          # a rounding tie may land on the neighbour
    assert ((q.float() - ref) != 0).float().mean() < 1e-3


def test_int8_gemm_is_exact_and_scaled():
    native = _dev()
    torch.manual_seed(1)
    M, N, K = 1000, 768, 3072
    a = torch.randint(-127, 128, (M, K), device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
    out = native.gemm(a, b, out_dtype=torch.float32)
    ref = (a.double() @ b.double().t())
    assert out.dtype == torch.float32 and (out.double() - ref).abs().max() == 0        # int32 accumulation, |sum| < 2^24
    rs, cs = torch.rand(M, device="cuda") + 0.5, torch.rand(N, device="cuda") + 0.5
    bias = torch.randn(N, device="cuda").bfloat16()
    y = native.gemm(a, b, row_scale=rs, col_scale=cs, bias=bias)
    ref2 = ref.float() * rs[:, None] * cs[None, :] + bias.float()
    assert (y.float() - ref2).abs().max() <= 1e-2 * ref2.abs().max()
    native.check_status()


def test_int8_widening_is_exact():
    native = _dev()
    q = torch.randint(-128, 128, (512, 4096), device="cuda", dtype=torch.int8)
    y = torch.empty(q.shape, device="cuda", dtype=torch.bfloat16)
    native.load().cast_int8_bf16(q, y)
    assert torch.equal(y.float(), q.float())


@pytest.mark.parametrize("group,compute", [(0, False), (0, True), (64, False), (64, True)])
def test_int8_linear_forward_backward(group, compute):
    _dev()
    torch.manual_seed(2)
    w = torch.randn(1536, 3072, device="cuda") * 0.03
    x = torch.randn(700, 3072, device="cuda").bfloat16().requires_grad_(True)
    bias = torch.randn(1536, device="cuda").bfloat16()
    iw = F.Int8Weight.from_dense(w, group, compute)
    y = iw.linear(x, bias)
    ref = x.float() @ w.t() + bias.float()
    assert (y.float() - ref).abs().max() <= (0.05 if compute else 0.03) * ref.abs().max()
    cpu = F.Int8Weight(iw.q.cpu(), iw.scale.cpu(), group, compute).linear(x.detach().float().cpu(), bias.float().cpu())
    assert (y.float().cpu() - cpu).abs().max() <= 2e-2 * cpu.abs().max()                  # same rounding points as the CPU path
    dy = torch.randn_like(y)
    y.backward(dy)
    gref = dy.float() @ iw.weight(torch.float32)
    assert (x.grad.float() - gref).abs().max() <= 2e-2 * gref.abs().max()


def test_mxfp8_quantiser_and_weight():
    native = _dev()
    torch.manual_seed(3)
    x = (torch.randn(300, 4096, device="cuda") * torch.logspace(-3, 2, 300, device="cuda")[:, None]).bfloat16()
    q, s = native.load().quantize_mxfp8(x)
    qr, sr = F.quantize_mxfp8(x.cpu().float())
    assert torch.equal(s.cpu(), sr)
    assert (q.float().cpu() - qr.float()).abs().max() == 0
    back = F.dequantize_mxfp8(q, s, torch.float32)
    rel = (back - x.float()).abs() / x.float().abs().clamp_min(1e-30)
    assert rel[x.float().abs() > 0].median() < 0.04
    w = torch.randn(512, 1024, device="cuda") * 0.05
    mx = F.MxFp8Weight.from_dense(w)
    xin = torch.randn(64, 1024, device="cuda").bfloat16().requires_grad_(True)
    y = mx.linear(xin, None)
    assert (y.float() - xin.float() @ w.t()).abs().max() <= 0.06 * (xin.float() @ w.t()).abs().max()
    y.sum().backward()
    assert xin.grad is not None and torch.isfinite(xin.grad).all()
