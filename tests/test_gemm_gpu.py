"""tcgen05 GEMM family against a plain PyTorch fp32 reference of the same product."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    return af @ bf


def _rel(x, y):
    return ((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 200, 136), (1000, 3072, 3072), (4352, 128, 3072), (77, 24, 520)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_bf16_layouts(M, N, K, a_mn, b_mn):
    from kohakumosstrainer_b200.ops import native

    if (a_mn and M % 8) or (b_mn and N % 8) or (not a_mn and K % 8) or (not b_mn and K % 8):
        pytest.skip("row stride must be a multiple of 16 bytes")
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g).bfloat16()
    out = native.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    native.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    assert _rel(out, ref) < 2e-3
    out16 = native.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert _rel(out16, ref) < 6e-3


@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("a_dtype,b_dtype", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
def test_fp8_per_tensor(a_dtype, b_dtype, b_mn):
    from kohakumosstrainer_b200.ops import native

    M, N, K = 520, 768, 1024
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g) * 0.05).bfloat16()
    xq, xs = native.quantize_fp8(x, a_dtype)
    wq, wsc = native.quantize_fp8(w, b_dtype)
    out = native.gemm(xq, wq, b_mn=b_mn, scale_a=xs[:1], scale_b=wsc[:1], out_dtype=torch.float32)
    native.check_status()
    # exact reference on the quantised values
    ref = _ref(xq.float() * xs[0], wq.float() * wsc[0], False, b_mn)
    assert _rel(out, ref) < 1e-4
    # and close to the unquantised product
    assert _rel(out, _ref(x, w, False, b_mn)) < 0.08


def test_quantize_matches_torch_cast():
    from kohakumosstrainer_b200.ops import native

    x = (torch.randn(333, 264, device="cuda") * 3).bfloat16()
    q, s = native.quantize_fp8(x)
    amax = x.float().abs().max()
    torch.testing.assert_close(s[0], amax / 448.0)
    ref = (x.float() * (448.0 / amax)).to(torch.float8_e4m3fn)
    assert (q.view(torch.uint8) != ref.view(torch.uint8)).float().mean() < 1e-3
    qr, rs = native.quantize_fp8_rows(x)
    ramax = x.float().abs().amax(1)
    torch.testing.assert_close(rs, ramax / 448.0)
    refr = (x.float() * (448.0 / ramax)[:, None]).to(torch.float8_e4m3fn)
    assert (qr.view(torch.uint8) != refr.view(torch.uint8)).float().mean() < 1e-3
    q5, rs5 = native.quantize_fp8_rows(x, torch.float8_e5m2, both=True)
    assert q5.dtype == torch.float8_e5m2 and rs5.shape == (2, 333)
    torch.testing.assert_close(rs5[0], ramax / 57344.0)
    torch.testing.assert_close(rs5[1], 57344.0 / ramax)
    ref5 = (x.float() * (57344.0 / ramax)[:, None]).to(torch.float8_e5m2)
    assert (q5.view(torch.uint8) != ref5.view(torch.uint8)).float().mean() < 1e-3
    for dim in (4104, 9216, 16384):       # rows wide enough for the one-CTA-per-row kernel
        xw = (torch.randn(37, dim, device="cuda") * 3).bfloat16()
        for dt, fmax in ((torch.float8_e4m3fn, 448.0), (torch.float8_e5m2, 57344.0)):
            qw, sw = native.quantize_fp8_rows(xw, dt, both=True)
            am = xw.float().abs().amax(1)
            torch.testing.assert_close(sw[0], am / fmax)
            refw = (xw.float() * (fmax / am)[:, None]).to(dt)
            assert (qw.view(torch.uint8) != refw.view(torch.uint8)).float().mean() < 1e-3


def test_linear_epilogue_scales_bias_gate_residual():
    from kohakumosstrainer_b200.ops import native

    M, N, K, B = 700, 384, 256, 3
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g).bfloat16()
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    mod = torch.randn(B, 6, N, device="cuda", generator=g)
    seg = torch.randint(0, B, (M,), device="cuda", generator=g, dtype=torch.int32).sort().values
    row_scale = torch.rand(M, device="cuda", generator=g) + 0.5
    col_scale = torch.rand(N, device="cuda", generator=g) + 0.5
    out = native.gemm(a, b, alpha=0.5, row_scale=row_scale, col_scale=col_scale, bias=bias, res=res,
                      beta=0.7, gate=mod[:, 2], seg=seg, out_dtype=torch.float32)
    native.check_status()
    acc = a.float() @ b.float().t()
    ref = (acc * 0.5 * row_scale[:, None] * col_scale[None] + bias.float()) * mod[:, 2][seg.long()] + 0.7 * res.float()
    assert _rel(out, ref) < 2e-3


def test_lowrank_bypass_accumulates_into_same_tile():
    from kohakumosstrainer_b200.ops import native

    M, N, K, R = 640, 512, 384, 16
    g = torch.Generator(device="cuda").manual_seed(2)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    t = torch.randn(M, R, device="cuda", generator=g).bfloat16()
    u = torch.randn(N, R, device="cuda", generator=g).bfloat16()
    out = native.gemm(a, b, t=t, u=u, out_dtype=torch.float32)
    native.check_status()
    ref = a.float() @ b.float().t() + t.float() @ u.float().t()
    assert _rel(out, ref) < 2e-3
    # rank 8 (one 16-byte row) exercises the zero-filled tail of the bypass box
    t8, u8 = t[:, :8].contiguous(), u[:, :8].contiguous()
    out8 = native.gemm(a, b, t=t8, u=u8, out_dtype=torch.float32)
    ref8 = a.float() @ b.float().t() + t8.float() @ u8.float().t()
    assert _rel(out8, ref8) < 2e-3


def test_split_k_skinny_problem():
    from kohakumosstrainer_b200.ops import native

    M, N, K = 3072, 16, 8192  # adapter wgrad shape: dU[out, r] = dY^T[out, tokens] . T[tokens, r]
    g = torch.Generator(device="cuda").manual_seed(3)
    dy = torch.randn(K, M, device="cuda", generator=g).bfloat16()
    t = torch.randn(K, N, device="cuda", generator=g).bfloat16()
    out = native.gemm(dy, t, a_mn=True, b_mn=True, out_dtype=torch.float32, splits=None)
    native.check_status()
    ref = dy.float().t() @ t.float()
    assert _rel(out, ref) < 2e-3
    out1 = native.gemm(dy, t, a_mn=True, b_mn=True, out_dtype=torch.float32, splits=1)
    assert _rel(out1, ref) < 2e-3


def test_situ_epilogue_pairs_up_and_gate():
    from kohakumosstrainer_b200.ops import eager, native

    M, F, K = 300, 256, 192
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * F, K, device="cuda", generator=g) * 0.3).bfloat16()
    aux = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    out = native.gemm(a, w, epilogue=native.EPI_SITU, aux=aux)
    native.check_status()
    h = (a.float() @ w.float().t())
    assert _rel(aux, h) < 6e-3
    ref = eager.situ_glu(aux.float())
    assert _rel(out, ref) < 6e-3


def test_qk_rope_epilogue_matches_eager():
    from kohakumosstrainer_b200.ops import eager, native

    M, H, K = 260, 2, 256
    D = H * 128
    g = torch.Generator(device="cuda").manual_seed(6)
    y = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(3 * D, K, device="cuda", generator=g) * 0.2).bfloat16()
    qw = (torch.rand(128, device="cuda", generator=g) + 0.5).bfloat16()
    kw = (torch.rand(128, device="cuda", generator=g) + 0.5).bfloat16()
    pos = torch.randn(M, 4, device="cuda", generator=g) * 20
    bands = 1.0 / (10000 ** (torch.arange(16, device="cuda", dtype=torch.float32) / 16))
    table = native.rope_table(pos, bands)
    rstd = torch.empty(M, 2 * H, device="cuda")
    out = native.gemm(y, w, epilogue=native.EPI_QK_ROPE, q_norm_w=qw, k_norm_w=kw, rope=table, rope_cols=2 * D,
                      eps=1e-6, head_rstd=rstd)
    native.check_status()
    lin = y.float() @ w.float().t()
    q, k, v = lin.split(D, 1)
    rq, rk = eager.qk_norm_rope(q.unflatten(1, (H, 128)), k.unflatten(1, (H, 128)), qw, kw, pos, bands, 1e-6)
    assert _rel(out[:, :D], rq.flatten(1)) < 8e-3
    assert _rel(out[:, D : 2 * D], rk.flatten(1)) < 8e-3
    assert _rel(out[:, 2 * D :], v) < 6e-3
    ref_rstd = torch.rsqrt(q.unflatten(1, (H, 128)).square().mean(-1) + 1e-6)
    assert _rel(rstd[:, :H], ref_rstd) < 1e-3


# ---- CTA-pair tiles (256 rows per pair): shapes large enough that the launcher picks them ----------------
PAIR_M = 4900   # 20 pair tiles, the last one ragged (a 128-row half with 36 rows, then nothing)


@pytest.mark.gpu
def test_pair_tiles_linear_epilogue_and_bypass_bf16():
    from kohakumosstrainer_b200.ops import native

    M, N, K, B, R = PAIR_M, 1024, 640, 3, 16
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    t = torch.randn(M, R, device="cuda", generator=g).bfloat16()
    u = torch.randn(N, R, device="cuda", generator=g).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g).bfloat16()
    res = torch.randn(M, N, device="cuda", generator=g).bfloat16()
    mod = torch.randn(B, 6, N, device="cuda", generator=g)
    seg = torch.randint(0, B, (M,), device="cuda", generator=g, dtype=torch.int32).sort().values
    row_scale = torch.rand(M, device="cuda", generator=g) + 0.5
    col_scale = torch.rand(N, device="cuda", generator=g) + 0.5
    acc = a.float() @ b.float().t() + t.float() @ u.float().t()
    ref = (acc * 0.5 * row_scale[:, None] * col_scale[None] + bias.float()) * mod[:, 2][seg.long()] + 0.7 * res.float()
    for dtype in (torch.float32, torch.bfloat16):       # direct stores, and the staged TMA-store path
        out = native.gemm(a, b, alpha=0.5, row_scale=row_scale, col_scale=col_scale, bias=bias, res=res, beta=0.7,
                          gate=mod[:, 2], seg=seg, t=t, u=u, out_dtype=dtype)
        native.check_status()
        assert _rel(out, ref) < (2e-3 if dtype == torch.float32 else 6e-3)
    plain = native.gemm(a, b)
    native.check_status()
    assert _rel(plain, a.float() @ b.float().t()) < 6e-3


@pytest.mark.gpu
def test_pair_tiles_fp8_rows_with_bypass():
    from kohakumosstrainer_b200.ops import native

    M, N, K, R = PAIR_M, 1280, 768, 8
    g = torch.Generator(device="cuda").manual_seed(12)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    xq, xs = native.quantize_fp8_rows(x, both=True)
    wq, ws = native.quantize_fp8(w)
    t = torch.randn(M, R, device="cuda", generator=g).bfloat16()
    u = torch.randn(N, R, device="cuda", generator=g).bfloat16()
    out = native.gemm(xq, wq, row_scale=xs[0], scale_b=ws[:1], t=t, u=u, out_dtype=torch.float32)
    native.check_status()
    deq = (xq.float() * xs[0][:, None]) @ (wq.float() * ws[0]).t()
    bypass = (t.float() @ u.float().t()) * xs[0][:, None] * ws[0]      # the bypass shares the rescaled accumulator
    assert _rel(out, deq + bypass) < 2e-3
    for e5 in (False, True):
        dq, ds = native.quantize_fp8_rows(x, torch.float8_e5m2 if e5 else torch.float8_e4m3fn, both=True)
        o = native.gemm(dq, wq, row_scale=ds[0], scale_b=ws[:1])
        native.check_status()
        assert _rel(o, (dq.float() * ds[0][:, None]) @ (wq.float() * ws[0]).t()) < 6e-3


@pytest.mark.gpu
def test_pair_tiles_situ_and_qk_rope_epilogues():
    from kohakumosstrainer_b200.ops import eager, native

    M, F, K = PAIR_M, 512, 640
    g = torch.Generator(device="cuda").manual_seed(13)
    a = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(2 * F, K, device="cuda", generator=g) * 0.1).bfloat16()
    t = (torch.randn(M, 8, device="cuda", generator=g) * 0.3).bfloat16()
    u = (torch.randn(2 * F, 8, device="cuda", generator=g) * 0.3).bfloat16()
    aux = torch.empty(M, 2 * F, device="cuda", dtype=torch.bfloat16)
    out = native.gemm(a, w, epilogue=native.EPI_SITU, aux=aux, t=t, u=u)
    native.check_status()
    h = a.float() @ w.float().t() + t.float() @ u.float().t()
    assert _rel(aux, h) < 6e-3
    assert _rel(out, eager.situ_glu(aux.float())) < 6e-3

    H = 3
    D = H * 128
    wq = (torch.randn(3 * D, K, device="cuda", generator=g) * 0.1).bfloat16()
    qw = (torch.rand(128, device="cuda", generator=g) + 0.5).bfloat16()
    kw = (torch.rand(128, device="cuda", generator=g) + 0.5).bfloat16()
    pos = torch.randn(M, 4, device="cuda", generator=g) * 20
    bands = 1.0 / (10000 ** (torch.arange(16, device="cuda", dtype=torch.float32) / 16))
    table = native.rope_table(pos, bands)
    rstd = torch.empty(M, 2 * H, device="cuda")
    o = native.gemm(a, wq, epilogue=native.EPI_QK_ROPE, q_norm_w=qw, k_norm_w=kw, rope=table, rope_cols=2 * D, eps=1e-6, head_rstd=rstd)
    native.check_status()
    lin = a.float() @ wq.float().t()
    q, k, v = lin.split(D, 1)
    rq, rk = eager.qk_norm_rope(q.unflatten(1, (H, 128)), k.unflatten(1, (H, 128)), qw, kw, pos, bands, 1e-6)
    assert _rel(o[:, :D], rq.flatten(1)) < 8e-3
    assert _rel(o[:, D : 2 * D], rk.flatten(1)) < 8e-3
    assert _rel(o[:, 2 * D :], v) < 6e-3


def test_pair_tiles_mn_major_b_dgrad_shape():
    from kohakumosstrainer_b200.ops import native

    M, N, K, R = PAIR_M, 1024, 768, 8
    g = torch.Generator(device="cuda").manual_seed(14)
    d = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(K, N, device="cuda", generator=g) * 0.05).bfloat16()      # [out, in]: dgrad reads it MN-major
    t = torch.randn(M, R, device="cuda", generator=g).bfloat16()
    u = torch.randn(N, R, device="cuda", generator=g).bfloat16()
    out = native.gemm(d, w, b_mn=True, t=t, u=u, out_dtype=torch.float32)
    native.check_status()
    assert _rel(out, d.float() @ w.float() + t.float() @ u.float().t()) < 2e-3
    dq, ds = native.quantize_fp8_rows(d, torch.float8_e5m2, both=True)
    wq, ws = native.quantize_fp8(w)
    o8 = native.gemm(dq, wq, b_mn=True, row_scale=ds[0], scale_b=ws[:1])
    native.check_status()
    assert _rel(o8, (dq.float() * ds[0][:, None]) @ (wq.float() * ws[0])) < 6e-3
