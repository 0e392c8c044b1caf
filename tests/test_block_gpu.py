"""Block ops and the fused layer path on CUDA against the eager fp32 reference."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from kohakumosstrainer_b200.types import MossArchConfig, build_seqinfo  # noqa: E402


def _rel(x, y):
    return ((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-12)).item()


def _seq(dev):
    hw = torch.tensor([[16, 16], [12, 20], [8, 8]])
    tl = torch.tensor([32, 17, 50])
    return build_seqinfo(hw, tl).to(dev)


def test_rms_norm_mod_forward_backward():
    from kohakumosstrainer_b200.ops import eager, native_ops

    seq = _seq("cuda")
    n, d = seq.n_joint, 256
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(n, d, device="cuda", generator=g).bfloat16().requires_grad_()
    w = (torch.rand(d, device="cuda", generator=g) + 0.5).bfloat16().requires_grad_()
    mod = torch.randn(3, 6, d, device="cuda", generator=g).requires_grad_()
    y = native_ops.rms_norm_mod(x, w, mod[:, 0], mod[:, 1], seq.seg_joint, 1e-6)
    xr, wr, mr = (t.detach().float().requires_grad_() for t in (x, w, mod))
    yr = eager.rms_norm_mod(xr, wr, mr[:, 0], mr[:, 1], seq.seg_joint, 1e-6)
    assert _rel(y, yr) < 5e-3
    dy = torch.randn(n, d, device="cuda", generator=g)
    y.backward(dy.bfloat16())
    yr.backward(dy.bfloat16().float())
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    assert _rel(mod.grad, mr.grad) < 1e-2


def test_qk_norm_rope_standalone_forward_backward():
    from kohakumosstrainer_b200.ops import eager, native_ops

    seq = _seq("cuda")
    n, h = seq.n_joint, 4
    g = torch.Generator(device="cuda").manual_seed(1)
    q = torch.randn(n, h, 128, device="cuda", generator=g).bfloat16().requires_grad_()
    k = torch.randn(n, h, 128, device="cuda", generator=g).bfloat16().requires_grad_()
    qw = (torch.rand(128, device="cuda", generator=g) + 0.5).bfloat16().requires_grad_()
    kw = (torch.rand(128, device="cuda", generator=g) + 0.5).bfloat16().requires_grad_()
    bands = 1.0 / (10000 ** (torch.arange(16, device="cuda", dtype=torch.float32) / 16))
    oq, ok = native_ops.qk_norm_rope(q, k, qw, kw, seq.pos_joint, bands, 1e-6)
    ref = [t.detach().float().requires_grad_() for t in (q, k, qw, kw)]
    rq, rk = eager.qk_norm_rope(ref[0], ref[1], ref[2], ref[3], seq.pos_joint, bands, 1e-6)
    assert _rel(oq, rq) < 6e-3 and _rel(ok, rk) < 6e-3
    dq = torch.randn_like(rq).bfloat16()
    dk = torch.randn_like(rk).bfloat16()
    torch.autograd.backward([oq, ok], [dq, dk])
    torch.autograd.backward([rq, rk], [dq.float(), dk.float()])
    assert _rel(q.grad, ref[0].grad) < 2e-2
    assert _rel(k.grad, ref[1].grad) < 2e-2
    assert _rel(qw.grad, ref[2].grad) < 2e-2


def test_situ_and_gated_residual_and_loss():
    from kohakumosstrainer_b200.ops import eager, native_ops

    seq = _seq("cuda")
    n, f = seq.n_joint, 512
    g = torch.Generator(device="cuda").manual_seed(2)
    h = (torch.randn(n, 2 * f, device="cuda", generator=g) * 3).bfloat16().requires_grad_()
    a = native_ops.situ_glu(h)
    hr = h.detach().float().requires_grad_()
    ar = eager.situ_glu(hr)
    assert _rel(a, ar) < 5e-3
    da = torch.randn(n, f, device="cuda", generator=g).bfloat16()
    a.backward(da)
    ar.backward(da.float())
    assert _rel(h.grad, hr.grad) < 1e-2

    x = torch.randn(n, f, device="cuda", generator=g).bfloat16().requires_grad_()
    o = torch.randn(n, f, device="cuda", generator=g).bfloat16().requires_grad_()
    mod = torch.randn(3, 6, f, device="cuda", generator=g).requires_grad_()
    out = native_ops.gated_residual(x, o, mod[:, 2], seq.seg_joint, 0.9)
    xr, orr, mr = (t.detach().float().requires_grad_() for t in (x, o, mod))
    outr = eager.gated_residual(xr, orr, mr[:, 2], seq.seg_joint, 0.9)
    assert _rel(out, outr) < 5e-3
    d = torch.randn(n, f, device="cuda", generator=g).bfloat16()
    out.backward(d)
    outr.backward(d.float())
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(o.grad, orr.grad) < 1e-2 and _rel(mod.grad, mr.grad) < 1e-2

    pred = torch.randn(seq.n_img, 128, device="cuda", generator=g).bfloat16().requires_grad_()
    target = torch.randn(seq.n_img, 128, device="cuda", generator=g)
    wt = torch.rand(3, device="cuda", generator=g)
    loss = native_ops.token_mse(pred, target, seq.seg_img, wt)
    pr = pred.detach().float().requires_grad_()
    lr = eager.token_mse(pr, target, seq.seg_img, wt)
    torch.testing.assert_close(loss, lr, rtol=1e-4, atol=1e-4)
    loss.backward()
    lr.backward()
    assert _rel(pred.grad, pr.grad) < 1e-2


def _pair(base: str, seed=0):
    """(bf16 model on the native op set, fp32 twin on the eager op set) with identical
    bf16-representable weights, the same fp8 bytes and the same LoRA factors."""
    import copy

    from kohakumosstrainer_b200 import adapters
    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import apply_param_dtypes
    from kohakumosstrainer_b200.ops import EagerOps
    from kohakumosstrainer_b200.quant import apply_base_precision

    cfg = MossArchConfig(dim=256, depth=2, heads=2, ffn_dim=512, text_dim=256, text_blocks=1)
    ref = build_backbone(cfg, device="cuda", dtype=torch.float32, seed=seed)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    model = copy.deepcopy(ref)
    apply_param_dtypes(model, torch.bfloat16)
    model.bind_ops()
    ref.bind_ops(EagerOps())
    if base == "fp8":
        apply_base_precision(model, "fp8_compute", "tensor")
        apply_base_precision(ref, "fp8_compute", "tensor")
    acfg = adapters.AdapterConfig(dim=8, alpha=8, preset="attn-mlp")
    aset = adapters.apply(model, adapters.AdapterConfig(dim=8, alpha=8, preset="attn-mlp", dtype=torch.bfloat16))
    with torch.no_grad():
        for _, _, mod in aset.items():
            mod.lora_up.weight.normal_(std=0.05)
    rset = adapters.apply(ref, acfg)
    rset.load_adapter_state({k: v.float() for k, v in aset.adapter_state().items()})
    return model, aset, ref, rset


@pytest.mark.parametrize("base", ["bf16", "fp8"])
def test_model_lora_step_matches_fp32_reference(base):
    """Tiny DiT, LoRA r8 on attn+mlp: native bf16 / fp8 forward + backward against the fp32
    eager twin (fp8: the twin multiplies by the dequantised weights)."""
    from kohakumosstrainer_b200.ops import native

    seq = _seq("cuda")
    g = torch.Generator(device="cuda").manual_seed(3)
    model, aset, ref, rset = _pair(base)
    assert model.ops.name == "native"
    z = torch.randn(seq.n_img, 128, device="cuda", generator=g).bfloat16()
    text = torch.randn(seq.n_txt, 256, device="cuda", generator=g).bfloat16()
    sigma = torch.rand(3, device="cuda", generator=g)
    target = torch.randn(seq.n_img, 128, device="cuda", generator=g)
    ones = torch.ones(3, device="cuda")

    v = model(z, text, sigma, seq)
    loss = model.ops.token_mse(v, target, seq.seg_img, ones) / seq.n_img
    loss.backward()
    native.check_status()
    rv = ref(z.float(), text.float(), sigma, seq)
    rloss = ref.ops.token_mse(rv, target, seq.seg_img, ones) / seq.n_img
    rloss.backward()

    tol = 0.03 if base == "bf16" else 0.08
    assert _rel(v, rv) < tol, (loss.item(), rloss.item())
    assert abs(loss.item() - rloss.item()) / abs(rloss.item()) < tol
    rg = dict(rset.named_parameters())
    bad = []
    for n, p in aset.named_parameters():
        assert p.grad is not None, n
        err = _rel(p.grad, rg[n].grad)
        if err > (0.1 if base == "bf16" else 0.3):
            bad.append((n, err))
    assert not bad, bad[:6]


def test_full_finetune_grads_match_fp32_reference():
    """ALGO=full: every trainable weight's gradient through the native path (wgrad on the
    tcgen05 GEMM, norm / modulation / qk-norm grads) against the fp32 eager twin."""
    import copy

    from kohakumosstrainer_b200.models import build_backbone
    from kohakumosstrainer_b200.models.build import apply_param_dtypes
    from kohakumosstrainer_b200.ops import EagerOps, native

    cfg = MossArchConfig(dim=256, depth=2, heads=2, ffn_dim=512, text_dim=256, text_blocks=1)
    ref = build_backbone(cfg, device="cuda", dtype=torch.float32, seed=5)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.bfloat16().float())
    model = copy.deepcopy(ref)
    apply_param_dtypes(model, torch.bfloat16)
    model.bind_ops()
    ref.bind_ops(EagerOps())
    seq = _seq("cuda")
    g = torch.Generator(device="cuda").manual_seed(4)
    z = torch.randn(seq.n_img, 128, device="cuda", generator=g).bfloat16()
    text = torch.randn(seq.n_txt, 256, device="cuda", generator=g).bfloat16()
    sigma = torch.rand(3, device="cuda", generator=g)
    target = torch.randn(seq.n_img, 128, device="cuda", generator=g)
    ones = torch.ones(3, device="cuda")
    v = model(z, text, sigma, seq)
    (model.ops.token_mse(v, target, seq.seg_img, ones) / seq.n_img).backward()
    native.check_status()
    rv = ref(z.float(), text.float(), sigma, seq)
    (ref.ops.token_mse(rv, target, seq.seg_img, ones) / seq.n_img).backward()
    assert _rel(v, rv) < 0.03
    rg = dict(ref.named_parameters())
    bad, checked = [], 0
    for n, p in model.named_parameters():
        assert p.grad is not None, n
        if rg[n].grad.norm() == 0:
            continue
        err = _rel(p.grad, rg[n].grad)
        checked += 1
        if err > 0.12:
            bad.append((n, round(err, 3)))
    assert checked > 40 and not bad, bad[:8]


def test_muon_newton_schulz_on_the_tcgen05_gemm_matches_torch():
    from kohakumosstrainer_b200.optim.muon import _ns_native, _ns_torch

    g = torch.Generator(device="cuda").manual_seed(8)
    x = torch.randn(256, 768, device="cuda", generator=g).bfloat16()
    x = (x / x.norm()).contiguous()
    a, b = _ns_native(x, 5).float(), _ns_torch(x, 5).float()
    assert _rel(a, b) < 0.05
    s = torch.linalg.svdvals(a)
    assert 0.4 < s.min() and s.max() < 1.4


def test_fused_adamw_kernel_matches_reference_math():
    from kohakumosstrainer_b200.optim import FusedAdamW

    g = torch.Generator(device="cuda").manual_seed(9)
    shapes = [(300, 17), (8192 * 3 + 5,), (64, 64)]
    ps = [torch.nn.Parameter(torch.randn(s, device="cuda", generator=g).bfloat16()) for s in shapes]
    rs = [torch.nn.Parameter(p.detach().float().cpu()) for p in ps]
    ours = FusedAdamW(ps, lr=1e-2, weight_decay=0.1, master_weights=True)
    ref = torch.optim.AdamW(rs, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ema = {id(p): p.detach().float().clone() for p in ps}
    ours.attach_ema(ema)
    ours.ema_decay = 0.9
    ema_ref = [r.detach().clone() for r in rs]
    scale = torch.tensor([0.5], device="cuda")
    for _ in range(4):
        for p, r in zip(ps, rs):
            gr = torch.randn(p.shape, device="cuda", generator=g).bfloat16()
            p.grad = gr
            r.grad = gr.float().cpu() * 0.5
        ours.step(grad_scale=scale)
        ref.step()
        for e, r in zip(ema_ref, rs):
            e.lerp_(r.detach(), 0.1)
    for p, r, e in zip(ps, rs, ema_ref):
        master = ours.state[p]["master"]
        torch.testing.assert_close(master.cpu(), r.detach(), rtol=2e-5, atol=2e-6)
        torch.testing.assert_close(p.detach().float().cpu(), r.detach().bfloat16().float(), rtol=1e-2, atol=1e-3)
        torch.testing.assert_close(ema[id(p)].cpu(), e, rtol=1e-4, atol=1e-5)
    skip = torch.ones(1, dtype=torch.int32, device="cuda")
    before = [p.detach().clone() for p in ps]
    ours.step(skip=skip)
    assert all(torch.equal(a, b) for a, b in zip(before, ps))


@pytest.mark.gpu
@pytest.mark.parametrize("states,writeback", [("8bit", "nearest"), ("fp32", "kahan"), ("fp32", "stochastic"), ("8bit", "kahan")])
def test_fused_adamw_state_formats_match_the_cpu_reference(states, writeback):
    """8-bit blockwise states and the bf16 writeback modes: the CUDA step against the same
    optimiser's plain PyTorch fp32 path on CPU, fed the same gradients."""
    from kohakumosstrainer_b200.optim import FusedAdamW

    g = torch.Generator().manual_seed(3)
    shapes = [(300, 17), (8192 + 77,), (64, 64)]
    init = [torch.randn(s, generator=g).bfloat16() for s in shapes]
    dev = [torch.nn.Parameter(t.clone().cuda()) for t in init]
    cpu = [torch.nn.Parameter(t.clone()) for t in init]
    kw = dict(lr=1e-2, weight_decay=0.1, states=states, writeback=writeback)
    a, b = FusedAdamW(dev, **kw), FusedAdamW(cpu, **kw)
    for _ in range(5):
        for p, r in zip(dev, cpu):
            gr = torch.randn(r.shape, generator=g).bfloat16()
            p.grad, r.grad = gr.cuda(), gr.clone()
        a.step()
        b.step()
    for p, r in zip(dev, cpu):
        # one bf16 ulp of slack: device and host may round a tie differently after five steps
        torch.testing.assert_close(p.detach().float().cpu(), r.detach().float(), rtol=8e-3, atol=1e-3)
        sa, sb = a.state[p], b.state[r]
        if states == "8bit":
            # a code that lands on the other side of a rounding boundary feeds the next step: after five
            # steps single codes may sit a few units apart, the bulk are equal
            for key in ("mq", "rq"):
                diff = (sa[key].cpu().int() - sb[key].int()).abs()
                assert diff.max() <= 4 and diff.float().mean() < 0.1, (key, int(diff.max()), float(diff.float().mean()))
            torch.testing.assert_close(sa["ms"].cpu(), sb["ms"], rtol=1e-3, atol=1e-12)
        if writeback == "kahan":
            full_a = p.detach().float().cpu() + sa["comp"].float().cpu()
            full_b = r.detach().float() + sb["comp"].float()
            # with 8-bit states a code on the other side of a rounding boundary moves a single element by a few 1e-4
            torch.testing.assert_close(full_a, full_b, rtol=1e-3, atol=2e-3 if states == "8bit" else 2e-4)



@pytest.mark.gpu
def test_gradient_producers_emit_the_row_quantised_copy():
    """SiTU backward and the gate scaling write bf16 d plus its per-row e5m2 copy in one pass: both equal the
    unfused kernel followed by the row quantiser."""
    from kohakumosstrainer_b200.ops import native

    ops = native.load()
    g = torch.Generator(device="cuda").manual_seed(21)
    for M, F in ((300, 8192), (77, 512)):
        aux = (torch.randn(M, 2 * F, device="cuda", generator=g) * 2).bfloat16()
        da = torch.randn(M, F, device="cuda", generator=g).bfloat16()
        d_ref = torch.empty_like(aux)
        ops.situ_bwd(da, aux[:, :F], aux[:, F:], d_ref[:, :F], d_ref[:, F:])
        q_ref, s_ref = native.quantize_fp8_rows(d_ref, torch.float8_e5m2, both=True)
        d = torch.empty_like(aux)
        q = torch.empty(M, 2 * F, dtype=torch.float8_e5m2, device="cuda")
        s = torch.empty(2, M, device="cuda")
        assert ops.situ_bwd_quant(da, aux[:, :F], aux[:, F:], d[:, :F], d[:, F:], q, s)
        assert torch.equal(d, d_ref)
        torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
        assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
    for M, D in ((513, 3072), (40, 256)):
        x = torch.randn(M, D, device="cuda", generator=g).bfloat16()
        mod = torch.randn(3, 6, D, device="cuda", generator=g)
        seg = torch.randint(0, 3, (M,), device="cuda", generator=g, dtype=torch.int32).sort().values
        y_ref = torch.empty_like(x)
        ops.seg_scale(x, mod[:, 2], seg, y_ref)
        q_ref, s_ref = native.quantize_fp8_rows(y_ref, torch.float8_e5m2, both=True)
        y, q, s = torch.empty_like(x), torch.empty(M, D, dtype=torch.float8_e5m2, device="cuda"), torch.empty(2, M, device="cuda")
        assert ops.seg_scale_quant(x, mod[:, 2], seg, y, q, s)
        assert torch.equal(y, y_ref)
        torch.testing.assert_close(s, s_ref, rtol=1e-6, atol=0)
        assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
    # a row wider than the fused kernel covers is declined, not mangled
    wide = torch.zeros(8, 8192, device="cuda", dtype=torch.bfloat16)
    assert not ops.seg_scale_quant(wide, torch.ones(1, 8192, device="cuda"), torch.zeros(8, dtype=torch.int32, device="cuda"), torch.empty_like(wide),
                                   torch.empty(8, 8192, dtype=torch.float8_e5m2, device="cuda"), torch.empty(2, 8, device="cuda"))
