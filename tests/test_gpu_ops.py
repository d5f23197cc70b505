"""GPU numerics of the autograd-level ops (conv, norms, gate update, CAM read, loss, linears, the
fused layer step) against autograd through the plain-PyTorch fp32 statement."""

import pytest
import torch
import torch.nn.functional as F

from gdnet_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _cu():
    from gdnet_b200.ops import cuda as cu

    return cu


def _rel(got, want):
    got, want = got.float(), want.float()
    return float((got - want).norm() / want.norm().clamp(min=1e-12))


def _check(got, want, tol, what):
    r = _rel(got, want)
    assert r < tol, f"{what}: relative error {r:.4g} (tol {tol}); max abs {float((got.float()-want.float()).abs().max()):.4g}"


# the last two shapes make the fused dx + dw backward walk 16 and 32 rows per warp (it picks the walk by the grid size)
@pytest.mark.parametrize("B,T,d,k", [(2, 64, 128, 4), (2, 300, 256, 7), (1, 129, 64, 9), (3, 40, 32, 1), (1, 5, 8, 4),
                                     (3, 200, 136, 4), (8, 4096, 1024, 4), (2, 8192, 4096, 4)])
@pytest.mark.parametrize("use_halo", [False, True])
def test_causal_dwconv_fwd_bwd(B, T, d, k, use_halo):
    cu = _cu()
    if k == 1 and use_halo:
        pytest.skip("no halo for k=1")
    x = torch.randn(B, T, d, device=DEV, dtype=BF, requires_grad=True)
    w = torch.randn(d, k, device=DEV, requires_grad=True)
    halo = torch.randn(B, k - 1, d, device=DEV, dtype=BF, requires_grad=True) if use_halo else None
    out = cu.causal_dwconv(x, w, halo)
    gy = torch.randn_like(out)
    out.backward(gy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().clone().requires_grad_()
    hr = halo.detach().float().requires_grad_() if use_halo else None
    want = ref.causal_dwconv(xr, wr, hr)
    want.backward(gy.float())
    _check(out, want, 1e-2, "conv out")
    _check(x.grad, xr.grad, 1e-2, "conv dx")
    _check(w.grad, wr.grad, 2e-2, "conv dw")
    if use_halo:
        _check(halo.grad, hr.grad, 1e-2, "conv dhalo")


@pytest.mark.parametrize("rows,d", [(300, 256), (4100, 1024), (130, 384), (203, 512), (77, 2048)])   # register paths (d = 256 * n) and the generic one
def test_rmsnorm_fwd_bwd(rows, d):
    cu = _cu()
    x = torch.randn(rows, d, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.rand(d, device=DEV) + 0.5).requires_grad_()
    y = cu.rmsnorm(x, w, 1e-6)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    want = ref.rmsnorm(xr, wr, 1e-6)
    want.backward(gy.float())
    _check(y, want, 1e-2, "rmsnorm y")
    _check(x.grad, xr.grad, 1e-2, "rmsnorm dx")
    _check(w.grad, wr.grad, 1e-2, "rmsnorm dw")


def test_fused_mem_read_fwd_bwd():
    cu = _cu()
    B, S, ds, dc = 5, 32, 64, 128
    mk = lambda *s: torch.randn(*s, device=DEV, requires_grad=True)
    q, gam, e, tags, vals = mk(B, ds), mk(B, ds), mk(S, ds), mk(B, S, ds), mk(B, S, dc)
    alpha = torch.tensor([0.7], device=DEV, requires_grad=True)
    out, w = cu.fused_mem_read(q, gam, e, tags, vals, alpha)
    assert not w.requires_grad
    gy = torch.randn_like(out)
    out.backward(gy)
    refs = [t.detach().clone().requires_grad_() for t in (q, gam, e, tags, vals, alpha)]
    out_r, w_r = ref.fused_mem_read(*refs)
    out_r.backward(gy)
    _check(out, out_r, 1e-4, "mem_read out")
    _check(w, w_r, 1e-4, "mem_read w")
    for name, a, b in zip("q gamma e tags vals alpha".split(), (q, gam, e, tags, vals, alpha), refs):
        _check(a.grad, b.grad, 1e-3, f"mem_read d{name}")


@pytest.mark.parametrize("V,Vp", [(1000, 1000), (250, 256)])
def test_cross_entropy(V, Vp):
    cu = _cu()
    n = 64
    logits = (torch.randn(n, Vp, device=DEV) * 3).to(BF).requires_grad_()
    tgt = torch.randint(0, V, (n,), device=DEV)
    tgt[::7] = -100
    lr = logits.detach().float()[:, :V].requires_grad_()
    want = F.cross_entropy(lr, tgt, ignore_index=-100)
    want.backward()
    loss = cu.cross_entropy(logits.clone(), tgt, -100, vocab=V)      # clone: the op consumes its input
    _check(loss, want, 2e-3, "ce loss")
    x = logits.detach().clone().requires_grad_()
    y = x * 1.0
    loss2 = cu.cross_entropy(y, tgt, -100, vocab=V)
    (2.0 * loss2).backward()
    _check(x.grad[:, :V], 2.0 * lr.grad, 2e-2, "ce grad")
    if Vp > V:
        assert x.grad[:, V:].abs().max() == 0


def test_cross_entropy_out_of_range_target_is_ignored_and_reported():
    """A class id outside [0, vocab) that is not the ignore index must never be used as an index: the row gives
    loss 0 and gradient 0, is left out of the mean, and the status word makes the host raise."""
    from gdnet_b200 import _ext

    cu = _cu()
    n, V, Vp = 32, 250, 256
    logits = (torch.randn(n, Vp, device=DEV) * 3).to(BF)
    tgt = torch.randint(0, V, (n,), device=DEV)
    tgt[3], tgt[5], tgt[9] = V, -7, 10**9          # first padded column, negative, far out of range
    good = tgt.clone()
    good[[3, 5, 9]] = -100
    want = F.cross_entropy(logits.float()[:, :V], good, ignore_index=-100)
    x = logits.clone().requires_grad_()
    loss = cu.cross_entropy(x * 1.0, tgt, -100, vocab=V)
    loss.backward()
    torch.cuda.synchronize()
    with pytest.raises(_ext.KernelArgumentError):
        _ext.check_status(logits)
    _ext.check_status(logits)                      # the status word was reset by the failed check
    _check(loss, want, 2e-3, "ce loss with bad targets dropped")
    assert float(x.grad[[3, 5, 9]].abs().max()) == 0.0
    # the kernels stay usable afterwards
    loss2 = cu.cross_entropy(logits.clone(), good, -100, vocab=V)
    _check(loss2, want, 2e-3, "ce after a reported bad target")
    _ext.check_status(logits)


@pytest.mark.parametrize("M,K,N,bias", [(256, 128, 256, True), (512, 384, 128, False)])
def test_linear_bf16_fwd_bwd(M, K, N, bias):
    cu = _cu()
    x = torch.randn(M, K, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(BF).requires_grad_()
    b = torch.randn(N, device=DEV, dtype=BF, requires_grad=True) if bias else None
    y = cu.linear_bf16(x, w, b)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    br = b.detach().float().requires_grad_() if bias else None
    F.linear(xr, wr, br).backward(gy.float())
    _check(y, F.linear(xr, wr, br), 1e-2, "linear y")
    _check(x.grad, xr.grad, 1e-2, "linear dx")
    _check(w.grad, wr.grad, 1e-2, "linear dw")
    if bias:
        _check(b.grad, br.grad, 1e-2, "linear db")


@pytest.mark.parametrize("recipe", ["block", "tensor"])
def test_fp8_linear_module_fwd_bwd(recipe):
    from gdnet_b200.ops.fp8_linear import FP8Linear

    M, K, N = 256, 256, 384
    lin = torch.nn.Linear(K, N).to(DEV)
    mod = FP8Linear(lin, recipe=recipe)
    x = torch.randn(M, K, device=DEV, dtype=BF, requires_grad=True)
    y = mod(x)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr = x.detach().float().requires_grad_()
    wr, br = mod.weight.detach().float().requires_grad_(), mod.bias.detach().float().requires_grad_()
    F.linear(xr, wr, br).backward(gy.float())
    tol = 0.08 if recipe == "block" else 0.12
    _check(y, F.linear(xr, wr, br), tol, "fp8 y")
    _check(x.grad, xr.grad, tol, "fp8 dx")
    _check(mod.weight.grad, wr.grad, tol, "fp8 dw")
    _check(mod.bias.grad, br.grad, 2e-2, "fp8 db")
    if recipe == "tensor":
        assert float(mod._amax_x) > 0 and float(mod._amax_w) > 0


def _make_layer(d, k, fp8):
    from gdnet_b200.layer import GDLayer
    from gdnet_b200.utils.fp8 import convert_to_fp8

    torch.manual_seed(0)
    layer = GDLayer(d, k)
    with torch.no_grad():   # make both gates and the recovery path matter
        for p in ("gf", "gb", "rf", "rb"):
            getattr(layer, f"{p}_W2").weight.mul_(30.0)
            getattr(layer, f"{p}_norm").weight.add_(torch.randn(d) * 0.2)
    layer = layer.to(DEV)
    if fp8:
        convert_to_fp8(layer)
    else:
        layer.to(BF)
    return layer


def _fake_q(x, block):
    """``x`` rounded to bf16, quantised to e4m3 with one power-of-two scale per ``block`` columns of a row, dequantised."""
    xb = x.to(BF).float()
    M, Kd = xb.shape
    v = xb.view(M, Kd // block, block)
    amax = v.abs().amax(dim=-1, keepdim=True)
    scale = torch.exp2(torch.ceil(torch.log2(amax.clamp(min=1e-30) / ref.FP8_MAX)))
    scale = torch.where(amax > 0, scale, torch.ones_like(scale))
    q = (v / scale).clamp(-ref.FP8_MAX, ref.FP8_MAX).to(ref.FP8_DTYPE).float()
    return (q * scale).view(M, Kd)


class _FakeFp8Linear(torch.autograd.Function):
    """fp32 statement of the block-scaled FP8 linear as the kernels run it: forward and data gradient on quantised
    operands, weight gradient on the bf16 operands."""

    @staticmethod
    def forward(ctx, x, w, b, block, bwd_block):
        shape = x.shape
        ctx.bwd_block = bwd_block
        x2 = x.reshape(-1, shape[-1])
        w8, sw = ref.quantize_128x128(w.to(BF).float(), pow2=True)
        wq = w8.float() * sw.repeat_interleave(128, 0).repeat_interleave(128, 1)[: w.shape[0], : w.shape[1]]
        ctx.save_for_backward(x2.to(BF).float(), wq)
        ctx.shape = shape
        return (_fake_q(x2, block) @ wq.t() + b).view(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, wq = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = _fake_q(dy2, ctx.bwd_block) @ wq
        dyb = dy2.to(BF).float()
        return dx.view(ctx.shape), dyb.t() @ x2, dyb.sum(0), None, None


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("step", ["fwd", "bwd"])
def test_layer_step_matches_reference(fp8, step):
    """Fused CUDA step (values and every gradient) against the fp32 composition on the same weights."""
    from gdnet_b200.models.layer import _STEP_PREFIXES

    B, T, d, k = 2, 128, 256, 4
    layer = _make_layer(d, k, fp8)
    x = torch.randn(B, T, d, device=DEV, dtype=BF, requires_grad=True)
    s = torch.randn(B, T, d, device=DEV, dtype=BF, requires_grad=True)
    fo, so, gm = layer._step(step, x, s, return_gate="mean")
    gF, gS = torch.randn_like(fo), torch.randn_like(so)
    (fo.float() * gF).sum().add((so.float() * gS).sum()).add(3.0 * gm).backward()

    conv, g, r = _STEP_PREFIXES[step]
    P = lambda n: getattr(layer, n)
    xr, sr = x.detach().float().requires_grad_(), s.detach().float().requires_grad_()
    prm = {}
    for name in (f"{r}_W1", f"{r}_W2", f"{g}_W1", f"{g}_W2"):
        prm[name + ".w"] = P(name).weight.detach().float().requires_grad_()
        prm[name + ".b"] = P(name).bias.detach().float().requires_grad_()
    prm["rn"] = P(f"{r}_norm").weight.detach().float().requires_grad_()
    prm["gn"] = P(f"{g}_norm").weight.detach().float().requires_grad_()
    prm["cw"] = P(conv).taps.detach().float().requires_grad_()
    # FP8 mode: the oracle's recovery linears see the same quantised operands as the kernels (e4m3 with power-of-two
    # block scales: 1x128 for the first GEMM's input, 1x64 for the second's, which its producer's epilogue writes;
    # 128x128 for the weights; 1x128 for the incoming gradient of the data-gradient GEMM), everything else in fp32.
    # What remains is bf16 rounding of stored intermediates, so the tolerances are the same order as in bf16 mode.
    calls = []

    def fake_fp8_linear(xin, w, b):
        calls.append(1)
        # (block of the input's scales, block of the incoming gradient's scales): operands written by a GEMM epilogue
        # (silu(h1) forward, dh1 backward) carry one scale per 64 columns, the others one per 128
        return _FakeFp8Linear.apply(xin, w, b, *((128, 64) if len(calls) == 1 else (64, 128)))

    fo_r, so_r, g_r, _ = ref.layer_step(
        xr, sr, prm["cw"], prm[f"{r}_W1.w"], prm[f"{r}_W1.b"], prm[f"{r}_W2.w"], prm[f"{r}_W2.b"], prm["rn"],
        prm[f"{g}_W1.w"], prm[f"{g}_W1.b"], prm["gn"], prm[f"{g}_W2.w"], prm[f"{g}_W2.b"],
        r_eps=ref.default_rms_eps(BF), linear_fn=fake_fp8_linear if fp8 else None)
    (fo_r * gF.float()).sum().add((so_r * gS.float()).sum()).add(3.0 * g_r.mean()).backward()

    tol = 0.03 if fp8 else 0.02
    _check(fo, fo_r, tol, "fwd'")
    _check(so, so_r, tol, "side'")
    _check(gm, g_r.mean(), 1e-2, "gate mean")
    _check(x.grad, xr.grad, tol * 2, "dx")
    _check(s.grad, sr.grad, tol * 2, "ds")
    pairs = [(P(conv).conv.weight.grad.squeeze(1), prm["cw"].grad, "dconv_w"),
             (P(f"{r}_norm").weight.grad, prm["rn"].grad, "drnorm"),
             (P(f"{g}_norm").weight.grad, prm["gn"].grad, "dgnorm")]
    for name in (f"{r}_W1", f"{r}_W2", f"{g}_W1", f"{g}_W2"):
        pairs.append((P(name).weight.grad, prm[name + ".w"].grad, f"d{name}.weight"))
        pairs.append((P(name).bias.grad, prm[name + ".b"].grad, f"d{name}.bias"))
    for got, want, what in pairs:
        assert got is not None, what
        _check(got, want, tol * 2.5, what)
    # parameters of the other step stay untouched
    other = "bwd" if step == "fwd" else "fwd"
    assert getattr(layer, _STEP_PREFIXES[other][0]).conv.weight.grad is None


@pytest.mark.parametrize("fp8", [False, True])
def test_zero_side_step_matches_explicit_zeros(fp8):
    """``side=None`` (the first forward step of a layer: its side stream is all zeros) leaves out the recovery gate,
    which only multiplies the side stream. Outputs must be bit-equal to the general step on an explicit zero tensor,
    the gradients equal up to the summation order of the weight-gradient GEMMs, and the recovery parameters must get
    no gradient from either."""
    import copy

    from gdnet_b200.models.layer import _STEP_PREFIXES

    B, T, d, k = 2, 128, 256, 4
    la = _make_layer(d, k, fp8)
    lb = copy.deepcopy(la)
    torch.manual_seed(3)
    x = torch.randn(B, T, d, device=DEV, dtype=BF)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    fa, sa, ga = la._step("fwd", xa, None, return_gate="mean")
    fb, sb, gb = lb._step("fwd", xb, torch.zeros_like(x), return_gate="mean")
    assert torch.equal(fa, fb) and torch.equal(sa, sb), "outputs differ from the step on explicit zeros"
    assert abs(float(ga) - float(gb)) < 1e-6
    gF, gS = torch.randn_like(fa), torch.randn_like(sa)
    (fa.float() * gF).sum().add((sa.float() * gS).sum()).add(3.0 * ga).backward()
    (fb.float() * gF).sum().add((sb.float() * gS).sum()).add(3.0 * gb).backward()
    _check(xa.grad, xb.grad, 2e-3, "dx")
    conv, g, r = _STEP_PREFIXES["fwd"]
    for name in (f"{g}_W1", f"{g}_W2"):
        _check(getattr(la, name).weight.grad, getattr(lb, name).weight.grad, 5e-3, f"d{name}.weight")
        _check(getattr(la, name).bias.grad, getattr(lb, name).bias.grad, 5e-3, f"d{name}.bias")
    _check(getattr(la, f"{g}_norm").weight.grad, getattr(lb, f"{g}_norm").weight.grad, 5e-3, "dgnorm")
    _check(getattr(la, conv).conv.weight.grad, getattr(lb, conv).conv.weight.grad, 5e-3, "dconv_w")
    for name in (f"{r}_W1", f"{r}_W2"):
        for prm in (getattr(lb, name).weight, getattr(lb, name).bias):
            assert prm.grad is None or float(prm.grad.float().abs().max()) == 0.0, f"{name}: non-zero gradient from a zero side stream"
        for prm in (getattr(la, name).weight, getattr(la, name).bias):
            assert prm.grad is None or float(prm.grad.float().abs().max()) == 0.0
    # the FP8 copy of side' that the step hands to the next one must be the one the general step hands over
    if fp8:
        f2a, s2a = la._step("bwd", fa.detach(), sa.detach())
        f2b, s2b = lb._step("bwd", fb.detach(), sb.detach())
        assert torch.equal(f2a, f2b) and torch.equal(s2a, s2b)


@pytest.mark.parametrize("fp8", [False, True])
def test_fused_layer_steps_keep_their_red_zones(fp8):
    """Every output and scratch buffer of the fused steps (general and zero-side, forward and backward) is allocated
    with a canary-filled red zone behind it; no kernel may write there."""
    from gdnet_b200.runtime.checked import RedZones

    B, T, d, k = 2, 128, 256, 4
    layer = _make_layer(d, k, fp8)
    x = torch.randn(B, T, d, device=DEV, dtype=BF, requires_grad=True)
    with RedZones(torch.device(DEV, torch.cuda.current_device())) as rz:
        f1, s1, g1 = layer._step("fwd", x, None, return_gate="mean")
        f2, s2 = layer._step("bwd", f1, s1)
        (f2.float().sum() + s2.float().sum() + g1).backward()
        torch.cuda.synchronize()
        assert rz.check() > 20
    _ext_status = __import__("gdnet_b200._ext", fromlist=["check_status"])
    _ext_status.check_status(x)


def test_layer_step_main_grad_accumulates():
    B, T, d, k = 1, 128, 128, 4
    layer = _make_layer(d, k, True)
    for p in layer.parameters():
        p.main_grad = torch.zeros(p.shape, dtype=torch.float32, device=DEV)
    x = torch.randn(B, T, d, device=DEV, dtype=BF, requires_grad=True)
    s = torch.randn(B, T, d, device=DEV, dtype=BF, requires_grad=True)
    for _ in range(2):
        fo, so = layer.fwd_step(x, s)
        (fo.float().sum() + so.float().pow(2).sum()).backward()
    g2 = layer.rf_W1.weight.main_grad.clone()
    assert layer.rf_W1.weight.grad is None and g2.abs().sum() > 0
    for p in layer.parameters():
        p.main_grad.zero_()
    fo, so = layer.fwd_step(x, s)
    (fo.float().sum() + so.float().pow(2).sum()).backward()
    _check(g2, 2 * layer.rf_W1.weight.main_grad, 1e-3, "main_grad accumulates over two backward passes")


def test_sigma_estimates_fwd_bwd():
    cu = _cu()
    mats = [torch.randn(64, 128, device=DEV).to(BF).requires_grad_(), torch.randn(32, 32, device=DEV).requires_grad_()]
    vecs = [F.normalize(torch.randn(m.shape[1], device=DEV), dim=0) for m in mats]
    sig = cu.sigma_estimates(mats, vecs)
    (sig * torch.tensor([1.0, -2.0], device=DEV)).sum().backward()
    refs = [m.detach().float().requires_grad_() for m in mats]
    want = torch.stack([(W @ v).norm() for W, v in zip(refs, vecs)])
    (want * torch.tensor([1.0, -2.0], device=DEV)).sum().backward()
    _check(sig, want, 1e-3, "sigma")
    for a, b in zip(mats, refs):
        _check(a.grad, b.grad, 1e-2, "dsigma/dW")


def test_optimizer_kernels():
    cu = _cu()
    n = 10_000
    gt, gi = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
    sums = torch.zeros(4, device=DEV)
    cu.K.grad_dots(gt, gi, sums)
    assert torch.allclose(sums[:3], torch.stack([(gt * gt).sum(), (gt * gi).sum(), (gi * gi).sum()]), rtol=1e-4)
    for dtype in (torch.bfloat16, torch.float32):
        p = torch.randn(n, device=DEV).to(dtype)
        p_ref = p.float().clone()
        m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        m_r, v_r = m.clone(), v.clone()
        coef = float(sums[1] / sums[0])
        scal = torch.tensor([coef, 0.5], device=DEV)
        for step in (1, 2):
            cu.K.projected_adamw(p, gt, gi, m, v, scal, 0.1, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
            ref.projected_adamw_(p_ref, gt, gi, m_r, v_r, coef=coef, beta_proj=0.1, grad_scale=0.5, lr=1e-2,
                                 beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
            if dtype == torch.bfloat16:
                p_ref = p_ref.to(dtype).float()
        assert torch.allclose(p.float(), p_ref, atol=1e-2 if dtype == torch.bfloat16 else 1e-5)
        assert torch.allclose(m, m_r, atol=1e-6) and torch.allclose(v, v_r, atol=1e-6)


def _ptr_table(t):
    return torch.tensor([t.data_ptr()], dtype=torch.int64, device=DEV)


def _status(t):
    from gdnet_b200 import _ext

    _ext.check_status(t)


def test_collective_kernels_single_rank():
    """The peer-memory kernels with a world of one (every "peer" table holds this GPU's own buffer, so no kernel
    waits for another): fused update against the plain optimizer kernel, in all phase combinations; gradient
    sinks of the epilogue reduce-scatter; the MAX all-reduce."""
    cu = _cu()
    n = 128 * 64
    torch.manual_seed(4)
    for phases in ((0,), (1, 2), (3, 4), (5,), (6, 0), (6, 1, 2)):
        gt, gi = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
        gt0, gi0 = gt.clone(), gi.clone()
        p = torch.randn(n, device=DEV).bfloat16()
        p_ref = p.clone()
        m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        m_r, v_r = m.clone(), v.clone()
        flags = torch.zeros(1024, dtype=torch.int32, device=DEV)
        scal = torch.tensor([0.3, 1.0], device=DEV)
        sums = torch.zeros(8, device=DEV)
        # phase 6 reduces the task gradient alone into t_red (here: a copy), the later phases then take it from there
        t_red = torch.full((n,), 7.0, device=DEV) if 6 in phases else None
        timing = torch.zeros(4, dtype=torch.int64, device=DEV)
        for ph in phases:
            cu.K.allreduce_adamw(_ptr_table(gt), _ptr_table(gi), _ptr_table(p), _ptr_table(flags), m, v, scal, n, 0, 1,
                                 8, ph, True, 0.1, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, sums, True, t_red if ph != 2 else None,
                                 timing if ph == 0 else None)
            if ph == 6:
                torch.cuda.synchronize()
                assert torch.equal(t_red, gt0), "task-only pass must leave the mean task gradient in t_red"
                gt.fill_(float("nan"))        # from here on the task gradient must come from t_red
        if 0 in phases:
            t = timing.tolist()
            assert 0 < t[0] <= t[1] <= t[2], t
        cu.K.projected_adamw(p_ref, gt0, gi0, m_r, v_r, scal, 0.1, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1)
        torch.cuda.synchronize()
        assert torch.equal(p, p_ref), f"phases {phases}: parameters differ from the plain update"
        assert torch.allclose(m, m_r, atol=1e-7) and torch.allclose(v, v_r, atol=1e-7)
        if phases != (2,):
            want = torch.stack([(gt0 * gt0).sum(), (gt0 * gi0).sum(), (gi0 * gi0).sum()])
            assert torch.allclose(sums[:3], want, rtol=1e-3), f"phases {phases}: shard dot products"
        if phases[-1] >= 4:
            assert float(gt.abs().max()) == 0.0 and float(gi.abs().max()) == 0.0, "consumed shard not cleared"

    # epilogue reduce-scatter with one rank: a weight-gradient GEMM into a registered flat buffer
    flat = torch.zeros(4 * 256 * 128, device=DEV)
    cu.K.clear_grad_sinks()
    cu.K.register_grad_sink(flat, _ptr_table(flat), flat.numel())
    try:
        M, N, Kd = 512, 256, 128
        dy, x = torch.randn(M, N, device=DEV, dtype=BF), torch.randn(M, Kd, device=DEV, dtype=BF)
        view = flat[256 * 128 : 2 * 256 * 128].view(N, Kd)
        cu.gemm_bf16(dy, x, a_mn=True, b_mn=True, out=view, accumulate=True)
        cu.gemm_bf16(dy, x, a_mn=True, b_mn=True, out=view, accumulate=True)
        small = torch.randn(1000, device=DEV)
        cu.K.peer_add(flat[3 * 256 * 128 : 3 * 256 * 128 + 1000], small)
        cu.K.peer_add(flat[3 * 256 * 128 : 3 * 256 * 128 + 1000], small.bfloat16())
        torch.cuda.synchronize()
        _status(dy)
        _check(view, 2.0 * (dy.float().t() @ x.float()), 1e-2, "wgrad through a gradient sink")
        assert float(flat[: 256 * 128].abs().max()) == 0.0, "the sink wrote outside the view"
        assert torch.allclose(flat[3 * 256 * 128 : 3 * 256 * 128 + 1000], small + small.bfloat16().float(), atol=1e-6)
    finally:
        cu.K.clear_grad_sinks()

    # MAX all-reduce, world of one: the vector comes back unchanged, twice (both slot sets)
    area = torch.zeros(2 * 512, device=DEV)
    fl = torch.zeros(64, dtype=torch.int32, device=DEV)
    vec = torch.rand(300, device=DEV)
    keep = vec.clone()
    for seq in (1, 2, 3):
        cu.K.max_allreduce(vec, _ptr_table(area), _ptr_table(fl), 512, 0, 1, seq)
    torch.cuda.synchronize()
    _status(vec)
    assert torch.equal(vec, keep)


@pytest.mark.parametrize("B,T,d", [(1, 64, 256), (3, 40, 128), (2, 8, 320)])
def test_conv_kernels_exchange_halo_in_kernel(B, T, d):
    """The sequence-parallel form of the conv kernels on one GPU: two "ranks" are two launches in stream order over
    two halves of one sequence, and every rank's slot and flag area is a plain local buffer. Forward: rank 0 stores
    its last rows into rank 1's slot and raises the flag, rank 1 finds it raised. Backward runs rank 1 first (its
    halo gradient goes to rank 0's slot). Outputs and all gradients must equal the conv over the whole sequence."""
    from gdnet_b200 import _ext

    cu = _cu()
    k = 4
    torch.manual_seed(B * 100 + T)
    x = torch.randn(B, 2 * T, d, device=DEV).to(BF)
    w = (torch.randn(d, k, device=DEV) * 0.5)
    dc = torch.randn(B, 2 * T, d, device=DEV).to(BF)
    xr = x.float().requires_grad_()
    wr = w.clone().requires_grad_()
    want = ref.causal_dwconv(xr, wr)
    want.backward(dc.float())
    wt = w.t().contiguous()
    nbytes = B * (k - 1) * d * 2
    slots = [torch.zeros(2 * nbytes, dtype=torch.uint8, device=DEV) for _ in range(2)]
    flags = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(2)]
    tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=DEV)
    cnt = torch.zeros(2, dtype=torch.int32, device=DEV)
    halves = [x[:, :T].clone(memory_format=torch.contiguous_format), x[:, T:].clone(memory_format=torch.contiguous_format)]
    outs, halos = [], []
    for rank in (0, 1):
        out = torch.empty(B, T, d, device=DEV, dtype=BF)
        halo = torch.full((B, k - 1, d), 9.0, device=DEV, dtype=BF)
        cu.K.dwconv_fwd_sp(halves[rank], wt, out, halo, tab(slots), tab(flags), cnt[0:1], 0, 0, rank, 2, 1, 50_000_000)
        outs.append(out)
        halos.append(halo)
    torch.cuda.synchronize()
    _ext.check_status(x)
    assert float(halos[0].abs().max()) == 0.0 and torch.equal(halos[1], x[:, T - (k - 1) : T])
    _check(torch.cat(outs, dim=1), want, 1e-2, "conv over two shards")
    assert int(cnt[0]) == 0 and int(flags[1][0]) == 1
    dxs = [None, None]
    dw = torch.zeros(d, k, device=DEV)
    dcs = [dc[:, :T].clone(memory_format=torch.contiguous_format), dc[:, T:].clone(memory_format=torch.contiguous_format)]
    for rank in (1, 0):
        dx = torch.empty(B, T, d, device=DEV, dtype=BF)
        cu.K.dwconv_bwd_sp(dcs[rank], halves[rank], halos[rank], wt, dx, dw, tab(slots), tab(flags), cnt[1:2], nbytes, 1,
                           rank, 2, 1, 50_000_000)
        dxs[rank] = dx
    torch.cuda.synchronize()
    _ext.check_status(x)
    _check(torch.cat(dxs, dim=1), xr.grad, 1e-2, "dx over two shards (halo gradient added in-kernel)")
    _check(dw, wr.grad, 1e-2, "dw over two shards")
    assert int(cnt[1]) == 0 and int(flags[0][1]) == 1


def test_cam_read_out_on_own_kernels_matches_composition():
    """``Memory.read`` on bf16 CUDA tensors (token-sized GEMMs on the tensor-core kernel, norm + sigmoid + blend in
    one kernel) against the same module in fp32, which takes the plain-PyTorch composition: output and the gradients
    of both streams, the buffers and the read-out parameters."""
    import copy

    from gdnet_b200.models.memory import Memory

    torch.manual_seed(3)
    B, T, d = 2, 128, 128
    mem = Memory(d, 32, 16, 8, T).to(DEV)
    with torch.no_grad():
        mem.rho.fill_(0.6)
        mem.W_pos.weight.normal_(std=0.3)
        mem.W_r2.weight.normal_(std=0.2)
    mem.eval()                                   # keeps the spectral-norm vectors fixed over the two evaluations
    m32, mbf = copy.deepcopy(mem), copy.deepcopy(mem).to(BF)
    fwd = torch.randn(B, T, d, device=DEV).to(BF)
    side = torch.randn(B, T, d, device=DEV).to(BF)
    tags = torch.randn(B, 8, 16, device=DEV).to(BF)
    vals = torch.randn(B, 8, 32, device=DEV).to(BF)
    wt = torch.randn(B, T, d, device=DEV).to(BF).float()
    res = []
    for m, dt in ((m32, torch.float32), (mbf, BF)):
        ins = [t.to(dt).clone().requires_grad_() for t in (fwd, side, tags, vals)]
        out, w = m.read(*ins)
        (out.float() * wt).sum().backward()
        grads = {n: p.grad.float() for n, p in m.named_parameters() if p.grad is not None}
        res.append((out.float(), [t.grad.float() for t in ins], grads, w))
    (o32, g32, p32, w32), (obf, gbf, pbf, wbf) = res
    _check(obf, o32, 1e-2, "blended forward stream")
    _check(wbf, w32, 1e-2, "retrieval weights")
    for name, a, b in zip(("fwd", "side", "tags", "vals"), gbf, g32):
        _check(a, b, 4e-2, f"gradient of {name}")
    assert set(pbf) == set(p32), sorted(set(pbf) ^ set(p32))
    for n in p32:
        if p32[n].norm() > 1e-6:
            _check(pbf[n], p32[n], 6e-2, f"gradient of {n}")
    _status(fwd)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_spectral_weight_matches_torch_hook(dtype):
    """The hard spectral norm of ``cam.W_r1`` on its own kernel against torch's spectral-norm hook: the normalised
    weight, the updated ``u`` / ``v`` buffers over three training iterations, the evaluation-mode weight, and the
    gradient that reaches ``weight_orig``."""
    import copy

    cu = _cu()
    torch.manual_seed(2)
    d = 64
    lin = torch.nn.utils.spectral_norm(torch.nn.Linear(3 * d + 1, d)).to(DEV).to(dtype)
    mine = copy.deepcopy(lin)
    tol = 2e-2 if dtype == BF else 1e-4
    for mode in ("train", "train", "train", "eval"):
        for m in (lin, mine):
            m.train(mode == "train")
            m.zero_grad(set_to_none=True)
        x = torch.randn(16, 3 * d + 1, device=DEV, dtype=dtype)
        want = lin(x)
        (want.float() ** 2).sum().backward()
        W = cu.spectral_weight(mine)
        got = torch.nn.functional.linear(x, W, mine.bias)
        (got.float() ** 2).sum().backward()
        _check(W, lin.weight, tol, f"normalised weight ({mode})")
        _check(got, want, tol, f"output ({mode})")
        _check(mine.weight_u, lin.weight_u, tol, "u")
        _check(mine.weight_v, lin.weight_v, tol, "v")
        _check(mine.weight_orig.grad, lin.weight_orig.grad, 5 * tol, f"gradient of weight_orig ({mode})")
    _status(x)


def test_peer_wait_runs_out_and_reports():
    """A wait for a flag that nothing sets ends after its time limit: the kernel returns, the host raises
    KernelTimeout naming the wait site, and the next launch works. The "peers" are this GPU's own zeroed
    buffers and the limit is 20 ms, so nothing hangs."""
    import time

    from gdnet_b200 import _ext

    cu = _cu()
    _ext.check_status(torch.zeros(1, device=DEV))
    budget = 20_000_000
    # halo exchange as rank 1 of 2: nothing to push (rank 1 is the last), waits for rank 0's flag
    slots = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    flags = torch.zeros(64, dtype=torch.int32, device=DEV)
    two = lambda t: torch.tensor([t.data_ptr(), t.data_ptr()], dtype=torch.int64, device=DEV)
    tail = torch.ones(2, 3, 64, device=DEV, dtype=BF)
    halo = torch.full_like(tail, 7.0)
    t0 = time.perf_counter()
    cu.K.halo_push_wait(tail, halo, two(slots), two(flags), 0, 0, 1, 2, 1, False, budget)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.5, "the wait did not honour its 20 ms limit"
    with pytest.raises(_ext.KernelTimeout, match="site 40"):
        _ext.check_status(tail)
    assert float(halo.abs().max()) == 0.0, "a halo that never arrived must read as zeros"
    # MAX all-reduce as rank 0 of 2: rank 1's flag never comes
    area = torch.zeros(2 * 2 * 256, device=DEV)
    fl = torch.zeros(64, dtype=torch.int32, device=DEV)
    vec = torch.rand(100, device=DEV)
    keep = vec.clone()
    cu.K.max_allreduce(vec, two(area), two(fl), 256, 0, 2, 1, budget)
    torch.cuda.synchronize()
    with pytest.raises(_ext.KernelTimeout, match="site 50"):
        _ext.check_status(vec)
    assert torch.equal(vec, keep), "after a timeout the vector keeps this rank's values"
    # the context is intact: a normal launch right after
    cu.K.max_allreduce(vec, _ptr_table(area), _ptr_table(fl), 256, 0, 1, 2)
    torch.cuda.synchronize()
    _ext.check_status(vec)
    assert torch.equal(vec, keep)


def test_engine_gradient_buffers_match_autograd():
    """Every parameter's task and information gradient, as the engine's kernels leave them in the two flat
    fp32 buffers (weight-gradient epilogues, packed small-parameter delivery, conv taps through their base
    parameter, batched spectral-penalty gradients), against plain autograd on the same model, over two steps
    (the second step would expose a gradient that went to the buffer of the other pass)."""
    import copy

    from gdnet_b200.model import GDNet
    from gdnet_b200.train.engine import TrainEngine
    from gdnet_b200.train.step import info_losses
    from gdnet_b200.utils.fp8 import autocast, cast_for_precision

    torch.manual_seed(0)
    base = GDNet(vocab_size=1024, d_embed=128, d=128, n_layers=2, n_cycles=2, kernel_size=4, chunk_size=256).to(DEV)
    cast_for_precision(base, "fp8")
    ref_model = copy.deepcopy(base)
    eng = TrainEngine(copy.deepcopy(base), precision="fp8")
    eng._update = lambda *a, **k: None            # keep the parameters: only the gradient buffers are compared
    g = torch.Generator().manual_seed(3)
    for step in range(2):
        tok = torch.randint(0, 1024, (2, 257), generator=g).to(DEV)
        inp, tgt = tok[:, :-1], tok[:, 1:]
        torch.manual_seed(100 + step)             # same random probe vectors of the spectral penalty in both runs
        eng.projected_step(inp, tgt)
        got = {}
        for which in ("task", "info"):
            eng._point_main_grad(which)
            got[which] = {n: p.main_grad.clone() for n, p in eng.module.named_parameters()}
        torch.manual_seed(100 + step)
        with autocast("fp8", "cuda"):
            logits, side, _, _, gate_vals, _, _ = ref_model(inp, None, None, return_gates="mean")
            loss_task = F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt.reshape(-1))
        params = dict(ref_model.named_parameters())
        names = list(params)
        g_task = torch.autograd.grad(loss_task, [params[n] for n in names], retain_graph=True, allow_unused=True)
        with autocast("fp8", "cuda"):
            loss_info = info_losses(ref_model, side, gate_vals)
        g_info = torch.autograd.grad(loss_info, [params[n] for n in names], allow_unused=True)
        for which, grads in (("task", g_task), ("info", g_info)):
            for n, gr in zip(names, grads):
                have = got[which][n].float()
                want = torch.zeros_like(have) if gr is None else gr.float()
                scale = float(want.norm())
                if scale < 1e-6:
                    assert float(have.norm()) < 1e-4, f"step {step} {which} {n}: expected no gradient"
                else:
                    rel = float((have - want).norm()) / scale
                    assert rel < 0.08, f"step {step} {which} gradient of {n}: relative error {rel:.3f}"


@pytest.mark.parametrize("fp8", [False, True])
def test_linear_cross_entropy_chunked(fp8):
    """Projection + loss in row chunks against the unfused path: loss, gradient of the input, gradient of the
    head (through autograd and through an installed fp32 gradient buffer)."""
    cu = _cu()
    M, Kd, V, Vp = 512, 256, 1000, 1024
    torch.manual_seed(1)
    x = torch.randn(M, Kd, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(Vp, Kd, device=DEV) * 0.05).to(BF).requires_grad_()
    tgt = torch.randint(0, V, (M,), device=DEV)
    tgt[::7] = -100
    loss = cu.linear_cross_entropy(x, w, tgt, V, fp8, chunk_rows=128)
    (2.0 * loss).backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    want = F.cross_entropy((xr @ wr.t())[:, :V], tgt, ignore_index=-100)
    (2.0 * want).backward()
    tol = 0.08 if fp8 else 0.02
    assert abs(float(loss) - float(want)) < tol * abs(float(want))
    _check(x.grad, xr.grad, tol, "d loss / d x")
    _check(w.grad, wr.grad, tol, "d loss / d W")
    w2 = w.detach().clone().requires_grad_()
    w2.main_grad = torch.zeros(Vp, Kd, device=DEV)
    cu.linear_cross_entropy(x.detach(), w2, tgt, V, fp8, chunk_rows=256).backward()
    assert w2.grad is None
    _check(w2.main_grad, 0.5 * wr.grad, tol, "head gradient in the fp32 buffer")
