"""The reference's public kernel entry points (gdnet/kernel/gated_causal_depthwise_conv: ``rmsnorm_fwd``,
``gate_stream_update_fwd``, ``gated_output`` / ``GatedCausalDepthwiseConvFunction``; gdnet/kernel/fp8_linear:
``fp8_gemm``) on CUDA tensors, and the fused update kernels of the layer step called directly, each against
the plain-PyTorch fp32 statement of the same arithmetic with autograd
(the cases of the reference's tests/test_gated_causal_dwconv.py:150-218, on the shapes the sm_100a kernels take)."""

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
    got, want = got.detach().float(), want.detach().float()
    return float((got - want).norm() / want.norm().clamp(min=1e-12))


def _check(got, want, tol, what):
    r = _rel(got, want)
    assert r < tol, f"{what}: relative error {r:.4g} (tol {tol})"


def _status(t):
    from gdnet_b200 import _ext

    _ext.check_status(t)


@pytest.mark.parametrize("rows,d", [(64, 128), (100, 256), (7, 1024)])
def test_rmsnorm_fwd_api(rows, d):
    from gdnet_b200.kernel.gated_causal_depthwise_conv import rmsnorm_fwd

    h = torch.randn(rows, d, device=DEV).to(BF)
    w = torch.rand(d, device=DEV) + 0.5
    y, rstd = rmsnorm_fwd(h, w, 1e-6)
    want_rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6)
    _check(rstd, want_rstd, 1e-5, "rstd")
    _check(y, h.float() * want_rstd[:, None] * w, 6e-3, "normalised rows")
    _status(h)


@pytest.mark.parametrize("rows,d", [(64, 128), (300, 256), (16, 8)])
def test_gate_stream_update_api_fwd_bwd(rows, d):
    from gdnet_b200.kernel.gated_causal_depthwise_conv import gate_stream_update_fwd

    ins = [torch.randn(rows, d, device=DEV).to(BF) for _ in range(3)] + [torch.rand(rows, d, device=DEV).to(BF)]
    leaves = [t.clone().requires_grad_() for t in ins]
    refs = [t.float().requires_grad_() for t in ins]
    fo, so = gate_stream_update_fwd(*leaves)
    fr, sr, _ = ref.gate_stream_update(*refs)
    _check(fo, fr, 6e-3, "fwd'")
    _check(so, sr, 6e-3, "side'")
    wf, ws = torch.randn_like(fr), torch.randn_like(sr)
    (fo.float() * wf.to(BF).float() + so.float() * ws.to(BF).float()).sum().backward()
    (fr * wf.to(BF).float() + sr * ws.to(BF).float()).sum().backward()
    for name, a, b in zip(("g_pre", "conv", "side", "R"), leaves, refs):
        _check(a.grad, b.grad, 1e-2, f"gradient of {name}")
    _status(fo)


@pytest.mark.parametrize("rows,d", [(256, 128), (512, 256)])
def test_gated_output_all_gradients(rows, d):
    """Outputs and the gradients of all eight differentiable inputs of ``gated_output``."""
    from gdnet_b200.kernel.gated_causal_depthwise_conv import GatedCausalDepthwiseConvFunction, gated_output

    torch.manual_seed(rows + d)
    c = torch.randn(rows, d, device=DEV).to(BF)
    s = torch.randn(rows, d, device=DEV).to(BF)
    R = torch.rand(rows, d, device=DEV).to(BF)
    W1 = (torch.randn(d, d, device=DEV) / d**0.5).to(BF)
    W2 = (torch.randn(d, d, device=DEV) * 0.05).to(BF)
    b1 = (torch.randn(d, device=DEV) * 0.1).to(BF)
    b2 = (torch.randn(d, device=DEV) * 0.1 + 1.0).to(BF)
    wn = (torch.rand(d, device=DEV) + 0.5).to(BF)
    ins = [c, s, R, W1, b1, wn, W2, b2]
    leaves = [t.clone().requires_grad_() for t in ins]
    refs = [t.float().requires_grad_() for t in ins]
    fo, so = gated_output(*leaves, 1e-6)
    assert fo.dtype == BF and fo.shape == (rows, d)
    g_pre = ref.gate_pre(refs[0], refs[3], refs[4], refs[5], refs[6], refs[7], 1e-6)
    fr, sr, _ = ref.gate_stream_update(g_pre, refs[0], refs[1], refs[2])
    _check(fo, fr, 1e-2, "fwd'")
    _check(so, sr, 1e-2, "side'")
    wf, ws = torch.randn_like(fr).to(BF).float(), torch.randn_like(sr).to(BF).float()
    (fo.float() * wf + so.float() * ws).sum().backward()
    (fr * wf + sr * ws).sum().backward()
    for name, a, b in zip("conv side R W1 b1 W_norm W2 b2".split(), leaves, refs):
        assert a.grad is not None, name
        _check(a.grad, b.grad, 3e-2, f"gradient of {name}")
    fo2, so2 = GatedCausalDepthwiseConvFunction.apply(*[t.detach() for t in leaves], 1e-6)
    assert torch.equal(fo2, fo.detach()) and torch.equal(so2, so.detach())
    _status(fo)


def test_fp8_gemm_per_tensor_fast_path():
    """Per-tensor scaled e4m3 GEMM on the hardware-scaled kernel; device scales, no host read."""
    from gdnet_b200.kernel.fp8_linear import fp8_gemm, quantize_fp8

    M, N, Kd = 256, 384, 512
    a, b = torch.randn(M, Kd, device=DEV), torch.randn(N, Kd, device=DEV) * 0.3
    sa = (448.0 / a.abs().max()).reshape(1)
    sb = (448.0 / b.abs().max()).reshape(1)
    a8, _, _ = quantize_fp8(a.to(BF), sa, need_col=False)
    b8, _, _ = quantize_fp8(b.to(BF), sb, need_col=False)
    got = fp8_gemm(a8, b8, 1.0 / sa, 1.0 / sb, out_dtype=torch.float32)
    want = (a8.float() @ b8.float().t()) / (sa * sb)
    _check(got, want, 2e-3, "per-tensor fp8 gemm")
    got2 = fp8_gemm(a8, b8, float(1.0 / sa), float(1.0 / sb))
    _check(got2, want, 1e-2, "per-tensor fp8 gemm, python scales, bf16 out")
    _status(a)


# ---------------------------------------------------------------------------------------
# the fused update kernels of the layer step, called directly
# ---------------------------------------------------------------------------------------
def _gate_oracle(g_pre, z, c, s, w_r, eps_r):
    zf = z.float()
    rstd = torch.rsqrt(zf.pow(2).mean(-1, keepdim=True) + eps_r)
    R = torch.sigmoid(zf * rstd * w_r.float())
    g = torch.sigmoid(g_pre.float())
    fo = c.float() * g + s.float() * R
    so = c.float() * (1 - g) + s.float() * (1 - R)
    return fo, so, g, rstd.squeeze(-1)


# d = 256 * n runs the kernel in which n warps share a row (see the backward test below)
@pytest.mark.parametrize("rows,d,quant", [(256, 128, True), (384, 256, True), (50, 64, False), (131, 256, False),
                                          (301, 512, False), (256, 512, True), (515, 1024, False), (384, 1024, True),
                                          (77, 2048, False), (128, 2048, True)])
def test_gate_update_fwd_kernel(rows, d, quant):
    cu = _cu()
    torch.manual_seed(rows)
    g_pre, z, c, s = (torch.randn(rows, d, device=DEV).to(BF) for _ in range(4))
    w_r = torch.rand(d, device=DEV) + 0.5
    fo = torch.empty(rows, d, device=DEV, dtype=BF)
    so = torch.empty_like(fo)
    gate = torch.empty_like(fo)
    rstd = torch.empty(rows, device=DEV)
    gsum = torch.zeros((), device=DEV)
    extra = ()
    if quant:
        kb = d // 128
        q = torch.empty(rows, d, dtype=torch.float8_e4m3fn, device=DEV)
        qs = torch.empty(kb, rows, device=DEV)
        qp = cu.packed_buffer(rows, d, DEV)
        extra = (q, qs, qp)
    cu.K.gate_update_fwd(g_pre, z, c, s, w_r, fo, so, gate, rstd, gsum, 1e-6, *extra)
    torch.cuda.synchronize()
    _status(fo)
    wf, ws, wg, wr = _gate_oracle(g_pre, z, c, s, w_r, 1e-6)
    _check(fo, wf, 6e-3, "fwd'")
    _check(so, ws, 6e-3, "side'")
    _check(gate, wg, 6e-3, "gate")
    _check(rstd, wr, 1e-4, "rstd of the recovery pre-activation")
    assert abs(float(gsum) - float(wg.sum())) < 2e-3 * float(wg.sum())
    if quant:
        # the FP8 copy of side' as the next step's recovery GEMM reads it: e4m3 values, power-of-two 1x128 scales,
        # the same scales packed as UE8M0 chunks
        q_ref, s_ref = ref.quantize_1x128(so.float(), pow2=True)
        assert torch.equal(qs.t().contiguous(), s_ref), "1x128 scales of the quantised side stream"
        assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
        assert torch.equal(qp, ref.pack_ue8m0_rows(s_ref)), "packed UE8M0 chunks of the quantised side stream"


# d = 256 * n runs the kernel in which n warps share a row (row counts that leave the last group of rows partly empty
# included); other widths the one-warp-per-row form
@pytest.mark.parametrize("rows,d,quant", [(256, 128, True), (384, 256, True), (131, 256, False), (301, 512, False),
                                          (256, 512, True), (515, 1024, False), (384, 1024, True), (77, 2048, False),
                                          (128, 2048, True), (64, 384, False)])
def test_gate_update_bwd_kernel(rows, d, quant):
    """Every output of the fused backward of the stream update against autograd through the fp32 statement."""
    cu = _cu()
    torch.manual_seed(rows + 1)
    g_pre, z, c, s = (torch.randn(rows, d, device=DEV).to(BF) for _ in range(4))
    dF, dS = (torch.randn(rows, d, device=DEV).to(BF) for _ in range(2))
    w_r = torch.rand(d, device=DEV) + 0.5
    b2g = torch.randn(d, device=DEV) * 0.2
    parts = d // 128
    ssq = torch.rand(rows, parts, device=DEV) * 40 + 20           # partial sums of squares of the gate's hidden layer
    eps_g, dgm = 1e-6, torch.tensor([0.37], device=DEV)
    rstd_z = torch.rsqrt(z.float().pow(2).mean(-1) + 1e-6)
    dq, dz = torch.empty(rows, d, device=DEV, dtype=BF), torch.empty(rows, d, device=DEV, dtype=BF)
    dsc = torch.empty(rows, 2 * d, device=DEV, dtype=BF)
    rowcoef = torch.empty(rows, device=DEV)
    db2g, dw_r, db2r = (torch.zeros(d, device=DEV) for _ in range(3))
    extra = ()
    if quant:
        dz8 = torch.empty(rows, d, dtype=torch.float8_e4m3fn, device=DEV)
        sdz = torch.empty(d // 128, rows, device=DEV)
        pdz = cu.packed_buffer(rows, d, DEV)
        extra = (dz8, sdz, pdz)
    cu.K.gate_update_bwd(dF, dS, g_pre, z, c, s, w_r, b2g, rstd_z, ssq, eps_g, dgm, dq, dz, dsc, rowcoef, db2g, dw_r, db2r, *extra)
    torch.cuda.synchronize()
    _status(dq)
    # oracle
    gp, zz, cc, ss, ww = (t.float().requires_grad_() for t in (g_pre, z, c, s, w_r))
    fo, so, g, _ = _gate_oracle(gp, zz, cc, ss, ww, 1e-6)
    loss = (fo * dF.float()).sum() + (so * dS.float()).sum() + dgm[0] * g.mean()
    loss.backward()
    _check(dz, zz.grad, 1e-2, "dz")
    _check(dsc[:, :d], ss.grad, 1e-2, "direct gradient of the side stream")
    _check(dsc[:, d:], cc.grad, 1e-2, "direct gradient of the conv output")
    r_g = torch.rsqrt(ssq.sum(-1) / d + eps_g)
    _check(dq, gp.grad * r_g[:, None], 1e-2, "dq = rstd_g * d g_pre")
    want_rc = r_g * r_g / d * (gp.grad * (g_pre.float() - b2g)).sum(-1)
    _check(rowcoef, want_rc, 1e-2, "row coefficient of the gate norm's backward")
    _check(db2g, gp.grad.sum(0), 1e-2, "db2 of the gate")
    _check(dw_r, ww.grad, 1e-2, "gradient of the recovery norm weight")
    _check(db2r, zz.grad.sum(0), 1e-2, "db2 of the recovery MLP")
    if quant:
        q_ref, s_ref = ref.quantize_1x128(dz.float(), pow2=True)
        assert torch.equal(sdz.t().contiguous(), s_ref)
        assert (dz8.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
        assert torch.equal(pdz, ref.pack_ue8m0_rows(s_ref))


def test_small_reduction_kernels():
    """colsum, segment_add, scale_cols / unscale_cols_bwd."""
    cu = _cu()
    x = torch.randn(1000, 384, device=DEV).to(BF)
    out = torch.full((384,), 2.0, device=DEV)
    cu.K.colsum(x, out)
    _check(out, x.float().sum(0) + 2.0, 1e-4, "colsum accumulates into its output")
    xs = torch.randn(512, 256, device=DEV).to(BF)[:, 64:192]          # a column range of a wider buffer
    out2 = torch.zeros(128, device=DEV)
    cu.K.colsum(xs, out2)
    _check(out2, xs.float().sum(0), 1e-4, "colsum over a strided view")

    src = torch.randn(300 + 128 + 40, device=DEV)
    dsts = [torch.ones(300, device=DEV), torch.ones(128, device=DEV), torch.ones(40, device=DEV)]
    addr = torch.tensor([t.data_ptr() for t in dsts], dtype=torch.int64, device=DEV)
    offs = torch.tensor([0, 300, 428], dtype=torch.int32, device=DEV)
    cu.K.segment_add(src, addr, offs)
    torch.cuda.synchronize()
    for t, lo in zip(dsts, (0, 300, 428)):
        assert torch.allclose(t, 1.0 + src[lo : lo + t.numel()])

    W2 = torch.randn(256, 384, device=DEV).to(BF)
    colw = torch.rand(384, device=DEV) + 0.5
    W2w = torch.empty_like(W2)
    cu.K.scale_cols(W2, colw, W2w)
    _check(W2w, W2.float() * colw, 6e-3, "scale_cols")
    dW2w = torch.randn(256, 384, device=DEV)
    dW2 = torch.full((256, 384), 0.5, device=DEV)
    dcolw = torch.full((384,), -1.0, device=DEV)
    cu.K.unscale_cols_bwd(dW2w, W2, colw, dW2, dcolw)
    _check(dW2, 0.5 + dW2w * colw, 1e-5, "dW2 accumulated")
    _check(dcolw, -1.0 + (dW2w * W2.float()).sum(0), 1e-4, "gradient of the column weights accumulated")
    _status(x)
