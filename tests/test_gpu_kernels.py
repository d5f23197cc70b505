"""GPU numerics of every sm_100a kernel against the plain-PyTorch fp32 statement of the same op."""

import pytest
import torch
import torch.nn.functional as F

from gdnet_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _cu():
    from gdnet_b200.ops import cuda as cu

    return cu


def _close(got, want, atol, rtol, what=""):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    bad = err > tol
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} mismatched, max err {float(err.max()):.4g} "
            f"(ref max {float(want.abs().max()):.4g}), first bad at {idx}: got {float(got[tuple(idx)]):.5g} "
            f"want {float(want[tuple(idx)]):.5g}"
        )


def _status_clean(t):
    from gdnet_b200 import _ext

    _ext.check_status(t)


# ---------------------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 128), (384, 512, 192), (1000, 128, 256), (4096, 1024, 1024)])
def test_gemm_bf16_kmajor(M, N, K):
    cu = _cu()
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    out = cu.gemm_bf16(a, b)
    torch.cuda.synchronize()
    _status_clean(a)
    _close(out, a.float() @ b.float().t(), atol=0.05 * K ** 0.5, rtol=2e-2, what=f"bf16 gemm {M}x{N}x{K}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 320), (1024, 1024, 4096)])
def test_gemm_bf16_mn_major(a_mn, b_mn, M, N, K):
    cu = _cu()
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    out = cu.gemm_bf16(a_in, b_in, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _status_clean(a)
    _close(out, a.float() @ b.float().t(), atol=0.05 * K ** 0.5, rtol=2e-2, what=f"mn gemm a_mn={a_mn} b_mn={b_mn}")


def test_gemm_bf16_epilogues():
    cu = _cu()
    M, N, K = 512, 512, 256
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16) * 0.5
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.1
    bias = torch.randn(N, device=DEV)
    base = a.float() @ b.float().t()

    # bias + silu + pre-activation copy + per-row partial sums of squares
    pre = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ssq = torch.zeros(M, N // 128, device=DEV)
    out = cu.gemm_bf16(a, b, bias=bias, act=cu.ACT_SILU, pre_out=pre, ssq_out=ssq)
    want_pre = base + bias
    _close(pre, want_pre, 2e-2, 2e-2, "pre_out")
    _close(out, F.silu(want_pre), 2e-2, 2e-2, "silu out")
    _close(ssq.sum(1), out.float().pow(2).sum(1), 1e-2, 1e-2, "ssq partials")

    # row scale from ssq partials: rstd * acc + bias
    out2 = cu.gemm_bf16(a, b, bias=bias, ssq_in=ssq, norm_dim=N, norm_eps=1e-6)
    rstd = torch.rsqrt(ssq.sum(1) / N + 1e-6)
    _close(out2, base * rstd[:, None] + bias, 2e-2, 2e-2, "row scale from ssq")

    # explicit row scale, bf16 bias
    rs = torch.rand(M, device=DEV) + 0.5
    out3 = cu.gemm_bf16(a, b, bias=bias.bfloat16(), row_scale=rs)
    _close(out3, base * rs[:, None] + bias.bfloat16().float(), 2e-2, 2e-2, "row scale")

    # aux modes
    aux = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    _close(cu.gemm_bf16(a, b, aux=aux, aux_mode=cu.AUX_ADD), base + aux.float(), 2e-2, 2e-2, "aux add")
    sg = torch.sigmoid(aux.float())
    dsilu = sg * (1 + aux.float() * (1 - sg))
    _close(cu.gemm_bf16(a, b, aux=aux, aux_mode=cu.AUX_MUL_SILU_GRAD), base * dsilu, 2e-2, 2e-2, "aux silu grad")
    rc = torch.randn(M, device=DEV) * 0.1
    want = (base - F.silu(aux.float()) * rc[:, None]) * dsilu
    _close(cu.gemm_bf16(a, b, aux=aux, aux_mode=cu.AUX_RMS_SILU_BWD, rowcoef=rc), want, 2e-2, 2e-2, "aux rms bwd")

    # fp32 output with accumulation, strided output view
    acc = torch.ones(M, 2 * N, device=DEV)
    cu.gemm_bf16(a, b, out=acc[:, N:], accumulate=True)
    _close(acc[:, N:], base + 1.0, 1e-2, 1e-2, "fp32 accumulate")
    assert torch.all(acc[:, :N] == 1.0)
    torch.cuda.synchronize()
    _status_clean(a)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (4096, 1024, 2048), (1000, 256, 256)])
def test_gemm_fp8_blockscaled(M, N, K):
    cu = _cu()
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.2
    a8, sa = ref.quantize_1x128(a.float())
    b8, sb = ref.quantize_128x128(b.float())
    want = ref.fp8_gemm_blockscaled(a8, sa, b8, sb, out_dtype=torch.float32)
    out = cu.gemm_fp8(a8, sa.t().contiguous(), b8, sb.contiguous(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    _status_clean(a)
    _close(out, want, 1e-2, 1e-3, f"fp8 gemm {M}x{N}x{K}")
    bias = torch.randn(N, device=DEV)
    out2 = cu.gemm_fp8(a8, sa.t().contiguous(), b8, sb.contiguous(), bias=bias, act=cu.ACT_SILU)
    _close(out2, F.silu(want + bias), 3e-2, 2e-2, "fp8 gemm bias+silu")


# ---------------------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------------------
def test_quantize_rows_matches_reference():
    cu = _cu()
    x = (torch.randn(384, 512, device=DEV) * 3).bfloat16()
    q, s = cu.quantize_rows(x)
    q_ref, s_ref = ref.quantize_1x128(x.float())
    _close(s.t(), s_ref, 0, 1e-5, "row scales")
    deq, deq_ref = ref.dequantize_1x128(q, s.t()), ref.dequantize_1x128(q_ref, s_ref)
    assert (deq - deq_ref).abs().max() <= 0.07 * x.float().abs().max()
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
    # silu fused in front of the quantiser
    q2, s2 = cu.quantize_rows(x, pre_silu=True)
    want = F.silu(x.float()).bfloat16().float()
    _close(ref.dequantize_1x128(q2, s2.t()), want, 0.02, 0.07, "silu + quant")


def test_quantize_transposed_modes():
    cu = _cu()
    x = (torch.randn(256, 384, device=DEV) * 2).bfloat16()
    xt = x.float().t().contiguous()
    qt, st = cu.quantize_transposed(x, cu.Q_BLOCK)
    q_ref, s_ref = ref.quantize_128x128(xt)
    _close(st, s_ref, 0, 1e-5, "block scales (transposed)")
    _close(ref.dequantize_128x128(qt, st), xt, 0.02, 0.07, "block transposed dequant")
    qc, sc = cu.quantize_transposed(x, cu.Q_COLS)
    qr, sr = ref.quantize_1x128(xt)            # rows of x^T in blocks of 128 original rows
    _close(sc.t(), sr, 0, 1e-5, "col scales")
    _close(ref.dequantize_1x128(qc, sc.t()), xt, 0.02, 0.07, "cols transposed dequant")
    q, s, qt2, st2 = cu.quantize_rows_and_transposed(x, cu.Q_COLS)
    assert torch.equal(qt2.view(torch.uint8), qc.view(torch.uint8)) and torch.equal(st2, sc)
    _close(ref.dequantize_1x128(q, s.t()), x.float(), 0.02, 0.07, "rows in combined call")


def test_quantize_weight_both_layouts():
    cu = _cu()
    w = torch.randn(256, 512, device=DEV).bfloat16()
    qw = cu.quantize_weight(w)
    _close(ref.dequantize_128x128(qw.q, qw.s), w.float(), 0.02, 0.07, "weight")
    _close(ref.dequantize_128x128(qw.qt, qw.st), w.float().t(), 0.02, 0.07, "weight^T")
    assert cu.quantize_weight(w) is qw


@pytest.mark.parametrize("rows,cols", [(70, 130), (192, 320)])    # ragged tiles; whole tiles (the 16-byte path)
def test_quantize_per_tensor(rows, cols):
    cu = _cu()
    x = torch.randn(rows, cols, device=DEV).bfloat16()
    scale = torch.tensor([448.0 / 4.0], device=DEV)
    q, qc, amax = cu.quantize_fp8_tensor(x, scale)
    want = (x.float() * scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert (q.view(torch.uint8) != want.view(torch.uint8)).float().mean() < 1e-3
    assert torch.equal(qc.view(torch.uint8), q.view(torch.uint8).t())
    assert torch.allclose(amax, x.float().abs().max())


# ---------------------------------------------------------------------------------------
# hardware block-scaled FP8 GEMM (UE8M0 scales applied by the tensor core)
# ---------------------------------------------------------------------------------------
def _mx_operands(M, N, K, vary_rows=True):
    a = torch.randn(M, K, device=DEV)
    if vary_rows:   # very different magnitudes per row and per K block, so a wrong scale mapping is visible
        a = a * torch.exp2(torch.randint(-6, 7, (M, K // 128), device=DEV).float()).repeat_interleave(128, dim=1)
    b = torch.randn(N, K, device=DEV) * 0.2
    if vary_rows:
        b = b * torch.exp2(torch.randint(-3, 4, (N // 128, K // 128), device=DEV).float()).repeat_interleave(
            128, dim=0).repeat_interleave(128, dim=1)
    a8, sa = ref.quantize_1x128(a, pow2=True)
    b8, sb = ref.quantize_128x128(b, pow2=True)
    return a8, sa, b8, sb


@pytest.mark.parametrize("vary", [False, True])
@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (4096, 1024, 2048)])
def test_gemm_fp8_mx_matches_oracle(M, N, K, vary):
    cu = _cu()
    a8, sa, b8, sb = _mx_operands(M, N, K, vary)
    want = ref.fp8_gemm_blockscaled(a8, sa, b8, sb, out_dtype=torch.float32)
    out = cu.gemm_fp8_mx(a8, ref.pack_ue8m0_rows(sa), b8, ref.pack_ue8m0_blocks(sb), out_dtype=torch.float32)
    torch.cuda.synchronize()
    _status_clean(a8)
    _close(out, want, 1e-2 * float(want.abs().max()) * 1e-2 + 1e-3, 2e-3, f"mx gemm {M}x{N}x{K} vary={vary}")


def test_quantizer_pow2_and_packed_chunks():
    cu = _cu()
    x = (torch.randn(256, 384, device=DEV) * torch.exp2(torch.randint(-4, 5, (256, 1), device=DEV).float())).bfloat16()
    packed = cu.packed_buffer(256, 384, DEV)
    q, s = cu.quantize_rows(x, pow2=True, packed=packed)
    q_ref, s_ref = ref.quantize_1x128(x.float(), pow2=True)
    _close(s.t(), s_ref, 0, 1e-6, "pow2 row scales")
    assert torch.equal(packed, ref.pack_ue8m0_rows(s_ref)), "packed UE8M0 chunks differ"
    assert (q.view(torch.uint8) != q_ref.view(torch.uint8)).float().mean() < 1e-3
    # weights: both layouts, constant-filled chunks
    w = torch.randn(256, 384, device=DEV).bfloat16()
    wq = torch.empty(256, 384, dtype=torch.float8_e4m3fn, device=DEV)
    ws = torch.empty(2, 3, device=DEV)
    wt = torch.empty(384, 256, dtype=torch.float8_e4m3fn, device=DEV)
    wts = torch.empty(3, 2, device=DEV)
    pw, pwt = cu.packed_buffer(256, 384, DEV), cu.packed_buffer(384, 256, DEV)
    cu.K.quant_tile(w, False, wq, ws, cu.Q_BLOCK, wt, wts, cu.Q_BLOCK, True, pw, pwt)
    _, ws_ref = ref.quantize_128x128(w.float(), pow2=True)
    _close(ws, ws_ref, 0, 1e-6, "pow2 block scales")
    assert torch.equal(pw, ref.pack_ue8m0_blocks(ws_ref)) and torch.equal(pwt, ref.pack_ue8m0_blocks(ws_ref.t()))
    # transposed with per-column scales (the A operand of a weight-gradient GEMM)
    xt = torch.empty(384, 256, dtype=torch.float8_e4m3fn, device=DEV)
    xts = torch.empty(2, 384, device=DEV)
    pxt = cu.packed_buffer(384, 256, DEV)
    cu.K.quant_tile(x, False, None, None, cu.Q_ROWS, xt, xts, cu.Q_COLS, True, None, pxt)
    _, st_ref = ref.quantize_1x128(x.float().t().contiguous(), pow2=True)
    _close(xts.t(), st_ref, 0, 1e-6, "pow2 col scales")
    assert torch.equal(pxt, ref.pack_ue8m0_rows(st_ref))


def test_gemm_fp8_mx_quantised_output():
    """The epilogue's e4m3 copy of silu(out): one power-of-two scale per 64 columns of a row, stored as the two
    UE8M0 bytes of the packed chunk that belong to those columns."""
    cu = _cu()
    M, N, K = 256, 384, 256
    a8, sa, b8, sb = _mx_operands(M, N, K, True)
    bias = torch.randn(N, device=DEV)
    q8 = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=DEV)
    p8 = cu.packed_buffer(M, N, DEV)
    out = cu.gemm_fp8_mx(a8, ref.pack_ue8m0_rows(sa), b8, ref.pack_ue8m0_blocks(sb), bias=bias, q8=q8, q8_p=p8,
                         q8_silu=True)
    torch.cuda.synchronize()
    _status_clean(a8)
    act = torch.nn.functional.silu(out.float()).bfloat16().float()
    # scale byte of row r, 32-column step j of chunk (r // 128, c // 128): (r % 32) * 16 + (r % 128 // 32) * 4 + j
    r = torch.arange(M, device=DEV)
    off = (r % 32) * 16 + (r % 128 // 32) * 4
    chunks = p8.view(M // 128, N // 128, 512)
    scale = torch.empty(M, N // 32, device=DEV)
    for cb in range(N // 128):
        for j in range(4):
            scale[:, cb * 4 + j] = torch.exp2(chunks[r // 128, cb, off + j].float() - 127.0)
    assert torch.equal(scale[:, 0::2], scale[:, 1::2]), "both 32-column steps of a 64-column group share a scale"
    amax = act.view(M, N // 64, 64).abs().amax(-1)
    s64 = scale[:, 0::2]
    ok = (s64 * 448.0 >= amax * (1 - 1e-3)) & ((s64 * 448.0 < 2.0 * amax * (1 + 1e-3)) | (amax == 0))
    assert bool(ok.all()), "scales are not the next power of two above amax/448"
    deq = q8.float().view(M, N // 64, 64) * s64[:, :, None]
    err = float((deq.view(M, N) - act).norm() / act.norm())
    assert err < 0.05, f"quantised copy differs from silu(out): rel err {err}"
    # the copy as the A operand of a second GEMM: every 32-column K step must be scaled by its own byte (the two
    # halves of a 128-column block differ here, unlike operands quantised in 1x128 blocks)
    assert bool((s64[:, 0::2] != s64[:, 1::2]).any()), "test needs rows whose two 64-column scales differ"
    w8, sw = ref.quantize_128x128(torch.randn(256, N, device=DEV) * 0.05, pow2=True)
    second = cu.gemm_fp8_mx(q8, p8, w8, ref.pack_ue8m0_blocks(sw), out_dtype=torch.float32)
    torch.cuda.synchronize()
    _status_clean(a8)
    wq = w8.float() * sw.repeat_interleave(128, 0).repeat_interleave(128, 1)
    want2 = deq.view(M, N) @ wq.t()
    _close(second, want2, 2e-3 * float(want2.abs().max()), 2e-3, "GEMM on the quantised copy")
    # without storing out
    q8b = torch.empty_like(q8)
    p8b = cu.packed_buffer(M, N, DEV)
    cu.gemm_fp8_mx(a8, ref.pack_ue8m0_rows(sa), b8, ref.pack_ue8m0_blocks(sb), bias=bias, q8=q8b, q8_p=p8b, q8_silu=True,
                   store_out=False)
    torch.cuda.synchronize()
    assert torch.equal(q8b.view(torch.uint8), q8.view(torch.uint8)) and torch.equal(p8b, p8)


@pytest.mark.parametrize("M,N,K", [(256, 128, 128), (256, 128, 640), (512, 256, 1536), (512, 384, 1024), (4096, 1024, 2048)])
def test_gemm_fp8_mx_pair_matches_single_cta(M, N, K):
    """The CTA-pair form (256 x 128 pair tiles, scale chunks fetched through a tensor map) against the single-CTA
    kernel on the same operands, plain and with bias + auxiliary add + quantised output."""
    cu = _cu()
    a8, sa, b8, sb = _mx_operands(M, N, K, True)
    pa, pb = ref.pack_ue8m0_rows(sa), ref.pack_ue8m0_blocks(sb)
    bias = torch.randn(N, device=DEV)
    aux = torch.randn(M, N, device=DEV).bfloat16()
    res = {}
    try:
        for pair in (0, 1):
            cu.K.gemm_set_mx_pair(pair)
            plain = cu.gemm_fp8_mx(a8, pa, b8, pb, out_dtype=torch.float32)
            q8 = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=DEV)
            p8 = cu.packed_buffer(M, N, DEV).zero_()
            fused = cu.gemm_fp8_mx(a8, pa, b8, pb, bias=bias, aux=aux, aux_mode=1, q8=q8, q8_p=p8)
            torch.cuda.synchronize()
            _status_clean(a8)
            res[pair] = (plain, fused, q8.view(torch.uint8).clone(), p8.clone())
    finally:
        cu.K.gemm_set_mx_pair(1)
    want = ref.fp8_gemm_blockscaled(a8, sa, b8, sb, out_dtype=torch.float32)
    _close(res[1][0], want, 1e-2 * float(want.abs().max()) * 1e-2 + 1e-3, 2e-3, f"mx pair gemm {M}x{N}x{K}")
    _close(res[1][0], res[0][0], 1e-5 * float(want.abs().max()), 1e-5, "pair against single CTA")
    _close(res[1][1].float(), res[0][1].float(), 1e-2 * float(want.abs().max()), 1e-2, "pair against single CTA, fused epilogue")
    assert (res[1][2] != res[0][2]).float().mean() < 1e-3 and torch.equal(res[1][3], res[0][3])


def test_gemm_bf16_strided_outputs_and_edges():
    """Outputs that are column slices of a wider buffer (the layer step writes into halves of its gradient buffer, in
    place over the auxiliary input) and shapes whose last tiles are partial: the bulk stores must clip at the matrix
    edge and leave the neighbouring columns alone."""
    cu = _cu()
    for M, N, K in ((1000, 160, 256), (512, 256, 128)):
        a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16) * 0.5
        b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.1
        base = a.float() @ b.float().t()
        wide = torch.randn(M, 2 * N, device=DEV, dtype=torch.bfloat16)
        keep, add = wide[:, :N].clone(), wide[:, N:].float().clone()
        view = wide[:, N:]
        cu.gemm_bf16(a, b, out=view, aux=view, aux_mode=cu.AUX_ADD)          # in place over the auxiliary input
        pre = torch.full((M, 2 * N), 7.0, device=DEV, dtype=torch.bfloat16)
        out = cu.gemm_bf16(a, b, pre_out=pre[:, :N], act=cu.ACT_SILU)
        torch.cuda.synchronize()
        _status_clean(a)
        _close(wide[:, N:], base + add, 3e-2, 2e-2, f"in-place aux add into a column slice {M}x{N}")
        assert torch.equal(wide[:, :N], keep), "columns beside the output slice were touched"
        _close(pre[:, :N], base, 2e-2, 2e-2, "pre_out slice")
        assert torch.all(pre[:, N:] == 7.0), "columns beside the pre_out slice were touched"
        _close(out, F.silu(base), 2e-2, 2e-2, "silu out")


# ---------------------------------------------------------------------------------------
# parameter gather carried by the GEMMs
# ---------------------------------------------------------------------------------------
def _jobs(src, dst, counters, first, chunks, chunk_bytes, subs):
    """Job rows (src, dst, counter, 16-byte vectors) for `chunks` ranges of `chunk_bytes`, each cut in `subs` pieces."""
    rows = []
    piece = chunk_bytes // subs
    for c in range(chunks):
        for j in range(subs):
            o = c * chunk_bytes + j * piece
            rows.append([src.data_ptr() + o, dst.data_ptr() + o, counters.data_ptr() + 4 * (first + c) if counters is not None else 0,
                         piece // 16])
    return rows


@pytest.mark.parametrize("M,N,K", [(512, 256, 256), (4096, 1024, 2048), (384, 256, 256)])
def test_gemm_fp8_mx_gathers_its_own_b_operand(M, N, K):
    """The hardware-scaled FP8 GEMM with its B operand (e4m3 rows and packed scales) arriving through gather jobs
    that the same launch carries: the producer warp waits for the per-128-row counters, so the result must equal
    the GEMM on the source buffers. The "owner's" memory is this GPU's own; M = 384 takes the single-CTA kernel,
    where the launcher copies first."""
    cu = _cu()
    a8, sa, b8, sb = _mx_operands(M, N, K, True)
    pa, pb = ref.pack_ue8m0_rows(sa), ref.pack_ue8m0_blocks(sb)
    want = cu.gemm_fp8_mx(a8, pa, b8, pb, out_dtype=torch.float32)
    nb = N // 128
    stage_q = torch.zeros_like(b8.view(torch.uint8))
    stage_p = torch.zeros_like(pb)
    cnt = torch.zeros(2 * nb, dtype=torch.int32, device=DEV)
    rows = _jobs(b8.view(torch.uint8), stage_q, cnt, 0, nb, 128 * K, 2) + _jobs(pb, stage_p, cnt, nb, nb, (K // 128) * 512, 1)
    table = torch.tensor(rows, dtype=torch.int64, device=DEV)
    for use in (1, 2):
        stage_q.zero_()
        stage_p.zero_()
        cu.K.attach_gather_jobs(table)
        cu.K.attach_b_ready(cnt[:nb], cnt[nb:], 2 * use, use)
        got = cu.gemm_fp8_mx(a8, pa, stage_q.view(torch.float8_e4m3fn), stage_p, out_dtype=torch.float32)
        torch.cuda.synchronize()
        _status_clean(a8)
        assert torch.equal(stage_q, b8.view(torch.uint8)) and torch.equal(stage_p, pb), "gathered bytes differ from the source"
        assert torch.equal(got, want), f"use {use}: GEMM on the gathered operand differs"
        assert cnt[:nb].tolist() == [2 * use] * nb and cnt[nb:].tolist() == [use] * nb


def test_gather_jobs_ride_on_bf16_gemm_and_stand_alone():
    cu = _cu()
    src = torch.randint(0, 255, (3 * 1024 * 1024 + 4096,), dtype=torch.uint8, device=DEV)
    dst = torch.zeros_like(src)
    cnt = torch.zeros(4, dtype=torch.int32, device=DEV)
    rows = _jobs(src, dst, cnt, 0, 3, 1024 * 1024, 16) + _jobs(src[3 * 1024 * 1024 :], dst[3 * 1024 * 1024 :], None, 0, 1, 4096, 1)
    table = torch.tensor(rows, dtype=torch.int64, device=DEV)
    a = torch.randn(1024, 512, device=DEV).bfloat16()
    b = torch.randn(256, 512, device=DEV).bfloat16()
    want = cu.gemm_bf16(a, b)
    cu.K.attach_gather_jobs(table)
    got = cu.gemm_bf16(a, b)
    torch.cuda.synchronize()
    _status_clean(a)
    assert torch.equal(got, want) and torch.equal(dst, src)
    assert cnt.tolist() == [16, 16, 16, 0]
    dst.zero_()
    cu.K.gather_jobs(table)
    torch.cuda.synchronize()
    assert torch.equal(dst, src) and cnt.tolist() == [32, 32, 32, 0]


def test_wgrad_into_virtual_gradient_sink():
    """A weight-gradient GEMM whose fp32 destination is addressed as (sink, flat offset) instead of a tensor: the
    form used when gradients are sharded over the ranks and no rank holds a full-size buffer."""
    cu = _cu()
    per = 4 * 256 * 128
    shard = torch.zeros(per, device=DEV)
    # a world of one whose shard starts at flat offset 0: the biased table is the plain address
    table = torch.tensor([shard.data_ptr()], dtype=torch.int64, device=DEV)
    cu.K.clear_grad_sinks()
    try:
        sink = int(cu.K.register_virtual_grad_sink(table, per, per))
        M, N, Kd = 512, 256, 256
        dy, x = torch.randn(M, N, device=DEV).bfloat16(), torch.randn(M, Kd, device=DEV).bfloat16()
        ref_ = cu.GradRef(sink, 256 * 128, N, Kd)
        cu.gemm_bf16(dy, x[:, :128], a_mn=True, b_mn=True, out=ref_.col_range(0, 128), accumulate=True)
        cu.gemm_bf16(dy, x[:, 128:], a_mn=True, b_mn=True, out=ref_.col_range(128, 128), accumulate=True)
        cu.accumulate_main_grad(cu.GradRef(sink, 0, 8, 128), torch.ones(8, 128, device=DEV))
        torch.cuda.synchronize()
        _status_clean(dy)
        want = dy.float().t() @ x.float()
        got = shard[256 * 128 : 256 * 128 + N * Kd].view(N, Kd)
        _close(got, want, 2e-2 * float(want.abs().max()) * 1e-1, 1e-2, "wgrad through a virtual sink")
        assert float(shard[: 8 * 128].min()) == 1.0 and float(shard[8 * 128 : 256 * 128].abs().max()) == 0.0
    finally:
        cu.K.clear_grad_sinks()
