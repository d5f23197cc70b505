"""CPU checks of the plain-PyTorch op statements against independent formulations."""

import math

import pytest
import torch
import torch.nn.functional as F

from gdnet_b200.ops import reference as ref


@pytest.mark.parametrize("B,T,d,k", [(2, 16, 8, 4), (1, 5, 3, 7), (3, 33, 16, 1)])
def test_causal_dwconv_matches_conv1d(B, T, d, k):
    x = torch.randn(B, T, d)
    w = torch.randn(d, k)
    want = F.conv1d(F.pad(x.transpose(1, 2), (k - 1, 0)), w.unsqueeze(1), groups=d).transpose(1, 2)
    assert torch.allclose(ref.causal_dwconv(x, w), want, atol=1e-5)


def test_causal_dwconv_halo_equals_longer_sequence():
    B, T, d, k = 2, 12, 8, 4
    x = torch.randn(B, 2 * T, d)
    w = torch.randn(d, k)
    full = ref.causal_dwconv(x, w)
    right = ref.causal_dwconv(x[:, T:], w, halo=ref.conv_tail(x[:, :T], k))
    assert torch.allclose(full[:, T:], right, atol=1e-6)


def test_stream_update_conserves_mass():
    c, s = torch.randn(7, 16), torch.randn(7, 16)
    f, so, g = ref.gate_stream_update(torch.randn(7, 16), c, s, torch.rand(7, 16))
    assert torch.allclose(f + so, c + s, atol=1e-5)
    assert g.min() > 0 and g.max() < 1


def test_rmsnorm_matches_torch():
    x, w = torch.randn(5, 32), torch.randn(32)
    want = torch.nn.functional.rms_norm(x, (32,), w, 1e-6)
    assert torch.allclose(ref.rmsnorm(x, w, 1e-6), want, atol=1e-5)


def test_fused_mem_read_einsum():
    B, S, ds, dc = 3, 5, 8, 4
    q, gam, e = torch.randn(B, ds), torch.rand(B, ds), torch.randn(S, ds)
    tags, vals, alpha = torch.randn(B, S, ds), torch.randn(B, S, dc), torch.tensor([0.7])
    out, w = ref.fused_mem_read(q, gam, e, tags, vals, alpha)
    sim = (tags * q[:, None]).sum(-1) + 0.7 * (gam @ e.t())
    assert torch.allclose(w, sim.softmax(-1), atol=1e-6)
    assert torch.allclose(out, (sim.softmax(-1)[..., None] * vals).sum(1), atol=1e-6)
    assert torch.allclose(w.sum(-1), torch.ones(B), atol=1e-6)


def test_block_quant_roundtrip_and_scales():
    x = torch.randn(64, 256) * 3
    q, s = ref.quantize_1x128(x)
    assert q.dtype == ref.FP8_DTYPE and s.shape == (64, 2)
    assert torch.allclose(s, x.view(64, 2, 128).abs().amax(-1) / 448)
    assert (ref.dequantize_1x128(q, s) - x).abs().max() <= x.abs().max() * 0.07
    w = torch.randn(256, 384)
    qw, sw = ref.quantize_128x128(w)
    assert sw.shape == (2, 3)
    assert (ref.dequantize_128x128(qw, sw) - w).abs().max() <= w.abs().max() * 0.07
    # odd sizes pad internally
    q2, s2 = ref.quantize_1x128(torch.randn(3, 130))
    assert q2.shape == (3, 130) and s2.shape == (3, 2)
    z, sz = ref.quantize_1x128(torch.zeros(2, 128))
    assert torch.all(sz == 1) and torch.all(z.float() == 0)


def test_fp8_gemm_blockscaled_equals_dequantised_matmul():
    a, b = torch.randn(48, 256), torch.randn(128, 256)
    a8, sa = ref.quantize_1x128(a)
    b8, sb = ref.quantize_128x128(b)
    got = ref.fp8_gemm_blockscaled(a8, sa, b8, sb, out_dtype=torch.float32)
    want = ref.dequantize_1x128(a8, sa) @ ref.dequantize_128x128(b8, sb).t()
    assert torch.allclose(got, want, atol=1e-3, rtol=1e-4)
    assert (got - a @ b.t()).abs().max() < 0.08 * (a @ b.t()).abs().max()


def test_fp8_linear_blockscaled_grads_close_to_exact():
    x = torch.randn(128, 128, requires_grad=True)
    w = torch.randn(256, 128, requires_grad=True) * 0.1
    w.retain_grad()
    b = torch.randn(256, requires_grad=True)
    y = ref.fp8_linear_blockscaled(x, w, b)
    gy = torch.randn_like(y)
    y.backward(gy)
    x2, w2, b2 = x.detach().requires_grad_(), w.detach().requires_grad_(), b.detach().requires_grad_()
    F.linear(x2, w2, b2).backward(gy)
    for got, want in ((x.grad, x2.grad), (w.grad, w2.grad), (b.grad, b2.grad)):
        assert (got - want).abs().max() < 0.1 * want.abs().max() + 1e-3


def test_projected_adamw_matches_torch_adamw():
    torch.manual_seed(1)
    p = torch.randn(100)
    ref_p = p.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    m, v = torch.zeros(100), torch.zeros(100)
    for step in range(1, 4):
        gt, gi = torch.randn(100), torch.randn(100)
        coef = float((gi * gt).sum() / (gt * gt).sum())
        ref_p.grad = gt + 0.1 * (gi - coef * gt)
        opt.step()
        ref.projected_adamw_(p, gt, gi, m, v, coef=coef, beta_proj=0.1, grad_scale=1.0, lr=1e-2,
                             beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        assert torch.allclose(p, ref_p.detach(), atol=1e-6)


def test_power_iteration_converges():
    W = torch.randn(20, 30)
    u, v = F.normalize(torch.randn(20), dim=0), F.normalize(torch.randn(30), dim=0)
    u, v, sigma = ref.power_iteration(W, u, v, n_iter=200)
    assert math.isclose(float(sigma), float(torch.linalg.matrix_norm(W, 2)), rel_tol=1e-3)
