"""Plain-PyTorch statement of every GDNet op.

This module is three things at once:

* the CPU execution path (the tiny copy-task configuration trains entirely here),
* the numerical oracle every sm_100a kernel is tested against (fp32 math, same
  rounding points as the kernels), and
* the timed CPU baseline.

Everything here is ordinary differentiable torch code, so autograd supplies the
backward that the hand-written backward kernels are checked against.

Parity notes (paths are inside the reference project):

* causal depthwise conv ............ gdnet/kernel/gated_causal_depthwise_conv/conv.py:10-69
* RMSNorm / gate stream update ..... gdnet/kernel/gated_causal_depthwise_conv/gate_norm.py:8-57
* gated output (gate MLP) .......... gdnet/kernel/gated_causal_depthwise_conv/function.py:35-40
* recovery gate .................... gdnet/layer.py:86-92
* fused memory read ................ gdnet/kernel/fused_mem_read/kernel.py:13-80
* per-tensor FP8 quantise .......... gdnet/kernel/fp8_linear/quantize.py:10-56
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

FP8_MAX = 448.0
FP8_DTYPE = torch.float8_e4m3fn
QBLOCK = 128  # edge of a quantisation block (1x128 activations, 128x128 weights)

GATE_EPS = 1e-6  # eps of the RMSNorm inside the gate MLP (function.py:99)


# --------------------------------------------------------------------------------------
# causal depthwise convolution
# --------------------------------------------------------------------------------------

def causal_dwconv(x: torch.Tensor, w: torch.Tensor, halo: torch.Tensor | None = None) -> torch.Tensor:
    """``out[b,t,c] = sum_i w[c,i] * x[b, t-(k-1)+i, c]`` with fp32 accumulation.

    Positions before the start of the shard read ``halo`` (``(B, k-1, d)``: the last
    ``k-1`` inputs of the previous sequence shard) or zeros when ``halo`` is None.
    The result is stored in ``x.dtype``.
    """
    B, T, d = x.shape
    k = w.shape[1]
    xf = x.float()
    if k > 1:
        left = halo.float() if halo is not None else xf.new_zeros(B, k - 1, d)
        xf = torch.cat([left, xf], dim=1)
    wf = w.float()
    acc = xf[:, 0:T] * wf[:, 0]
    for i in range(1, k):
        acc = acc + xf[:, i : i + T] * wf[:, i]
    return acc.to(x.dtype)


def conv_tail(x: torch.Tensor, k: int) -> torch.Tensor:
    """The ``k-1`` trailing inputs a shard hands to the next shard as its left halo."""
    return x[:, x.shape[1] - (k - 1) :, :]


# --------------------------------------------------------------------------------------
# normalisation and gates
# --------------------------------------------------------------------------------------

def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype)


RMS_EPS_DEFAULT = float(torch.finfo(torch.float32).eps)


def default_rms_eps(dtype: torch.dtype | None = None) -> float:
    """The epsilon of an ``nn.RMSNorm(eps=None)`` as the reference runs it, i.e. on a CUDA tensor: torch's fused
    CUDA kernel does not take the machine epsilon of the *input* dtype (7.8e-3 for bfloat16, which is what the
    CPU composite uses) but a float32-sized one, whatever the input dtype. The difference is not cosmetic: the
    streams of a freshly initialised model have an RMS of a few hundredths, so 7.8e-3 under the square root would
    scale every normalised activation down several times. The same value is used on every device and dtype here, so
    the CPU statement of an op and its CUDA kernel agree."""
    return RMS_EPS_DEFAULT


def gate_stream_update(g_pre, c, s, R):
    """``g = sigmoid(g_pre)``; route ``c`` and ``s`` between the two streams.

    ``fwd' + side' == c + s`` exactly in real arithmetic: nothing is discarded.
    """
    g = torch.sigmoid(g_pre.float())
    cf, sf, Rf = c.float(), s.float(), R.float()
    fwd_out = cf * g + sf * Rf
    side_out = cf * (1.0 - g) + sf * (1.0 - Rf)
    return fwd_out.to(c.dtype), side_out.to(c.dtype), g


def linear(x, w, b=None):
    """y = x w^T + b computed in the dtype of ``x`` (weights are cast to it)."""
    return F.linear(x, w.to(x.dtype), None if b is None else b.to(x.dtype))


def gate_pre(c, W1, b1, w_norm, W2, b2, eps: float = GATE_EPS):
    """Pre-activation of the forward gate: ``W2 . RMSNorm(silu(W1 c + b1)) + b2``."""
    h = F.silu(linear(c, W1, b1))
    return linear(rmsnorm(h, w_norm, eps), W2, b2)


def recovery_gate(s, c, W1, b1, W2, b2, w_norm, eps: float | None = None):
    """``R = sigmoid(RMSNorm(W2 silu(W1 [s ; c] + b1) + b2))`` (norm after W2)."""
    u = torch.cat([s, c], dim=-1)
    z = linear(F.silu(linear(u, W1, b1)), W2, b2)
    eps = default_rms_eps(z.dtype) if eps is None else eps
    return torch.sigmoid(rmsnorm(z, w_norm, eps).float()).to(z.dtype)


def layer_step(x, s, conv_w, rW1, rb1, rW2, rb2, rnorm_w, gW1, gb1, gnorm_w, gW2, gb2,
               halo=None, r_eps: float | None = None, g_eps: float = GATE_EPS,
               linear_fn=None):
    """One GDLayer step. Returns ``(fwd', side', g, c)``.

    ``linear_fn(x, w, b)`` replaces the recovery-path linears (the ones that are FP8
    in FP8 mode); the gate MLP always runs in the activation dtype, as in the
    reference (gdnet/layer.py:130-139).
    """
    lin = linear if linear_fn is None else linear_fn
    c = causal_dwconv(x, conv_w, halo)
    u = torch.cat([s.to(c.dtype), c], dim=-1)
    z = lin(F.silu(lin(u, rW1, rb1)), rW2, rb2)
    eps_r = default_rms_eps(z.dtype) if r_eps is None else r_eps
    R = torch.sigmoid(rmsnorm(z, rnorm_w, eps_r).float())
    g_pre = gate_pre(c, gW1, gb1, gnorm_w, gW2, gb2, g_eps)
    fwd_out, side_out, g = gate_stream_update(g_pre, c, s.to(c.dtype), R)
    return fwd_out, side_out, g, c


# --------------------------------------------------------------------------------------
# content-addressed memory read
# --------------------------------------------------------------------------------------

def fused_mem_read(q, gamma, e, tags, vals, alpha):
    """``w = softmax_s(<tags_s, q> + alpha <e_s, gamma>)``, ``out = sum_s w_s vals_s``.

    Computed in fp32; ``out`` is returned in ``q.dtype`` and ``w`` in fp32.
    """
    qf, gf, ef = q.float(), gamma.float(), e.float()
    sim = torch.einsum("bsd,bd->bs", tags.float(), qf)
    sim = sim + alpha.float().reshape(()) * torch.einsum("sd,bd->bs", ef, gf)
    w = torch.softmax(sim, dim=-1)
    out = torch.einsum("bs,bsd->bd", w, vals.float())
    return out.to(q.dtype), w


def retrieval_entropy(w: torch.Tensor, n_slots: int) -> torch.Tensor:
    return -(w * (w + 1e-8).log()).sum(-1) / math.log(n_slots)


# --------------------------------------------------------------------------------------
# FP8 (e4m3) quantisation: per-tensor and block-scaled
# --------------------------------------------------------------------------------------

def quantize_per_tensor(x: torch.Tensor, scale: torch.Tensor):
    """``clamp(x*scale, +-448) -> e4m3`` plus the observed amax (delayed scaling)."""
    xf = x.float()
    amax = xf.abs().amax()
    q = (xf * scale.float()).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q, amax


def _pad_to(x: torch.Tensor, dim: int, mult: int) -> torch.Tensor:
    pad = (-x.shape[dim]) % mult
    if pad == 0:
        return x
    shape = list(x.shape)
    shape[dim] = pad
    return torch.cat([x, x.new_zeros(shape)], dim=dim)


def _block_scale(amax: torch.Tensor, pow2: bool) -> torch.Tensor:
    """``amax/448`` per block (1 for an all-zero block); with ``pow2`` rounded up to a power of two,
    the form the tensor core's UE8M0 block scaling needs."""
    s = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    if pow2:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    return s


def quantize_1x128(x: torch.Tensor, pow2: bool = False):
    """Row-wise blocks of 128 along the last dim.

    Returns ``(q (M,K) e4m3, s (M, ceil(K/128)) fp32)`` with ``x ~= q * s`` and
    ``s = amax/448`` (1.0 for an all-zero block).
    """
    M, K = x.shape
    xp = _pad_to(x.float(), 1, QBLOCK).view(M, -1, QBLOCK)
    amax = xp.abs().amax(dim=-1)
    s = _block_scale(amax, pow2)
    q = (xp / s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q.view(M, -1)[:, :K].contiguous(), s


def quantize_128x128(w: torch.Tensor, pow2: bool = False):
    """Square 128x128 blocks. Returns ``(q (N,K) e4m3, s (ceil(N/128), ceil(K/128)))``."""
    N, K = w.shape
    wp = _pad_to(_pad_to(w.float(), 0, QBLOCK), 1, QBLOCK)
    nb, kb = wp.shape[0] // QBLOCK, wp.shape[1] // QBLOCK
    blocks = wp.view(nb, QBLOCK, kb, QBLOCK)
    amax = blocks.abs().amax(dim=(1, 3))
    s = _block_scale(amax, pow2)
    q = (blocks / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q.view(wp.shape)[:N, :K].contiguous(), s


def pack_ue8m0_rows(s: torch.Tensor) -> torch.Tensor:
    """Pack power-of-two row scales ``s (M, KB)`` (M a multiple of 128) into the 512-byte chunks the
    block-scaled tensor-core MMA reads: chunk ``(m // 128, kb)``, the four bytes of row ``r = m % 128``
    at ``(r % 32) * 16 + (r // 32) * 4``."""
    M, KB = s.shape
    e = (torch.log2(s.float()).round() + 127).clamp(0, 254).to(torch.uint8)          # (M, KB)
    out = torch.zeros(M // 128, KB, 512, dtype=torch.uint8, device=s.device)
    r = torch.arange(128, device=s.device)
    pos = (r % 32) * 16 + (r // 32) * 4
    blocks = e.view(M // 128, 128, KB).permute(0, 2, 1)                                # (MB, KB, 128)
    for j in range(4):
        out[:, :, pos + j] = blocks
    return out


def pack_ue8m0_blocks(s: torch.Tensor) -> torch.Tensor:
    """Pack 128x128 block scales ``s (NB, KB)`` into constant-filled 512-byte chunks."""
    e = (torch.log2(s.float()).round() + 127).clamp(0, 254).to(torch.uint8)
    return e.unsqueeze(-1).expand(*s.shape, 512).contiguous()


def dequantize_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return q.float() * s.repeat_interleave(QBLOCK, dim=1)[:, :K]


def dequantize_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    full = s.repeat_interleave(QBLOCK, dim=0).repeat_interleave(QBLOCK, dim=1)
    return q.float() * full[:N, :K]


def fp8_gemm_blockscaled(a8, sa, b8, sb, out_dtype=torch.bfloat16, bias=None):
    """``D = (a8*sa) (b8*sb)^T`` accumulated block by block in fp32.

    ``a8 (M,K)`` with 1x128 scales ``sa (M,K/128)``; ``b8 (N,K)`` with 128x128 scales
    ``sb (N/128,K/128)``. The sum over K runs in blocks of 128, each partial product
    scaled before it is added, which is the order the tensor-core kernel uses.
    """
    M, K = a8.shape
    N = b8.shape[0]
    acc = torch.zeros(M, N, dtype=torch.float32, device=a8.device)
    sb_rows = sb.repeat_interleave(QBLOCK, dim=0)[:N]
    for kb in range(0, K, QBLOCK):
        j = kb // QBLOCK
        part = a8[:, kb : kb + QBLOCK].float() @ b8[:, kb : kb + QBLOCK].float().t()
        acc += part * sa[:, j : j + 1] * sb_rows[:, j].unsqueeze(0)
    if bias is not None:
        acc += bias.float()
    return acc.to(out_dtype)


def fp8_linear_blockscaled(x, w, b=None):
    """Emulated block-scaled FP8 linear with a straight-through backward.

    Forward: quantise ``x`` 1x128 and ``w`` 128x128, multiply the dequantised
    operands. Backward: gradients of the equivalent full-precision linear with the
    incoming gradient and the saved operands passed through the same quantisers
    (dgrad: 1x128 grad x 128x128 weight; wgrad: 1x128 grad^T x 128x128 x^T).
    """
    return _BlockFp8LinearFn.apply(x, w, b)


class _BlockFp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        xq, xs = quantize_1x128(x2)
        wq, ws = quantize_128x128(w)
        y = fp8_gemm_blockscaled(xq, xs, wq, ws, out_dtype=x.dtype, bias=b)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = b is not None
        ctx.in_shape = shape
        return y.reshape(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        gq, gs = quantize_1x128(g2)
        wtq, wts = quantize_128x128(w.t().contiguous())
        dx = fp8_gemm_blockscaled(gq, gs, wtq, wts, out_dtype=x2.dtype)
        gtq, gts = quantize_1x128(g2.t().contiguous())
        xtq, xts = quantize_128x128(x2.t().contiguous())
        dw = fp8_gemm_blockscaled(gtq, gts, xtq, xts, out_dtype=torch.float32)
        db = g2.float().sum(0).to(gy.dtype) if ctx.has_bias else None
        return dx.reshape(ctx.in_shape), dw.to(w.dtype), db


# --------------------------------------------------------------------------------------
# loss, spectral norm, optimiser
# --------------------------------------------------------------------------------------

def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100):
    """Mean token cross-entropy in fp32 over ``logits (n, V)``."""
    return F.cross_entropy(logits.float(), targets, ignore_index=ignore_index)


def sn_sigma(W: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """One-matvec estimate of the top singular value: ``||W v||`` for unit ``v``."""
    return (W.float() @ v.float()).norm()


def power_iteration(W: torch.Tensor, u: torch.Tensor, v: torch.Tensor, n_iter: int = 1, eps: float = 1e-12):
    """``v <- W^T u / ||.||``, ``u <- W v / ||.||``; returns ``(u, v, sigma = u^T W v)``."""
    Wf = W.float()
    u, v = u.float(), v.float()
    for _ in range(n_iter):
        v = F.normalize(Wf.t() @ u, dim=0, eps=eps)
        u = F.normalize(Wf @ v, dim=0, eps=eps)
    return u, v, torch.dot(u, Wf @ v)


def projected_adamw_(p, gt, gi, m, v, *, coef, beta_proj, grad_scale, lr, beta1, beta2, eps,
                     weight_decay, step):
    """In-place AdamW on ``g = grad_scale * (gt + beta_proj * (gi - coef * gt))``.

    ``m``/``v`` are fp32 moments; ``p`` is updated in its own dtype from an fp32
    computation. Decoupled weight decay, bias-corrected (matches torch.optim.AdamW).
    """
    g = (gt.float() + beta_proj * (gi.float() - coef * gt.float())) * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    pf = p.float() * (1 - lr * weight_decay)
    pf = pf - (lr / bc1) * m / ((v / bc2).sqrt() + eps)
    p.copy_(pf.to(p.dtype))
    return p
