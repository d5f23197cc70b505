"""Gated causal depthwise conv: names kept from the reference package
(gdnet/kernel/gated_causal_depthwise_conv/__init__.py). CUDA tensors run the sm_100a kernels,
CPU tensors the plain-PyTorch statement."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ...ops import functional as ops
from ...ops import reference as ref

MAX_K = 16


def causal_dwconv_fwd(x, W_conv, T=None, k=None, BLOCK_T=None):
    """``x (B,T,d)``, ``W_conv (d,k)`` -> ``(B,T,d)``. ``T``, ``k`` and ``BLOCK_T`` are accepted for call
    compatibility with the reference launchers and ignored (shapes are read from the tensors)."""
    return ops.causal_dwconv(x, W_conv)


def causal_dwconv_fwd_sp(x, halo, W_conv, T=None, k=None, BLOCK_T=None):
    return ops.causal_dwconv(x, W_conv, halo)


class CausalDWConvFunction:
    """``CausalDWConvFunction.apply(x, W_conv, T, k, BLOCK_T)`` as in the reference."""

    @staticmethod
    def apply(x, W_conv, T=None, k=None, BLOCK_T=None):
        return ops.causal_dwconv(x, W_conv)


class CausalDWConvFunctionSP:
    """Sequence-parallel variant taking the left halo explicitly; the halo receives a gradient."""

    @staticmethod
    def apply(x, halo, W_conv, T=None, k=None, BLOCK_T=None):
        return ops.causal_dwconv(x, W_conv, halo)


def _cuda_rows(*ts) -> bool:
    return all(t.is_cuda for t in ts) and ts[0].dim() == 2 and ts[0].shape[1] % 8 == 0


def rmsnorm_fwd(H, W_norm, eps, BLOCK_D=None):
    """Returns ``(H_norm, rstd)`` like the reference's launcher (gate_norm.py:133-152); bf16 CUDA rows run the
    sm_100a kernel."""
    if H.is_cuda and H.dtype == torch.bfloat16 and H.dim() == 2 and H.shape[1] % 8 == 0 and H.is_contiguous():
        from ...ops import cuda as cu

        return cu.rmsnorm_fwd(H, W_norm, eps)
    rstd = torch.rsqrt(H.float().pow(2).mean(-1) + eps)
    return ops.rmsnorm(H, W_norm, eps), rstd


def gate_stream_update_fwd(g_pre, conv_flat, side_flat, R_flat, BLOCK_D=None):
    """``(fwd', side')`` from the gate pre-activation and both streams (gate_norm.py:155-190); differentiable in all
    four inputs. CUDA tensors run the sm_100a kernel (bf16), CPU tensors the plain-PyTorch statement."""
    if _cuda_rows(g_pre, conv_flat, side_flat, R_flat):
        from ...ops import cuda as cu

        return cu.gate_stream_update(g_pre, conv_flat, side_flat, R_flat)
    fo, so, _ = ref.gate_stream_update(g_pre, conv_flat, side_flat, R_flat)
    return fo, so


def gated_output(conv_flat, side, R, W1, b1, W_norm, W2, b2, eps: float = 1e-6):
    """Gate MLP + stream update over a pre-computed conv output ``(n_rows, d)``
    (reference: gdnet/kernel/gated_causal_depthwise_conv/function.py:90-131). On CUDA with ``d`` and the row count
    multiples of 128 this is one autograd node on the tensor-core GEMMs and the update kernels; other shapes and
    CPU tensors take the plain-PyTorch statement."""
    n, d = conv_flat.shape
    dt = conv_flat.dtype
    if conv_flat.is_cuda:
        from ...ops import cuda as cu

        if cu.gated_output_ok(conv_flat, W1, W2):
            fo, so = cu.gated_output(conv_flat, side.reshape(n, d), R.reshape(n, d), W1, b1, W_norm, W2, b2, eps)
            return fo.to(dt), so.to(dt)
    g_pre = ref.gate_pre(conv_flat, W1, b1, W_norm, W2, b2, eps)
    fo, so, _ = ref.gate_stream_update(g_pre, conv_flat, side.to(dt).reshape(n, d), R.to(dt).reshape(n, d))
    return fo, so


class GatedCausalDepthwiseConvFunction:
    @staticmethod
    def apply(conv_flat, side_flat, R_flat, W1, b1, W_norm, W2, b2, eps):
        return gated_output(conv_flat, side_flat, R_flat, W1, b1, W_norm, W2, b2, eps)


def gated_causal_depthwise_conv(x, side, R, W_conv, W1, b1, W_norm, W2, b2, eps: float = 1e-6):
    """Causal depthwise conv followed by the gated stream update; ``(fwd', side')`` in ``x.dtype``."""
    B, T, d = x.shape
    if W_conv.shape[1] > MAX_K:
        raise ValueError(f"kernel size {W_conv.shape[1]} exceeds MAX_K={MAX_K}")
    c = ops.causal_dwconv(x, W_conv).reshape(B * T, d)
    fo, so = gated_output(c, side, R, W1, b1, W_norm, W2, b2, eps)
    return fo.view(B, T, d).to(x.dtype), so.view(B, T, d).to(x.dtype)


__all__ = [
    "gated_causal_depthwise_conv", "gated_output", "GatedCausalDepthwiseConvFunction",
    "CausalDWConvFunction", "CausalDWConvFunctionSP", "causal_dwconv_fwd", "causal_dwconv_fwd_sp",
    "rmsnorm_fwd", "gate_stream_update_fwd",
]
