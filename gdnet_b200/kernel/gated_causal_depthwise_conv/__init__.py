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


def rmsnorm_fwd(H, W_norm, eps, BLOCK_D=None):
    """Returns ``(H_norm, rstd)`` like the reference's launcher (gate_norm.py:133-152)."""
    rstd = torch.rsqrt(H.float().pow(2).mean(-1) + eps)
    return ops.rmsnorm(H, W_norm, eps), rstd


def gate_stream_update_fwd(g_pre, conv_flat, side_flat, R_flat, BLOCK_D=None):
    fo, so, _ = ref.gate_stream_update(g_pre, conv_flat, side_flat, R_flat)
    return fo, so


def gated_output(conv_flat, side, R, W1, b1, W_norm, W2, b2, eps: float = 1e-6):
    """Gate MLP + stream update over a pre-computed conv output ``(n_rows, d)``
    (reference: gdnet/kernel/gated_causal_depthwise_conv/function.py:90-131)."""
    n, d = conv_flat.shape
    dt = conv_flat.dtype
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
