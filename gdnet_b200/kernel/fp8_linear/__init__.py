"""FP8 linear building blocks (reference: gdnet/kernel/fp8_linear/__init__.py).

``quantize_fp8`` is the reference's per-tensor quantiser (row-major and transposed e4m3 copies plus
amax); ``fp8_gemm`` multiplies e4m3 operands with per-tensor scales on the sm_100a block-scaled
tensor-core kernel (the reference's SM90 wgmma kernel cannot be built for this GPU);
``FP8Linear`` is the module."""

from __future__ import annotations

import torch

from ...ops import reference as ref
from ...ops.fp8_linear import FP8Linear

FP8_MAX = ref.FP8_MAX


def quantize_fp8(x, scale, need_col: bool = True, out_row=None, out_col=None, amax_buf=None):
    if x.is_cuda:
        from ...ops import cuda as cu

        return cu.quantize_fp8_tensor(x, scale, need_col, out_row, out_col, amax_buf)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    q, amax = ref.quantize_per_tensor(x2, scale)
    if out_row is not None:
        out_row.copy_(q)
        q = out_row
    qc = q.t().contiguous() if need_col else q
    if need_col and out_col is not None:
        out_col.copy_(qc)
        qc = out_col
    if amax_buf is not None:
        amax_buf.copy_(torch.maximum(amax_buf, amax.reshape(1)))
        amax = amax_buf.squeeze()
    return q.reshape(shape), qc, amax


def _as_scale(v, device):
    if torch.is_tensor(v):
        return v.reshape(-1)[:1].to(device=device, dtype=torch.float32)
    return torch.full((1,), float(v), dtype=torch.float32, device=device)


_unit_scales: dict = {}


def _unit_packed(rows: int, cols: int, device):
    """Packed UE8M0 chunks that all say 2^0, cached per shape: per-tensor scaling applies the two dequantisation
    factors as one per-row epilogue scale instead."""
    key = (rows, cols, str(device))
    t = _unit_scales.get(key)
    if t is None:
        t = torch.full((rows // 128, cols // 128, 512), 127, dtype=torch.uint8, device=device)
        _unit_scales[key] = t
    return t


def fp8_gemm(a, b, scale_a=1.0, scale_b=1.0, out_dtype=torch.bfloat16):
    """``D = (a * scale_a) (b * scale_b)^T`` for e4m3 ``a (M,K)``, ``b (N,K)``; scales are the
    dequantisation factors (reference: gdnet/kernel/fp8_linear/gemm.py:697-777). On CUDA with all three sizes
    multiples of 128 this is the hardware-scaled tcgen05 kernel with unit block scales and the product of the two
    factors applied in the epilogue; the factors stay on the device (no host synchronisation)."""
    M, Kd = a.shape
    N = b.shape[0]
    if a.is_cuda and Kd % 128 == 0 and N % 128 == 0 and M % 128 == 0:
        from ...ops import cuda as cu

        both = (_as_scale(scale_a, a.device) * _as_scale(scale_b, a.device)).expand(M).contiguous()
        return cu.gemm_fp8_mx(a.contiguous(), _unit_packed(M, Kd, a.device), b.contiguous(), _unit_packed(N, Kd, a.device),
                              out_dtype=out_dtype, row_scale=both)
    sa_v = float(scale_a) if not torch.is_tensor(scale_a) else float(scale_a.reshape(-1)[0])
    sb_v = float(scale_b) if not torch.is_tensor(scale_b) else float(scale_b.reshape(-1)[0])
    if a.is_cuda and Kd % 128 == 0 and N % 128 == 0:
        from ...ops import cuda as cu

        sa = torch.full(((Kd + 127) // 128, M), sa_v, dtype=torch.float32, device=a.device)
        sb = torch.full(((N + 127) // 128, (Kd + 127) // 128), sb_v, dtype=torch.float32, device=a.device)
        return cu.gemm_fp8(a, sa, b, sb, out_dtype=out_dtype)
    return ((a.float() @ b.float().t()) * (sa_v * sb_v)).to(out_dtype)


__all__ = ["quantize_fp8", "fp8_gemm", "FP8Linear", "FP8_MAX"]
