"""FP8 (e4m3) linear layer with bf16 master weights.

Two recipes:

``block`` (default)
    Current scaling in blocks: 1x128 along the reduction for activations and
    gradients, 128x128 for weights; fp32 scales; fp32 accumulation with the partial
    product of each 128-deep block scaled before it is added. This is the recipe of the
    sm_100a tensor-core GEMM (``csrc/gemm_sm100.cu``).

``tensor``
    The reference's recipe (gdnet/kernel/fp8_linear/linear.py:9-73): one delayed
    scale per tensor for ``x`` and ``w`` (``scale = 448/amax`` refreshed by
    ``update_fp8_scales`` from a running amax window) and a current scale for the
    incoming gradient.

The module keeps the reference's buffers (``scale_x, scale_w, inv_scale_x,
inv_scale_w, _w_fp8_row, _w_fp8_col, _amax_w, _amax_x``) under the same names so FP8
checkpoints load in both directions; the block recipe does not read the scale buffers.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import reference as ref

RECIPES = ("block", "tensor")


class _TensorScaledLinearFn(torch.autograd.Function):
    """Per-tensor delayed-scaling FP8 linear, plain-PyTorch arithmetic."""

    @staticmethod
    def forward(ctx, x, w, scale_x, scale_w, amax_x, amax_w):
        xq, ax = ref.quantize_per_tensor(x, scale_x)
        wq, aw = ref.quantize_per_tensor(w, scale_w)
        amax_x.copy_(torch.maximum(amax_x, ax.reshape(1)))
        amax_w.copy_(torch.maximum(amax_w, aw.reshape(1)))
        ctx.save_for_backward(xq, wq, scale_x, scale_w)
        y = (xq.float() @ wq.float().t()) / (scale_x.float() * scale_w.float())
        return y.to(torch.bfloat16)

    @staticmethod
    def backward(ctx, gy):
        xq, wq, scale_x, scale_w = ctx.saved_tensors
        gyf = gy.float()
        scale_g = ref.FP8_MAX / gyf.abs().amax().clamp(min=1e-12)
        gq, _ = ref.quantize_per_tensor(gyf, scale_g)
        dx = (gq.float() @ wq.float()) / (scale_g * scale_w.float())
        dw = (gq.float().t() @ xq.float()) / (scale_g * scale_x.float())
        return dx.to(torch.bfloat16), dw.to(torch.bfloat16), None, None, None, None


class FP8Linear(nn.Module):
    """Drop-in replacement for ``nn.Linear`` built from an existing linear."""

    def __init__(self, linear: nn.Linear, recipe: str = "block"):
        super().__init__()
        if recipe not in RECIPES:
            raise ValueError(f"unknown FP8 recipe {recipe!r}; expected one of {RECIPES}")
        self.recipe = recipe
        out_f, in_f = linear.weight.shape
        self.in_features, self.out_features = in_f, out_f
        self.weight = nn.Parameter(linear.weight.data.to(torch.bfloat16))
        self.bias = nn.Parameter(linear.bias.data.to(torch.bfloat16)) if linear.bias is not None else None
        dev = linear.weight.device
        for name in ("scale_x", "scale_w", "inv_scale_x", "inv_scale_w"):
            self.register_buffer(name, torch.ones(1, device=dev))
        self.register_buffer("_w_fp8_row", torch.zeros(out_f, in_f, dtype=ref.FP8_DTYPE, device=dev))
        self.register_buffer("_w_fp8_col", torch.zeros(in_f, out_f, dtype=ref.FP8_DTYPE, device=dev))
        self.register_buffer("_amax_w", torch.zeros(1, dtype=torch.float32, device=dev))
        self.register_buffer("_amax_x", torch.zeros(1, dtype=torch.float32, device=dev))

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, recipe={self.recipe}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]).to(torch.bfloat16)
        if x2.is_cuda:
            from . import cuda as cuda_ops

            y = cuda_ops.fp8_linear(x2, self)
        elif self.recipe == "block":
            y = ref.fp8_linear_blockscaled(x2, self.weight, self.bias)
        else:
            y = _TensorScaledLinearFn.apply(
                x2, self.weight, self.scale_x, self.scale_w, self._amax_x, self._amax_w
            )
            if self.bias is not None:
                y = y + self.bias
        return y.reshape(*shape[:-1], self.out_features)
