"""Precision policy and FP8 module conversion.

Parity with the reference's ``gdnet/utils/fp8.py``: ``Precision`` literal, ``autocast``
(bf16 autocast for both the bf16 and the fp8 mode), ``convert_to_fp8`` (same
eligibility rule: plain ``nn.Linear``, not spectral-normalised, both dims multiples of
16, not under ``cam.``; spectral-normalised modules, non-CAM RMSNorm weights and the
whole CAM are cast to bf16) and ``update_fp8_scales`` (one MAX all-reduce over all amax
buffers, ``scale = 448/amax``, reset).

Differences: ``convert_to_fp8`` takes a ``recipe`` (``block`` = 1x128/128x128 current
scaling, the default; ``tensor`` = the reference's per-tensor delayed scaling), works on
CPU too (emulated arithmetic), and keeps ``head.weight`` tied to ``embed.weight``
unless ``untie_head=True`` (the reference's conversion silently unties them,
gdnet/kernel/fp8_linear/linear.py:80).
"""

from __future__ import annotations

from contextlib import nullcontext
from typing import Literal

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops.fp8_linear import FP8Linear
from ..ops.reference import FP8_MAX, QBLOCK

Precision = Literal["fp32", "bf16", "fp8"]


def autocast(precision: Precision = "fp32", device_type: str | None = None):
    if precision == "fp32":
        return nullcontext()
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    return torch.autocast(device_type, dtype=torch.bfloat16)


def _under_cam(fqn: str) -> bool:
    return fqn.startswith("cam.") or ".cam." in fqn


def fp8_eligible(mod: nn.Module, fqn: str, recipe: str = "block") -> bool:
    if not isinstance(mod, nn.Linear) or "weight_orig" in mod._parameters or _under_cam(fqn):
        return False
    mult = QBLOCK if recipe == "block" else 16
    return mod.in_features % mult == 0 and mod.out_features % mult == 0


def convert_to_fp8(model: nn.Module, recipe: str = "block", untie_head: bool = False) -> nn.Module:
    """Swap eligible linears for :class:`FP8Linear` in place. Call before wrapping."""
    tied = (
        getattr(model, "head", None) is not None
        and getattr(model, "embed", None) is not None
        and model.head.weight is model.embed.weight
    )
    for fqn, mod in list(model.named_modules()):
        if not fp8_eligible(mod, fqn, recipe):
            continue
        parent_name, _, attr = fqn.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, attr, FP8Linear(mod, recipe=recipe))

    if tied and not untie_head and isinstance(model.head, FP8Linear):
        model.embed.weight.data = model.embed.weight.data.to(torch.bfloat16)
        model.head.weight = model.embed.weight

    for mod in model.modules():
        if "weight_orig" in mod._parameters:
            mod.to(torch.bfloat16)
    for fqn, mod in model.named_modules():
        if isinstance(mod, nn.RMSNorm) and mod.weight is not None and not _under_cam(fqn):
            mod.weight.data = mod.weight.data.to(torch.bfloat16)
    cam = getattr(model, "cam", None)
    if cam is not None:
        cam.to(torch.bfloat16)
    return model


@torch.no_grad()
def _peer_max_ok() -> bool:
    """The peer-memory MAX all-reduce needs torch's symmetric memory; ``GDNET_AMAX_NCCL=1`` forces NCCL."""
    import os

    if os.environ.get("GDNET_AMAX_NCCL", "0") == "1":
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return True


def update_fp8_scales(model: nn.Module, group=None) -> None:
    """Refresh the delayed per-tensor scales from the amax windows (tensor recipe).

    One MAX all-reduce carries every amax of the model. Modules on the block recipe
    compute their scales on the fly and are skipped.
    """
    mods = [m for m in model.modules() if isinstance(m, FP8Linear) and m.recipe == "tensor"]
    if not mods:
        return
    amax = torch.cat([t for m in mods for t in (m._amax_x, m._amax_w)]).clamp_(min=1e-12)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if amax.is_cuda and _peer_max_ok():
            from ..parallel.symm import max_allreduce_

            max_allreduce_(amax, group)      # one peer-memory kernel instead of an NCCL call
        else:
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    for i, m in enumerate(mods):
        m.scale_x.copy_(FP8_MAX / amax[2 * i])
        m.scale_w.copy_(FP8_MAX / amax[2 * i + 1])
        m.inv_scale_x.copy_(m.scale_x.reciprocal())
        m.inv_scale_w.copy_(m.scale_w.reciprocal())
        m._amax_x.zero_()
        m._amax_w.zero_()


def cast_for_precision(model: nn.Module, precision: Precision, recipe: str = "block") -> nn.Module:
    """Apply the reference's per-mode casts (scripts/training.py:384-389)."""
    if precision == "bf16":
        model.to(torch.bfloat16)
    elif precision == "fp8":
        model.embed.weight.data = model.embed.weight.data.to(torch.bfloat16)
        convert_to_fp8(model, recipe=recipe)
    return model
