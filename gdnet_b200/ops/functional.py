"""Op entry points used by the model code.

One rule decides the implementation: the device of the tensors. CUDA tensors run the
hand-written sm_100a kernels (``gdnet_b200.ops.cuda``, which refuses to work without
the compiled extension rather than fall back); CPU tensors run the plain-PyTorch
statement in ``gdnet_b200.ops.reference``. There is no other backend.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import reference as ref


def _on_gpu(t: torch.Tensor) -> bool:
    return t.is_cuda


def _cuda():
    from . import cuda as cuda_ops  # deferred: needs the compiled extension

    return cuda_ops


# --------------------------------------------------------------------------------------
# single ops
# --------------------------------------------------------------------------------------

def causal_dwconv(x, w, halo=None):
    if _on_gpu(x):
        return _cuda().causal_dwconv(x, w, halo)
    return ref.causal_dwconv(x, w, halo)


def rmsnorm(x, w, eps):
    if _on_gpu(x):
        return _cuda().rmsnorm(x, w, eps)
    return ref.rmsnorm(x, w, eps)


def fused_mem_read(q, gamma, e, tags, vals, alpha):
    if _on_gpu(q):
        return _cuda().fused_mem_read(q, gamma, e, tags, vals, alpha)
    out, w = ref.fused_mem_read(q, gamma, e, tags, vals, alpha)
    return out, w.detach()


def cross_entropy(logits, targets, ignore_index: int = -100):
    if _on_gpu(logits):
        return _cuda().cross_entropy(logits, targets, ignore_index)
    return ref.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index)


def linear_cross_entropy(x, head, targets, vocab: int, ignore_index: int = -100):
    """Mean cross-entropy of ``head(x)[..., :vocab]`` against ``targets``. On CUDA, for a bias-free bf16 or
    block-scaled FP8 head, the projection, the loss and the head's gradients run chunk by chunk over the rows
    without ever holding all logits (``ops/cuda.py:_LinearCrossEntropyFn``)."""
    x2 = x.reshape(-1, x.shape[-1])
    if _on_gpu(x2) and ignore_index == -100 and getattr(head, "bias", None) is None:
        from .fp8_linear import FP8Linear

        cu = _cuda()
        fp8 = isinstance(head, FP8Linear) and head.recipe == "block"
        plain = type(head) is torch.nn.Linear or fp8
        if plain and cu.linear_cross_entropy_ok(x2, head.weight, fp8):
            return cu.linear_cross_entropy(x2, head.weight, targets, vocab, fp8)
    logits = head(x)[..., :vocab]
    return cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1), ignore_index)


def sample_top_p(logits: torch.Tensor, top_p: float, generator=None) -> torch.Tensor:
    """Nucleus sampling of one id from ``logits (1, V)``."""
    probs = F.softmax(logits, dim=-1)
    sp, si = torch.sort(probs, descending=True)
    before = torch.cumsum(sp, dim=-1) - sp
    sp = torch.where(before < top_p, sp, torch.zeros_like(sp))
    sp = sp / sp.sum(dim=-1, keepdim=True)
    pick = torch.multinomial(sp[0], 1, generator=generator)
    return si[0, pick]


# --------------------------------------------------------------------------------------
# one GDLayer step
# --------------------------------------------------------------------------------------

def _module_linear(mod, x):
    """``mod(x)`` for a plain ``nn.Linear`` (weights cast to ``x.dtype``) or an FP8 linear."""
    from .fp8_linear import FP8Linear

    if isinstance(mod, FP8Linear):
        return mod(x)
    return ref.linear(x, mod.weight, mod.bias)


def layer_step(fwd, side, layer, conv_name: str, g: str, r: str, sp_group=None, sp_slot=None,
               return_gate: bool | str = False):
    """Run one step of ``layer`` with the parameter set ``(conv_name, g, r)``.

    Returns ``(fwd', side')`` or ``(fwd', side', gate)`` where ``gate`` is the forward
    gate tensor (``return_gate=True``) or its mean (``return_gate="mean"``). ``side=None`` stands for an
    all-zero side stream: the CUDA path then leaves out the recovery gate, which only ever multiplies it.
    """
    conv = getattr(layer, conv_name)
    k = conv.size
    if _on_gpu(fwd):
        return _cuda().layer_step(fwd, side, layer, conv_name, g, r, sp_group, sp_slot, return_gate)
    if side is None:          # ``None`` stands for an all-zero side stream (the first forward step of a layer)
        side = torch.zeros_like(fwd)

    halo = None
    if sp_group is not None and k > 1:
        from ..parallel.sp import halo_exchange

        halo = halo_exchange(ref.conv_tail(fwd, k).contiguous(), sp_group)

    c = ref.causal_dwconv(fwd, conv.taps, halo)
    s = side.to(c.dtype)
    u = torch.cat([s, c], dim=-1)
    w1r, w2r, nr = getattr(layer, f"{r}_W1"), getattr(layer, f"{r}_W2"), getattr(layer, f"{r}_norm")
    z = _module_linear(w2r, F.silu(_module_linear(w1r, u)))
    eps_r = nr.eps if nr.eps is not None else ref.default_rms_eps(z.dtype)
    R = torch.sigmoid(ref.rmsnorm(z, nr.weight, eps_r).float())
    w1g, w2g, ng = getattr(layer, f"{g}_W1"), getattr(layer, f"{g}_W2"), getattr(layer, f"{g}_norm")
    g_pre = ref.gate_pre(c, w1g.weight, w1g.bias, ng.weight, w2g.weight, w2g.bias)
    fwd_out, side_out, gate = ref.gate_stream_update(g_pre, c, s, R)
    if return_gate == "mean":
        return fwd_out, side_out, gate.mean()
    if return_gate:
        return fwd_out, side_out, gate.to(c.dtype)
    return fwd_out, side_out
