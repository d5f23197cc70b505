"""Sequence parallelism: contiguous T shards and the conv-halo / memory-state exchange.

The only cross-token mixing in GDNet is a causal depthwise conv of width ``k``, so a
shard needs just the previous shard's last ``k-1`` conv inputs (reference:
gdnet/utils/sp.py:102-143). Two transports implement the same differentiable
exchange:

* **symmetric-memory kernels** (CUDA tensors, extension built): the conv kernels push
  the tail rows into the next rank's slot and wait on a sequence-numbered flag, all
  from inside the kernel over NVLink peer memory (``csrc/elementwise.cu``: ``dwconv_fwd_sw_kernel<.., true>``,
  ``dwconv_dx_sw_kernel<.., true>``; stand-alone form ``csrc/comm.cu``: ``halo_push_wait_kernel``);
* **point-to-point messages** (CPU/gloo, or NCCL when ``GDNET_SP_TRANSPORT=p2p``): plain
  ``isend``/``irecv``; this is what the CPU tests run.

Differences from the reference, on purpose:

* the gradient of a halo is delivered to the owning rank *inside* the backward of the
  exchange and added to the tail rows before autograd consumes them (the reference
  queues the add until after ``backward()`` has returned, gdnet/utils/sp.py:44-55,167,
  which drops it);
* every exchange of a pass has its own slot and a monotonically increasing sequence
  number, so a fast producer cannot overwrite a halo that has not been read.

``flush_bwd_halos`` is therefore a no-op kept for call-site compatibility.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist


def shard_range(T: int, sp_rank: int, sp_size: int) -> tuple[int, int]:
    """``[start, end)`` of a rank's contiguous slice of a length-``T`` sequence."""
    if T % sp_size != 0:
        raise ValueError(f"sequence length {T} not divisible by sp_size {sp_size}")
    t_local = T // sp_size
    return sp_rank * t_local, (sp_rank + 1) * t_local


def shard_sequence(seq: torch.Tensor, sp_rank: int, sp_size: int, dim: int = 1) -> torch.Tensor:
    s, e = shard_range(seq.shape[dim], sp_rank, sp_size)
    return seq.narrow(dim, s, e - s)


def _neighbours(group) -> tuple[int, int, int | None, int | None]:
    """``(rank_in_group, size, global_rank_of_prev, global_rank_of_next)``."""
    r, n = dist.get_rank(group), dist.get_world_size(group)
    prev_g = dist.get_global_rank(group, r - 1) if r > 0 else None
    next_g = dist.get_global_rank(group, r + 1) if r < n - 1 else None
    return r, n, prev_g, next_g


class _HaloExchangeP2P(torch.autograd.Function):
    """tail -> next rank's halo; gradient of the halo -> previous rank's tail."""

    @staticmethod
    def forward(ctx, tail: torch.Tensor, group) -> torch.Tensor:
        r, n, prev_g, next_g = _neighbours(group)
        ctx.group = group
        reqs = []
        halo = torch.zeros_like(tail)
        if next_g is not None:
            reqs.append(dist.isend(tail.contiguous(), dst=next_g, group=group))
        if prev_g is not None:
            reqs.append(dist.irecv(halo, src=prev_g, group=group))
        for q in reqs:
            q.wait()
        return halo

    @staticmethod
    def backward(ctx, d_halo: torch.Tensor):
        r, n, prev_g, next_g = _neighbours(ctx.group)
        reqs = []
        d_tail = torch.zeros_like(d_halo)
        if prev_g is not None:
            reqs.append(dist.isend(d_halo.contiguous(), dst=prev_g, group=ctx.group))
        if next_g is not None:
            reqs.append(dist.irecv(d_tail, src=next_g, group=ctx.group))
        for q in reqs:
            q.wait()
        return d_tail, None


def halo_exchange(tail: torch.Tensor, group, slot: int | None = None) -> torch.Tensor:
    """Send this shard's conv tail ``(B, k-1, d)`` right, return the halo from the left.

    Rank 0 of the group gets zeros. Differentiable (see the module docstring).
    """
    if group is None or dist.get_world_size(group) == 1:
        return torch.zeros_like(tail)
    if tail.is_cuda and os.environ.get("GDNET_SP_TRANSPORT", "symm") == "symm":
        from .symm import halo_exchange_symm

        return halo_exchange_symm(tail, group, slot)
    return _HaloExchangeP2P.apply(tail, group)


def state_exchange(summary: torch.Tensor, group) -> torch.Tensor:
    """Pass a per-shard state vector (the CAM chunk summary) to the next rank.

    Returns the previous rank's ``summary`` (zeros on the first rank). Not
    differentiable: the memory-filling passes run without a graph.
    """
    if group is None or dist.get_world_size(group) == 1:
        return torch.zeros_like(summary)
    with torch.no_grad():
        return _HaloExchangeP2P.apply(summary.detach(), group)


def gather_states(payload: torch.Tensor, group) -> torch.Tensor:
    """``(sp_size, *payload.shape)``: every shard's state vector (the chunk summary a shard would write into the
    content-addressed memory), in shard order, on every rank. Not differentiable: the reference fills the memory
    without a graph (gdnet/loss.py:54-85). On CUDA one peer-memory kernel (push to all, flags, bounded wait)."""
    n = dist.get_world_size(group)
    with torch.no_grad():
        flat = payload.detach().float().contiguous().view(-1)
        if flat.is_cuda and os.environ.get("GDNET_SP_TRANSPORT", "symm") == "symm":
            from .symm import all_gather_small

            out = all_gather_small(flat, group)
        else:
            parts = [torch.empty_like(flat) for _ in range(n)]
            dist.all_gather(parts, flat, group=group)
            out = torch.stack(parts)
    return out.view(n, *payload.shape)


# -- names kept from the reference ---------------------------------------------------

class FusedHaloConvSP:
    """Sequence-parallel causal conv under the reference's name and call form
    (gdnet/utils/sp.py:102-170): ``FusedHaloConvSP.apply(x, W_conv, T, k, BLOCK_T, sp_group)`` exchanges the
    ``k-1`` tail rows with the neighbours and convolves with the received halo. ``T`` and ``BLOCK_T`` are
    accepted for call-site compatibility (the kernels here pick their own tiling). Differentiable in ``x``,
    ``W_conv`` and, through the exchange, the previous rank's tail rows."""

    @staticmethod
    def apply(x, W_conv, T, k, BLOCK_T, sp_group, slot: int = 0):
        from ..ops import functional as ops
        from ..ops import reference as ref

        halo = halo_exchange(ref.conv_tail(x, k).contiguous(), sp_group, slot) if k > 1 else None
        return ops.causal_dwconv(x, W_conv, halo)


def flush_bwd_halos(sp_group) -> None:
    """No-op: halo gradients are applied inside the exchange's backward."""
    return None


def clear_symm_handles() -> None:
    """Free every cached symmetric buffer (collective over the SP group)."""
    from . import symm

    symm.release_all()
