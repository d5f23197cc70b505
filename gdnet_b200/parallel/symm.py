"""Symmetric (peer-mapped) buffers for the in-kernel collectives.

Allocation and handle exchange go through ``torch.distributed._symmetric_memory`` (CUDA
VMM allocations mapped into every rank of the group, plus a signal pad and, when the
switch supports it, an NVLS multicast address). The kernels only see raw pointers:
``buffer_ptrs[r]`` is rank ``r``'s buffer as mapped into this process.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

_HANDLES: dict = {}


class SymmBuffer:
    """A ``nbytes`` buffer that exists on every rank of ``group`` and is mapped in all of them."""

    def __init__(self, nbytes: int, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.local, group)
        self.local.zero_()
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.ptr_table = torch.tensor(self.ptrs, dtype=torch.int64, device=device)
        self.signal_table = torch.tensor(self.signal_ptrs, dtype=torch.int64, device=device)

    def view(self, dtype: torch.dtype, numel: int, offset_bytes: int = 0) -> torch.Tensor:
        item = torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes : offset_bytes + numel * item].view(dtype)

    def barrier(self) -> None:
        self.handle.barrier()


def get_buffer(key, nbytes: int, group, device) -> SymmBuffer:
    """Cached symmetric buffer; grows (collectively) when a larger size is asked for."""
    k = (key, id(group))
    buf = _HANDLES.get(k)
    if buf is None or buf.nbytes < nbytes:
        buf = SymmBuffer(nbytes, group, device)
        _HANDLES[k] = buf
    return buf


def release_all() -> None:
    _HANDLES.clear()
    _MAXRED.clear()


def halo_exchange_symm(tail: torch.Tensor, group, slot):
    from ..ops import cuda as cuda_ops

    return cuda_ops.halo_exchange(tail, group, slot)


_MAXRED: dict = {}


def max_allreduce_(vec: torch.Tensor, group=None, gather_out: torch.Tensor | None = None) -> torch.Tensor:
    """In-place element-wise MAX of a small fp32 CUDA vector over the ranks of ``group``: every rank stores
    its vector into every peer's exchange area and waits (bounded) for the peers' flags, one kernel, no
    NCCL call (``csrc/comm.cu:max_allreduce_kernel``). Reference counterpart: the MAX all-reduce of the amax
    windows in gdnet/utils/fp8.py:16-44."""
    from ..ops import cuda as cuda_ops

    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = vec.numel()
    st = _MAXRED.get(id(group))
    if st is None or st["slot"] < n:
        slot = max(256, 1 << (n - 1).bit_length())
        st = {"slot": slot, "area": SymmBuffer(2 * world * slot * 4, group, vec.device),
              "flags": SymmBuffer(max(256, world * 4), group, vec.device), "seq": 0}
        st["area"].barrier()
        _MAXRED[id(group)] = st
    st["seq"] += 1
    cuda_ops.K.max_allreduce(vec, st["area"].ptr_table, st["flags"].ptr_table, st["slot"], rank, world, st["seq"], 0, gather_out)
    return vec if gather_out is None else gather_out


def all_gather_small(vec: torch.Tensor, group=None) -> torch.Tensor:
    """``(world, n)``: every rank's small fp32 CUDA vector, in rank order. Same kernel and exchange area as
    :func:`max_allreduce_` (every rank stores its vector into its slot of every peer's area, flags, bounded wait),
    reading the slots out instead of reducing them."""
    group = group if group is not None else dist.group.WORLD
    out = torch.empty(dist.get_world_size(group), vec.numel(), dtype=torch.float32, device=vec.device)
    return max_allreduce_(vec.contiguous().view(-1), group, gather_out=out)
