"""Spectral-norm estimates for the soft penalty and the hard-SN power iteration.

``sigma_estimates`` evaluates ``||W_i v_i||`` for a fresh random unit vector per matrix
(reference: gdnet/loss.py:15-31). On CUDA all matrices are handled by one batched
matrix-vector kernel and its rank-1 backward (``csrc/loss_optim.cu``: ``batched_gemv_kernel``,
``batched_outer_add_kernel``); on CPU it is a
loop of fp32 matvecs.
"""

from __future__ import annotations

import torch


def _unit_vectors(mats, generator=None):
    vs = []
    for W in mats:
        v = torch.randn(W.shape[1], device=W.device, dtype=torch.float32, generator=generator)
        vs.append(v / v.norm())
    return vs


def sigma_estimates(mats, generator: torch.Generator | None = None, vectors=None) -> torch.Tensor:
    """fp32 tensor ``(len(mats),)`` of ``||W_i v_i||``; differentiable w.r.t. each ``W_i``."""
    if mats and mats[0].is_cuda:
        from . import cuda as cuda_ops

        return cuda_ops.sigma_estimates(mats, vectors, generator)      # probe vectors drawn in one batch
    vs = vectors if vectors is not None else _unit_vectors(mats, generator)
    return torch.stack([(W.float() @ v).norm() for W, v in zip(mats, vs)])
