"""Parameter sharding (ZeRO / FSDP) for GDNet.

``wrap_fsdp`` keeps the reference's entry point (gdnet/utils/distributed.py:112-178):
PyTorch FSDP with bf16 parameters, fp32 reduction, ``use_orig_params`` (needed by the
spectral-norm parametrisation). The reference wraps every ``GDLayer`` as its own unit,
but ``GDNet`` never calls ``layer(...)`` (it calls ``layer.fwd_step`` / ``bwd_step``), so
a per-layer unit would never be unsharded; the wrap here is therefore root-only unless
``auto_wrap=True`` is requested.

The B200 sharded engine (flat bf16 shards, all-gather fused in front of the first
GEMM that consumes a layer, gradient reduce-scatter fused with the AdamW update of
the shard) is :class:`gdnet_b200.train.engine.TrainEngine` with ``shard="full"``.
"""

from __future__ import annotations

import functools
import logging
import os

import torch
import torch.distributed as dist
import torch.nn as nn

log = logging.getLogger(__name__)


def wrap_fsdp(model: nn.Module, sharding_strategy=None, offload: bool = False,
              min_num_params: int = 1_000_000, auto_wrap: bool = False):
    from torch.distributed.fsdp import (
        BackwardPrefetch,
        CPUOffload,
        FullyShardedDataParallel as FSDP,
        MixedPrecision,
        ShardingStrategy,
    )
    from torch.distributed.fsdp.wrap import size_based_auto_wrap_policy

    if not dist.is_initialized():
        raise RuntimeError("wrap_fsdp needs an initialised process group: call init_distributed() first")
    if sharding_strategy is None:
        sharding_strategy = ShardingStrategy.SHARD_GRAD_OP
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    on_gpu = torch.cuda.is_available()
    policy = functools.partial(size_based_auto_wrap_policy, min_num_params=min_num_params) if auto_wrap else None
    wrapped = FSDP(
        model,
        auto_wrap_policy=policy,
        sharding_strategy=sharding_strategy,
        mixed_precision=MixedPrecision(
            param_dtype=torch.bfloat16, reduce_dtype=torch.float32, buffer_dtype=torch.bfloat16
        ),
        backward_prefetch=BackwardPrefetch.BACKWARD_PRE,
        cpu_offload=CPUOffload(offload_params=True) if offload else None,
        device_id=torch.device("cuda", local_rank) if on_gpu else None,
        use_orig_params=True,
        sync_module_states=on_gpu,
    )
    log.info("FSDP wrap: strategy=%s offload=%s", sharding_strategy.name, offload)
    return wrapped


def shard_bounds(numel: int, rank: int, world: int, align: int = 128) -> tuple[int, int]:
    """``[start, end)`` of ``rank``'s slice of a flat buffer of ``numel`` elements.

    Every shard but the last has ``ceil(numel/world)`` rounded up to ``align`` elements,
    so shard starts are 256-byte aligned for bf16 and vector loads never straddle ranks.
    """
    per = -(-numel // world)
    per = -(-per // align) * align
    start = min(rank * per, numel)
    return start, min(start + per, numel)
