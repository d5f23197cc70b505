"""Multi-GPU tests (2 ranks on 2 GPUs, spawned as child processes): fused gradient collective +
AdamW against the NCCL path, and the sequence-parallel halo exchange over symmetric memory against
the single-GPU model. Skipped with fewer than 2 GPUs. NVLS is off in NCCL for these runs and the
kernels use plain peer loads/stores only (``GDNET_MULTIMEM=0``), except in the one test of the multicast path."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(worker: str, nproc: int = 2, timeout: int = 600):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", GDNET_MULTIMEM="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(ROOT, "tests", "multi_gpu_workers.py"), worker]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "WORKER_OK" in proc.stdout, proc.stdout[-2000:]


def test_fused_collective_matches_nccl():
    _run("engine_fused_vs_nccl")


def test_multicast_update_matches_peer_loads():
    """The one test that uses ``multimem`` instructions (the worker switches them on for one of its two engines)."""
    _run("engine_multimem_vs_peer")


def test_epilogue_reduce_scatter_matches_nccl():
    _run("engine_scatter_vs_nccl")


def test_shared_fp8_weights_match_private_caches():
    _run("engine_shared_fp8_weights")


def test_peer_max_allreduce_matches_nccl():
    _run("peer_max_allreduce")


def test_sequence_parallel_matches_single_gpu():
    _run("sp_matches_single")


def test_engine_sp_step_runs():
    _run("sp_engine_step")


def test_full_shard_engine_matches_replicated():
    _run("engine_full_shard_vs_replicated")


def test_sharded_checkpoint_resume_matches_uninterrupted():
    _run("engine_ckpt_roundtrip")
