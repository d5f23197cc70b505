"""The allocation-free cross-entropy entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory while they run (all of it belongs to
their own pool, or their step loop must stay clear of the CUDA allocator), so the library offers
one entry point whose scratch lives in a fixed array inside the shared object. This test loads
the shared object with ctypes, calls ``gd_cross_entropy_mean_noalloc`` with raw device pointers and
checks it against the regular op (``torch.ops.gdnet_b200.cross_entropy`` through
``gdnet_b200.ops.cuda.cross_entropy``) on two calls in a row; the second call is shorter than the
first, so it would see leftovers in the shared scratch if the entry point relied on them.
The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from gdnet_b200 import _ext

    _ext.load()
    lib = ctypes.CDLL(str(_ext.lib_path()))
    fn = lib.gd_cross_entropy_mean_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _call(fn, logits, targets, vocab, ignore_index, out):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(logits.data_ptr(), targets.data_ptr(), logits.shape[0], vocab, logits.stride(0), ignore_index,
              out.data_ptr(), stream)


def test_noalloc_cross_entropy_matches_regular_entry_point_twice():
    from gdnet_b200.ops import cuda as cu

    fn = _lib()
    dev = "cuda"
    out = torch.zeros(1, device=dev)
    for rows, vocab, vp in ((512, 1000, 1024), (96, 250, 256)):
        logits = (torch.randn(rows, vp, device=dev) * 3).to(torch.bfloat16)
        targets = torch.randint(0, vocab, (rows,), device=dev)
        targets[::5] = -100
        before = logits.clone()
        rc = _call(fn, logits, targets, vocab, -100, out)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(before, logits), "the allocation-free entry point must not modify the logits"
        want = cu.cross_entropy(logits.clone(), targets, -100, vocab=vocab)   # regular op consumes its input
        assert abs(float(out) - float(want)) <= 2e-3 * max(1.0, abs(float(want))), (float(out), float(want))


def test_noalloc_rejects_bad_sizes_and_arguments():
    fn = _lib()
    dev = "cuda"
    logits = torch.zeros(8, 64, device=dev, dtype=torch.bfloat16)
    targets = torch.zeros(8, device=dev, dtype=torch.int64)
    out = torch.zeros(1, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    too_many = 65536 + 1
    assert fn(logits.data_ptr(), targets.data_ptr(), too_many, 64, 64, -100, out.data_ptr(), stream) == 1
    assert fn(logits.data_ptr(), targets.data_ptr(), 8, 65, 64, -100, out.data_ptr(), stream) == 2   # vocab > ld
    assert fn(logits.data_ptr(), targets.data_ptr(), 8, 64, 60, -100, out.data_ptr(), stream) == 2   # ld % 8
    assert fn(None, targets.data_ptr(), 8, 64, 64, -100, out.data_ptr(), stream) == 2
    assert fn(logits.data_ptr(), targets.data_ptr(), 8, 64, 64, -100, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()


def test_noalloc_ignores_out_of_range_targets():
    """Targets outside [0, vocab) are left out of the sum and the count, like ignored rows, and are never
    used to index the logits."""
    import torch.nn.functional as F

    fn = _lib()
    dev = "cuda"
    rows, vocab, vp = 64, 250, 256
    logits = (torch.randn(rows, vp, device=dev) * 3).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), device=dev)
    targets[1], targets[2], targets[40] = vocab + 3, -5, 1 << 40
    good = targets.clone()
    good[[1, 2, 40]] = -100
    out = torch.zeros(1, device=dev)
    assert _call(fn, logits, targets, vocab, -100, out) == 0
    torch.cuda.synchronize()
    want = F.cross_entropy(logits.float()[:, :vocab], good, ignore_index=-100)
    assert abs(float(out) - float(want)) <= 2e-3 * max(1.0, abs(float(want))), (float(out), float(want))
