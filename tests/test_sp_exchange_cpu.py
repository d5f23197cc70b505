"""Slot / ring / sequence-number bookkeeping of the in-kernel halo exchange (``ops/cuda.py:SpExchange``) on CPU, with
the symmetric buffers replaced by placeholders. What must hold so that a fast rank can never overwrite a message that
was not read, and so that all ranks agree on the numbers without talking to each other: sequence numbers of a slot
increase with every use; a forward use and the (at most two) gradient exchanges that answer it have ring positions
of their own; two uses of a slot less than a ring apart never share a position."""

import types

import pytest
import torch

from gdnet_b200.ops import cuda as cu


@pytest.fixture
def ctx(monkeypatch):
    st = {"data": types.SimpleNamespace(ptr_table="D"), "flags": types.SimpleNamespace(ptr_table="F"),
          "counters": torch.zeros(2 * cu.HALO_RING * cu.HALO_SLOTS, dtype=torch.int32), "slot_bytes": 96, "rank": 1, "world": 4,
          "pass_fwd": {}}
    monkeypatch.setattr(cu, "_halo_ctx", lambda group, nbytes, device: st)
    return st


def _fields(args):
    data, flags, counter, byte_off, idx, rank, world, seq = args
    return dict(idx=idx, byte_off=byte_off, seq=seq, rank=rank, world=world, counter=counter)


def test_forward_uses_get_increasing_sequence_numbers_and_their_own_ring_position(ctx):
    seen = {}
    for use in range(1, 3 * cu.HALO_RING):
        for slot in (0, 5, cu.HALO_SLOTS - 1):
            f = _fields(cu.SpExchange(None, slot, 96, "cpu").fwd_args())
            assert f["seq"] == use and f["rank"] == 1 and f["world"] == 4
            assert 0 <= f["idx"] < cu.HALO_RING * cu.HALO_SLOTS and f["idx"] % cu.HALO_SLOTS == slot
            assert f["byte_off"] == f["idx"] * 96 and f["counter"].numel() == 1
            # a position is reused only a whole ring of uses later
            last = seen.get(f["idx"])
            assert last is None or use - last == cu.HALO_RING
            seen[f["idx"]] = use


def test_gradient_exchanges_live_in_the_second_half_with_two_numbers_per_forward_use(ctx):
    seqs = set()
    for use in range(1, 2 * cu.HALO_RING):
        ex = cu.SpExchange(None, 7, 96, "cpu")
        first, second, third = (_fields(ex.bwd_args()) for _ in range(3))
        assert first["seq"] == 2 * use and second["seq"] == 2 * use + 1
        assert third["seq"] == second["seq"], "a graph is differentiated at most twice per forward use"
        for f in (first, second):
            assert cu.HALO_RING * cu.HALO_SLOTS <= f["idx"] < 2 * cu.HALO_RING * cu.HALO_SLOTS
            assert f["idx"] % cu.HALO_SLOTS == 7
            assert f["seq"] not in seqs
            seqs.add(f["seq"])
        assert first["idx"] != second["idx"]


def test_slot_index_is_bounded(ctx):
    with pytest.raises(ValueError, match="HALO_SLOTS"):
        cu.SpExchange(None, cu.HALO_SLOTS, 96, "cpu")
