"""Red zones behind the tensors the op layer allocates (gdnet_b200/runtime/checked.py), on CPU: an intact run
passes, a write behind a tensor is reported. The overwrite is made through a view of the padded allocation itself,
so nothing outside the test's own memory is touched."""

import pytest
import torch

from gdnet_b200.runtime.checked import CANARY, PAD, RedZoneError, RedZones


def test_red_zones_pass_when_nothing_writes_past_the_end():
    with RedZones("cpu") as rz:
        a = torch.empty(10, 7)
        b = torch.zeros(33, dtype=torch.bfloat16)
        c = torch.empty_like(a)
        d = a.new_empty(5)
        e = a.new_zeros(3, 3)
        a.fill_(1.0)
        c.copy_(a * 2)
        assert float(b.float().abs().sum()) == 0.0 and float(e.abs().sum()) == 0.0
        assert a.is_contiguous() and a.shape == (10, 7) and d.numel() == 5
        assert rz.check() == 5
        assert rz.check() == 0          # nothing new since the last check


def test_red_zone_violation_is_reported():
    with pytest.raises(RedZoneError, match="1 byte"):
        with RedZones("cpu") as rz:
            t = torch.empty(16, dtype=torch.float32)
            t.zero_()
            whole = torch.empty(0, dtype=torch.uint8).set_(t.untyped_storage())   # payload + red zone
            assert whole.numel() == 16 * 4 + PAD and int(whole[-1]) == CANARY
            whole[16 * 4 + 3] = 0           # what a kernel storing one element too many would do
            rz.check()


def test_layer_step_under_red_zones_cpu():
    """The plain-PyTorch layer step allocates through the same calls; it must run unchanged under the mode."""
    from gdnet_b200.layer import GDLayer

    torch.manual_seed(0)
    layer = GDLayer(32, 4)
    x = torch.randn(2, 16, 32, requires_grad=True)
    want_f, want_s = layer.fwd_step(x, torch.zeros(2, 16, 32))
    with RedZones("cpu") as rz:
        got_f, got_s = layer.fwd_step(x, torch.zeros(2, 16, 32))
        (got_f.sum() + got_s.sum()).backward()
        assert rz.check() > 0
    assert torch.allclose(got_f, want_f) and torch.allclose(got_s, want_s)


class _FakeFlags:
    def __init__(self, words):
        self.words = torch.tensor(words, dtype=torch.int32)

    def view(self, dtype, n):
        return self.words[:n]


def _fake_engine(flag_words, counter=0, comm_seq=5, task_seq=5, world=2, rank=0, n_groups=2):
    import types

    sums = torch.zeros(8)
    sums[4:5].view(torch.int32)[0] = counter
    groups = [types.SimpleNamespace(sums=sums.clone()) for _ in range(n_groups)]
    eng = types.SimpleNamespace(groups=groups, world=world, rank=rank, comm="fused", comm_seq=comm_seq, task_seq=task_seq,
                                overlap_task_reduce=True, pg=None, _flags=_FakeFlags(flag_words))
    eng.parameters = lambda: iter([torch.zeros(1)])
    return eng


def test_engine_invariants_accept_a_finished_step_and_name_what_is_off():
    """Flag words are [slot][writer]; after a step every peer's word equals seq * 8 + (number of groups - 1)."""
    from gdnet_b200.runtime.checked import engine_invariants

    want = 5 * 8 + 1
    good = [0, want, 0, want, 0, want]          # rank 0 of 2: its own words are never written
    engine_invariants(_fake_engine(good))
    with pytest.raises(AssertionError, match="a signal is missing"):
        engine_invariants(_fake_engine([0, want, 0, want - 8, 0, want]))
    with pytest.raises(AssertionError, match="a rank ran ahead"):
        engine_invariants(_fake_engine([0, want + 8, 0, want, 0, want]))
    with pytest.raises(AssertionError, match="block counter"):
        engine_invariants(_fake_engine(good, counter=3))
    engine_invariants(_fake_engine([0] * 6, world=1))          # one rank: nothing to check beyond the counters
