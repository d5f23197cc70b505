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
