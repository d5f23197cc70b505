"""Copy-with-gap with rotary position encoding of every conv input.

    python experiments/copy_task/run_rope.py [--gaps ...] [--epochs 80] [--hard-sn]

Variant of ``run.py`` (reference: experiments/copy_task/run_rope.py:47-123): each layer step first rotates
the halves ``(x1, x2)`` of the forward stream by the angle ``t * 10000^(-i / (d/2))`` and runs the conv,
the gates and the stream update on the rotated stream. ``--hard-sn`` additionally wraps the four ``W1``
matrices of every layer in hard spectral normalisation and re-derives the normalised weight before each
step (``_sync_sn``), which is the state of the layer the reference's script was written against.
"""

from __future__ import annotations

import argparse

import torch
import torch.nn as nn

import run as base          # the shared harness (puts the repo root on sys.path)
from gdnet_b200.layer import GDLayer, _sync_sn, apply_hard_sn


def rope(x: torch.Tensor) -> torch.Tensor:
    """Rotate ``(x[..., :d/2], x[..., d/2:])`` pairs of a (B, T, d) tensor by their position."""
    T, half = x.shape[1], x.shape[2] // 2
    theta = 10000.0 ** (-torch.arange(half, device=x.device, dtype=torch.float32) / half)
    ang = torch.outer(torch.arange(T, device=x.device, dtype=torch.float32), theta)
    cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


class GDLayerRoPE(GDLayer):
    """GDLayer whose forward and backward steps see the rotated stream."""

    def _step(self, which, fwd, side, sp_group=None, return_gate=False, sp_slot=None):
        for name in ("gf_W1", "gb_W1", "rf_W1", "rb_W1"):
            _sync_sn(getattr(self, name))          # no-op unless the matrix is SN-wrapped
        return super()._step(which, rope(fwd), side, sp_group, return_gate, sp_slot)


def make_rope_net(T: int, hard_sn: bool = False):
    net = base.make_net(T)
    layers = [GDLayerRoPE(base.D, base.KSIZE) for _ in range(base.LAYERS)]
    net.layers = nn.ModuleList([apply_hard_sn(l) for l in layers] if hard_sn else layers)
    return net


def main():
    ap = argparse.ArgumentParser()
    base.add_common_args(ap)
    ap.add_argument("--hard-sn", action="store_true")
    args = ap.parse_args()
    base.compare({"gdnet": base.make_net, "gdnet+rope": lambda T: make_rope_net(T, args.hard_sn)}, args)


if __name__ == "__main__":
    main()
