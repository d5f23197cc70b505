"""Copy-with-gap with sinusoidal position codes fed into the side streams.

    python experiments/copy_task/run_sin.py [--gaps ...] [--epochs 80]

Variant of ``run.py`` (reference: experiments/copy_task/run_sin.py:44-68): before every layer step of
every cycle the fixed code ``pe[t, 2i] = sin(t / 10000^(2i/d))``, ``pe[t, 2i+1] = cos(...)`` is added to
that layer's side stream, so the recovery gate sees absolute position while the forward stream stays
position-free. The sweep trains the plain net and the variant at every gap and prints both.
"""

from __future__ import annotations

import argparse
import math

import torch

import run as base          # the shared harness (puts the repo root on sys.path)
from gdnet_b200.model import GDNet


def sinusoidal_pe(T: int, d: int, device, dtype=torch.float32) -> torch.Tensor:
    pos = torch.arange(T, device=device, dtype=torch.float32).unsqueeze(1)
    freq = torch.exp(torch.arange(0, d, 2, device=device, dtype=torch.float32) * (-math.log(10000.0) / d))
    return torch.stack([(pos * freq).sin(), (pos * freq).cos()], dim=-1).flatten(-2).to(dtype)    # (T, d)


class GDNetSinPE(GDNet):
    """GDNet whose side streams receive the position code before each layer step."""

    def one_cycle(self, fwd, side, sp_group=None, gate_sink=None, gate_mode=True, cycle=0):
        pe = sinusoidal_pe(fwd.shape[1], fwd.shape[2], fwd.device, fwd.dtype).unsqueeze(0)
        n = len(self.layers)
        for i in range(n):
            fwd, side[i] = self.layers[i].fwd_step(fwd, side[i] + pe)
        for i in range(n - 1, -1, -1):
            fwd, side[i] = self.layers[i].bwd_step(fwd, side[i] + pe)
        return fwd, side


def main():
    ap = argparse.ArgumentParser()
    base.add_common_args(ap)
    base.compare({"gdnet": base.make_net, "gdnet+sin": lambda T: base.make_net(T, GDNetSinPE)}, ap.parse_args())


if __name__ == "__main__":
    main()
