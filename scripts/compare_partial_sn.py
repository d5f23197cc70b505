"""Hard spectral normalisation on all four gate W1 matrices against only the forward-step pair plus clipping.

    python scripts/compare_partial_sn.py [--steps 300] [--d 256] [--device cpu|cuda]

"Full": ``nn.utils.spectral_norm`` on gf/gb/rf/rb ``W1``. "Partial": only on gf/rf (the matrices the timed
``fwd_step`` uses), the other two left plain, with gradient-norm clipping at 1.0 to make up for the missing
constraint. Reported: mean step time of each and the two loss curves' end points.
Reference counterpart: scripts/compare_partial_sn.py.
"""

from __future__ import annotations

import argparse
import os
import sys
import time

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.layer import GDLayer, apply_hard_sn  # noqa: E402


def run(partial: bool, steps: int, d: int, device: str):
    torch.manual_seed(0)
    layer = apply_hard_sn(GDLayer(d, 7))
    if partial:
        for prefix in ("gb", "rb"):
            nn.utils.remove_spectral_norm(getattr(layer, f"{prefix}_W1"))
    layer = layer.to(device)
    opt = torch.optim.AdamW(layer.parameters(), lr=1e-4)
    g = torch.Generator(device="cpu").manual_seed(42)
    times, loss = [], 0.0
    for _ in range(steps):
        fwd = torch.randn(2, 128, d, generator=g).to(device)
        side = torch.randn(2, 128, d, generator=g).to(device)
        t0 = time.perf_counter()
        f2, s2 = layer.fwd_step(fwd, side)
        loss_t = f2.float().sum() + s2.float().sum()
        opt.zero_grad()
        loss_t.backward()
        if partial:
            nn.utils.clip_grad_norm_(layer.parameters(), max_norm=1.0)
        opt.step()
        if device == "cuda":
            torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
        loss = float(loss_t)
    warm = times[min(10, len(times) - 1):]
    return 1e3 * sum(warm) / len(warm), loss


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--d", type=int, default=256)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    t_full, l_full = run(False, args.steps, args.d, args.device)
    t_part, l_part = run(True, args.steps, args.d, args.device)
    print(f"full SN:            {t_full:8.3f} ms/step, last loss {l_full:.3f}")
    print(f"partial SN + clip:  {t_part:8.3f} ms/step, last loss {l_part:.3f}")
    print(f"speed-up:           {t_full / t_part:.2f}x")


if __name__ == "__main__":
    main()
