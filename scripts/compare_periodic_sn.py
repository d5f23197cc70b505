"""Hard spectral normalisation of the gate W1 matrices: power iteration every step against every K-th step.

    python scripts/compare_periodic_sn.py [--steps 300] [--every 1,4,16] [--d 256] [--device cpu|cuda] [--csv out.csv]

One GDLayer with ``nn.utils.spectral_norm`` on its four gate ``W1`` (``apply_hard_sn``) is trained on random
streams; on the steps that are not a multiple of K the iteration is skipped (``freeze_sn_iteration``: the
stored u/v are reused). Reported per K: mean step time, final loss, and the largest true singular value of
the four normalised matrices along the way (how far the stale estimate lets sigma drift above 1).
Reference counterpart: scripts/compare_periodic_sn.py.
"""

from __future__ import annotations

import argparse
import contextlib
import csv
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.layer import GDLayer, apply_hard_sn, freeze_sn_iteration  # noqa: E402

PREFIXES = ("gf", "gb", "rf", "rb")


def true_sigma(layer) -> float:
    return max(float(torch.linalg.matrix_norm(getattr(layer, f"{p}_W1").weight.detach().float(), ord=2)) for p in PREFIXES)


def run(every: int, steps: int, d: int, device: str):
    torch.manual_seed(0)
    layer = apply_hard_sn(GDLayer(d, 7)).to(device)
    opt = torch.optim.AdamW(layer.parameters(), lr=1e-4)
    g = torch.Generator(device="cpu").manual_seed(42)
    times, sig_max, loss = [], 0.0, 0.0
    for step in range(steps):
        fwd = torch.randn(2, 128, d, generator=g).to(device)
        side = torch.randn(2, 128, d, generator=g).to(device)
        t0 = time.perf_counter()
        ctx = contextlib.nullcontext() if step % every == 0 else freeze_sn_iteration(layer)
        with ctx:
            f2, s2 = layer.fwd_step(fwd, side)
        loss_t = f2.float().pow(2).mean() + s2.float().pow(2).mean()
        opt.zero_grad()
        loss_t.backward()
        opt.step()
        if device == "cuda":
            torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
        loss = float(loss_t)
        if step % 10 == 0:
            with freeze_sn_iteration(layer):
                layer.fwd_step(fwd, side)          # refresh .weight from the stored u/v without iterating
            sig_max = max(sig_max, true_sigma(layer))
    warm = times[min(10, len(times) - 1):]
    return dict(every=every, ms_per_step=1e3 * sum(warm) / len(warm), final_loss=loss, max_sigma=sig_max)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--every", default="1,4,16")
    ap.add_argument("--d", type=int, default=256)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--csv", default="")
    args = ap.parse_args()
    rows = [run(int(k), args.steps, args.d, args.device) for k in args.every.split(",")]
    for r in rows:
        print(f"iteration every {r['every']:3d} steps: {r['ms_per_step']:8.3f} ms/step, final loss {r['final_loss']:.4f}, "
              f"largest sigma seen {r['max_sigma']:.4f}")
    if args.csv:
        with open(args.csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0]))
            w.writeheader()
            w.writerows(rows)


if __name__ == "__main__":
    main()
