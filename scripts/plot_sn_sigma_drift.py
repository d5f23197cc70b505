"""How far do the spectral norms of the gate W1 matrices drift during training without hard normalisation?

    python scripts/plot_sn_sigma_drift.py [--steps 300] [--d 256] [--device cpu|cuda] [--csv sigma.csv] [--png sigma.png]

Trains one GDLayer (soft penalty only, as the training step applies it) on random streams and records the
largest singular value of gf/gb/rf/rb ``W1`` every 10 steps. Writes a CSV; draws a PNG when matplotlib is
installed. Reference counterpart: scripts/plot_sn_sigma_drift.py.
"""

from __future__ import annotations

import argparse
import csv
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200.layer import GDLayer  # noqa: E402
from gdnet_b200.loss import sn_soft_penalty  # noqa: E402

PREFIXES = ("gf", "gb", "rf", "rb")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--d", type=int, default=256)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--csv", default="sn_sigma_drift.csv")
    ap.add_argument("--png", default="")
    args = ap.parse_args()
    torch.manual_seed(0)
    layer = GDLayer(args.d, 7).to(args.device)
    opt = torch.optim.AdamW(layer.parameters(), lr=1e-3)
    rows = []
    for step in range(args.steps):
        fwd = torch.randn(4, 128, args.d, device=args.device)
        side = torch.randn(4, 128, args.d, device=args.device)
        f2, s2 = layer.fwd_step(fwd, side)
        f3, s3 = layer.bwd_step(f2, s2)
        loss = f3.float().pow(2).mean() + s3.float().pow(2).mean() + sn_soft_penalty([layer])
        opt.zero_grad()
        loss.backward()
        opt.step()
        if step % 10 == 0:
            sig = {p: float(torch.linalg.matrix_norm(getattr(layer, f"{p}_W1").weight.detach().float(), ord=2)) for p in PREFIXES}
            rows.append(dict(step=step, loss=float(loss), **sig))
    with open(args.csv, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0]))
        w.writeheader()
        w.writerows(rows)
    last = rows[-1]
    print("step %d: " % last["step"] + ", ".join(f"sigma({p}_W1) = {last[p]:.4f}" for p in PREFIXES))
    if args.png:
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except ImportError:
            print("matplotlib is not installed: CSV only")
            return
        for p in PREFIXES:
            plt.plot([r["step"] for r in rows], [r[p] for r in rows], label=f"{p}_W1")
        plt.axhline(1.0, color="k", lw=0.5)
        plt.xlabel("step")
        plt.ylabel("largest singular value")
        plt.legend()
        plt.savefig(args.png, dpi=120)


if __name__ == "__main__":
    main()
