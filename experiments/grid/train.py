"""4x4 grid world: do the transition operators specialise by move type?

    python experiments/grid/train.py [--steps 2000] [--n-ops 8] [--variant ctr|ctr-weak|ctr-delta|mse]

16 positions with learned embeddings; four moves (up/down/left/right with wrap). A sample is
``(z_t, z_t1) = (embed(pos), embed(next_pos).detach())``. Variants (reference: experiments/grid/train.py):
``mse`` regresses the routed prediction on ``z_t1``; ``ctr`` is the InfoNCE + load-balance loss of
``TransitionOperators.loss``; ``ctr-weak`` uses ``balance_coef=0.001``; ``ctr-delta`` lets the router see
``z_t1 - z_t`` (an oracle ceiling: the move is visible to the router). Reported: loss, next-position
accuracy by nearest embedding, and the purity of operator use per move type (1.0 = each move has its
own operator).
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gdnet_b200.operators import TransitionOperators  # noqa: E402

GRID, D = 4, 64
MOVES = {"up": (-1, 0), "down": (1, 0), "left": (0, -1), "right": (0, 1)}


def next_pos(pos: torch.Tensor, move: torch.Tensor) -> torch.Tensor:
    dr = torch.tensor([m[0] for m in MOVES.values()])[move]
    dc = torch.tensor([m[1] for m in MOVES.values()])[move]
    r, c = pos // GRID, pos % GRID
    return ((r + dr) % GRID) * GRID + (c + dc) % GRID


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--n-ops", type=int, default=8)
    ap.add_argument("--variant", choices=["ctr", "ctr-weak", "ctr-delta", "mse"], default="ctr")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    torch.manual_seed(args.seed)
    embed = nn.Embedding(GRID * GRID, D)
    ops = TransitionOperators(D, args.n_ops, balance_coef=0.001 if args.variant == "ctr-weak" else 0.01)
    opt = torch.optim.Adam(list(embed.parameters()) + list(ops.parameters()), lr=3e-3)

    def routed(z_t, z_t1):
        w = ops.routing(z_t1 - z_t if args.variant == "ctr-delta" else z_t)
        return ops.predict(z_t, w), w

    for step in range(1, args.steps + 1):
        pos = torch.randint(0, GRID * GRID, (args.batch,))
        move = torch.randint(0, 4, (args.batch,))
        z_t, z_t1 = embed(pos), embed(next_pos(pos, move)).detach()
        if args.variant == "mse":
            loss = F.mse_loss(routed(z_t, z_t1)[0], z_t1)
        elif args.variant == "ctr-delta":
            pred, w = routed(z_t, z_t1)
            temp = ops.log_temp.exp().clamp(min=0.01)
            logits = F.normalize(pred, dim=-1) @ F.normalize(z_t1, dim=-1).t() / temp
            mw = w.mean(0)
            loss = F.cross_entropy(logits, torch.arange(args.batch)) + ops.balance_coef * (mw * mw.log()).sum()
        else:
            loss = ops.loss(z_t, z_t1)
        opt.zero_grad()
        loss.backward()
        opt.step()
        if step % max(args.steps // 10, 1) == 0:
            print(f"step {step}: loss {loss.item():.4f}", flush=True)

    with torch.no_grad():
        pos = torch.arange(GRID * GRID).repeat(4)
        move = torch.arange(4).repeat_interleave(GRID * GRID)
        z_t, z_t1 = embed(pos), embed(next_pos(pos, move))
        pred, w = routed(z_t, z_t1)
        nearest = (F.normalize(pred, dim=-1) @ F.normalize(embed.weight, dim=-1).t()).argmax(-1)
        acc = (nearest == next_pos(pos, move)).float().mean().item()
        win = w.argmax(-1)
        purity = sum(torch.bincount(win[move == m], minlength=args.n_ops).max().item() for m in range(4)) / len(pos)
        print(f"{args.variant}: next-position accuracy {acc:.3f}, operator purity per move {purity:.3f}, "
              f"operators used {len(torch.unique(win))}/{args.n_ops}")


if __name__ == "__main__":
    main()
