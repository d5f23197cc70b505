"""Copy-with-gap: where does GDNet's recall fall off relative to its receptive field?

    python experiments/copy_task/run.py [--gaps 0,8,16,32,48,64,96,128] [--pe none|sin|rope] [--epochs 80]
                                        [--task gap|selective] [--out results.json]

Task (reference: experiments/copy_task/dataset.py): ``seq_len`` signal tokens (ids 0..9), ``gap`` noise
tokens (ids 10..49), then a recall token (50); the model must name the signal tokens from the
representation at the recall position (one linear head per signal position). ``selective`` interleaves
distractors between the signal tokens. Model: GDNet d=64, 3 layers, 3 cycles, k=7, so the receptive
field is 3*7*3 = 63 positions; the reference reports accuracy 1.0 up to gap 64 and a cliff after
(experiments/copy_task/CONCLUDE.md). ``--pe sin`` adds fixed sinusoidal position codes to the
embedding, ``--pe rope`` rotates pairs of embedding channels by position (the reference's run_sin.py /
run_rope.py variants).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gdnet_b200.model import GDNet  # noqa: E402

N_SIGNAL, N_NOISE, RECALL, VOCAB = 10, 40, 50, 52
D, LAYERS, CYCLES, KSIZE = 64, 3, 3, 7


def make_copy_data(n, seq_len, gap, task="gap", ratio=1, gen=None):
    sig = torch.randint(0, N_SIGNAL, (n, seq_len), generator=gen)
    noise = torch.randint(0, N_NOISE, (n, gap), generator=gen) + N_SIGNAL
    recall = torch.full((n, 1), RECALL)
    if task == "selective":
        dis = torch.randint(0, N_NOISE, (n, seq_len, ratio), generator=gen) + N_SIGNAL
        head = torch.cat([sig.unsqueeze(-1), dis], dim=-1).reshape(n, -1)
    else:
        head = sig
    return torch.cat([head, noise, recall], dim=1), sig


def position_codes(T, d, device):
    pos = torch.arange(T, device=device, dtype=torch.float32).unsqueeze(1)
    freq = torch.exp(torch.arange(0, d, 2, device=device, dtype=torch.float32) * (-math.log(10000.0) / d))
    return pos * freq            # (T, d/2)


class CopyModel(nn.Module):
    def __init__(self, T, seq_len, pe="none"):
        super().__init__()
        self.net = GDNet(VOCAB, D, D, LAYERS, n_cycles=CYCLES, chunk_size=T, kernel_size=KSIZE)
        self.heads = nn.ModuleList([nn.Linear(D, VOCAB) for _ in range(seq_len)])
        self.pe = pe

    def forward(self, tokens):
        net = self.net
        emb = net.embed(tokens)
        if self.pe != "none":
            ang = position_codes(tokens.shape[1], D, tokens.device)
            if self.pe == "sin":
                emb = emb + torch.cat([ang.sin(), ang.cos()], dim=-1)
            else:   # rope on channel pairs
                a, b = emb[..., 0::2], emb[..., 1::2]
                emb = torch.stack([a * ang.cos() - b * ang.sin(), a * ang.sin() + b * ang.cos()], dim=-1).flatten(-2)
        fwd = net.proj_in(emb)
        side = [torch.zeros_like(fwd) for _ in net.layers]
        for cyc in range(net.n_cycles):
            fwd, side = net.one_cycle(fwd, side, cycle=cyc)
        rep = net.norm_out(fwd)[:, -1]
        return [h(rep) for h in self.heads]


def run_gap(gap, args, dev):
    g = torch.Generator().manual_seed(args.seed)
    xtr, ytr = make_copy_data(args.n_train, args.seq_len, gap, args.task, gen=g)
    xva, yva = make_copy_data(args.n_val, args.seq_len, gap, args.task, gen=g)
    model = CopyModel(xtr.shape[1], args.seq_len, args.pe).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    acc = 0.0
    for epoch in range(args.epochs):
        perm = torch.randperm(len(xtr), generator=g)
        for i in range(0, len(xtr), args.batch):
            idx = perm[i : i + args.batch]
            x, y = xtr[idx].to(dev), ytr[idx].to(dev)
            logits = model(x)
            loss = sum(F.cross_entropy(logits[j], y[:, j]) for j in range(args.seq_len)) / args.seq_len
            opt.zero_grad()
            loss.backward()
            opt.step()
        if (epoch + 1) % args.eval_every == 0 or epoch + 1 == args.epochs:
            with torch.no_grad():
                logits = model(xva.to(dev))
                acc = sum((logits[j].argmax(-1).cpu() == yva[:, j]).float().mean().item()
                          for j in range(args.seq_len)) / args.seq_len
            print(f"  gap={gap:3d} epoch={epoch + 1:3d} loss={loss.item():.3f} acc={acc:.3f}", flush=True)
            if acc >= 0.99:
                break
    return acc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gaps", default="0,8,16,32,48,64,96,128")
    ap.add_argument("--pe", choices=["none", "sin", "rope"], default="none")
    ap.add_argument("--task", choices=["gap", "selective"], default="gap")
    ap.add_argument("--epochs", type=int, default=80)
    ap.add_argument("--eval-every", type=int, default=20)
    ap.add_argument("--seq-len", type=int, default=3)
    ap.add_argument("--n-train", type=int, default=8000)
    ap.add_argument("--n-val", type=int, default=2000)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    print(f"receptive field {CYCLES * KSIZE * LAYERS} positions, pe={args.pe}, task={args.task}")
    results = {}
    for gap in (int(v) for v in args.gaps.split(",")):
        results[gap] = run_gap(gap, args, dev)
        print(f"gap={gap:3d} FINAL acc={results[gap]:.3f}")
    if args.out:
        json.dump(results, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
