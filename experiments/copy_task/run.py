"""Copy-with-gap: where does GDNet's recall fall off relative to its receptive field?

    python experiments/copy_task/run.py [--gaps 0,8,16,32,48,64,96,128] [--epochs 80]
                                        [--task gap|selective] [--out results.json]

Task (reference: experiments/copy_task/dataset.py): ``seq_len`` signal tokens (ids 0..9), ``gap`` noise
tokens (ids 10..49), then a recall token (50); the model must name the signal tokens from the
representation at the recall position (one linear head per signal position). ``selective`` interleaves
distractors between the signal tokens. Model: GDNet d=64, 3 layers, 3 cycles, k=7, so the receptive
field is 3*7*3 = 63 positions; the reference reports accuracy 1.0 up to gap 64 and a cliff after
(experiments/copy_task/CONCLUDE.md). ``run_sin.py`` and ``run_rope.py`` repeat the sweep with position
information added (sinusoidal codes in the side streams, rotary conv inputs) and share this harness.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(_HERE)))
sys.path.insert(0, _HERE)

from dataset import VOCAB_SIZE, CopyWithGapDataset, SelectiveCopyDataset  # noqa: E402

from gdnet_b200.model import GDNet  # noqa: E402

D, LAYERS, CYCLES, KSIZE = 64, 3, 3, 7
RECEPTIVE_FIELD = CYCLES * KSIZE * LAYERS


def make_net(T: int, cls=GDNet) -> GDNet:
    return cls(VOCAB_SIZE, D, D, LAYERS, n_cycles=CYCLES, chunk_size=T, kernel_size=KSIZE)


class CopyProbe(nn.Module):
    """A GDNet trunk read at the recall position by one classifier per signal position
    (reference: experiments/copy_task/run.py:44-78, which taps ``norm_out`` with a forward hook)."""

    def __init__(self, net: GDNet, seq_len: int):
        super().__init__()
        self.net = net
        self.heads = nn.ModuleList([nn.Linear(D, VOCAB_SIZE) for _ in range(seq_len)])

    def forward(self, tokens):
        fwd, _, _ = self.net.trunk(tokens)
        rep = self.net.norm_out(fwd)[:, -1]
        return [h(rep) for h in self.heads]


def metrics(logits, targets):
    """(mean per-token accuracy, fraction of samples with every token right)."""
    pred = torch.stack([l.argmax(-1) for l in logits], dim=1)
    hit = pred == targets
    return hit.float().mean().item(), hit.all(dim=1).float().mean().item()


def train_gap(net_factory, gap, args, dev, label=""):
    """Train one probe at one gap; returns (token accuracy, exact-match accuracy) on held-out data."""
    g = torch.Generator().manual_seed(args.seed)
    ds_cls = SelectiveCopyDataset if args.task == "selective" else CopyWithGapDataset
    train, val = ds_cls(args.n_train, args.seq_len, gap, generator=g), ds_cls(args.n_val, args.seq_len, gap, generator=g)
    model = CopyProbe(net_factory(train.inputs.shape[1]), args.seq_len).to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    acc = exact = 0.0
    for epoch in range(args.epochs):
        perm = torch.randperm(len(train), generator=g)
        for i in range(0, len(train), args.batch):
            idx = perm[i : i + args.batch]
            x, y = train.inputs[idx].to(dev), train.targets[idx].to(dev)
            logits = model(x)
            loss = sum(F.cross_entropy(logits[j], y[:, j]) for j in range(args.seq_len)) / args.seq_len
            opt.zero_grad()
            loss.backward()
            opt.step()
        if (epoch + 1) % args.eval_every == 0 or epoch + 1 == args.epochs:
            with torch.no_grad():
                acc, exact = metrics(model(val.inputs.to(dev)), val.targets.to(dev))
            print(f"  {label}gap={gap:3d} epoch={epoch + 1:3d} loss={loss.item():.3f} acc={acc:.3f} exact={exact:.3f}",
                  flush=True)
            if acc >= 0.99:
                break
    return acc, exact


def add_common_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--gaps", default="0,8,16,32,48,64,96,128")
    ap.add_argument("--task", choices=["gap", "selective"], default="gap")
    ap.add_argument("--epochs", type=int, default=80)
    ap.add_argument("--eval-every", type=int, default=20)
    ap.add_argument("--seq-len", type=int, default=3)
    ap.add_argument("--n-train", type=int, default=8000)
    ap.add_argument("--n-val", type=int, default=2000)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="")


def compare(variants: dict, args) -> dict:
    """Run the gap sweep for every named net factory and print a table (used by the PE variants)."""
    dev = torch.device(args.device)
    print(f"receptive field {RECEPTIVE_FIELD} positions; expected cliff near gap {RECEPTIVE_FIELD - args.seq_len}")
    results: dict = {name: {} for name in variants}
    for gap in (int(v) for v in args.gaps.split(",")):
        for name, factory in variants.items():
            results[name][gap] = train_gap(factory, gap, args, dev, label=f"[{name}] ")
    print("gap  " + "  ".join(f"{n:>14s}" for n in variants))
    for gap in results[next(iter(variants))]:
        print(f"{gap:3d}  " + "  ".join(f"{results[n][gap][0]:.3f} / {results[n][gap][1]:.3f}" for n in variants))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(results, f, indent=1)
    return results


def main():
    ap = argparse.ArgumentParser()
    add_common_args(ap)
    compare({"gdnet": make_net}, ap.parse_args())


if __name__ == "__main__":
    main()
