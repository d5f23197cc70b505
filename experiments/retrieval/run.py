"""Key-value retrieval across chunks: content-only memory against the position-gated memory.

    python experiments/retrieval/run.py [--epochs 60] [--eval-every 10] [--device cpu] [--out curves.json]

Three conditions (``dataset.py``): C1 unique key (content retrieval), C2 the same key at two ages (the
newer value must win: needs a recency signal), C3 key never written (what matters is how far the blend
gate R stays shut and how diffuse the retrieval is). Both memories (``cam.py``) are trained on C1 + C2 and
evaluated on all three; per condition the script reports accuracy, mean R at the recall position and
the retrieval entropy ``-sum w log w`` (reference: experiments/retrieval/run.py:1-17, 85-200, which
reports ContentCAM ~0.48 and PosGateCAM 1.000 on C2). Curves go to a JSON file, and to a PNG beside it when
matplotlib is importable.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.nn.functional as F

_HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(_HERE)))
sys.path.insert(0, _HERE)

from dataset import CHUNK_SIZE, N_VALUES, VOCAB_SIZE, RetrievalDataset  # noqa: E402
from model import RetrievalModel  # noqa: E402

D, D_SIG, D_C, N_LAYERS, KERNEL_SIZE, N_CYCLES = 32, 8, 8, 1, 7, 2      # receptive field 14 of the 16-token chunk
AMBIGUOUS_K = 2


def entropy(w: torch.Tensor) -> torch.Tensor:
    return -(w * (w + 1e-8).log()).sum(-1)


def add_common_args(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--epochs", type=int, default=60)
    ap.add_argument("--eval-every", type=int, default=10)
    ap.add_argument("--n-train", type=int, default=10000)
    ap.add_argument("--n-val", type=int, default=2000)
    ap.add_argument("--n-slots", type=int, default=8)
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out", default="")


def make_sets(args, conditions, n, seed0, value_in_query=False):
    return {c: RetrievalDataset(n, args.n_slots, CHUNK_SIZE, c, AMBIGUOUS_K, seed0 + c, value_in_query)
            for c in conditions}


@torch.no_grad()
def evaluate(model, ds, dev):
    """(accuracy or nan, mean R, mean retrieval entropy) over a dataset; the model returns (logits, r, w)
    or (logits, w)."""
    model.eval()
    hits, rs, hs, n = 0.0, 0.0, 0.0, 0
    for i in range(0, len(ds), 256):
        x, y = ds.chunks[i : i + 256].to(dev), ds.targets[i : i + 256].to(dev)
        out = model(x)
        logits, w = out[0], out[-1]
        b = x.shape[0]
        hits += (logits.argmax(-1) == y).float().sum().item()
        rs += out[1].float().sum().item() if len(out) == 3 else float("nan")
        hs += entropy(w.float()).sum().item()
        n += b
    model.train()
    acc = hits / n if int(ds.targets[0]) >= 0 else float("nan")
    return acc, rs / n, hs / n


def fit(model, train_sets, val_sets, args, label=""):
    """Train on the concatenated training sets; returns the evaluation history."""
    dev = torch.device(args.device)
    model.to(dev)
    x = torch.cat([d.chunks for d in train_sets.values()])
    y = torch.cat([d.targets for d in train_sets.values()])
    g = torch.Generator().manual_seed(args.seed)
    opt = torch.optim.Adam(model.parameters(), lr=args.lr)
    hist: dict = {"epoch": []}
    for epoch in range(args.epochs):
        t0 = time.perf_counter()
        perm = torch.randperm(len(x), generator=g)
        for i in range(0, len(x), args.batch):
            idx = perm[i : i + args.batch]
            loss = F.cross_entropy(model(x[idx].to(dev))[0], y[idx].to(dev))
            opt.zero_grad()
            loss.backward()
            opt.step()
        if (epoch + 1) % args.eval_every == 0 or epoch + 1 == args.epochs:
            hist["epoch"].append(epoch + 1)
            line = f"{label}epoch={epoch + 1:3d} ({time.perf_counter() - t0:.1f}s/epoch)"
            for c, ds in val_sets.items():
                acc, r, h = evaluate(model, ds, dev)
                for k, v in (("acc", acc), ("r", r), ("h", h)):
                    hist.setdefault(f"c{c}_{k}", []).append(v)
                line += f"  C{c} acc={acc:.3f} R={r:.3f} H={h:.2f}"
            print(line, flush=True)
    return hist


def save_curves(results: dict, out: str) -> None:
    if not out:
        return
    with open(out, "w") as f:
        json.dump(results, f, indent=1)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return
    keys = sorted({k for h in results.values() for k in h if k != "epoch"})
    fig, axes = plt.subplots(1, len(keys), figsize=(3 * len(keys), 3))
    for ax, k in zip(axes, keys):
        for name, h in results.items():
            ax.plot(h["epoch"], h[k], label=name)
        ax.set_title(k)
    axes[0].legend()
    fig.tight_layout()
    fig.savefig(os.path.splitext(out)[0] + ".png", dpi=120)


def main():
    ap = argparse.ArgumentParser()
    add_common_args(ap)
    args = ap.parse_args()
    train = make_sets(args, (1, 2), args.n_train // 2, 0)
    val = make_sets(args, (1, 2, 3), args.n_val, 10)
    results = {}
    for name, pos_gate in (("ContentCAM", False), ("PosGateCAM", True)):
        torch.manual_seed(args.seed)
        model = RetrievalModel(VOCAB_SIZE, N_VALUES, D, D_SIG, D_C, args.n_slots, N_LAYERS, KERNEL_SIZE, N_CYCLES,
                               use_pos_gate=pos_gate)
        print(f"--- {name} ---")
        results[name] = fit(model, train, val, args)
    save_curves(results, args.out)


if __name__ == "__main__":
    main()
