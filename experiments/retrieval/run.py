"""Key-value retrieval across chunks through the content-addressed memory.

    python experiments/retrieval/run.py [--condition 1|2|3|all] [--epochs 20] [--no-entropy-gate] [--no-pos-gate]

A sample is ``n_slots`` chunks followed by a query chunk (reference: experiments/retrieval/dataset.py):
a signal chunk starts ``[SIGNAL, key, value, noise...]``, the query chunk ``[QUERY, key, noise...]``.
Condition 1: one signal chunk, the rest noise (unique key). Condition 2: the same key twice with
different values, the later one must win (recency). Condition 3: no signal chunk; what is evaluated
is how closed the blend gate stays and how diffuse the retrieval is. Every chunk is encoded by a
small stack of GDLayers and its summary written into the CAM; the query chunk reads the CAM and a
linear head names the value. ``--no-pos-gate`` zeroes the positional term (content-only retrieval, the
reference's ContentCAM); the default is the input-conditioned position gate (PosGateCAM);
``--no-entropy-gate`` hides the retrieval entropy from the blend gate (the v1 experiment; v2 feeds it).
Reported per condition: accuracy, mean blend-gate value R, normalised retrieval entropy H.
"""

from __future__ import annotations

import argparse
import math
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gdnet_b200.layer import GDLayer  # noqa: E402
from gdnet_b200.memory import Memory  # noqa: E402
from gdnet_b200.ops import reference as ref  # noqa: E402

N_KEYS = N_VALUES = N_NOISE = 16
CHUNK = 16
NOISE0 = N_KEYS + N_VALUES
SIGNAL, QUERY = NOISE0 + N_NOISE, NOISE0 + N_NOISE + 1
VOCAB = QUERY + 1


def make_samples(n, n_slots, condition, gap=2, gen=None):
    chunks = torch.randint(NOISE0, NOISE0 + N_NOISE, (n, n_slots + 1, CHUNK), generator=gen)
    key = torch.randint(0, N_KEYS, (n,), generator=gen)
    val = torch.randint(0, N_VALUES, (n,), generator=gen)
    target = val.clone()
    rows = torch.arange(n)
    if condition in (1, 2):
        chunks[rows, 0, 0], chunks[rows, 0, 1], chunks[rows, 0, 2] = SIGNAL, key, N_KEYS + val
    if condition == 2:
        new = (val + torch.randint(1, N_VALUES, (n,), generator=gen)) % N_VALUES
        j = gap + 1
        chunks[rows, j, 0], chunks[rows, j, 1], chunks[rows, j, 2] = SIGNAL, key, N_KEYS + new
        target = new
    if condition == 3:
        target = torch.full((n,), -1)
    chunks[rows, n_slots, 0], chunks[rows, n_slots, 1] = QUERY, key
    return chunks, target


class ChunkEncoder(nn.Module):
    """A GDLayer stack without embeddings (reference: experiments/retrieval/model.py:10-23)."""

    def __init__(self, d, n_layers, k, n_cycles):
        super().__init__()
        self.layers = nn.ModuleList([GDLayer(d, k) for _ in range(n_layers)])
        self.n_cycles = n_cycles

    def forward(self, x):
        side = [torch.zeros_like(x) for _ in self.layers]
        for _ in range(self.n_cycles):
            for i, layer in enumerate(self.layers):
                x, side[i] = layer.fwd_step(x, side[i])
            for i in range(len(self.layers) - 1, -1, -1):
                x, side[i] = self.layers[i].bwd_step(x, side[i])
        return x, side


class RetrievalModel(nn.Module):
    def __init__(self, d=64, n_slots=8, pos_gate=True, entropy_gate=True):
        super().__init__()
        self.embed = nn.Embedding(VOCAB, d)
        self.enc = ChunkEncoder(d, 2, 4, 2)
        self.cam = Memory(d, d // 4, d // 8, n_slots, CHUNK)
        self.head = nn.Linear(d, N_VALUES)
        self.pos_gate, self.entropy_gate, self.n_slots = pos_gate, entropy_gate, n_slots
        self.last_R = self.last_H = None

    def forward(self, chunks):
        B, C, T = chunks.shape
        # all context chunks are encoded in one batched call (the reference's retrieval note: ~4x faster
        # than a per-chunk loop), then written in order
        ctx, _ = self.enc(self.embed(chunks[:, :-1].reshape(B * (C - 1), T)))
        ctx_fwd = ctx.view(B, C - 1, T, -1)
        tags = torch.zeros(B, self.n_slots, self.cam.d_sig)
        vals = torch.zeros(B, self.n_slots, self.cam.d_c)
        for j in range(C - 1):
            tags, vals = self.cam.write(ctx_fwd[:, j, -1], ctx_fwd[:, j].mean(1), tags, vals)
        fwd, side = self.enc(self.embed(chunks[:, -1]))
        cam = self.cam
        q = cam.W_tag(fwd[:, 1])                       # the key sits at position 1 of the query chunk
        gamma = torch.sigmoid(cam.W_pos(q))
        alpha = cam._alpha() if self.pos_gate else cam.rho * 0.0
        out_c, w = ref.fused_mem_read(q, gamma, cam.W_slot.weight, tags, vals, alpha)
        retrieved = cam.W_up(out_c)
        h = ref.retrieval_entropy(w, self.n_slots)
        h_in = h if self.entropy_gate else torch.zeros_like(h)
        R = cam._blend_gate(side[0], fwd, retrieved, h_in)
        mixed = fwd * (1 - R) + retrieved.unsqueeze(1) * R
        self.last_R, self.last_H = R.mean().item(), h.mean().item()
        return self.head(mixed[:, 1])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--condition", default="all")
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--n-train", type=int, default=4000)
    ap.add_argument("--n-slots", type=int, default=8)
    ap.add_argument("--no-pos-gate", action="store_true")
    ap.add_argument("--no-entropy-gate", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    torch.manual_seed(args.seed)
    g = torch.Generator().manual_seed(args.seed)
    model = RetrievalModel(n_slots=args.n_slots, pos_gate=not args.no_pos_gate, entropy_gate=not args.no_entropy_gate)
    opt = torch.optim.Adam(model.parameters(), lr=2e-3)
    train = [make_samples(args.n_train // 2, args.n_slots, c, gen=g) for c in (1, 2)]
    x = torch.cat([t[0] for t in train])
    y = torch.cat([t[1] for t in train])
    for epoch in range(args.epochs):
        perm = torch.randperm(len(x), generator=g)
        for i in range(0, len(x), 64):
            idx = perm[i : i + 64]
            loss = F.cross_entropy(model(x[idx]), y[idx])
            opt.zero_grad()
            loss.backward()
            opt.step()
        print(f"epoch {epoch + 1}: loss {loss.item():.3f}", flush=True)
    conds = (1, 2, 3) if args.condition == "all" else (int(args.condition),)
    model.eval()
    with torch.no_grad():
        for c in conds:
            xe, ye = make_samples(512, args.n_slots, c, gen=g)
            pred = model(xe).argmax(-1)
            acc = (pred == ye).float().mean().item() if c != 3 else float("nan")
            print(f"C{c}: acc {acc:.3f}  R {model.last_R:.3f}  H {model.last_H:.3f}")


if __name__ == "__main__":
    main()
