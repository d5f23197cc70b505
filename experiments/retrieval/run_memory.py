"""The retrieval experiment on the framework's own ``Memory`` module, written to chunk by chunk.

    python experiments/retrieval/run_memory.py [--epochs 60] [--device cpu]

``run.py`` builds the tag / value buffers in one batched pass with the small memories of ``cam.py``. This
script checks the production path instead (reference: experiments/retrieval/run_memory.py:55-99): every
context chunk is encoded on its own and stored with ``Memory.write`` (shift + insert), the query chunk goes
through ``Memory.read`` (the fused read op, entropy-conditioned blend gate). Reported: C1 / C2 accuracy
and the retrieval entropy of all three conditions.
"""

from __future__ import annotations

import argparse

import torch
import torch.nn as nn

import run as base          # shared harness; puts the repo root and this folder on sys.path
from dataset import CHUNK_SIZE, N_VALUES, VOCAB_SIZE
from model import ChunkEncoder

from gdnet_b200.memory import Memory


class SequentialMemoryModel(nn.Module):
    """forward(chunks) -> (logits, retrieval weights)."""

    def __init__(self, vocab_size: int, n_values: int, d: int, d_sig: int, d_c: int, n_slots: int):
        super().__init__()
        self.n_slots, self.d_sig, self.d_c = n_slots, d_sig, d_c
        self.embed = nn.Embedding(vocab_size, d)
        self.encoder = ChunkEncoder(d, base.N_LAYERS, base.KERNEL_SIZE, base.N_CYCLES)
        self.cam = Memory(d, d_c, d_sig, n_slots, chunk_size=CHUNK_SIZE)
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, n_values)

    def forward(self, chunks):
        B, n_chunks, _ = chunks.shape
        tags = torch.zeros(B, self.n_slots, self.d_sig, device=chunks.device)
        vals = torch.zeros(B, self.n_slots, self.d_c, device=chunks.device)
        for j in range(n_chunks - 1):
            fwd, side = self.encoder(self.embed(chunks[:, j]))
            tags, vals = self.cam.write(fwd[:, -1], side[0].mean(1), tags, vals)
        fwd, side = self.encoder(self.embed(chunks[:, -1]))
        mixed, w = self.cam.read(fwd, side[0], tags, vals)
        return self.head(self.norm(mixed[:, -1])), w


def main():
    ap = argparse.ArgumentParser()
    base.add_common_args(ap)
    args = ap.parse_args()
    torch.manual_seed(args.seed)
    model = SequentialMemoryModel(VOCAB_SIZE, N_VALUES, base.D, base.D_SIG, base.D_C, args.n_slots)
    hist = base.fit(model, base.make_sets(args, (1, 2), args.n_train // 2, 0),
                    base.make_sets(args, (1, 2, 3), args.n_val, 10), args)
    base.save_curves({"Memory": hist}, args.out)


if __name__ == "__main__":
    main()
