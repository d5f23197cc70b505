"""Models of the retrieval experiment: a GDLayer stack as chunk encoder plus a pluggable memory."""

from __future__ import annotations

import torch
import torch.nn as nn

from cam import ContentCAM, PosGateCAM

from gdnet_b200.layer import GDLayer


class ChunkEncoder(nn.Module):
    """A GDLayer stack without embeddings (reference: experiments/retrieval/model.py:10-23): ``n_cycles``
    sweeps of forward steps up the stack and backward steps down it, side streams starting at zero."""

    def __init__(self, d: int, n_layers: int, kernel_size: int, n_cycles: int):
        super().__init__()
        self.layers = nn.ModuleList([GDLayer(d, kernel_size) for _ in range(n_layers)])
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
    """Encode every context chunk, fill the memory, read it from the query chunk, classify the value.

    All context chunks go through the encoder as one batch (the reference measured about 4x per epoch
    against a per-chunk loop, experiments/retrieval/CONCLUDE.md:60-64); their tags and values are laid out
    newest-first, which is what sequential writes would have produced (reference:
    experiments/retrieval/model.py:73-98).

    forward(chunks (B, n_chunks, T)) -> (logits (B, n_values), mean gate value at the last query token (B,),
    retrieval weights (B, n_slots)).
    """

    def __init__(self, vocab_size: int, n_values: int, d: int, d_sig: int, d_c: int, n_slots: int, n_layers: int,
                 kernel_size: int, n_cycles: int, use_pos_gate: bool, entropy_gate: bool = False):
        super().__init__()
        self.n_slots = n_slots
        self.embed = nn.Embedding(vocab_size, d)
        self.encoder = ChunkEncoder(d, n_layers, kernel_size, n_cycles)
        self.cam = (PosGateCAM if use_pos_gate else ContentCAM)(d, d_sig, d_c, n_slots, entropy_gate)
        self.norm = nn.RMSNorm(d)
        self.head = nn.Linear(d, n_values)

    def forward(self, chunks):
        B, n_chunks, T = chunks.shape
        n_write = n_chunks - 1
        ctx_fwd, ctx_side = self.encoder(self.embed(chunks[:, :n_write].reshape(B * n_write, T)))
        tag_in = ctx_fwd[:, -1].view(B, n_write, -1).flip(1)
        val_in = ctx_side[0].mean(1).view(B, n_write, -1).flip(1)
        tags, vals = self.cam.W_tag(tag_in), self.cam.W_c(val_in)
        fwd, side = self.encoder(self.embed(chunks[:, -1]))
        mixed, R, w = self.cam.read(fwd, side[0], tags, vals)
        return self.head(self.norm(mixed[:, -1])), R[:, -1].mean(-1), w
