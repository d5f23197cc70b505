"""GDNet language model.

Parity with the reference's ``gdnet/model.py``: ``embed`` (vocabulary padded to a
multiple of 16) -> ``proj_in`` -> ``n_cycles`` x [all layers ``fwd_step`` ascending,
then all layers ``bwd_step`` descending] -> CAM read -> ``norm_out`` -> ``proj_out``
-> ``head`` (weight tied to ``embed``) -> slice to ``vocab_size``. ``forward``
returns the same 7-tuple; ``state_dict`` keys are identical, so checkpoints move in
both directions.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..ops import reference as ref
from .layer import GDLayer
from .memory import Memory as CAM
from .operators import TransitionOperators


class GDNet(nn.Module):
    """Gated Dissipative Network.

    Args mirror the reference (gdnet/model.py:35-72). ``cam_enabled`` and
    ``trans_enabled`` start True.
    """

    def __init__(
        self,
        vocab_size: int,
        d_embed: int,
        d: int,
        n_layers: int,
        n_cycles: int = 3,
        chunk_size: int = 512,
        d_c: int | None = None,
        d_sig: int | None = None,
        n_slots: int = 32,
        kernel_size: int = 7,
        n_ops: int = 8,
    ) -> None:
        super().__init__()
        d_c = d_c or d // 4
        d_sig = d_sig or d // 8
        vocab_padded = vocab_size + (-vocab_size % 16)

        self.embed = nn.Embedding(vocab_padded, d_embed)
        self.proj_in = nn.Linear(d_embed, d, bias=False)
        self.layers = nn.ModuleList([GDLayer(d, kernel_size) for _ in range(n_layers)])
        self.proj_out = nn.Linear(d, d_embed, bias=False)
        self.head = nn.Linear(d_embed, vocab_padded, bias=False)
        self.head.weight = self.embed.weight

        self.cam = CAM(d, d_c, d_sig, n_slots, chunk_size)
        self.trans_ops = TransitionOperators(d, n_ops)
        self.norm_out = nn.RMSNorm(d)

        self.vocab_size, self.vocab_padded = vocab_size, vocab_padded
        self.d, self.d_embed = d, d_embed
        self.n_layers, self.n_cycles = n_layers, n_cycles
        self.chunk_size, self.kernel_size = chunk_size, kernel_size
        self.cam_enabled = True
        self.trans_enabled = True
        # sequence parallel: a shard reads a memory that already holds the summaries of the shards before it, as if the
        # shards had been processed one after the other as chunks (False: every shard sees only the buffers it is
        # given, which is what the reference does, scripts/training.py:379)
        self.sp_state_carry = True

    # -- trunk ------------------------------------------------------------------------

    def _embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.proj_in(self.embed(tokens))

    def one_cycle(self, fwd, side, sp_group=None, gate_sink=None, gate_mode=True, cycle=0):
        """All layers forward-step in order, then backward-step in reverse order.

        ``gate_sink``: list receiving the forward-gate value of every layer.
        ``cycle`` only numbers the sequence-parallel halo slots.
        """
        L = len(self.layers)
        for i, layer in enumerate(self.layers):
            slot = (cycle * 2 * L + i) if sp_group is not None else None
            if gate_sink is not None:
                fwd, side[i], g = layer._step("fwd", fwd, side[i], sp_group, gate_mode, slot)
                gate_sink.append(g)
            else:
                fwd, side[i] = layer._step("fwd", fwd, side[i], sp_group, False, slot)
        for i in range(L - 1, -1, -1):
            slot = (cycle * 2 * L + L + i) if sp_group is not None else None
            fwd, side[i] = self.layers[i]._step("bwd", fwd, side[i], sp_group, False, slot)
        return fwd, side

    def trunk(self, tokens, return_gates: bool | str = False, sp_group=None):
        """Embedding plus all cycles. Returns ``(fwd, side, gate_vals)``."""
        B, T = tokens.shape
        fwd = self._embed(tokens)
        # every layer's side stream starts at zero (reference: gdnet/model.py:142-146); ``None`` says so to the first
        # forward step, which then leaves out the recovery gate (it only multiplies the side stream) instead of
        # reading a tensor of zeros
        if type(self).one_cycle is GDNet.one_cycle:
            side: list = [None for _ in self.layers]
        else:          # a subclass with its own cycle (the experiments add position codes to the side stream) gets tensors
            side = [torch.zeros(B, T, self.d, dtype=fwd.dtype, device=fwd.device) for _ in self.layers]
        gate_vals: list[torch.Tensor] = []
        for cyc in range(self.n_cycles):
            fwd, side = self.one_cycle(
                fwd, side, sp_group,
                gate_sink=gate_vals if return_gates else None,
                gate_mode=return_gates, cycle=cyc,
            )
        return fwd, side, gate_vals

    def features_from(self, fwd: torch.Tensor) -> torch.Tensor:
        """Input of the vocabulary projection: ``proj_out(norm_out(fwd))``."""
        eps = self.norm_out.eps if self.norm_out.eps is not None else ref.default_rms_eps(fwd.dtype)
        return self.proj_out(ops.rmsnorm(fwd, self.norm_out.weight, eps))

    def logits_from(self, fwd: torch.Tensor) -> torch.Tensor:
        return self.head(self.features_from(fwd))[..., : self.vocab_size]

    # -- public API -------------------------------------------------------------------

    def forward(self, tokens, buffer_tags=None, buffer_vals=None, return_gates: bool | str = False,
                sp_group=None, need_logits: bool | str = True):
        """Returns ``(logits, side, buffer_tags, buffer_vals, gate_vals, cam_weights, fwd_last)``.

        ``return_gates=True`` collects the forward-gate tensors ``(B,T,d)`` of every
        forward step (gradients flow through them); ``return_gates="mean"`` collects
        only their means (0-dim tensors), which is what the information loss needs.
        ``need_logits=False`` skips the read-out (logits is None) for callers that only
        want the chunk summary, e.g. the memory-filling passes; ``need_logits="features"`` returns
        the input of the vocabulary projection in place of the logits (the caller fuses the
        projection with the loss, ``ops.linear_cross_entropy``).
        """
        B, T = tokens.shape
        fwd, side, gate_vals = self.trunk(tokens, return_gates, sp_group)
        dtype, device = fwd.dtype, fwd.device
        if buffer_tags is None:
            buffer_tags = torch.zeros(B, self.cam.n_slots, self.cam.d_sig, dtype=dtype, device=device)
        if buffer_vals is None:
            buffer_vals = torch.zeros(B, self.cam.n_slots, self.cam.d_c, dtype=dtype, device=device)

        fwd_last = fwd[:, -1, :]
        cam_weights = None
        logits = None
        if need_logits and sp_group is not None and self.cam_enabled and self.sp_state_carry:
            buffer_tags, buffer_vals = self.carry_sp_state(fwd_last, side, buffer_tags, buffer_vals, sp_group)
        if need_logits:
            if self.cam_enabled:
                fwd, cam_weights = self.cam.read(fwd, side[0], buffer_tags, buffer_vals)
            # "features": stop before the vocabulary projection (the caller fuses it with the loss)
            logits = self.features_from(fwd) if need_logits == "features" else self.logits_from(fwd)
        return logits, side, buffer_tags, buffer_vals, gate_vals, cam_weights, fwd_last

    @torch.no_grad()
    def carry_sp_state(self, fwd_last, side, buffer_tags, buffer_vals, sp_group, upto: int | None = None):
        """Sequence parallel: write the chunk summaries of the shards before this one (all shards with
        ``upto="all"``) into the buffers, in shard order. Every shard computes its summary
        ``(W_tag fwd_last, W_c mean_t side[0])`` locally; one small all-gather hands them round."""
        import torch.distributed as dist

        from ..parallel.sp import gather_states

        n = dist.get_world_size(sp_group)
        if n == 1:
            return buffer_tags, buffer_vals
        states = gather_states(self.cam.summary(fwd_last, side[0].mean(dim=1)), sp_group)     # (n, B, d_sig + d_c)
        last = n if upto == "all" else dist.get_rank(sp_group)
        for r in range(last):
            buffer_tags, buffer_vals = self.cam.push(states[r, :, : self.cam.d_sig], states[r, :, self.cam.d_sig :],
                                                     buffer_tags, buffer_vals)
        return buffer_tags, buffer_vals

    def write_cam(self, fwd_last, side, buffer_tags, buffer_vals):
        """Store this chunk's summary ``(fwd_last, mean_t side[0])``; no-op when CAM is off."""
        if self.cam_enabled:
            buffer_tags, buffer_vals = self.cam.write(
                fwd_last, side[0].mean(dim=1), buffer_tags, buffer_vals
            )
        return buffer_tags, buffer_vals

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int = 200, top_p: float = 0.9,
                 temperature: float = 1.0, generator: torch.Generator | None = None):
        """Nucleus sampling, batch 1 (reference: gdnet/model.py:209-255).

        Every step re-runs the model on the last ``chunk_size`` ids; the CAM receives a
        chunk summary every ``chunk_size`` steps.
        """
        self.eval()
        device = next(self.parameters()).device
        ids = input_ids.to(device)
        tags = torch.zeros(1, self.cam.n_slots, self.cam.d_sig, device=device)
        vals = torch.zeros(1, self.cam.n_slots, self.cam.d_c, device=device)
        for step in range(max_new_tokens):
            ctx = ids[:, -self.chunk_size :]
            logits, side, tags, vals, _, _, fwd_last = self.forward(ctx, tags, vals)
            if step % self.chunk_size == 0:
                tags, vals = self.write_cam(fwd_last, side, tags, vals)
            next_id = ops.sample_top_p(logits[:, -1, :].float() / temperature, top_p, generator)
            ids = torch.cat([ids, next_id.view(1, 1)], dim=1)
        return ids
