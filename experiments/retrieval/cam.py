"""Two small content-addressed memories compared by the retrieval experiment.

``ContentCAM`` scores a slot by tag similarity alone; ``PosGateCAM`` adds the input-conditioned
position term ``alpha * <sigmoid(W_pos q), e_s>`` with learned slot embeddings that decay with slot
age (reference: experiments/retrieval/cam.py:8-131). Both blend the retrieved vector into the
forward stream through a gate that starts mostly closed. ``entropy_gate=True`` also feeds the
normalised retrieval entropy to that gate (the second version of the experiment, reference:
experiments/retrieval_v2/run.py:137-186). The scoring / softmax / read-out is the framework's
``fused_mem_read`` op, so on a GPU the experiment runs the same kernel as the full model.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from gdnet_b200.ops import functional as ops


class ContentCAM(nn.Module):
    uses_position = False

    def __init__(self, d: int, d_sig: int, d_c: int, n_slots: int, entropy_gate: bool = False):
        super().__init__()
        self.n_slots, self.d_sig, self.d_c, self.entropy_gate = n_slots, d_sig, d_c, entropy_gate
        self.W_tag = nn.Linear(d, d_sig, bias=False)
        self.W_c = nn.Linear(d, d_c, bias=False)
        self.W_up = nn.Linear(d_c, d, bias=False)
        self.W_r1 = nn.utils.spectral_norm(nn.Linear(3 * d + (1 if entropy_gate else 0), d))
        self.W_r2 = nn.Linear(d, d)
        self.r_norm = nn.RMSNorm(d)
        nn.init.normal_(self.W_r2.weight, std=0.01)
        nn.init.constant_(self.W_r2.bias, -2.0)

    def write(self, tag_input, val_input, buffer_tags, buffer_vals):
        """Shift every slot one place older and store the new (tag, value) in slot 0."""
        tags = torch.cat([self.W_tag(tag_input).unsqueeze(1), buffer_tags[:, :-1]], dim=1)
        vals = torch.cat([self.W_c(val_input).detach().unsqueeze(1), buffer_vals[:, :-1]], dim=1)
        return tags, vals

    def _position_terms(self, q):
        gamma = torch.zeros_like(q)
        e = torch.zeros(self.n_slots, self.d_sig, dtype=q.dtype, device=q.device)
        return gamma, e, torch.zeros(1, dtype=q.dtype, device=q.device)

    def read(self, fwd, side, buffer_tags, buffer_vals):
        """Returns (blended stream, gate R, retrieval weights w)."""
        q = self.W_tag(fwd[:, -1])
        gamma, e, alpha = self._position_terms(q)
        out_c, w = ops.fused_mem_read(q, gamma, e, buffer_tags, buffer_vals, alpha)
        retrieved = self.W_up(out_c).unsqueeze(1).expand_as(fwd)
        parts = [side, fwd, retrieved]
        if self.entropy_gate:
            h = -(w * (w + 1e-8).log()).sum(-1) / math.log(self.n_slots)
            parts.append(h.view(-1, 1, 1).expand(-1, fwd.shape[1], 1).to(fwd.dtype))
        R = torch.sigmoid(self.r_norm(self.W_r2(F.silu(self.W_r1(torch.cat(parts, dim=-1))))))
        return fwd * (1 - R) + retrieved * R, R, w


class PosGateCAM(ContentCAM):
    uses_position = True

    def __init__(self, d: int, d_sig: int, d_c: int, n_slots: int, entropy_gate: bool = False, decay: float = 0.85):
        super().__init__(d, d_sig, d_c, n_slots, entropy_gate)
        self.W_slot = nn.Embedding(n_slots, d_sig)
        self.W_pos = nn.Linear(d_sig, d_sig, bias=False)
        nn.init.zeros_(self.W_pos.weight)                  # gamma starts at 0.5 everywhere
        self.rho = nn.Parameter(torch.zeros(1))
        with torch.no_grad():
            self.W_slot.weight.mul_(decay ** torch.arange(n_slots, dtype=torch.float32).unsqueeze(1))

    def _position_terms(self, q):
        return torch.sigmoid(self.W_pos(q)), self.W_slot.weight, torch.exp(self.rho)
