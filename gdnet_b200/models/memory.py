"""Content-addressed memory (CAM) with an input-conditioned position gate.

Parity with the reference's ``gdnet/memory.py``: same parameters and names
(``W_tag, W_pos, W_slot, rho, W_c, W_d, W_up, W_r1 (spectral-normalised), W_r2,
r_norm``), same initialisation, same ``write`` / ``read`` / ``recon_loss``.

Retrieval for a batch row::

    q      = W_tag(fwd[:, -1])                 content query
    gamma  = sigmoid(W_pos q)                  position gate (0.5 at init: W_pos = 0)
    e_s    = W_slot[s]                         slot embedding, rows decayed by 0.85**s
    w      = softmax_s(<tags_s, q> + alpha <e_s, gamma>)
    out    = W_up(sum_s w_s vals_s)
    h      = H(w) / log(n_slots)               normalised retrieval entropy
    R      = sigmoid(r_norm(W_r2 silu(W_r1 [side, fwd, out, h])))
    fwd'   = fwd (1-R) + out R

``alpha`` is ``rho`` itself, not ``exp(rho)``: the reference passes the raw
parameter (gdnet/memory.py:125) although its docstring says ``exp(rho)``; with
``rho`` initialised to 0 the position term starts switched off. Kept for checkpoint
and loss-curve compatibility; ``alpha_mode="exp"`` selects the documented form.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..ops import reference as ref


class Memory(nn.Module):
    def __init__(self, d: int, d_c: int, d_sig: int, n_slots: int, chunk_size: int,
                 alpha_mode: str = "raw") -> None:
        super().__init__()
        assert alpha_mode in ("raw", "exp")
        self.d, self.d_c, self.d_sig = d, d_c, d_sig
        self.n_slots, self.chunk_size = n_slots, chunk_size
        self.alpha_mode = alpha_mode

        self.W_tag = nn.Linear(d, d_sig, bias=False)
        self.W_pos = nn.Linear(d_sig, d_sig, bias=False)
        nn.init.zeros_(self.W_pos.weight)
        self.W_slot = nn.Embedding(n_slots, d_sig)
        with torch.no_grad():
            decay = 0.85 ** torch.arange(n_slots, dtype=self.W_slot.weight.dtype)
            self.W_slot.weight.mul_(decay.unsqueeze(1))
        self.rho = nn.Parameter(torch.zeros(1))

        self.W_c = nn.Linear(d, d_c, bias=False)
        self.W_d = nn.Linear(d_c, d, bias=False)
        self.W_up = nn.Linear(d_c, d, bias=False)
        self.W_r1 = nn.utils.spectral_norm(nn.Linear(3 * d + 1, d))
        self.W_r2 = nn.Linear(d, d)
        self.r_norm = nn.RMSNorm(d)
        nn.init.normal_(self.W_r2.weight, std=0.01)
        nn.init.constant_(self.W_r2.bias, -2.0)

    # -- write ------------------------------------------------------------------------

    def write(self, tag_input, val_input, buffer_tags, buffer_vals):
        """Shift every slot one place towards the end and store the new chunk summary in
        slot 0 (reference: gdnet/memory.py:74-101)."""
        tag = self.W_tag(tag_input).to(buffer_tags.dtype)
        val = self.W_c(val_input).to(buffer_vals.dtype)
        new_tags = torch.cat([tag.unsqueeze(1), buffer_tags[:, :-1]], dim=1)
        new_vals = torch.cat([val.unsqueeze(1), buffer_vals[:, :-1]], dim=1)
        return new_tags, new_vals

    def push(self, tag, val, buffer_tags, buffer_vals):
        """The slot shift of :meth:`write` for an already projected ``(tag (B, d_sig), val (B, d_c))`` pair."""
        new_tags = torch.cat([tag.to(buffer_tags.dtype).unsqueeze(1), buffer_tags[:, :-1]], dim=1)
        new_vals = torch.cat([val.to(buffer_vals.dtype).unsqueeze(1), buffer_vals[:, :-1]], dim=1)
        return new_tags, new_vals

    @torch.no_grad()
    def summary(self, tag_input, val_input):
        """``[W_tag(tag_input) | W_c(val_input)]`` ``(B, d_sig + d_c)``: what :meth:`write` would store, as one
        vector (the state a sequence shard hands to the shards after it)."""
        return torch.cat([self.W_tag(tag_input).float(), self.W_c(val_input).float()], dim=-1)

    # -- read -------------------------------------------------------------------------

    def _alpha(self) -> torch.Tensor:
        return self.rho.exp() if self.alpha_mode == "exp" else self.rho

    def read(self, fwd, side, buffer_tags, buffer_vals):
        """Query the buffer, blend the retrieved vector into ``fwd``.

        Returns ``(fwd', w.detach())`` with ``w (B, n_slots)`` the retrieval weights
        (reference: gdnet/memory.py:103-139).
        """
        B, T, d = fwd.shape
        q = self.W_tag(fwd[:, -1, :])
        gamma = torch.sigmoid(self.W_pos(q))
        e = self.W_slot.weight
        retrieved_c, w = ops.fused_mem_read(q, gamma, e, buffer_tags, buffer_vals, self._alpha())
        retrieved = self.W_up(retrieved_c.to(q.dtype))
        h = ref.retrieval_entropy(w, self.n_slots).to(fwd.dtype)
        if fwd.is_cuda:
            from ..ops import cuda as cu

            if cu.cam_readout_ok(fwd, self.W_r2.weight):
                return self._read_out_cuda(cu, side, fwd, retrieved, h), w.detach()
        R = self._blend_gate(side, fwd, retrieved, h)
        rexp = retrieved.unsqueeze(1)
        return fwd * (1 - R) + rexp * R, w.detach()

    def _sn_weight(self):
        """``W_r1.weight`` after the spectral-norm pre-forward hook, run by hand: it refreshes ``weight`` from
        ``weight_orig`` (one power iteration in training mode), as a module call would."""
        w = self.W_r1.weight_orig
        if w.is_cuda and w.dtype in (torch.bfloat16, torch.float32):
            from ..ops import cuda as cu

            return cu.spectral_weight(self.W_r1)     # same arithmetic, one kernel for the iteration and sigma
        for hook in self.W_r1._forward_pre_hooks.values():
            hook(self.W_r1, None)
        return self.W_r1.weight

    def _read_out_cuda(self, cu, side, fwd, retrieved, h):
        """The blend on the sm_100a kernels (``ops/cuda.py:_CamReadoutFn``): the two token-sized blocks of
        ``W_r1`` and ``W_r2`` on the tensor-core GEMM, norm + sigmoid + blend in one kernel."""
        d = self.d
        W = self._sn_weight().to(fwd.dtype)
        row_bias = F.linear(retrieved, W[:, 2 * d : 3 * d]) + h.unsqueeze(1) * W[:, 3 * d] + self.W_r1.bias.to(fwd.dtype)
        eps = self.r_norm.eps if self.r_norm.eps is not None else ref.default_rms_eps(fwd.dtype)
        return cu.cam_readout(side, fwd, retrieved, row_bias, W[:, :d], W[:, d : 2 * d], self.W_r2.weight, self.W_r2.bias,
                              self.r_norm.weight, eps)

    def _blend_gate(self, side, fwd, retrieved, h):
        """``sigmoid(r_norm(W_r2 silu(W_r1 [side, fwd, retrieved, h])))``.

        ``retrieved`` and ``h`` are constant along T, so their share of ``W_r1`` is a
        per-row bias: only the ``[side, fwd]`` part is a token-sized GEMM and the
        ``(B, T, 3d+1)`` concatenation is never built.
        """
        d = self.d
        W = self._sn_weight().to(fwd.dtype)          # (d, 3d+1), already divided by sigma
        b = self.W_r1.bias.to(fwd.dtype)
        row_bias = F.linear(retrieved, W[:, 2 * d : 3 * d]) + h.unsqueeze(1) * W[:, 3 * d] + b
        pre = F.linear(side.to(fwd.dtype), W[:, :d]) + F.linear(fwd, W[:, d : 2 * d]) + row_bias.unsqueeze(1)
        z = self.W_r2(F.silu(pre))
        return torch.sigmoid(self.r_norm(z))

    def recon_loss(self, val_input: torch.Tensor) -> torch.Tensor:
        """MSE of the value auto-encoder ``W_d(W_c(v))`` against ``v``."""
        return F.mse_loss(self.W_d(self.W_c(val_input)), val_input)
