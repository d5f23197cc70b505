"""Transition operators over chunk summaries.

Parity with the reference's ``gdnet/operators.py``: a bank ``W (n_ops, d, d)`` of
near-identity linear maps, a bias-free router, and two learned log-temperatures.
``loss`` is InfoNCE across the batch for the softly-routed prediction of ``z_t1`` from
``z_t``, plus ``balance_coef * sum_m m log m`` on the mean routing weights (negative
entropy: pushes the router towards uniform use). Dense mixture; no token dispatch.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class TransitionOperators(nn.Module):
    def __init__(self, d: int, n_ops: int = 8, balance_coef: float = 0.01):
        super().__init__()
        self.n_ops, self.d, self.balance_coef = n_ops, d, balance_coef
        bank = torch.eye(d).expand(n_ops, d, d) + 0.01 * torch.randn(n_ops, d, d)
        self.W = nn.Parameter(bank.contiguous())
        self.router = nn.Linear(d, n_ops, bias=False)
        self.log_tau = nn.Parameter(torch.tensor(0.0))
        self.log_temp = nn.Parameter(torch.tensor(-2.66))

    def routing(self, z_t: torch.Tensor) -> torch.Tensor:
        """Soft assignment ``(B, n_ops)``; router temperature floored at 0.1."""
        tau = self.log_tau.exp().clamp(min=0.1)
        return F.softmax(self.router(z_t) / tau, dim=-1)

    def predict(self, z_t: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``sum_o w[b,o] W_o z_t[b]``: route first, then one batched matmul."""
        mixed = torch.einsum("bo,oij->bij", w, self.W.to(z_t.dtype))
        return torch.einsum("bij,bj->bi", mixed, z_t)

    def loss(self, z_t: torch.Tensor, z_t1: torch.Tensor) -> torch.Tensor:
        w = self.routing(z_t)
        z_pred = self.predict(z_t, w.to(z_t.dtype))
        temp = self.log_temp.exp().clamp(min=0.01)
        logits = F.normalize(z_pred, dim=-1) @ F.normalize(z_t1, dim=-1).t() / temp
        labels = torch.arange(z_t.shape[0], device=z_t.device)
        nce = F.cross_entropy(logits.float(), labels)
        mean_w = w.float().mean(dim=0)
        return nce + self.balance_coef * (mean_w * mean_w.log()).sum()

    @torch.no_grad()
    def winning_operator(self, z_t: torch.Tensor) -> torch.Tensor:
        return self.routing(z_t).argmax(dim=-1)
