"""The GDNet training step: task gradient plus a projected information gradient.

Parity with the reference's ``gdnet/loss.py`` (same function names and signatures).

One step computes two gradients of the same forward pass::

    g_task = d loss_task / d theta                      loss_task = CE(logits, targets)
    g_info = d (loss_info + loss_trans) / d theta       loss_info = prod_l mean(gate_l) (last cycle)
                                                                   + sn_soft_penalty
                                                                   + 0.1 * cam.recon_loss(mean_t side[0])
                                                        loss_trans = 0.1 * trans_ops.loss(z_t, z_t1)
    c      = <g_info, g_task> / max(<g_task, g_task>, 1e-8)
    grad   = g_task + beta * (g_info - c * g_task)

so the information gradient can only move the solution inside the task level set.

The reference runs three backward passes over the retained graph (task, info,
transition; gdnet/loss.py:168-219) and sums the last two into ``g_info``. Here the info
and transition losses are added *before* the backward, which gives the same ``g_info``
from two passes instead of three.

The generic implementation below works with any optimizer on CPU and GPU. The B200
training engine (``gdnet_b200.train.engine``) runs the same arithmetic on flat
parameter/gradient buffers with fused projection + AdamW kernels and the fused
gradient collective.
"""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import functional as ops
from ..ops import spectral
from ..utils.fp8 import Precision
from ..utils.fp8 import autocast as make_autocast

SN_ATTRS = ("gf_W1", "gb_W1", "rf_W1", "rb_W1")


def unwrap(model: nn.Module) -> nn.Module:
    """Strip DDP / compile / engine wrappers down to the GDNet."""
    for attr in ("module", "_orig_mod", "module"):
        model = getattr(model, attr, model)
    return model


def sn_soft_penalty(layers, scale: float = 0.1, generator: torch.Generator | None = None) -> torch.Tensor:
    """``scale * sum relu(sigma_hat - 1)^2`` over the four gate ``W1`` of every layer.

    ``sigma_hat = ||W v||`` for one fresh random unit ``v`` per matrix, in fp32
    (reference: gdnet/loss.py:15-31).
    """
    mats = [getattr(layer, a).weight for layer in layers for a in SN_ATTRS]
    if mats and getattr(mats[0], "_gd_owner", None) is not None:
        # matrices spread over the ranks (full-shard engine): every matrix is probed by its owner alone. The
        # ranks' gradients are averaged afterwards, so the owner's term counts `world` times to weigh the same
        # as in the replicated case, where every rank adds it.
        world = mats[0]._gd_world
        mats = [W for W in mats if W._gd_owner == W._gd_rank]
        if not mats:
            return torch.zeros((), device=layers[0].gf_norm.weight.device)
        scale = scale * world
    sig = spectral.sigma_estimates(mats, generator=generator)
    return scale * torch.relu(sig - 1.0).pow(2).sum()


def gate_info_loss_from_vals(gate_vals, n_layers: int) -> torch.Tensor:
    """Product over the last cycle's layers of the mean forward-gate value.

    Accepts gate tensors or their pre-reduced means (reference: gdnet/loss.py:34-51).
    """
    last_cycle = gate_vals[-n_layers:]
    return torch.stack([g.float().mean() for g in last_cycle]).prod()


@torch.no_grad()
def build_cam_buffer(model: nn.Module, write_chunks: torch.Tensor, sp_group=None, max_rows: int = 1 << 18):
    """Fill the CAM from the write chunks ``(B, n_write, T)``, in order, no graph.

    Only the chunk summary is needed, so the read-out (norm, projection, vocabulary
    GEMM) of these passes is skipped (reference: gdnet/loss.py:54-85 computes and
    discards the logits). Without the read-out the trunk does not look at the memory, so
    the chunks are independent until the write: they run through the trunk stacked on the
    batch dimension (as many at a time as ``max_rows`` token rows allow) and only the
    cheap slot writes happen one after the other.
    """
    raw = unwrap(model)
    B, n_write, T = write_chunks.shape
    dev = write_chunks.device
    tags = torch.zeros(B, raw.cam.n_slots, raw.cam.d_sig, device=dev)
    vals = torch.zeros(B, raw.cam.n_slots, raw.cam.d_c, device=dev)
    if not raw.cam_enabled:
        return tags, vals
    group = max(1, min(n_write, max_rows // max(1, B * T)))
    for g0 in range(0, n_write, group):
        n = min(group, n_write - g0)
        stacked = write_chunks[:, g0 : g0 + n].transpose(0, 1).reshape(n * B, T)      # chunk-major
        _, side, _, _, _, _, fwd_last = raw(stacked, None, None, sp_group=sp_group, need_logits=False)
        summary = side[0].mean(dim=1)
        if sp_group is not None and getattr(raw, "sp_state_carry", False) and dist.get_world_size(sp_group) > 1:
            # sequence parallel with state carry: every write chunk is one earlier sequence cut into shards; all of
            # its shards' summaries go into the memory, in order, on every rank
            from ..parallel.sp import gather_states

            states = gather_states(raw.cam.summary(fwd_last, summary), sp_group)       # (shards, n * B, d_sig + d_c)
            ds = raw.cam.d_sig
            for i in range(n):
                for r in range(states.shape[0]):
                    tags, vals = raw.cam.push(states[r, i * B : (i + 1) * B, :ds], states[r, i * B : (i + 1) * B, ds:], tags, vals)
            continue
        for i in range(n):
            tags, vals = raw.cam.write(fwd_last[i * B : (i + 1) * B], summary[i * B : (i + 1) * B], tags, vals)
    return tags, vals


def info_losses(base: nn.Module, side, gate_vals, accum_steps: int = 1):
    """``loss_info + loss_trans`` of one micro-batch (see the module docstring)."""
    loss = gate_info_loss_from_vals(gate_vals, base.n_layers)
    if len(base.layers) > 0:
        loss = loss + sn_soft_penalty(base.layers)
    side0 = side[0]
    if base.cam_enabled:
        loss = loss + 0.1 * base.cam.recon_loss(side0.mean(dim=1))
    T = side0.shape[1]
    if base.trans_enabled and T >= 2:
        mid = T // 2
        z_t = side0[:, :mid].mean(dim=1)
        z_t1 = side0[:, mid:].mean(dim=1).detach()
        loss = loss + 0.1 * base.trans_ops.loss(z_t, z_t1)
    return loss / accum_steps


def _dots(g_task, g_info):
    denom = torch.zeros((), device=g_task[0].device, dtype=torch.float32)
    num = torch.zeros((), device=g_task[0].device, dtype=torch.float32)
    for gt, gi in zip(g_task, g_info):
        gtf = gt.float()
        denom += gtf.pow(2).sum()
        num += (gi.float() * gtf).sum()
    return denom, num


def projected_step(
    model: nn.Module,
    params: list[nn.Parameter],
    optimizer: torch.optim.Optimizer,
    tokens: torch.Tensor,
    targets: torch.Tensor,
    beta: float = 0.1,
    scaler=None,
    precision: Precision = "bf16",
    write_chunks: torch.Tensor | None = None,
    sp_group=None,
    grad_clip: float = 0.0,
    accum_steps: int = 1,
    loss_mask: torch.Tensor | None = None,
) -> float:
    """One optimizer step; returns the task loss (reference: gdnet/loss.py:88-264).

    ``loss_mask`` (optional, ``(B, T)`` bool) drops positions from the task loss, e.g.
    targets that cross a document boundary in packed data.
    """
    engine = getattr(model, "projected_step", None)
    if engine is not None and getattr(model, "is_gdnet_engine", False):
        return engine(tokens, targets, beta=beta, write_chunks=write_chunks, grad_clip=grad_clip,
                      accum_steps=accum_steps, loss_mask=loss_mask)

    base = unwrap(model)
    no_sync = getattr(model, "no_sync", contextlib.nullcontext)
    B = tokens.shape[0]
    if B % accum_steps != 0:
        raise ValueError(f"batch size {B} not divisible by accum_steps {accum_steps}")
    mb = B // accum_steps
    dev_type = tokens.device.type

    g_task = [torch.zeros_like(p) for p in params]
    g_info = [torch.zeros_like(p) for p in params]
    total_loss = torch.zeros((), device=tokens.device)
    optimizer.zero_grad(set_to_none=True)

    def _bank(acc):
        for a, p in zip(acc, params):
            if p.grad is not None:
                a.add_(p.grad)
        optimizer.zero_grad(set_to_none=True)

    for i in range(accum_steps):
        sl = slice(i * mb, (i + 1) * mb)
        tok_i, tgt_i = tokens[sl], targets[sl]
        wc_i = write_chunks[sl] if write_chunks is not None else None
        with make_autocast(precision, dev_type):
            tags = vals = None
            if wc_i is not None and base.cam_enabled:
                tags, vals = build_cam_buffer(model, wc_i, sp_group=sp_group)
            logits, side, _, _, gate_vals, _, _ = model(
                tok_i, tags, vals, return_gates="mean", sp_group=sp_group
            )
            tgt_flat = tgt_i.reshape(-1)
            if loss_mask is not None:
                tgt_flat = torch.where(loss_mask[sl].reshape(-1), tgt_flat, torch.full_like(tgt_flat, -100))
            loss_task = ops.cross_entropy(logits.reshape(-1, logits.shape[-1]), tgt_flat) / accum_steps
        with no_sync():
            (scaler.scale(loss_task) if scaler else loss_task).backward(retain_graph=True)
        _bank(g_task)

        with make_autocast(precision, dev_type):
            loss_info = info_losses(base, side, gate_vals, accum_steps)
        with no_sync():
            (scaler.scale(loss_info) if scaler else loss_info).backward()
        _bank(g_info)
        total_loss += loss_task.detach().float()

    denom, num = _dots(g_task, g_info)
    distributed = dist.is_available() and dist.is_initialized()
    if distributed:
        both = torch.stack([denom, num])
        dist.all_reduce(both)
        denom, num = both[0], both[1]
    coef = num / denom.clamp(min=1e-8)
    for p, gt, gi in zip(params, g_task, g_info):
        p.grad = (gt + beta * (gi - coef.to(gt.dtype) * gt)).to(p.dtype)

    if distributed:
        world = dist.get_world_size()
        flat = torch.cat([p.grad.reshape(-1).float() for p in params])
        dist.all_reduce(flat)
        flat.div_(world)
        off = 0
        for p in params:
            n = p.numel()
            p.grad.copy_(flat[off : off + n].view_as(p.grad))
            off += n

    if grad_clip > 0.0:
        if scaler:
            scaler.unscale_(optimizer)
        torch.nn.utils.clip_grad_norm_(params, grad_clip)
    if scaler:
        scaler.step(optimizer)
        scaler.update()
    else:
        optimizer.step()
    return float(total_loss)
