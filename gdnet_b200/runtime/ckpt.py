"""Checkpoints: the reference's single-file format plus a sharded format with reshard-on-load.

Single file (reference: scripts/training.py:318-339): ``torch.save({"step", "model", "optimizer",
"scheduler"})`` written by rank 0, loaded with ``weights_only=True``. Model keys are identical to
the reference's, so files move in both directions. Added here: ``extra`` (data cursor, RNG state)
so a resumed run continues the data stream instead of restarting it.

Sharded (``save_sharded`` / ``load_sharded``): every rank writes the pieces of the training engine's flat
parameter and AdamW-moment buffers that it holds (with several GPUs a rank holds the moments of its shard
only, and with ``shard="full"`` also only its own layer matrices), rank 0 writes a manifest that names every
parameter with its place in the flat layout. Loading goes through the parameter *names*: each saved piece is
cut along the parameters it covers and copied to wherever those parameters sit in the loading engine's
layout, as far as the loading rank holds them. A run can therefore resume on a different number of GPUs or
with a different sharding mode; one shard file is in memory at a time.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from ..train.step import unwrap


class CheckpointError(RuntimeError):
    """A checkpoint file is missing, truncated or does not match the model."""


def _invalidate_cuda_caches(model) -> None:
    """Parameters were written behind autograd's back: drop the derived copies (FP8 weights, fp32 vectors,
    folded gate matrices) that the CUDA ops cache per parameter version."""
    try:
        dev = next(unwrap(model).parameters()).device
    except StopIteration:
        return
    if dev.type == "cuda":
        from ..ops import cuda as cu

        cu.invalidate_param_caches()


def save_ckpt(path, step: int, model, optimizer=None, scheduler=None, extra: dict | None = None) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    payload = {"step": int(step), "model": unwrap(model).state_dict()}
    if optimizer is not None:
        payload["optimizer"] = optimizer.state_dict() if hasattr(optimizer, "state_dict") else optimizer
    if scheduler is not None:
        payload["scheduler"] = scheduler.state_dict()
    if extra:
        payload["extra"] = extra
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(payload, tmp)
    os.replace(tmp, path)  # a crash mid-write never leaves a truncated checkpoint under the final name


def _load_file(path):
    try:
        return torch.load(path, map_location="cpu", weights_only=True)
    except FileNotFoundError as exc:
        raise CheckpointError(f"checkpoint file {path} is missing") from exc
    except Exception as exc:      # truncated zip archive, bad pickle, ...
        raise CheckpointError(f"checkpoint file {path} cannot be read (truncated or corrupt): {exc}") from exc


def load_ckpt(path, model, optimizer=None, scheduler=None, strict: bool = True) -> tuple[int, dict]:
    ckpt = _load_file(path)
    if not isinstance(ckpt, dict) or "model" not in ckpt or "step" not in ckpt:
        raise CheckpointError(f"{path} is not a training checkpoint (no 'model' / 'step' entries)")
    unwrap(model).load_state_dict(ckpt["model"], strict=strict)
    if optimizer is not None and "optimizer" in ckpt and hasattr(optimizer, "load_state_dict"):
        optimizer.load_state_dict(ckpt["optimizer"])
    if scheduler is not None and "scheduler" in ckpt:
        scheduler.load_state_dict(ckpt["scheduler"])
    _invalidate_cuda_caches(model)
    return int(ckpt["step"]), ckpt.get("extra", {})


# -- sharded --------------------------------------------------------------------------------------

def flat_layout(engine) -> list[dict]:
    """Per engine group: every parameter's name, shape and flat offset, and the padded length."""
    out = []
    names = {id(p): n for n, p in unwrap(engine).named_parameters()}
    for g in engine.groups:
        out.append({
            "dtype": str(g.dtype).replace("torch.", ""),
            "numel": int(g.n),
            "params": [{"name": names[id(p)], "offset": int(o), "shape": list(p.shape), "numel": int(p.numel())}
                       for p, o in zip(g.params, g.offsets)],
        })
    return out


def reslice(total: int, rank: int, world: int, align: int = 128) -> tuple[int, int]:
    """``[lo, hi)`` of ``rank``'s share of a flat buffer of ``total`` elements cut into ``world`` aligned shards."""
    per = -(-total // world)
    per = -(-per // align) * align
    lo = min(rank * per, total)
    return lo, min(lo + per, total)


def _local_pieces(engine, g) -> dict:
    """What this rank contributes for group ``g``: the flat ranges it holds and their values."""
    p_lo, p_hi = g.p_range
    mv_lo, mv_hi = g.mv_range
    write_p = g.sharded or engine.rank == 0        # replicated parameters are written once, by rank 0
    p = g.flat[: p_hi - p_lo] if g.sharded else g.flat[p_lo:p_hi]
    if not write_p:
        p_lo = p_hi = 0
        p = g.flat[:0]
    return {"p_lo": int(p_lo), "p_hi": int(p_hi), "p": p.detach().cpu().clone(),
            "mv_lo": int(mv_lo), "mv_hi": int(mv_hi),
            "m": g.m[: mv_hi - mv_lo].detach().cpu().clone(), "v": g.v[: mv_hi - mv_lo].detach().cpu().clone()}


def save_sharded(directory, step: int, engine, extra: dict | None = None) -> None:
    """Every rank writes ``shard_{rank:05d}.pt``; rank 0 also writes the buffers and, last, ``manifest.json``.
    Collective only in the sense that every rank must call it (no communication happens)."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    rank, world = engine.rank, engine.world
    shard = {"rank": rank, "world": world, "groups": [_local_pieces(engine, g) for g in engine.groups]}
    tmp = d / f"shard_{rank:05d}.pt.tmp"
    torch.save(shard, tmp)
    os.replace(tmp, d / f"shard_{rank:05d}.pt")
    if rank == 0:
        buffers = {n: b.detach().cpu() for n, b in unwrap(engine).named_buffers()}
        torch.save(buffers, d / "buffers.pt")
        manifest = {"step": int(step), "world": world, "layout": flat_layout(engine),
                    "optim_step": engine.step_count, "lr": engine.lr, "extra": extra or {}}
        tmp = d / "manifest.json.tmp"
        tmp.write_text(json.dumps(manifest))
        os.replace(tmp, d / "manifest.json")


def _copy_overlap(src, src_lo, params, where, dst, dst_lo, dst_hi, dst_group) -> None:
    """``src`` holds the saved flat range ``[src_lo, src_lo + len(src))``. For every saved parameter inside it,
    copy the part that the destination range ``[dst_lo, dst_hi)`` of group ``dst_group`` holds."""
    src_hi = src_lo + src.numel()
    for prm in params:
        o, n = prm["offset"], prm["numel"]
        a, b = max(o, src_lo), min(o + n, src_hi)
        if a >= b:
            continue
        tgt = where.get(prm["name"])
        if tgt is None or tgt[0] != dst_group:
            continue
        new_off = tgt[1]
        # element range [a - o, b - o) of the parameter -> flat [new_off + a - o, new_off + b - o) of the new layout
        na, nb_ = new_off + (a - o), new_off + (b - o)
        ca, cb = max(na, dst_lo), min(nb_, dst_hi)
        if ca >= cb:
            continue
        dst[ca - dst_lo : cb - dst_lo].copy_(src[a - src_lo + (ca - na) : a - src_lo + (cb - na)])


def load_sharded(directory, engine) -> tuple[int, dict]:
    """Load a sharded checkpoint written with any world size and sharding mode into ``engine``."""
    d = Path(directory)
    try:
        manifest = json.loads((d / "manifest.json").read_text())
    except FileNotFoundError as exc:
        raise CheckpointError(f"{d} holds no manifest.json: not a sharded checkpoint, or its save did not finish") from exc
    except json.JSONDecodeError as exc:
        raise CheckpointError(f"{d / 'manifest.json'} is truncated or corrupt: {exc}") from exc
    old_world = int(manifest["world"])
    new_layout = flat_layout(engine)
    where = {prm["name"]: (gi, prm["offset"]) for gi, lay in enumerate(new_layout) for prm in lay["params"]}
    saved_names = {prm["name"] for lay in manifest["layout"] for prm in lay["params"]}
    if saved_names != set(where):
        missing, extra_ = sorted(set(where) - saved_names)[:5], sorted(saved_names - set(where))[:5]
        raise CheckpointError(f"checkpoint and model disagree on the parameters (missing {missing}, unexpected {extra_})")
    shapes = {prm["name"]: prm["shape"] for lay in new_layout for prm in lay["params"]}
    for lay in manifest["layout"]:
        for prm in lay["params"]:
            if list(prm["shape"]) != list(shapes[prm["name"]]):
                raise CheckpointError(f"shape of {prm['name']} differs: checkpoint {prm['shape']}, model {shapes[prm['name']]}")

    for g in engine.groups:           # ranges nothing is saved for (alignment padding) stay zero
        g.m.zero_()
        g.v.zero_()
    for r in range(old_world):
        sh = _load_file(d / f"shard_{r:05d}.pt")
        if not isinstance(sh, dict) or len(sh.get("groups", [])) != len(manifest["layout"]):
            raise CheckpointError(f"{d / f'shard_{r:05d}.pt'} does not match the manifest")
        for lay, part in zip(manifest["layout"], sh["groups"]):
            params = lay["params"]
            if "numel" not in params[0]:
                for prm in params:
                    n = 1
                    for s_ in prm["shape"]:
                        n *= s_
                    prm["numel"] = n
            for gi, g in enumerate(engine.groups):
                p_lo, p_hi = g.p_range
                mv_lo, mv_hi = g.mv_range
                dev = g.flat.device
                if part["p"].numel():
                    dst = g.flat[: p_hi - p_lo] if g.sharded else g.flat[p_lo:p_hi]
                    _copy_overlap(part["p"].to(dev), part["p_lo"], params, where, dst, p_lo, p_hi, gi)
                if part["m"].numel():
                    _copy_overlap(part["m"].to(dev), part["mv_lo"], params, where, g.m[: mv_hi - mv_lo], mv_lo, mv_hi, gi)
                    _copy_overlap(part["v"].to(dev), part["mv_lo"], params, where, g.v[: mv_hi - mv_lo], mv_lo, mv_hi, gi)
    buf_path = d / "buffers.pt"
    if buf_path.exists():
        bufs = _load_file(buf_path)
        for n, b in unwrap(engine).named_buffers():
            if n in bufs:
                b.copy_(bufs[n])
    engine.step_count = int(manifest["optim_step"])
    engine.lr = float(manifest["lr"])
    _invalidate_cuda_caches(engine)
    ws = getattr(engine, "weight_stream", None)
    if ws is not None:
        ws.refresh()          # owners re-derive the GEMM operands from the loaded masters (collective)
        ws.end_step()
    return int(manifest["step"]), manifest.get("extra", {})
