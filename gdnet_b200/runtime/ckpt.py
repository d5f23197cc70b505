"""Checkpoints: the reference's single-file format plus a sharded format with reshard-on-load.

Single file (reference: scripts/training.py:318-339): ``torch.save({"step", "model", "optimizer",
"scheduler"})`` written by rank 0, loaded with ``weights_only=True``. Model keys are identical to
the reference's, so files move in both directions. Added here: ``extra`` (data cursor, RNG state)
so a resumed run continues the data stream instead of restarting it.

Sharded (``save_sharded`` / ``load_sharded``): every rank writes its slice of the engine's flat
parameter and AdamW-moment buffers, rank 0 writes a manifest with the flat layout. Loading
re-slices for the current world size, so a run can resume on a different number of GPUs.
"""

from __future__ import annotations

import json
import os
from pathlib import Path

import torch

from ..train.step import unwrap


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


def load_ckpt(path, model, optimizer=None, scheduler=None, strict: bool = True) -> tuple[int, dict]:
    ckpt = torch.load(path, map_location="cpu", weights_only=True)
    unwrap(model).load_state_dict(ckpt["model"], strict=strict)
    if optimizer is not None and "optimizer" in ckpt and hasattr(optimizer, "load_state_dict"):
        optimizer.load_state_dict(ckpt["optimizer"])
    if scheduler is not None and "scheduler" in ckpt:
        scheduler.load_state_dict(ckpt["scheduler"])
    return int(ckpt["step"]), ckpt.get("extra", {})


# -- sharded --------------------------------------------------------------------------------------

def flat_layout(engine) -> list[dict]:
    out = []
    names = {id(p): n for n, p in unwrap(engine).named_parameters()}
    for g in engine.groups:
        out.append({
            "dtype": str(g.dtype).replace("torch.", ""),
            "numel": int(sum(-(-p.numel() // 128) * 128 for p in g.params)),
            "params": [{"name": names[id(p)], "offset": int(o), "shape": list(p.shape)}
                       for p, o in zip(g.params, g.offsets)],
        })
    return out


def reslice(total: int, rank: int, world: int, align: int = 128) -> tuple[int, int]:
    per = -(-total // world)
    per = -(-per // align) * align
    lo = min(rank * per, total)
    return lo, min(lo + per, total)


def save_sharded(directory, step: int, engine, extra: dict | None = None) -> None:
    """Each rank writes ``shard_{rank:05d}.pt``; rank 0 also writes ``manifest.json`` and the buffers."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    rank, world = engine.rank, engine.world
    shard = {"rank": rank, "world": world, "groups": []}
    for g in engine.groups:
        total = int(sum(-(-p.numel() // 128) * 128 for p in g.params))
        lo, hi = reslice(total, rank, world)
        full_m = g.m.numel() == g.n  # moments cover the whole buffer (1 GPU / nccl) or only this rank's shard
        m = g.m[lo:hi] if full_m else g.m[: hi - lo]
        v = g.v[lo:hi] if full_m else g.v[: hi - lo]
        shard["groups"].append({"lo": lo, "hi": hi, "p": g.flat[lo:hi].cpu().clone(),
                                "m": m.cpu().clone(), "v": v.cpu().clone()})
    torch.save(shard, d / f"shard_{rank:05d}.pt")
    if rank == 0:
        buffers = {n: b.cpu() for n, b in unwrap(engine).named_buffers()}
        torch.save(buffers, d / "buffers.pt")
        manifest = {"step": int(step), "world": world, "layout": flat_layout(engine),
                    "optim_step": engine.step_count, "lr": engine.lr, "extra": extra or {}}
        (d / "manifest.json").write_text(json.dumps(manifest))


def load_sharded(directory, engine) -> tuple[int, dict]:
    """Load a sharded checkpoint written with any world size into ``engine`` (any world size)."""
    d = Path(directory)
    manifest = json.loads((d / "manifest.json").read_text())
    old_world = int(manifest["world"])
    shards = [torch.load(d / f"shard_{r:05d}.pt", map_location="cpu", weights_only=True) for r in range(old_world)]
    for gi, g in enumerate(engine.groups):
        lay = manifest["layout"][gi]
        if [p["name"] for p in lay["params"]] != [p["name"] for p in flat_layout(engine)[gi]["params"]]:
            raise ValueError("checkpoint and model disagree on the flat parameter layout")
        total = int(lay["numel"])
        p_full = torch.zeros(total, dtype=g.dtype)
        m_full, v_full = torch.zeros(total), torch.zeros(total)
        for sh in shards:
            part = sh["groups"][gi]
            p_full[part["lo"] : part["hi"]] = part["p"]
            m_full[part["lo"] : part["hi"]] = part["m"]
            v_full[part["lo"] : part["hi"]] = part["v"]
        g.flat[:total].copy_(p_full)
        if g.m.numel() == g.n:
            g.m[:total].copy_(m_full)
            g.v[:total].copy_(v_full)
        else:
            lo, hi = reslice(total, engine.rank, engine.world)
            g.m.zero_()
            g.v.zero_()
            g.m[: hi - lo].copy_(m_full[lo:hi])
            g.v[: hi - lo].copy_(v_full[lo:hi])
    buf_path = d / "buffers.pt"
    if buf_path.exists():
        bufs = torch.load(buf_path, map_location="cpu", weights_only=True)
        for n, b in unwrap(engine).named_buffers():
            if n in bufs:
                b.copy_(bufs[n])
    engine.step_count = int(manifest["optim_step"])
    engine.lr = float(manifest["lr"])
    return int(manifest["step"]), manifest.get("extra", {})
