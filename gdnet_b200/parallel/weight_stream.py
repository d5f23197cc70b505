"""Fully sharded layer weights: every matrix has one owner rank, the others pull what a layer step needs.

This is the parameter side of the full-shard engine (``TrainEngine(shard="full")``; the reference's counterpart
is the per-``GDLayer`` FSDP wrap of gdnet/utils/distributed.py:112-178, whose unshard hooks never fire
because ``GDNet`` calls ``layer.fwd_step`` / ``bwd_step`` instead of ``layer(...)``).

* The eight large matrices of a layer (``{gf,gb,rf,rb}_{W1,W2}``) are spread over the ranks, whole matrices,
  balanced by size. A rank keeps bf16 masters, fp32 gradients and AdamW moments only for what it owns.
* After every optimizer update the owner derives the operands the GEMMs read from its masters, once: for the
  recovery MLP the e4m3 copies in both layouts with packed power-of-two block scales, for the gate MLP the
  norm-folded ``W2``. They live in a symmetric arena that every rank has mapped.
* A layer step asks for its set of operands (``acquire``). Operands owned by this rank are used in place; the
  others are copied from the owners' memory into a local staging slot by *gather jobs*. The jobs do not get a
  kernel of their own: they ride on the tensor-core GEMMs (``csrc/gemm_sm100.cu``: the second CTA of every
  pair has a warp that issues no MMAs; it runs ``run_gather_jobs``), so the NVLink transfer overlaps the math.
* The order in which sets are asked for is the same in every training step. It is recorded during the first
  step; from then on the GEMMs of a step carry the jobs of the *next* set into the other staging slot
  (prefetch), and a set that was not prefetched (first of a pass, evaluation, a change of order) is gathered by
  the first GEMM of its own step, whose producer warp waits for the per-128-row counters of its own B operand
  before each tile (bounded wait).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import cuda as cu
from .symm import SymmBuffer, max_allreduce_

BF16, F32, FP8 = torch.bfloat16, torch.float32, torch.float8_e4m3fn
JOB_BYTES = 64 * 1024       # a range is cut into jobs of at most this size (many jobs keep every gather warp busy)
CARRIERS = 4                # GEMMs over which the jobs of a prefetched set are spread


def _align(n: int, a: int = 1024) -> int:
    return -(-n // a) * a


class LayerSet:
    """What one layer step reads: the two recovery matrices (FP8) and the two gate matrices (bf16)."""

    def __init__(self, rW1, rW2, gW1, gW2, gnw):
        self.rW1, self.rW2, self.gW1, self.gW2, self.gnw = rW1, rW2, gW1, gW2, gnw


class Operands:
    """Result of ``acquire``: tensors a layer step hands to its GEMMs."""

    __slots__ = ("q1", "p1", "q2", "p2", "gW1", "W2w", "gW2")


class WeightStream:
    def __init__(self, group, device, sharded_group, layer_sets):
        """``sharded_group``: the engine's group of sharded parameters (owners, flat offsets, symmetric master
        buffer); ``layer_sets``: one :class:`LayerSet` per (layer, step direction)."""
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.g = sharded_group
        self.sets = {s.rW1.data_ptr(): s for s in layer_sets}
        self.info = sharded_group.index           # id(param) -> (owner, flat offset)

        # ---- arena plan: compute copies of every FP8 matrix and the folded W2 of every gate, per owner -------
        offs = [0] * self.world
        self.arena_off: dict[tuple[int, str], int] = {}

        def take(owner, nbytes):
            o = offs[owner]
            offs[owner] += _align(nbytes)
            return o

        for s in layer_sets:
            for w in (s.rW1, s.rW2):
                N, Kd = w.shape
                owner = self._owner(w)
                nbk = (N // 128) * (Kd // 128)
                for part, nb in (("q", N * Kd), ("p", nbk * 512), ("qt", N * Kd), ("pt", nbk * 512)):
                    self.arena_off[(id(w), part)] = take(owner, nb)
            self.arena_off[(id(s.gW2), "w2w")] = take(self._owner(s.gW2), s.gW2.numel() * 2)
        self.arena = SymmBuffer(max(max(offs), 1024), group, device)

        # ---- staging: two slots that hold one set each, plus the counters of the self-gathered B operand ------
        need = 0
        for s in layer_sets:
            fwd = sum(_align(w.numel()) + _align((w.shape[0] // 128) * (w.shape[1] // 128) * 512) for w in (s.rW1, s.rW2))
            gate = _align(s.gW1.numel() * 2) + 2 * _align(s.gW2.numel() * 2)
            need = max(need, fwd + gate)
        self.slot_bytes = need
        self.slots = [torch.empty(need, dtype=torch.uint8, device=device) for _ in range(2)]
        self.plans: dict = {}
        self.scratch_s: dict = {}
        self.order: list = []
        self.recording: list | None = []
        self.pos = 0
        self.cur_slot = 0
        self.prefetched = None          # (set key, mode, slot) whose jobs have been handed to carriers
        self.pending: list = []         # job slices not yet attached to a GEMM
        self.pending_ready = None       # (b_ready, sfb_ready, b_target, sfb_target) for the first carrier
        self.recording = []
        self._token = torch.zeros(1, dtype=F32, device=device)
        self.gathered_bytes = 0
        self.arena.barrier()
        self.refresh()

    # ---- ownership ------------------------------------------------------------------------------------------
    def _owner(self, w) -> int:
        return self.info[id(w)][0]

    def _master_ptr(self, w, rank) -> int:
        """Address of ``w``'s bf16 master in its owner's shard, as mapped into this process."""
        owner, off = self.info[id(w)]
        return self.g._sp.ptrs[owner] + (off - owner * self.g.per) * 2

    def _arena_view(self, w, part, shape, dtype):
        o = self.arena_off[(id(w), part)]
        n = 1
        for d in shape:
            n *= d
        item = torch.empty((), dtype=dtype).element_size()
        return self.arena.local[o : o + n * item].view(dtype).view(shape)

    # ---- owner side: derive the GEMM operands from the masters, once per update ---------------------------
    def refresh(self) -> None:
        """Collective. Every rank re-derives the operands of the matrices it owns, then all ranks exchange one
        flag (bounded wait) so that no rank gathers before its peers' copies are complete."""
        for s in self.sets.values():
            for w in (s.rW1, s.rW2):
                if self._owner(w) != self.rank:
                    continue
                N, Kd = w.shape
                nb, kb = N // 128, Kd // 128
                key = (nb, kb)
                sc = self.scratch_s.get(key)
                if sc is None:
                    sc = (torch.empty(nb, kb, dtype=F32, device=self.device), torch.empty(kb, nb, dtype=F32, device=self.device))
                    self.scratch_s[key] = sc
                cu.K.quant_tile(w.detach(), False, self._arena_view(w, "q", (N, Kd), FP8), sc[0], cu.Q_BLOCK,
                                self._arena_view(w, "qt", (Kd, N), FP8), sc[1], cu.Q_BLOCK, True,
                                self._arena_view(w, "p", (nb, kb, 512), torch.uint8),
                                self._arena_view(w, "pt", (kb, nb, 512), torch.uint8))
            if self._owner(s.gW2) == self.rank:
                cu.K.scale_cols(s.gW2.detach(), cu.f32(s.gnw), self._arena_view(s.gW2, "w2w", tuple(s.gW2.shape), BF16))
        max_allreduce_(self._token, self.group)
        self._flush()                   # (jobs handed out are always run: the counters count every table run)
        self.prefetched = None

    # ---- plans: job tables of a set for a slot --------------------------------------------------------------
    def _plan(self, key, mode, slot):
        pk = (key, mode, slot)
        plan = self.plans.get(pk)
        if plan is not None:
            return plan
        s = self.sets[key]
        base = self.slots[slot].data_ptr()
        jobs: list[tuple[int, int, int, int]] = []
        ops = Operands()
        off = 0
        counters: list[tuple[str, int, int]] = []       # (operand, first counter index, chunks)
        n_counters = 0
        layout = []

        def add(name, w, part, shape, dtype, chunk_rows_bytes, flagged):
            """One operand: local view when owned, else a staging range plus its jobs."""
            nonlocal off, n_counters
            owner = self._owner(w)
            n = 1
            for d in shape:
                n *= d
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            if owner == self.rank:
                if part == "master":
                    t = w.detach()
                else:
                    t = self._arena_view(w, part, shape, dtype)
                layout.append((name, t, None))
                return
            src = self._master_ptr(w, owner) if part == "master" else self.arena.ptrs[owner] + self.arena_off[(id(w), part)]
            dst_off = off
            off += _align(nbytes)
            t = self.slots[slot][dst_off : dst_off + nbytes].view(dtype).view(shape)
            chunks = nbytes // chunk_rows_bytes if flagged else 1
            cb = chunk_rows_bytes if flagged else nbytes
            first = n_counters
            if flagged:
                n_counters += chunks
            subs = -(-cb // JOB_BYTES)
            for c in range(chunks):
                for j in range(subs):
                    lo = c * cb + j * JOB_BYTES
                    hi = min(c * cb + cb, lo + JOB_BYTES)
                    jobs.append((src + lo, base + dst_off + lo, (first + c) if flagged else -1, (hi - lo) // 16))
            layout.append((name, t, (first, chunks, subs) if flagged else None))

        def fp8(prefix, w, transposed, flagged):
            N, Kd = w.shape
            rows, cols = (Kd, N) if transposed else (N, Kd)
            add(prefix + "q", w, "qt" if transposed else "q", (rows, cols), FP8, 128 * cols, flagged)
            add(prefix + "p", w, "pt" if transposed else "p", (rows // 128, cols // 128, 512), torch.uint8,
                (cols // 128) * 512, flagged)

        if mode == "F":
            fp8("1", s.rW1, False, True)       # the first GEMM of a forward step reads this one: per-tile counters
            fp8("2", s.rW2, False, False)
            add("gW1", s.gW1, "master", tuple(s.gW1.shape), BF16, 0, False)
            add("W2w", s.gW2, "w2w", tuple(s.gW2.shape), BF16, 0, False)
        else:
            add("W2w", s.gW2, "w2w", tuple(s.gW2.shape), BF16, 0, False)
            add("gW2", s.gW2, "master", tuple(s.gW2.shape), BF16, 0, False)
            add("gW1", s.gW1, "master", tuple(s.gW1.shape), BF16, 0, False)
            fp8("2", s.rW2, True, False)
            fp8("1", s.rW1, True, False)
        if off > self.slot_bytes:
            raise RuntimeError("staging slot too small for a layer set")
        cnt = torch.zeros(max(n_counters, 1), dtype=torch.int32, device=self.device)
        cbase = cnt.data_ptr()
        table = None
        if jobs:
            table = torch.tensor([[a, b, (cbase + 4 * c) if c >= 0 else 0, n] for a, b, c, n in jobs], dtype=torch.int64,
                                 device=self.device)
        for name, t, _ in layout:
            setattr(ops, {"1q": "q1", "1p": "p1", "2q": "q2", "2p": "p2"}.get(name, name), t)
        if mode == "F":
            ops.gW2 = None
        ready = None
        flagged = {name: f for name, _, f in layout if f is not None}
        if "1q" in flagged and "1p" in flagged:
            fq, fp_ = flagged["1q"], flagged["1p"]
            ready = (cnt[fq[0] : fq[0] + fq[1]], cnt[fp_[0] : fp_[0] + fp_[1]], fq[2], fp_[2])
        plan = {"ops": ops, "table": table, "counters": cnt, "ready": ready, "uses": 0,
                "bytes": sum(j[3] for j in jobs) * 16}
        self.plans[pk] = plan
        return plan

    # ---- consumer side --------------------------------------------------------------------------------------
    def owns(self, rW1) -> bool:
        return rW1.data_ptr() in self.sets

    def acquire(self, rW1, mode: str) -> Operands:
        """The operands of the layer step whose first recovery matrix is ``rW1``; ``mode`` "F" (forward: row-major
        e4m3 copies) or "B" (backward: transposed e4m3 copies plus the raw gate ``W2``)."""
        key = rW1.data_ptr()
        want = (key, mode)
        if self.recording is not None:
            self.recording.append(want)
        predicted = self.order and self.pos < len(self.order) and self.order[self.pos] == want
        hit = self.prefetched is not None and self.prefetched[:2] == want
        self._flush()                   # jobs of this set that found no carrier run now, in stream order
        if hit:
            slot = self.prefetched[2]
            plan = self._plan(key, mode, slot)
        else:
            slot = 1 - self.cur_slot
            plan = self._plan(key, mode, slot)
            if plan["table"] is not None:
                # gathered by the first GEMM of this very step; in a forward step that GEMM reads the first
                # operand while it arrives, so it gets the counters to wait on
                plan["uses"] += 1
                self.gathered_bytes += plan["bytes"]
                self.pending = [plan["table"]]
                if plan["ready"] is not None:
                    br, sr, sq, sp = plan["ready"]
                    self.pending_ready = (br, sr, plan["uses"] * sq, plan["uses"] * sp)
        self.cur_slot = slot
        self.prefetched = None
        if predicted:
            self.pos += 1
            if self.pos < len(self.order):
                nk, nm = self.order[self.pos]
                nplan = self._plan(nk, nm, 1 - slot)
                if nplan["table"] is not None:
                    nplan["uses"] += 1
                    self.gathered_bytes += nplan["bytes"]
                    t = nplan["table"]
                    per = -(-t.shape[0] // CARRIERS)
                    self.pending += [t[i : i + per] for i in range(0, t.shape[0], per)]
                self.prefetched = (nk, nm, 1 - slot)
        elif self.order:
            self.order = []             # the order changed: stop predicting until it has been recorded again
            if self.recording is None:
                self.recording = [want]
        return plan["ops"]

    def attach(self) -> None:
        """Called right before a tensor-core GEMM is launched: hand it the next slice of pending jobs."""
        if self.pending:
            cu.K.attach_gather_jobs(self.pending.pop(0))
            if self.pending_ready is not None:
                cu.K.attach_b_ready(*self.pending_ready)
                self.pending_ready = None

    def settle(self) -> None:
        """For a step whose first GEMM cannot wait for operands that are still arriving (it is not the block-scaled
        FP8 GEMM): the jobs of the current set that were meant to ride on that GEMM run now, as a launch of their
        own; jobs that prefetch the next set stay pending."""
        if self.pending_ready is not None:
            cu.K.gather_jobs(self.pending.pop(0))
            self.pending_ready = None

    def _flush(self) -> None:
        while self.pending:
            cu.K.gather_jobs(self.pending.pop(0))
        self.pending_ready = None

    def end_step(self) -> None:
        """End of a training step (after the update and ``refresh``): restart the prediction."""
        self._flush()
        if self.recording is not None and self.recording:
            self.order = self.recording
        self.recording = None if self.order else []
        self.pos = 0
        self.prefetched = None
