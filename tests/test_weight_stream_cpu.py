"""The request / prefetch state machine of the weight stream (gdnet_b200/parallel/weight_stream.py) on CPU: plans
and kernel calls are replaced by recorders, so only the bookkeeping runs (which set is gathered by which GEMM, what is
prefetched, what a step without an FP8 first GEMM settles before its GEMMs, how a changed order is handled)."""

import types

import pytest
import torch

from gdnet_b200.parallel import weight_stream as ws_mod


class _Rec:
    def __init__(self):
        self.calls = []

    def attach_gather_jobs(self, t):
        self.calls.append(("attach", int(t[0, 0]), t.shape[0]))

    def attach_b_ready(self, *a):
        self.calls.append(("ready", a[2], a[3]))

    def gather_jobs(self, t):
        self.calls.append(("launch", int(t[0, 0]), t.shape[0]))


class _Key:
    """Stands in for a parameter: ``acquire`` only asks for its ``data_ptr``."""

    def __init__(self, k):
        self.k = k

    def data_ptr(self):
        return self.k


def _stream(monkeypatch, remote=True):
    rec = _Rec()
    monkeypatch.setattr(ws_mod, "cu", types.SimpleNamespace(K=rec))
    st = object.__new__(ws_mod.WeightStream)
    st.order, st.pos, st.cur_slot = [], 0, 0
    st.prefetched, st.pending, st.pending_ready, st.recording, st.gathered_bytes = None, [], None, [], 0
    st.plans = {}

    def plan(key, mode, slot):
        pk = (key, mode, slot)
        if pk not in st.plans:
            table = torch.full((8, 4), key * 10 + (0 if mode == "F" else 1), dtype=torch.int64) if remote else None
            ready = ("b", "s", 3, 2) if (remote and mode == "F") else None
            st.plans[pk] = {"ops": (key, mode, slot), "table": table, "ready": ready, "uses": 0, "bytes": 100}
        return st.plans[pk]

    st._plan = plan
    return st, rec


def _run_step(st, requests, gemms_per_step=3, settle=()):
    got = []
    for key, mode in requests:
        got.append(st.acquire(_Key(key), mode))
        if (key, mode) in settle:
            st.settle()
        for _ in range(gemms_per_step):
            st.attach()
    st.end_step()
    return got


def test_first_step_gathers_every_set_in_its_own_step(monkeypatch):
    st, rec = _stream(monkeypatch)
    reqs = [(1, "F"), (2, "F"), (2, "B"), (1, "B")]
    ops = _run_step(st, reqs)
    assert [o[:2] for o in ops] == reqs
    # nothing is predicted yet: every set rides on the first GEMM of its own step, forward sets with the counters to wait on
    assert [c for c in rec.calls if c[0] != "ready"] == [("attach", 10, 8), ("attach", 20, 8), ("attach", 21, 8), ("attach", 11, 8)]
    assert [c for c in rec.calls if c[0] == "ready"] == [("ready", 3, 2), ("ready", 3, 2)]
    assert st.order == reqs and st.gathered_bytes == 400


def test_later_steps_prefetch_the_next_set(monkeypatch):
    st, rec = _stream(monkeypatch)
    reqs = [(1, "F"), (2, "F"), (2, "B"), (1, "B")]
    _run_step(st, reqs)
    rec.calls.clear()
    ops = _run_step(st, reqs, gemms_per_step=6)
    # the first set of the step is gathered by its own first GEMM; every later one arrives as CARRIERS slices on the
    # GEMMs of the step before it, into the other staging slot
    first = rec.calls[0]
    assert first == ("attach", 10, 8) and rec.calls[1][0] == "ready"
    slices = [c for c in rec.calls[2:] if c[0] == "attach"]
    assert [c[1] for c in slices] == [20] * ws_mod.CARRIERS + [21] * ws_mod.CARRIERS + [11] * ws_mod.CARRIERS
    assert sum(c[2] for c in slices if c[1] == 20) == 8
    assert not [c for c in rec.calls if c[0] == "launch"]
    slots = [o[2] for o in ops]
    assert all(a != b for a, b in zip(slots, slots[1:])), "consecutive sets must use different staging slots"


def test_too_few_gemms_flush_the_rest_as_a_launch(monkeypatch):
    st, rec = _stream(monkeypatch)
    reqs = [(1, "F"), (2, "F")]
    _run_step(st, reqs)
    rec.calls.clear()
    _run_step(st, reqs, gemms_per_step=2)          # own table + one slice ride; the other slices find no carrier
    launched = [c for c in rec.calls if c[0] == "launch"]
    assert launched and all(c[1] == 20 for c in launched)
    assert sum(c[2] for c in rec.calls if c[1] == 20) == 8, "every job of the prefetched set ran exactly once"


def test_settle_runs_the_own_gather_before_a_step_without_an_fp8_first_gemm(monkeypatch):
    st, rec = _stream(monkeypatch)
    reqs = [(1, "F"), (2, "F")]
    _run_step(st, reqs, settle={(1, "F")})
    # the set of the settled step never reaches a GEMM with counters to wait on: it ran as a launch of its own
    assert rec.calls[0] == ("launch", 10, 8)
    assert ("ready", 3, 2) in rec.calls and rec.calls.index(("ready", 3, 2)) > 1      # the second step's, not the first's
    rec.calls.clear()
    _run_step(st, reqs, settle={(1, "F")}, gemms_per_step=6)
    assert rec.calls[0] == ("launch", 10, 8)
    # the prefetch of the next set still rides on the settled step's GEMMs
    assert [c[1] for c in rec.calls[1:] if c[0] == "attach"] == [20] * ws_mod.CARRIERS
    assert not [c for c in rec.calls if c[0] == "ready"]


def test_a_changed_order_stops_the_prediction_until_it_is_recorded_again(monkeypatch):
    st, rec = _stream(monkeypatch)
    _run_step(st, [(1, "F"), (2, "F"), (3, "F")])
    rec.calls.clear()
    _run_step(st, [(1, "F"), (3, "F"), (2, "F")], gemms_per_step=6)      # e.g. an evaluation pass in between
    # set 2 had been prefetched for nothing; sets 3 and 2 are gathered in their own steps
    own = [c for c in rec.calls if c[0] == "attach" and c[2] == 8]
    assert [c[1] for c in own] == [10, 30, 20]
    assert st.order == [(3, "F"), (2, "F")], "recording restarts at the request that broke the prediction"
    _run_step(st, [(1, "F"), (3, "F"), (2, "F")], gemms_per_step=6)     # a whole step in the new order is recorded
    assert st.order == [(1, "F"), (3, "F"), (2, "F")]
    rec.calls.clear()
    _run_step(st, st.order, gemms_per_step=6)
    assert [c for c in rec.calls if c[0] == "attach" and c[2] < 8], "prefetching resumes once the new order is known"


def test_local_sets_need_no_jobs(monkeypatch):
    st, rec = _stream(monkeypatch, remote=False)
    _run_step(st, [(1, "F"), (2, "F")])
    _run_step(st, [(1, "F"), (2, "F")])
    assert rec.calls == [] and st.gathered_bytes == 0
