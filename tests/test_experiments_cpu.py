"""The small-scale experiments: data layouts, model variants and one-epoch runs of every script on CPU."""

import importlib.util
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXP = os.path.join(ROOT, "experiments")


def _load(folder, name):
    """Import experiments/<folder>/<name>.py under a unique module name (two folders have a dataset.py)."""
    path = os.path.join(EXP, folder, name + ".py")
    spec = importlib.util.spec_from_file_location(f"exp_{folder}_{name}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_copy_datasets_layout():
    ds = _load("copy_task", "dataset")
    g = torch.Generator().manual_seed(0)
    d = ds.CopyWithGapDataset(32, seq_len=3, gap=5, generator=g)
    assert d.inputs.shape == (32, 9) and d.targets.shape == (32, 3)
    assert torch.equal(d.inputs[:, :3], d.targets) and int(d.targets.max()) < 10
    assert (d.inputs[:, 3:8] >= 10).all() and (d.inputs[:, 3:8] < 50).all()
    assert (d.inputs[:, -1] == ds.RECALL_TOKEN).all()
    s = ds.SelectiveCopyDataset(16, seq_len=3, gap=4, distractor_ratio=2, generator=g)
    assert s.inputs.shape == (16, 3 * 3 + 4 + 1)
    assert torch.equal(s.inputs[:, 0:9:3], s.targets)          # signal every third token
    assert (s.inputs[:, 1:9:3] >= 10).all() and (s.inputs[:, 2:9:3] >= 10).all()
    x, y = d[3]
    assert x.shape == (9,) and y.shape == (3,) and len(d) == 32


def test_retrieval_dataset_conditions():
    ds = _load("retrieval", "dataset")
    c1 = ds.RetrievalDataset(64, 8, condition=1, seed=1)
    assert c1.chunks.shape == (64, 9, 16)
    assert (c1.chunks[:, 0, 0] == ds.SIGNAL_TOKEN).all() and (c1.chunks[:, -1, 0] == ds.QUERY_TOKEN).all()
    assert torch.equal(c1.chunks[:, 0, 1], c1.chunks[:, -1, 1])                 # the query asks for the written key
    assert torch.equal(c1.chunks[:, 0, 2] - ds.VALUE_OFFSET, c1.targets)
    assert (c1.chunks[:, 1:-1] >= ds.NOISE_OFFSET).all() and (c1.chunks[:, 1:-1] < ds.SIGNAL_TOKEN).all()
    c2 = ds.RetrievalDataset(64, 8, condition=2, ambiguous_k=2, seed=2)
    old, new = c2.chunks[:, 0, 2] - ds.VALUE_OFFSET, c2.chunks[:, 3, 2] - ds.VALUE_OFFSET
    assert (c2.chunks[:, 3, 0] == ds.SIGNAL_TOKEN).all() and (old != new).all() and torch.equal(new, c2.targets)
    c3 = ds.RetrievalDataset(64, 8, condition=3, seed=3)
    assert (c3.targets == -1).all() and not (c3.chunks[:, :-1] == ds.SIGNAL_TOKEN).any()
    c3v = ds.RetrievalDataset(64, 8, condition=3, seed=3, value_in_query=True)
    assert torch.equal(c3v.chunks[:, -1, 2] - ds.VALUE_OFFSET, c3v.targets) and (c3v.targets >= 0).all()
    with pytest.raises(ValueError):
        ds.RetrievalDataset(4, 8, condition=4)


def test_rope_is_a_rotation_and_sin_codes():
    sys.path.insert(0, os.path.join(EXP, "copy_task"))
    try:
        rope_mod = _load("copy_task", "run_rope")
        sin_mod = _load("copy_task", "run_sin")
    finally:
        sys.path.remove(os.path.join(EXP, "copy_task"))
        sys.modules.pop("run", None)
        sys.modules.pop("dataset", None)
    x = torch.randn(2, 11, 16)
    y = rope_mod.rope(x)
    assert torch.allclose(y[:, 0], x[:, 0])                                     # position 0 is not rotated
    pair_norm = lambda t: (t[..., :8] ** 2 + t[..., 8:] ** 2)                   # noqa: E731
    assert torch.allclose(pair_norm(y), pair_norm(x), atol=1e-5)
    pe = sin_mod.sinusoidal_pe(7, 16, "cpu")
    assert pe.shape == (7, 16) and torch.allclose(pe[0, 0::2], torch.zeros(8)) and torch.allclose(pe[0, 1::2], torch.ones(8))
    assert torch.allclose(pe[3, 0], torch.sin(torch.tensor(3.0)))
    net = rope_mod.make_rope_net(12, hard_sn=True)
    fwd, _, _ = net.trunk(torch.randint(0, 52, (2, 12)))
    assert fwd.shape == (2, 12, 64) and torch.isfinite(fwd).all()


def test_position_gate_prefers_recent_slot():
    sys.path.insert(0, os.path.join(EXP, "retrieval"))
    try:
        cam = _load("retrieval", "cam")
    finally:
        sys.path.remove(os.path.join(EXP, "retrieval"))
    torch.manual_seed(0)
    m = cam.PosGateCAM(16, 4, 4, 6, entropy_gate=True)
    tags, vals = torch.zeros(3, 6, 4), torch.zeros(3, 6, 4)
    t2, v2 = m.write(torch.randn(3, 16), torch.randn(3, 16), tags, vals)
    assert t2.shape == tags.shape and (t2[:, 1:] == 0).all() and not (t2[:, 0] == 0).all()
    t3, _ = m.write(torch.randn(3, 16), torch.randn(3, 16), t2, v2)
    assert torch.equal(t3[:, 1], t2[:, 0])                                      # older entries move one slot back
    fwd, side = torch.randn(3, 5, 16), torch.randn(3, 5, 16)
    out, R, w = m.read(fwd, side, t3, v2)
    assert out.shape == fwd.shape and R.shape == fwd.shape and torch.allclose(w.sum(-1), torch.ones(3), atol=1e-5)
    assert float(R.mean()) < 0.5                                                # the gate starts mostly shut
    c = cam.ContentCAM(16, 4, 4, 6)
    _, _, wc = c.read(fwd, side, torch.zeros(3, 6, 4), vals)
    assert torch.allclose(wc, torch.full((3, 6), 1 / 6), atol=1e-6)             # no tags, no position term: uniform


SCRIPTS = [
    ("copy_task/run.py", ["--gaps", "4", "--n-train", "128", "--n-val", "32"]),
    ("copy_task/run_sin.py", ["--gaps", "4", "--n-train", "128", "--n-val", "32"]),
    ("copy_task/run_rope.py", ["--gaps", "4", "--n-train", "128", "--n-val", "32"]),
    ("retrieval/run.py", ["--n-train", "128", "--n-val", "32"]),
    ("retrieval/run_memory.py", ["--n-train", "128", "--n-val", "32"]),
    ("retrieval_v2/run.py", ["--n-train", "126", "--n-val", "32"]),
    ("grid/train.py", ["--steps", "20"]),
]


@pytest.mark.parametrize("script,extra", SCRIPTS, ids=[s for s, _ in SCRIPTS])
def test_script_runs_one_epoch(script, extra):
    cmd = [sys.executable, os.path.join(EXP, script), *extra]
    if not script.startswith("grid"):
        cmd += ["--epochs", "1", "--device", "cpu"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip()


def test_gpu_monitor_and_live_tables_with_a_fake_nvml():
    """The throughput sweep's GPU monitor only reads, and does so through a handful of NVML calls: run it against a
    stand-in, and render the tables as plain lines."""
    import io
    import types

    from gdnet_b200.runtime.monitor import GpuMonitor, LiveTables

    calls = []

    class FakeNvml:
        NVML_CLOCK_SM = 1

        def nvmlInit(self):
            calls.append("init")

        def nvmlDeviceGetCount(self):
            return 2

        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetUtilizationRates(self, h):
            return types.SimpleNamespace(gpu=90 + h, memory=10)

        def nvmlDeviceGetMemoryInfo(self, h):
            return types.SimpleNamespace(used=(40 + h) * 2**30, total=180 * 2**30)

        def nvmlDeviceGetPowerUsage(self, h):
            return 900_000

        def nvmlDeviceGetClockInfo(self, h, which):
            return 1700

        def __getattr__(self, name):          # anything that would change a setting is not part of the stand-in
            raise AssertionError(f"unexpected NVML call {name}")

    mon = GpuMonitor(period=0.01, nvml=FakeNvml())
    rows = mon.sample()
    assert [r["util"] for r in rows] == [90, 91] and rows[1]["mem_gib"] == 41.0 and rows[0]["sm_mhz"] == 1700
    mon.latest = rows
    buf = io.StringIO()
    t = LiveTables("sweep", mon, force_plain=True, stream=buf)
    t.add(dict(B=8, T=4096, ms=432.1, tok_s=75800.0, params=300.5e6, mem_gib=61.2))
    t.add(dict(B=64, T=8192, ms=float("nan"), tok_s=float("nan"), params=0, mem_gib=0.0, oom=True))
    t.close()
    text = buf.getvalue()
    assert "sweep" in text and "75,800" in text and "OOM" in text and "gpu 1: util 91 %" in text
