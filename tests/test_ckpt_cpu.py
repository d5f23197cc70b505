"""Checkpoint IO on CPU: the single-file format (reference: scripts/training.py:318-339) and the sharded format
with re-slicing for another world size. The sharded tests build the engine's flat groups for several "ranks" in
one process (no collectives are involved in saving or loading) and compare parameters and AdamW moments."""

import copy
import types

import pytest
import torch

from gdnet_b200.model import GDNet
from gdnet_b200.runtime.ckpt import CheckpointError, load_ckpt, load_sharded, save_ckpt, save_sharded
from gdnet_b200.train.engine import TrainEngine, _Group


def _model(seed=0):
    torch.manual_seed(seed)
    return GDNet(vocab_size=64, d_embed=32, d=32, n_layers=2, n_cycles=1, kernel_size=3, chunk_size=16, n_slots=4)


def test_single_file_round_trip_with_extra(tmp_path):
    m = _model(0)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3)
    m(torch.randint(0, 64, (2, 16)))[0].sum().backward()
    opt.step()
    extra = {"phase": 1, "windows_done": 1234, "rng": torch.get_rng_state()}
    save_ckpt(tmp_path / "a.pt", 7, m, opt, None, extra)
    assert not (tmp_path / "a.pt.tmp").exists()
    m2 = _model(1)
    opt2 = torch.optim.AdamW(m2.parameters(), lr=1e-3)
    step, got = load_ckpt(tmp_path / "a.pt", m2, opt2)
    assert step == 7 and got["phase"] == 1 and got["windows_done"] == 1234 and torch.equal(got["rng"], extra["rng"])
    for (n1, a), (n2, b) in zip(m.state_dict().items(), m2.state_dict().items()):
        assert n1 == n2 and torch.equal(a, b), n1
    s1, s2 = opt.state_dict()["state"], opt2.state_dict()["state"]
    assert s1.keys() == s2.keys()
    for k in s1:
        assert torch.equal(s1[k]["exp_avg"], s2[k]["exp_avg"]) and torch.equal(s1[k]["exp_avg_sq"], s2[k]["exp_avg_sq"])


def test_single_file_keys_are_the_references(tmp_path):
    """The saved model keys are the reference's parameter names (gdnet/model.py, gdnet/layer.py, gdnet/memory.py,
    gdnet/operators.py); spot-check the ones that differ most from a plain module tree."""
    m = _model(0)
    save_ckpt(tmp_path / "a.pt", 0, m)
    keys = set(torch.load(tmp_path / "a.pt", weights_only=True)["model"])
    for k in ("embed.weight", "head.weight", "proj_in.weight", "norm_out.weight", "layers.0.conv_fwd.conv.weight",
              "layers.1.rb_W1.weight", "layers.0.gf_norm.weight", "cam.W_r1.weight_orig", "cam.W_r1.weight_u",
              "cam.W_r1.weight_v", "cam.rho", "trans_ops.W", "trans_ops.log_tau", "trans_ops.router.weight"):
        assert k in keys, k


def test_truncated_single_file_raises_clear_error(tmp_path):
    m = _model(0)
    save_ckpt(tmp_path / "a.pt", 3, m)
    raw = (tmp_path / "a.pt").read_bytes()
    (tmp_path / "cut.pt").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(CheckpointError, match="truncated or corrupt"):
        load_ckpt(tmp_path / "cut.pt", _model(1))
    with pytest.raises(CheckpointError, match="missing"):
        load_ckpt(tmp_path / "nope.pt", _model(1))


def _fake_rank_engine(model, world, rank, shard_moments):
    """The engine's flat groups as rank ``rank`` of ``world`` would build them, without a process group."""
    by_dtype = {}
    for p in model.parameters():
        by_dtype.setdefault(p.dtype, []).append(p)
    groups = []
    for dt, ps in by_dtype.items():
        g = _Group(ps, dt, torch.device("cpu"), world, rank, False, None)
        if shard_moments:      # what the symmetric-memory modes do: moments for this rank's shard only
            g.m, g.v = torch.zeros(g.per), torch.zeros(g.per)
            g.mv_range = g.shard
        groups.append(g)
    eng = types.SimpleNamespace(groups=groups, rank=rank, world=world, step_count=0, lr=1e-3, module=model)
    return eng


def _fill(engines):
    """Same parameters on all ranks, moments that are a known function of the flat index."""
    for eng in engines:
        for gi, g in enumerate(eng.groups):
            lo, hi = g.mv_range
            idx = torch.arange(lo, hi, dtype=torch.float32)
            g.m.copy_(idx * 0.5 + gi)
            g.v.copy_(idx * 0.25 + 10 * gi)
        eng.step_count, eng.lr = 11, 3e-4


def _full_moments(engines):
    """name -> (m, v) per parameter, assembled from all ranks."""
    out = {}
    names = {id(p): n for n, p in engines[0].module.named_parameters()}
    for gi, g0 in enumerate(engines[0].groups):
        m_full, v_full = torch.zeros(g0.n), torch.zeros(g0.n)
        for eng in engines:
            g = eng.groups[gi]
            lo, hi = g.mv_range
            m_full[lo:hi], v_full[lo:hi] = g.m[: hi - lo], g.v[: hi - lo]
        for p, o in zip(g0.params, g0.offsets):
            out[names[id(p)]] = (m_full[o : o + p.numel()].clone(), v_full[o : o + p.numel()].clone())
    return out


@pytest.mark.parametrize("new_world", [1, 4])
def test_sharded_save_on_two_ranks_loads_on_one_and_four(tmp_path, new_world):
    base = _model(0)
    old = [_fake_rank_engine(copy.deepcopy(base), 2, r, True) for r in range(2)]
    _fill(old)
    for eng in old:
        save_sharded(tmp_path / "ck", 42, eng, {"windows_done": 99})
    want_p = {n: p.detach().clone() for n, p in old[0].module.named_parameters()}
    want_mv = _full_moments(old)

    new = [_fake_rank_engine(_model(5), new_world, r, new_world > 1) for r in range(new_world)]
    for eng in new:
        step, extra = load_sharded(tmp_path / "ck", eng)
        assert step == 42 and extra == {"windows_done": 99} and eng.step_count == 11 and eng.lr == 3e-4
    for eng in new:
        for n, p in eng.module.named_parameters():
            assert torch.equal(p.detach(), want_p[n]), n
    got_mv = _full_moments(new)
    for n, (m, v) in want_mv.items():
        assert torch.equal(got_mv[n][0], m) and torch.equal(got_mv[n][1], v), n


def test_truncated_or_missing_shard_raises_clear_error(tmp_path):
    base = _model(0)
    old = [_fake_rank_engine(copy.deepcopy(base), 2, r, True) for r in range(2)]
    _fill(old)
    for eng in old:
        save_sharded(tmp_path / "ck", 1, eng)
    f = tmp_path / "ck" / "shard_00001.pt"
    raw = f.read_bytes()
    f.write_bytes(raw[: len(raw) // 3])
    with pytest.raises(CheckpointError, match="shard_00001.pt.*truncated or corrupt"):
        load_sharded(tmp_path / "ck", _fake_rank_engine(_model(1), 1, 0, False))
    f.unlink()
    with pytest.raises(CheckpointError, match="missing"):
        load_sharded(tmp_path / "ck", _fake_rank_engine(_model(1), 1, 0, False))
    (tmp_path / "ck" / "manifest.json").unlink()
    with pytest.raises(CheckpointError, match="manifest"):
        load_sharded(tmp_path / "ck", _fake_rank_engine(_model(1), 1, 0, False))


def test_sharded_load_rejects_another_model(tmp_path):
    eng = _fake_rank_engine(_model(0), 1, 0, False)
    save_sharded(tmp_path / "ck", 1, eng)
    torch.manual_seed(0)
    other = GDNet(vocab_size=64, d_embed=32, d=32, n_layers=3, n_cycles=1, kernel_size=3, chunk_size=16, n_slots=4)
    with pytest.raises(CheckpointError, match="disagree on the parameters"):
        load_sharded(tmp_path / "ck", _fake_rank_engine(other, 1, 0, False))


def test_engine_optimizer_state_guards():
    eng = TrainEngine(_model(0), precision="bf16")
    sd = eng.state_dict_optim()
    eng.load_state_dict_optim(sd)
    bad = dict(sd, world=2)
    with pytest.raises(ValueError, match="sharded checkpoint"):
        eng.load_state_dict_optim(bad)
    bad = dict(sd, m=[m[:-1] for m in sd["m"]])
    with pytest.raises(ValueError, match="moments"):
        eng.load_state_dict_optim(bad)
