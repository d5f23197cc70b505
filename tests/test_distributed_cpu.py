"""Host-side distributed logic on CPU ranks (gloo, world size 2 and 4): group construction, sequence
parallelism with the point-to-point halo transport, the generic distributed projected step, and
failure detection by heartbeats. No GPU involved."""

import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gdnet_b200.parallel import groups
from gdnet_b200.parallel.fsdp import shard_bounds
from gdnet_b200.parallel.sp import shard_range, shard_sequence
from gdnet_b200.runtime.watchdog import Heartbeat, Watchdog, find_stalled, find_stragglers, read_heartbeats


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    groups.init_distributed(backend="gloo", timeout_minutes=2)
    try:
        fn(rank, world, *args)
    finally:
        groups.destroy()


def _spawn(fn, world, *args):
    mp.spawn(_entry, args=(world, _free_port(), fn, args), nprocs=world, join=True)


def test_group_layout_pure():
    sp, dp = groups.sp_dp_ranks(8, 4)
    assert sp == [[0, 1, 2, 3], [4, 5, 6, 7]] and dp == [[0, 4], [1, 5], [2, 6], [3, 7]]
    with pytest.raises(ValueError):
        groups.sp_dp_ranks(6, 4)
    assert shard_range(64, 1, 4) == (16, 32)
    assert shard_sequence(torch.arange(12).view(1, 12), 2, 3).tolist() == [[8, 9, 10, 11]]
    lo, hi = shard_bounds(1000, 1, 4)
    assert lo % 128 == 0 and (lo, hi) == (256, 512)
    assert shard_bounds(1000, 3, 4) == (768, 1000)


def _groups_worker(rank, world):
    groups.init_process_groups(sp_size=2)
    sp, dp = groups.get_sp_group(), groups.get_dp_group()
    assert dist.get_world_size(sp) == 2 and dist.get_world_size(dp) == world // 2
    assert dist.get_rank(sp) == rank % 2 and dist.get_rank(dp) == rank // 2
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=sp)
    assert t.item() == (rank // 2) * 4 + 1          # ranks 2b and 2b+1


def test_process_groups_four_ranks():
    _spawn(_groups_worker, 4)


def _sp_worker(rank, world):
    from gdnet_b200.model import GDNet

    torch.manual_seed(0)
    T = 32 * world
    model = GDNet(vocab_size=64, d_embed=16, d=32, n_layers=2, n_cycles=2, chunk_size=T, kernel_size=4)
    model.cam_enabled = False
    tok = torch.randint(0, 64, (2, T), generator=torch.Generator().manual_seed(1))
    full = model(tok)[0]
    full.pow(2).mean().backward()
    want = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad(set_to_none=True)
    t_loc = T // world
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    loc = model(tok[:, sl], sp_group=dist.group.WORLD)[0]
    assert torch.allclose(loc, full[:, sl], atol=1e-5), (loc - full[:, sl]).abs().max()
    (loc.pow(2).sum() / full.numel()).backward()
    for n, p in model.named_parameters():
        if n in want:
            g = p.grad.clone() if p.grad is not None else torch.zeros_like(want[n])
            dist.all_reduce(g)
            assert torch.allclose(g, want[n], atol=1e-5), n


def test_sequence_parallel_equals_unsplit_cpu():
    """Values and (summed) gradients over a sequence split across ranks equal the unsplit run: the halo
    gradient reaches the previous shard inside backward."""
    _spawn(_sp_worker, 2)


def _sp_carry_worker(rank, world):
    """State carry: shard r reads a memory that holds the summaries of shards 0..r-1, exactly what processing the
    shards one after the other as chunks would have written."""
    from gdnet_b200.model import GDNet
    from gdnet_b200.train.step import build_cam_buffer

    torch.manual_seed(0)
    T = 32 * world
    model = GDNet(vocab_size=64, d_embed=16, d=32, n_layers=2, n_cycles=2, chunk_size=T, kernel_size=4, n_slots=6)
    with torch.no_grad():
        model.cam.rho.fill_(0.7)
        model.cam.W_pos.weight.normal_(std=0.3)
    model.eval()      # the spectral norm of the read-out gate would otherwise advance its power iteration per call
    tok = torch.randint(0, 64, (2, T), generator=torch.Generator().manual_seed(1))
    t_loc = T // world
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    with torch.no_grad():
        # oracle from the unsplit trunk: summaries of the shards before this one, then the read-out of this shard
        fwd, side, _ = model.trunk(tok)
        tags = torch.zeros(2, 6, model.cam.d_sig)
        vals = torch.zeros(2, 6, model.cam.d_c)
        for r in range(rank):
            seg = slice(r * t_loc, (r + 1) * t_loc)
            tags, vals = model.cam.write(fwd[:, seg][:, -1], side[0][:, seg].mean(dim=1), tags, vals)
        out, _ = model.cam.read(fwd[:, sl], side[0][:, sl], tags, vals)
        want = model.logits_from(out)
        got, _, gt, gv, _, _, _ = model(tok[:, sl], sp_group=dist.group.WORLD)
        assert torch.allclose(got, want, atol=1e-5), (got - want).abs().max()
        assert torch.allclose(gt, tags, atol=1e-6) and torch.allclose(gv, vals, atol=1e-6)
        if rank > 0:
            model.sp_state_carry = False
            plain = model(tok[:, sl], sp_group=dist.group.WORLD)[0]
            model.sp_state_carry = True
            assert not torch.allclose(plain, want, atol=1e-4), "the carried state made no difference"
        else:
            model.sp_state_carry = False
            model(tok[:, sl], sp_group=dist.group.WORLD)
            model.sp_state_carry = True
        # memory-filling passes: every shard of every write chunk ends up in the buffers, chunk by chunk
        wc = torch.randint(0, 64, (2, 2, T), generator=torch.Generator().manual_seed(2))
        ft, fv = build_cam_buffer(model, wc[:, :, sl], sp_group=dist.group.WORLD)
        tags = torch.zeros(2, 6, model.cam.d_sig)
        vals = torch.zeros(2, 6, model.cam.d_c)
        for i in range(2):
            fwd, side, _ = model.trunk(wc[:, i])
            for r in range(world):
                seg = slice(r * t_loc, (r + 1) * t_loc)
                tags, vals = model.cam.write(fwd[:, seg][:, -1], side[0][:, seg].mean(dim=1), tags, vals)
        assert torch.allclose(ft, tags, atol=1e-5) and torch.allclose(fv, vals, atol=1e-5)


def test_sequence_parallel_state_carry_equals_sequential_chunks():
    _spawn(_sp_carry_worker, 2)


def _step_worker(rank, world, tmp):
    from gdnet_b200.loss import projected_step
    from gdnet_b200.model import GDNet

    torch.manual_seed(0)
    model = GDNet(vocab_size=64, d_embed=16, d=32, n_layers=1, n_cycles=1, chunk_size=16, kernel_size=4)
    params = list(model.parameters())
    opt = torch.optim.SGD(params, lr=0.1)
    g = torch.Generator().manual_seed(10 + rank)
    tok, tgt = torch.randint(0, 64, (2, 16), generator=g), torch.randint(0, 64, (2, 16), generator=g)
    torch.manual_seed(3)
    projected_step(model, params, opt, tok, tgt, precision="fp32")
    flat = torch.cat([p.detach().reshape(-1) for p in params])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    assert torch.allclose(flat, ref, atol=1e-6), "ranks diverged after the distributed step"
    Heartbeat(tmp, rank).beat(1)


def test_distributed_projected_step_keeps_ranks_in_sync(tmp_path):
    _spawn(_step_worker, 2, str(tmp_path))
    beats = read_heartbeats(str(tmp_path))
    assert sorted(beats) == [0, 1] and all(b["step"] == 1 for b in beats.values())


def test_watchdog_names_the_rank_that_stopped(tmp_path):
    d = str(tmp_path)
    hb = [Heartbeat(d, r) for r in range(3)]
    for h in hb:
        h.beat(5)
    assert find_stalled(read_heartbeats(d), 3, stall_s=60) == []
    assert find_stalled(read_heartbeats(d), 4, stall_s=60) == [3]          # a rank that never joined
    hb[0].beat(9)
    hb[2].beat(9)                                                            # rank 1 stops beating
    assert find_stragglers(read_heartbeats(d), max_lag=2) == [1]
    later = time.time() + 100
    beats = read_heartbeats(d)
    beats[0]["time"] = beats[2]["time"] = later
    assert find_stalled(beats, 3, stall_s=60, now=later) == [1]
    seen = []
    wd = Watchdog(d, world=4, stall_s=0.0, period_s=0.05, on_failure=seen.append)
    wd.start()
    time.sleep(0.3)
    wd.stop()
    assert seen and 3 in seen[0]


def _timeout_worker(rank, world):
    # rank 1 never joins the collective: rank 0 must get an error from the short timeout, not hang
    if rank == 0:
        t = torch.ones(1)
        try:
            dist.all_reduce(t)
            raise AssertionError("all_reduce returned although a rank was missing")
        except RuntimeError:
            pass
    else:
        time.sleep(8)


def _entry_short(rank, world, port, fn, args):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    groups.init_distributed(backend="gloo", timeout_minutes=3.0 / 60.0)
    fn(rank, world, *args)
    os._exit(0)            # skip the collective teardown: the peer is gone on purpose


def test_missing_rank_ends_collective_with_error():
    mp.spawn(_entry_short, args=(2, _free_port(), _timeout_worker, ()), nprocs=2, join=True)
