"""Workers for tests/test_gpu_multi.py (run under torch.distributed.run, one process per GPU)."""

import copy
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdnet_b200 import _ext  # noqa: E402
from gdnet_b200.model import GDNet  # noqa: E402
from gdnet_b200.train.engine import TrainEngine  # noqa: E402
from gdnet_b200.utils.fp8 import cast_for_precision  # noqa: E402


def _gap(a, b, a0, what):
    """Two engines that should have taken the same steps: AdamW turns a gradient whose sign is decided by rounding
    noise (atomics add in a different order from run to run) into a full-size step of either sign, so single
    elements may differ by 2 * lr * steps. What must hold: such elements are rare, and the difference is small
    against the distance the parameters moved."""
    a, b, a0 = a.float(), b.float(), a0.float()
    d = (a - b).abs()
    frac = (d > 5e-3).float().mean().item()
    rel = d.norm().item() / ((a - a0).norm().item() + 1e-12)
    assert frac < 2e-2 and rel < 0.15, f"{what}: {frac:.2%} of the elements differ by more than 5e-3, relative gap {rel:.3f}"
    return rel


def _model(dev, seed=0, T=256):
    torch.manual_seed(seed)
    m = GDNet(vocab_size=1024, d_embed=128, d=128, n_layers=2, n_cycles=2, kernel_size=4, chunk_size=T).to(dev)
    return cast_for_precision(m, "fp8")


def engine_fused_vs_nccl(rank, world, dev):
    """Two engines from identical weights, one per comm backend, fed the same per-rank data: parameters
    must agree after several steps, and all ranks must hold identical parameters."""
    base = _model(dev)
    e_fused = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="fused")
    e_nccl = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="nccl")
    init = [gr.flat.float().clone() for gr in e_nccl.groups]
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    for step in range(3):
        tok = torch.randint(0, 1024, (2, 256), generator=g).to(dev)
        tgt = torch.randint(0, 1024, (2, 256), generator=g).to(dev)
        clip = 1.0 if step == 2 else 0.0          # also exercise the two-phase (clipped) path
        torch.manual_seed(7 + step)
        l1 = e_fused.projected_step(tok, tgt, grad_clip=clip)
        torch.manual_seed(7 + step)
        l2 = e_nccl.projected_step(tok, tgt, grad_clip=clip)
        assert abs(float(l1) - float(l2)) < 5e-2 * max(1.0, abs(float(l2))), (float(l1), float(l2))
    torch.cuda.synchronize()
    _ext.check_status(tok)
    for ga, gb, a0 in zip(e_fused.groups, e_nccl.groups, init):
        a, b = ga.flat.float(), gb.flat.float()
        _gap(a, b, a0, "fused vs nccl parameters")
        ref = a.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, a), "ranks hold different parameters after the fused all-gather"
    # what the update kernels must leave behind: clean status, counters at zero, every peer's flags at the last sequence number
    from gdnet_b200.runtime.checked import engine_invariants

    engine_invariants(e_fused)


def engine_multimem_vs_peer(rank, world, dev):
    """The update kernel reading its shard through the NVLink multicast address (sum formed inside the switch, updated
    parameters broadcast by one store) against the same kernel on plain peer loads and stores. Without a multicast
    address on the box there is nothing to compare."""
    import os

    base = _model(dev)
    os.environ["GDNET_MULTIMEM"] = "1"
    e_mc = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="fused")
    os.environ["GDNET_MULTIMEM"] = "0"
    e_pp = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="fused")
    assert not any(any(gr.mc) for gr in e_pp.groups)
    if not all(all(gr.mc) for gr in e_mc.groups):
        print("no multicast address for the gradient buffers on this box: nothing to compare", flush=True)
        return
    init = [gr.flat.float().clone() for gr in e_pp.groups]
    g = torch.Generator(device="cpu").manual_seed(300 + rank)
    for step in range(3):
        tok = torch.randint(0, 1024, (2, 256), generator=g).to(dev)
        tgt = torch.randint(0, 1024, (2, 256), generator=g).to(dev)
        clip = 1.0 if step == 2 else 0.0          # also the two-phase (clipped) path
        torch.manual_seed(7 + step)
        l1 = e_mc.projected_step(tok, tgt, grad_clip=clip)
        torch.manual_seed(7 + step)
        l2 = e_pp.projected_step(tok, tgt, grad_clip=clip)
        assert abs(float(l1) - float(l2)) < 5e-2 * max(1.0, abs(float(l2))), (float(l1), float(l2))
    torch.cuda.synchronize()
    _ext.check_status(tok)
    for ga, gb, a0 in zip(e_mc.groups, e_pp.groups, init):
        a, b = ga.flat.float(), gb.flat.float()
        _gap(a, b, a0, "multicast vs peer-load parameters")
        ref = a.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, a), "ranks hold different parameters after the multicast store"
    e_mc.close()
    e_pp.close()


def engine_scatter_vs_nccl(rank, world, dev):
    """Gradients reduce-scattered from the weight-gradient GEMM epilogues (NVLink atomics into the owner's
    shard) against NCCL all-reduce, both with the projection coefficient of the reduced gradients."""
    base = _model(dev)
    e_nccl = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="nccl", projection="global")
    e_fused = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="fused", projection="global")
    e_sc = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="scatter")
    init = [gr.flat.float().clone() for gr in e_nccl.groups]
    g = torch.Generator(device="cpu").manual_seed(200 + rank)
    from gdnet_b200.ops import cuda as cu

    for step in range(3):
        tok = torch.randint(0, 1024, (2, 256), generator=g).to(dev)
        tgt = torch.randint(0, 1024, (2, 256), generator=g).to(dev)
        clip = 1.0 if step == 2 else 0.0
        losses = []
        for eng in (e_nccl, e_fused, e_sc):
            torch.manual_seed(7 + step)
            losses.append(float(eng.projected_step(tok, tgt, grad_clip=clip)))
        assert max(losses) - min(losses) < 5e-2 * max(1.0, abs(losses[0])), losses
    torch.cuda.synchronize()
    _ext.check_status(tok)
    for ga, gb, gc, a0 in zip(e_nccl.groups, e_fused.groups, e_sc.groups, init):
        a, b, c = ga.flat.float(), gb.flat.float(), gc.flat.float()
        _gap(a, b, a0, "fused(global) vs nccl(global) parameters")
        _gap(a, c, a0, "scatter vs nccl parameters")
        ref = c.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, c), "ranks hold different parameters after the all-gather"
        lo, hi = gc.shard
        assert float(gc.g_task[lo:hi].abs().max()) == 0.0, "the consumed shard was not cleared"


def engine_shared_fp8_weights(rank, world, dev):
    """FP8 weights quantised by their owner and stored into every rank's cache by the quantisation kernel:
    same losses and bit-identical parameters as every rank quantising everything itself."""
    from gdnet_b200.ops import cuda as cu

    base = _model(dev)
    g = torch.Generator(device="cpu").manual_seed(300 + rank)
    data = [(torch.randint(0, 1024, (2, 256), generator=g).to(dev), torch.randint(0, 1024, (2, 256), generator=g).to(dev))
            for _ in range(3)]
    results = []
    for shared in (False, True):
        eng = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="fused", share_fp8_weights=shared)
        assert (eng._shared is not None) == shared
        if not shared:
            init = [gr.flat.float().clone() for gr in eng.groups]
        losses = []
        for step, (tok, tgt) in enumerate(data):
            torch.manual_seed(7 + step)
            losses.append(float(eng.projected_step(tok, tgt)))
        torch.cuda.synchronize()
        _ext.check_status(tok)
        results.append((losses, [gr.flat.clone() for gr in eng.groups]))
        if shared:
            assert len(eng._shared.owned) < len(eng._shared.entries), "this rank quantised every weight"
    (l0, p0), (l1, p1) = results
    # the weight-gradient GEMMs add their split-K shares with atomics, so two runs agree to rounding noise only
    assert l0[0] == l1[0] and all(abs(a - b) < 5e-3 * abs(a) for a, b in zip(l0, l1)), (l0, l1)
    for a, b, a0 in zip(p0, p1, init):
        _gap(a, b, a0, "parameters with private and with shared caches")
    # the arena must hold exactly what a private quantisation of the current weights gives, on every rank
    sw = eng._shared
    sw.refresh()
    torch.cuda.synchronize()
    for (_, _, _), qw in sw.entries.items():
        w = qw.source
        N, Kd = w.shape
        q, qt = torch.empty_like(qw.q), torch.empty_like(qw.qt)
        s_, st = torch.empty_like(qw.s), torch.empty_like(qw.st)
        pp, pt = torch.empty_like(qw.p), torch.empty_like(qw.pt)
        cu.K.quant_tile(w.detach(), False, q, s_, cu.Q_BLOCK, qt, st, cu.Q_BLOCK, True, pp, pt)
        for got, want, what in ((qw.q, q, "q"), (qw.qt, qt, "qt"), (qw.p, pp, "p"), (qw.pt, pt, "pt")):
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), f"shared copy {what} of a {N}x{Kd} weight is stale"
        assert torch.equal(qw.s, s_) and torch.equal(qw.st, st)
    _ext.check_status(tok)
    dist.barrier()
    cu.clear_caches()


def peer_max_allreduce(rank, world, dev):
    """One-kernel MAX all-reduce over peer memory against NCCL, repeated (the slot sets alternate), and through
    update_fp8_scales on the per-tensor recipe."""
    from gdnet_b200.parallel.symm import max_allreduce_

    for it in range(5):
        g = torch.Generator().manual_seed(1000 * it + rank)
        v = torch.rand(300 + 17 * it, generator=g).to(dev)
        want = v.clone()
        dist.all_reduce(want, op=dist.ReduceOp.MAX)
        got = max_allreduce_(v.clone())
        torch.cuda.synchronize()
        _ext.check_status(v)
        assert torch.equal(got, want), f"iteration {it}: peer MAX all-reduce differs from NCCL"
    from gdnet_b200.utils.fp8 import update_fp8_scales

    torch.manual_seed(0)
    m = GDNet(vocab_size=1024, d_embed=128, d=128, n_layers=1, n_cycles=1, kernel_size=4, chunk_size=256).to(dev)
    cast_for_precision(m, "fp8", recipe="tensor")
    tok = torch.randint(0, 1024, (2, 256), generator=torch.Generator().manual_seed(rank)).to(dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        m(tok)
    update_fp8_scales(m)
    torch.cuda.synchronize()
    _ext.check_status(tok)
    scales = torch.cat([b.reshape(-1) for n, b in m.named_buffers() if n.endswith("scale_x") or n.endswith("scale_w")])
    ref = scales.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(ref, scales), "ranks disagree on the FP8 scales after the amax exchange"


def sp_matches_single(rank, world, dev):
    """Forward + backward of the model over a sequence split across ranks equals the unsplit run."""
    T = 256 * world
    model = _model(dev, T=T)
    model.cam_enabled = False
    tok = torch.randint(0, 1024, (2, T), generator=torch.Generator().manual_seed(5)).to(dev)
    # unsplit reference on every rank
    logits_full = model(tok)[0]
    loss_full = logits_full.float().pow(2).mean()
    loss_full.backward()
    g_full = {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad(set_to_none=True)
    # sequence parallel
    t_loc = T // world
    tok_loc = tok[:, rank * t_loc : (rank + 1) * t_loc]
    logits_loc = model(tok_loc, sp_group=dist.group.WORLD)[0]
    want = logits_full[:, rank * t_loc : (rank + 1) * t_loc]
    err = (logits_loc.float() - want.float()).abs().max().item()
    assert err < 0.03 * want.float().abs().max().item() + 1e-2, f"SP logits differ: {err}"
    (logits_loc.float().pow(2).sum() / logits_full.numel()).backward()
    torch.cuda.synchronize()
    _ext.check_status(tok)
    for n, p in model.named_parameters():
        if p.grad is None or n not in g_full:
            continue
        g = p.grad.float().clone()
        dist.all_reduce(g)
        denom = g_full[n].norm().item() + 1e-6
        rel = (g - g_full[n]).norm().item() / denom
        assert rel < 0.05, f"SP gradient of {n} differs: rel {rel}"


def sp_engine_step(rank, world, dev):
    T = 256 * world
    model = _model(dev, T=256)
    engine = TrainEngine(model, lr=1e-3, precision="fp8", sp_group=dist.group.WORLD, comm="fused")
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, 1024, (2, T + 1), generator=g).to(dev)
    wc = torch.randint(0, 1024, (2, 2, T), generator=g).to(dev)
    sl = slice(rank * 256, (rank + 1) * 256)
    losses = []
    for _ in range(3):
        losses.append(float(engine.projected_step(tok[:, :-1][:, sl], tok[:, 1:][:, sl], write_chunks=wc[:, :, sl])))
    torch.cuda.synchronize()
    _ext.check_status(tok)
    assert all(l == l for l in losses), losses
    assert losses[-1] < losses[0] + 1.0


def engine_full_shard_vs_replicated(rank, world, dev):
    """Layer matrices, their gradients and AdamW moments spread over the ranks, operands gathered by the GEMMs that
    consume them, against the same engine with everything replicated (both reduce gradients from the epilogues):
    same losses, same parameters after three steps with memory write chunks, 1/world of the matrices resident."""
    from gdnet_b200.ops import cuda as cu

    base = _model(dev)
    g = torch.Generator(device="cpu").manual_seed(400 + rank)
    data = [(torch.randint(0, 1024, (2, 256), generator=g).to(dev), torch.randint(0, 1024, (2, 256), generator=g).to(dev),
             torch.randint(0, 1024, (2, 2, 256), generator=g).to(dev)) for _ in range(3)]
    results = {}
    for shard in ("none", "full"):
        eng = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="scatter", shard=shard)
        losses = []
        for step, (tok, tgt, wc) in enumerate(data):
            torch.manual_seed(7 + step)
            losses.append(float(eng.projected_step(tok, tgt, write_chunks=wc, grad_clip=1.0 if step == 2 else 0.0)))
        torch.cuda.synchronize()
        _ext.check_status(tok)
        sd = {k: v.float().clone() for k, v in eng.full_state_dict().items() if v.is_floating_point()}
        results[shard] = (losses, sd, eng.resident_bytes(),
                          sum(p.numel() * 2 for p in eng.groups[-1].params) if shard == "full" else 0)
        if shard == "full":
            ws = eng.weight_stream
            assert ws is not None and ws.order, "the order of the layer sets was not learnt"
            assert ws.gathered_bytes > 0, "nothing was gathered from the owner ranks"
            sg = eng.groups[-1]
            assert sg.sharded and sg.flat.numel() * world == sg.n
            owned = sum(o == rank for o in sg.owner)
            assert 0 < owned < len(sg.owner), "this rank owns all or none of the layer matrices"
            # a forward outside the training step (other order of requests) still finds its weights
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                out = eng(tok)[0]
            assert bool(torch.isfinite(out.float()).all())
            torch.cuda.synchronize()
            _ext.check_status(tok)
        dist.barrier()
        eng.close()
        cu.clear_caches()
        del eng
    (l0, p0, b0, _), (l1, p1, b1, layer_bytes) = results["none"], results["full"]
    assert all(abs(a - b) < 5e-3 * max(1.0, abs(a)) for a, b in zip(l0, l1)), (l0, l1)
    sd0 = {k: v.float() for k, v in base.state_dict().items() if v.is_floating_point()}
    moved = [k for k in p0 if (p0[k] - sd0[k]).norm().item() > 0]
    worst = max(_gap(p0[k], p1[k], sd0[k], f"full-shard vs replicated {k}") for k in moved if p0[k].numel() >= 1024)
    # of the sharded matrices a rank keeps 1 / world (whole matrices, balanced by size)
    assert b0["params"] - b1["params"] >= layer_bytes * (world - 1) // world - 4096 * world, (b0, b1, layer_bytes)
    assert b0["grads"] - b1["grads"] >= 4 * layer_bytes * (world - 1) // world - 4096 * world, (b0, b1, layer_bytes)
    if rank == 0:
        print(f"full-shard: losses {l1}, largest relative parameter gap {worst:.3g}, resident bytes {b1} against {b0}")


def engine_ckpt_roundtrip(rank, world, dev):
    """Step, save a sharded checkpoint, step again; then a fresh engine loads the checkpoint and takes the same
    step: both end with the same parameters and moments (every rank holds only its shard of the moments, so a
    checkpoint that kept one rank's moments for everybody would show here)."""
    import tempfile

    from gdnet_b200.ops import cuda as cu
    from gdnet_b200.runtime.ckpt import load_sharded, save_sharded

    base = _model(dev)
    g = torch.Generator(device="cpu").manual_seed(500 + rank)
    data = [(torch.randint(0, 1024, (2, 256), generator=g).to(dev), torch.randint(0, 1024, (2, 256), generator=g).to(dev))
            for _ in range(3)]
    box = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    path = box[0]
    for shard in ("none", "full"):
        eng = TrainEngine(copy.deepcopy(base), lr=1e-2, precision="fp8", comm="scatter" if shard == "full" else "fused", shard=shard)
        for step in range(2):
            torch.manual_seed(7 + step)
            eng.projected_step(*data[step])
        save_sharded(os.path.join(path, shard), 2, eng, {"cursor": 5})
        torch.manual_seed(9)
        eng.projected_step(*data[2])
        torch.cuda.synchronize()
        want_p = {k: v.float().clone() for k, v in eng.full_state_dict().items() if v.is_floating_point()}
        want_m = [gr.m.clone() for gr in eng.groups]
        dist.barrier()
        eng.close()
        cu.clear_caches()
        del eng
        torch.manual_seed(123)       # other initial weights: everything must come from the checkpoint
        eng2 = TrainEngine(_model(dev, seed=1), lr=1e-2, precision="fp8", comm="scatter" if shard == "full" else "fused", shard=shard)
        step, extra = load_sharded(os.path.join(path, shard), eng2)
        assert step == 2 and extra == {"cursor": 5} and eng2.step_count == 2
        torch.manual_seed(9)
        eng2.projected_step(*data[2])
        torch.cuda.synchronize()
        _ext.check_status(data[0][0])
        got_p = {k: v.float() for k, v in eng2.full_state_dict().items() if v.is_floating_point()}
        sd0 = {k: v.float() for k, v in base.state_dict().items() if v.is_floating_point()}
        for k in want_p:
            if want_p[k].numel() >= 1024 and (want_p[k] - sd0[k]).norm().item() > 0:
                _gap(want_p[k], got_p[k], sd0[k], f"{shard}: {k} after resume")
        for a, b in zip(want_m, [gr.m for gr in eng2.groups]):
            assert (a - b).abs().max().item() < 1e-3 * (a.abs().max().item() + 1e-6) + 1e-6, f"{shard}: AdamW moments differ after resume"
        dist.barrier()
        eng2.close()
        cu.clear_caches()
        del eng2


if __name__ == "__main__":
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        globals()[sys.argv[1]](rank, world, dev)
        dist.barrier()
        if rank == 0:
            print("WORKER_OK")
    finally:
        dist.destroy_process_group()
