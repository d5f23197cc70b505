"""Parity with the unmodified reference package (alcxpr/gdnet), imported from ``baseline/_ref`` when that
install exists (it is not part of the source tree; the tests are skipped without it).

CPU: the reference's ``GDNet.state_dict()`` loads into this framework's model with ``strict=True`` and back,
plain and after the FP8 module swap. GPU: from one ``state_dict`` both models give the same logits, the same
task gradient and, through their own ``projected_step`` with the same optimizer and batch (memory write chunks,
gradient accumulation), the same loss and the same parameter update.
"""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "gdnet")), reason="reference package not installed")

ARGS = dict(vocab_size=512, d_embed=128, d=128, n_layers=2, n_cycles=2, chunk_size=128, n_slots=8, kernel_size=4)


def _ref():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    if not os.path.exists(os.path.join(REF, "gdnet", "kernel", "fp8_linear", "gemm.py")):
        import types        # the reference's unused SM90 GEMM file may be absent from a snapshot: provide the name

        stub = types.ModuleType("gdnet.kernel.fp8_linear.gemm")
        stub.fp8_gemm = lambda *a, **k: (_ for _ in ()).throw(NotImplementedError("not part of this snapshot"))
        sys.modules.setdefault("gdnet.kernel.fp8_linear.gemm", stub)
    import gdnet
    import gdnet.loss
    import gdnet.model

    return gdnet


def test_state_dict_interchange_both_directions():
    ref = _ref()
    from gdnet_b200.model import GDNet

    torch.manual_seed(0)
    r = ref.model.GDNet(**ARGS)
    o = GDNet(**ARGS)
    assert list(r.state_dict()) == list(o.state_dict())
    o.load_state_dict(r.state_dict(), strict=True)
    for (k, a), b in zip(r.state_dict().items(), o.state_dict().values()):
        assert torch.equal(a, b), k
    torch.manual_seed(1)
    o2 = GDNet(**ARGS)
    r.load_state_dict(o2.state_dict(), strict=True)
    for (k, a), b in zip(o2.state_dict().items(), r.state_dict().values()):
        assert torch.equal(a, b), k


def test_fp8_converted_state_dict_interchange():
    """After the FP8 module swap the reference's per-linear buffers (scales, amax windows, cached e4m3 weights)
    appear under the same keys here when the reference's recipe (per-tensor scales, untied head) is selected."""
    ref = _ref()
    from gdnet.utils.fp8 import convert_to_fp8 as ref_convert

    from gdnet_b200.model import GDNet
    from gdnet_b200.utils.fp8 import convert_to_fp8

    torch.manual_seed(0)
    r = ref.model.GDNet(**ARGS)
    ref_convert(r)
    o = GDNet(**ARGS)
    convert_to_fp8(o, recipe="tensor", untie_head=True)
    rk, ok = set(r.state_dict()), set(o.state_dict())
    assert rk == ok, (sorted(rk - ok)[:8], sorted(ok - rk)[:8])
    o.load_state_dict(r.state_dict(), strict=True)
    r.load_state_dict(o.state_dict(), strict=True)


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp(min=1e-12))


def _pair(dev, seed=0):
    ref = _ref()
    from gdnet_b200.model import GDNet

    torch.manual_seed(seed)
    r = ref.model.GDNet(**ARGS).to(dev).to(torch.bfloat16)
    o = GDNet(**ARGS).to(dev).to(torch.bfloat16)
    o.load_state_dict(r.state_dict(), strict=True)
    # rho = 0 switches the position term of the memory read off; give it a value so that path is compared too
    with torch.no_grad():
        r.cam.rho.fill_(0.5)
        o.cam.rho.fill_(0.5)
    # the reference's projection (gdnet/loss.py:238-239) multiplies by a 0-dim float32 coefficient, which turns the
    # gradient of a 0-dim bfloat16 parameter into float32 and torch refuses to assign it: its step only runs when
    # the two 0-dim parameters are float32, as they are in its FP8 mode (which leaves trans_ops untouched)
    for m in (r, o):
        for name in ("log_tau", "log_temp"):
            prm = getattr(m.trans_ops, name)
            prm.data = prm.data.float()
    return ref, r, o


@pytest.mark.gpu
def test_forward_and_task_gradient_match_reference():
    dev = "cuda"
    ref, r, o = _pair(dev)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, 512, (4, 128), generator=g).to(dev)
    tgt = torch.randint(0, 512, (4, 128), generator=g).to(dev)
    tags = (torch.randn(4, 8, 16, generator=g) * 0.5).to(dev).bfloat16()
    vals = (torch.randn(4, 8, 32, generator=g) * 0.5).to(dev).bfloat16()
    outs = []
    for m in (r, o):
        m.train()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits, side, _, _, gates, w, fwd_last = m(tok, tags, vals, return_gates=True)
            loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt.reshape(-1))
        loss.backward()
        grads = {n: p.grad.float().clone() for n, p in m.named_parameters() if p.grad is not None}
        m.zero_grad(set_to_none=True)
        outs.append((logits.float(), [s.float() for s in side], [g_.float() for g_ in gates], w.float(), fwd_last.float(),
                     float(loss), grads))
    (lr, sr, gr, wr, fr, lossr, grr), (lo, so, go, wo, fo, losso, gro) = outs
    assert _rel(lo, lr) < 0.03, f"logits differ: {_rel(lo, lr)}"
    assert _rel(fo, fr) < 0.03 and _rel(wo, wr) < 0.02
    for a, b in zip(so, sr):
        assert _rel(a, b) < 0.03, "side stream differs"
    assert len(go) == len(gr)
    for a, b in zip(go, gr):
        assert _rel(a, b) < 0.02, "gate values differ"
    assert abs(losso - lossr) < 5e-3 * abs(lossr)
    assert set(gro) == set(grr), sorted(set(gro) ^ set(grr))
    worst = max((n for n in grr if grr[n].norm() > 1e-6), key=lambda n: _rel(gro[n], grr[n]))
    assert _rel(gro[worst], grr[worst]) < 0.08, f"task gradient of {worst} differs: {_rel(gro[worst], grr[worst])}"
    flat_r = torch.cat([grr[n].reshape(-1) for n in sorted(grr)])
    flat_o = torch.cat([gro[n].reshape(-1) for n in sorted(grr)])
    assert _rel(flat_o, flat_r) < 0.03, f"whole task gradient differs: {_rel(flat_o, flat_r)}"


@pytest.mark.gpu
@pytest.mark.parametrize("n_write,accum", [(0, 1), (2, 1), (2, 2)])
def test_projected_step_matches_reference(n_write, accum):
    """One step of the reference's ``gdnet.loss.projected_step`` (three backward passes) against this
    framework's (two passes: information and transition losses summed first); the optimizer is SGD with a zero
    learning rate, so the projected gradient both steps hand to it can be read from ``p.grad`` afterwards."""
    dev = "cuda"
    ref, r, o = _pair(dev, seed=1)
    from gdnet_b200.loss import projected_step

    g = torch.Generator().manual_seed(11)
    tok = torch.randint(0, 512, (4, 128), generator=g).to(dev)
    tgt = torch.randint(0, 512, (4, 128), generator=g).to(dev)
    wc = torch.randint(0, 512, (4, n_write, 128), generator=g).to(dev) if n_write else None
    res = []
    for m, step in ((r, ref.loss.projected_step), (o, projected_step)):
        m.train()
        params = [p for p in m.parameters() if p.requires_grad]
        opt = torch.optim.SGD(params, lr=0.0)       # the step leaves the projected gradient in p.grad
        torch.manual_seed(5)
        loss = step(m, params, opt, tok, tgt, beta=0.1, precision="bf16", write_chunks=wc, accum_steps=accum)
        res.append((float(loss), {n: p.grad.detach().float().clone() for n, p in m.named_parameters() if p.grad is not None}))
    (lr_, dr), (lo_, do) = res
    assert abs(lo_ - lr_) < 5e-3 * abs(lr_), (lo_, lr_)
    assert set(dr) == set(do)
    flat_r = torch.cat([dr[n].reshape(-1) for n in sorted(dr)])
    flat_o = torch.cat([do[n].reshape(-1) for n in sorted(dr)])
    assert _rel(flat_o, flat_r) < 0.05, f"projected gradient differs: {_rel(flat_o, flat_r)}"
    for n in ("layers.0.rf_W1.weight", "layers.1.gf_W2.weight", "layers.0.conv_fwd.conv.weight", "proj_out.weight",
              "embed.weight", "cam.W_up.weight"):
        assert _rel(do[n], dr[n]) < 0.10, f"projected gradient of {n} differs: {_rel(do[n], dr[n])}"
