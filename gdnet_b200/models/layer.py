"""GDLayer: one gated-dissipative layer (forward stream + side stream).

Behavioural parity with the reference's ``gdnet/layer.py`` (module and parameter
names, initialisation, the four step entry points). The arithmetic itself lives in
``gdnet_b200.ops``: on a CUDA tensor a step is a single autograd node backed by the
sm_100a kernels, on a CPU tensor it is the plain-PyTorch oracle.

A "step" with prefix pair ``(conv_p, g_p, r_p)``::

    c     = causal_dwconv(fwd; Wc_p)
    R     = sigmoid(RMSNorm_r(W2_r silu(W1_r [side ; c] + b1_r) + b2_r))
    g     = sigmoid(W2_g RMSNorm_g(silu(W1_g c + b1_g)) + b2_g)
    fwd'  = c*g     + side*R
    side' = c*(1-g) + side*(1-R)
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import functional as ops

_STEP_PREFIXES = {"fwd": ("conv_fwd", "gf", "rf"), "bwd": ("conv_bwd", "gb", "rb")}


class CausalDepthWiseConv1d(nn.Module):
    """Holder of the depthwise taps ``conv.weight (d, 1, k)``.

    ``forward`` is the stand-alone causal conv (reference: gdnet/layer.py:14-42); the
    layer steps read the taps directly.
    """

    def __init__(self, d: int, size: int = 7):
        super().__init__()
        self.size = size
        self.conv = nn.Conv1d(d, d, kernel_size=size, padding=size - 1, groups=d, bias=False)

    @property
    def taps(self) -> torch.Tensor:
        """The ``(d, k)`` view of the conv weight. It remembers the parameter it views (``base_param``), so a
        kernel's backward can look up the flat fp32 gradient buffer a training engine has installed on the
        parameter at that time (``main_grad``) and add the tap gradients in place."""
        w = self.conv.weight
        t = w.squeeze(1)
        t.base_param = w
        return t

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.causal_dwconv(x, self.taps)


class GDLayer(nn.Module):
    """A single gated-dissipative layer (reference: gdnet/layer.py:45-215).

    Args:
        d: hidden width.
        size: causal depthwise conv width ``k``.
    """

    def __init__(self, d: int, size: int = 7):
        super().__init__()
        self.d = d
        self.conv_fwd = CausalDepthWiseConv1d(d, size)
        self.conv_bwd = CausalDepthWiseConv1d(d, size)
        # gates start open (bias +2), recovery starts mostly closed (bias -2)
        for prefix, fan_in, bias0 in (("gf", d, 2.0), ("gb", d, 2.0), ("rf", 2 * d, -2.0), ("rb", 2 * d, -2.0)):
            w1 = nn.Linear(fan_in, d)
            nn.init.orthogonal_(w1.weight)
            w2 = nn.Linear(d, d)
            nn.init.normal_(w2.weight, std=0.01)
            nn.init.constant_(w2.bias, bias0)
            setattr(self, f"{prefix}_W1", w1)
            setattr(self, f"{prefix}_W2", w2)
            setattr(self, f"{prefix}_norm", nn.RMSNorm(d))

    # -- pieces, exposed for tests and experiments ------------------------------------

    def _gate(self, prefix: str, x: torch.Tensor) -> torch.Tensor:
        """Gate value through the modules (FP8 linears in FP8 mode; layer.py:80-84)."""
        w1, w2 = getattr(self, f"{prefix}_W1"), getattr(self, f"{prefix}_W2")
        norm = getattr(self, f"{prefix}_norm")
        return torch.sigmoid(w2(norm(torch.nn.functional.silu(w1(x)))))

    def _recovery(self, prefix: str, side: torch.Tensor, fwd: torch.Tensor) -> torch.Tensor:
        w1, w2 = getattr(self, f"{prefix}_W1"), getattr(self, f"{prefix}_W2")
        norm = getattr(self, f"{prefix}_norm")
        z = w2(torch.nn.functional.silu(w1(torch.cat([side, fwd], dim=-1))))
        return torch.sigmoid(norm(z))

    # -- steps ------------------------------------------------------------------------

    def _step(self, which: str, fwd, side, sp_group=None, return_gate=False, sp_slot=None):
        conv_name, g, r = _STEP_PREFIXES[which]
        out = ops.layer_step(
            fwd, side, self, conv_name, g, r,
            sp_group=sp_group, sp_slot=sp_slot, return_gate=return_gate,
        )
        return out

    def fwd_step(self, fwd, side, return_gate: bool | str = False):
        return self._step("fwd", fwd, side, return_gate=return_gate)

    def bwd_step(self, fwd, side):
        return self._step("bwd", fwd, side)

    def fwd_step_sp(self, fwd, side, sp_group, return_gate: bool | str = False, sp_slot=None):
        return self._step("fwd", fwd, side, sp_group=sp_group, return_gate=return_gate, sp_slot=sp_slot)

    def bwd_step_sp(self, fwd, side, sp_group, sp_slot=None):
        return self._step("bwd", fwd, side, sp_group=sp_group, sp_slot=sp_slot)


# --------------------------------------------------------------------------------------
# hard spectral-norm helpers used by the reference's SN study scripts
# (scripts/compare_periodic_sn.py:12,45 and experiments/copy_task/run_rope.py:28,70
# import them from gdnet.layer although the reference's layer.py no longer has them).
# --------------------------------------------------------------------------------------

_SN_ATTRS = ("gf_W1", "gb_W1", "rf_W1", "rb_W1")


def apply_hard_sn(layer: GDLayer) -> GDLayer:
    """Wrap the four gate ``W1`` linears of ``layer`` in ``nn.utils.spectral_norm``."""
    for attr in _SN_ATTRS:
        mod = getattr(layer, attr)
        if "weight_orig" not in mod._parameters:
            setattr(layer, attr, nn.utils.spectral_norm(mod))
    return layer


class freeze_sn_iteration:
    """Context manager: skip the power iteration of every SN-wrapped ``W1`` of ``layer``.

    Inside the block the spectral-norm hooks reuse the stored ``u``/``v`` (the modules
    are put in eval mode, which is how torch's hook decides), so ``sigma`` is still
    applied but not refreshed: "periodic" SN runs the iteration only every K-th step.
    """

    def __init__(self, layer: nn.Module):
        self._mods = [m for m in layer.modules() if "weight_orig" in getattr(m, "_parameters", {})]
        self._was_training: list[bool] = []

    def __enter__(self):
        self._was_training = [m.training for m in self._mods]
        for m in self._mods:
            m.training = False
        return self

    def __exit__(self, *exc):
        for m, t in zip(self._mods, self._was_training):
            m.training = t
        return False


def _sync_sn(mod: nn.Module) -> None:
    """Recompute ``mod.weight`` from ``weight_orig`` and the stored ``u``/``v`` without
    advancing the power iteration (used after loading weights or an optimizer step)."""
    if "weight_orig" not in getattr(mod, "_parameters", {}):
        return
    with torch.no_grad():
        w = mod.weight_orig
        sigma = torch.dot(mod.weight_u, torch.mv(w.reshape(w.shape[0], -1), mod.weight_v))
        mod.weight = (w / sigma).detach()
