"""Loader of the compiled sm_100a extension (``gdnet_b200/_C.so``).

The library is built in-tree by ``python -m gdnet_b200.build``. On a machine with a GPU a
missing library is an error, not a reason to fall back: the CUDA ops import this module
and raise if it cannot be loaded.
"""

from __future__ import annotations

from pathlib import Path

import torch

import os

# GDNET_LIB: another build of the same library (kernel experiments compare two builds in one session)
_LIB = Path(os.environ["GDNET_LIB"]) if os.environ.get("GDNET_LIB") else Path(__file__).resolve().parent / "_C.so"
_loaded = False


def lib_path() -> Path:
    return _LIB


def load() -> None:
    """Load the extension once; raises ``RuntimeError`` with the build command if absent."""
    global _loaded
    if _loaded:
        return
    if not _LIB.exists():
        raise RuntimeError(
            f"{_LIB} is missing: build the sm_100a extension with `python -m gdnet_b200.build`"
        )
    torch.ops.load_library(str(_LIB))
    _loaded = True


def available() -> bool:
    return _LIB.exists()


def ops():
    load()
    return torch.ops.gdnet_b200


class KernelTimeout(RuntimeError):
    """A bounded wait inside a kernel ran out; the kernel returned early."""


class KernelArgumentError(ValueError):
    """A kernel met data it refuses to use (e.g. a class index outside the vocabulary); it skipped the
    offending element instead of touching memory out of bounds."""


_STATUS_NAMES = {
    1: "TMA stage never arrived (consumer wait)",
    2: "shared-memory stage never released (producer wait)",
    3: "accumulator never completed (epilogue wait)",
    4: "accumulator never drained (MMA wait)",
    5: "peer flag never written",
    6: "bad argument",
}


def check_status(like: torch.Tensor, reset: bool = True) -> None:
    """Read the device status word (synchronises) and raise if a kernel reported a problem."""
    st = ops().kernel_status(like)
    code, site, block, detail = st.tolist()
    if code != 0:
        if reset:
            st.zero_()
        if code == 6:
            raise KernelArgumentError(
                f"kernel status 6 (bad argument) at site {site}, block {block}, detail {detail}"
                + (": cross-entropy target outside [0, vocab); that row was ignored" if site == 60 else "")
            )
        raise KernelTimeout(
            f"kernel status {code} ({_STATUS_NAMES.get(code, '?')}) at site {site}, block {block}, detail {detail}"
        )
