"""Import path kept from the reference (``gdnet.utils.sp``)."""

from ..parallel.sp import (  # noqa: F401
    FusedHaloConvSP,
    clear_symm_handles,
    flush_bwd_halos,
    halo_exchange,
    shard_range,
    shard_sequence,
    state_exchange,
)
