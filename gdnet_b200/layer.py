"""Import path kept from the reference (``gdnet.layer``)."""
from .models.layer import (  # noqa: F401
    CausalDepthWiseConv1d,
    GDLayer,
    _sync_sn,
    apply_hard_sn,
    freeze_sn_iteration,
)
