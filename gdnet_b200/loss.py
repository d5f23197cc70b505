"""Import path kept from the reference (``gdnet.loss``)."""
from .train.step import (  # noqa: F401
    build_cam_buffer,
    gate_info_loss_from_vals,
    info_losses,
    projected_step,
    sn_soft_penalty,
)
