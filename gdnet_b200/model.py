"""Import path kept from the reference (``gdnet.model``)."""
from .models.gdnet import CAM, GDNet, GDLayer, TransitionOperators  # noqa: F401
