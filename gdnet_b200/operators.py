"""Import path kept from the reference (``gdnet.operators``)."""
from .models.operators import TransitionOperators  # noqa: F401
