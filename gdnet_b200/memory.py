"""Import path kept from the reference (``gdnet.memory``)."""
from .models.memory import Memory  # noqa: F401
