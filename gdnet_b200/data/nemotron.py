"""Import path kept from the reference (``gdnet.data.nemotron``)."""
from .streaming import NemotronDataset  # noqa: F401
