"""Import path kept from the reference (``gdnet.data.fineweb_edu``)."""
from .streaming import FineWebEduDataset  # noqa: F401
