"""gdnet_b200: a Blackwell (sm_100a) native GDNet pretraining framework.

Public surface follows the reference package ``gdnet`` (gdnet/__init__.py:1-25) so
``import gdnet_b200 as gdnet`` is a drop-in change for scripts written against it.
"""

from .utils import (  # noqa: F401
    Precision,
    autocast,
    barrier,
    destroy,
    get_rank,
    get_world_size,
    init_distributed,
    is_main_process,
    launch,
    wrap_fsdp,
)

__version__ = "0.1.0"

__all__ = [
    "autocast", "Precision", "init_distributed", "wrap_fsdp", "launch", "get_rank",
    "get_world_size", "is_main_process", "barrier", "destroy",
]
