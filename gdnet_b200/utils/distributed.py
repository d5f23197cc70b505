"""Import path kept from the reference (``gdnet.utils.distributed``)."""

from ..parallel.fsdp import wrap_fsdp  # noqa: F401
from ..parallel.groups import (  # noqa: F401
    barrier,
    destroy,
    get_dp_group,
    get_rank,
    get_sp_group,
    get_world_size,
    init_distributed,
    init_process_groups,
    is_main_process,
    launch,
    sp_dp_ranks,
)
