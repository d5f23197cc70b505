from .distributed import (  # noqa: F401
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
    wrap_fsdp,
)
from .fp8 import Precision, autocast, cast_for_precision, convert_to_fp8, update_fp8_scales  # noqa: F401
