from .mixed import MixedDataset  # noqa: F401
from .packed import PackedTokenDataset  # noqa: F401
from .streaming import FineWebEduDataset, NemotronDataset, pack_token_stream  # noqa: F401
from .synthetic import CopyTaskDataset, SyntheticPackedDataset, copy_task_batch, synthetic_packed_batch  # noqa: F401
