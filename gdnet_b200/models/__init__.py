from .gdnet import GDNet  # noqa: F401
from .layer import CausalDepthWiseConv1d, GDLayer  # noqa: F401
from .memory import Memory  # noqa: F401
from .operators import TransitionOperators  # noqa: F401
