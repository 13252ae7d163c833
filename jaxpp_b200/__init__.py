"""B200-native MPMD pipeline-parallel training framework."""
from . import primitives as _primitives  # registers the pp:: marker ops
from .ops import core as _ops_core  # registers the b200:: ops
from .api import *  # noqa: F401,F403
from .api import __all__ as _api_all

__version__ = "0.1.0"
__all__ = list(_api_all)
