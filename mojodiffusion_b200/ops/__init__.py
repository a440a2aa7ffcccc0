"""Ops: hand-written sm_100a kernels (GPU) with pure-torch fp32 references (CPU path and test oracle)."""
from . import native, reference
from .functional import *  # noqa: F401,F403
from .native import check_status
