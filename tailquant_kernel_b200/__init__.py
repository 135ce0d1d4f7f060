"""B200-native split W4A4 + tail linear (hand-written sm_100a CUDA behind a C ABI)."""
from . import ops, policy, weights_io  # noqa: F401
from .linear import SplitLinear, interleave_gate_up, split_linear_forward  # noqa: F401
from ._lib import (TQ_HAD_BLOCK128, TQ_HAD_KRON12, TQ_HAD_NONE, TQ_HAD_WHT)  # noqa: F401
