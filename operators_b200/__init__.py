"""Host-side binding of the B200 `nv-gpu` backend for the InfiniOperators
decode hot path (RMSNorm, RoPE, SwiGLU, Add, causal softmax, random sample).

The product is the C-ABI shared library built from `csrc/`; this package only
loads it and mirrors the reference's Python wrapper (same names: open_lib,
to_tensor, create_handle, ...), plus `ops`, thin per-operator functions that
run the create / workspace / compute / destroy stages on torch tensors.
"""
from .data_layout import *  # noqa: F401,F403
from .devices import DeviceEnum  # noqa: F401
from .liboperators import CTensor, infiniopHandle_t, infiniopTensorDescriptor_t, open_lib  # noqa: F401
from .utils import *  # noqa: F401,F403
