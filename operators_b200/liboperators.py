"""Loading the shared library and the ctypes types of its C ABI.

Same names and meaning as the reference wrapper (reference
operatorspy/liboperators.py:14-73): `open_lib()` returns a `ctypes.CDLL` with
the handle and tensor-descriptor entry points typed.  The library is looked up
in `$INFINI_ROOT/lib` when INFINI_ROOT is set (the reference's install
convention) and otherwise in this package's own `lib/` directory, where
`python -m operators_b200.build` puts it.  There is no CPU fallback: if the
CUDA library is missing, open_lib raises.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_int, c_int64, c_uint64

from .data_layout import DataLayout

Device = c_int

_PKG_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")


class TensorDescriptor(Structure):
    _fields_ = [
        ("dt", DataLayout),
        ("ndim", c_uint64),
        ("shape", POINTER(c_uint64)),
        ("pattern", POINTER(c_int64)),
    ]


infiniopTensorDescriptor_t = POINTER(TensorDescriptor)


class CTensor:
    """A tensor descriptor plus the raw data pointer it describes."""

    def __init__(self, desc, data):
        self.descriptor = desc
        self.data = data


class Handle(Structure):
    _fields_ = [("device", c_int)]


infiniopHandle_t = POINTER(Handle)


def library_path(lib_dir=None):
    if lib_dir is None:
        root = os.environ.get("INFINI_ROOT")
        lib_dir = os.path.join(root, "lib") if root else _PKG_LIB_DIR
    for d in lib_dir.split(os.pathsep):
        p = os.path.join(d, "libinfiniop.so")
        if os.path.isfile(p):
            return p
    raise FileNotFoundError(
        "libinfiniop.so not found in %r: build it with `python -m operators_b200.build` "
        "or point INFINI_ROOT at an install" % lib_dir
    )


def open_lib(lib_dir=None):
    lib = ctypes.CDLL(library_path(lib_dir))
    lib.infiniopCreateTensorDescriptor.argtypes = [
        POINTER(infiniopTensorDescriptor_t),
        c_uint64,
        POINTER(c_uint64),
        POINTER(c_int64),
        DataLayout,
    ]
    lib.infiniopCreateTensorDescriptor.restype = c_int
    lib.infiniopDestroyTensorDescriptor.argtypes = [infiniopTensorDescriptor_t]
    lib.infiniopDestroyTensorDescriptor.restype = c_int
    lib.infiniopCreateHandle.argtypes = [POINTER(infiniopHandle_t), c_int, c_int]
    lib.infiniopCreateHandle.restype = c_int
    lib.infiniopDestroyHandle.argtypes = [infiniopHandle_t]
    lib.infiniopDestroyHandle.restype = c_int
    return lib
