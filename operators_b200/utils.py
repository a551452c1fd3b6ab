"""Helpers shared by callers of the C ABI; same names and behaviour as the
reference's (reference operatorspy/utils.py:6-108)."""
import ctypes

from .data_layout import BF16, F16, F32, F64, I8, I16, I32, I64, U8, U16, U32, U64
from .liboperators import CTensor, infiniopHandle_t, infiniopTensorDescriptor_t

STATUS_NAMES = {
    0: "STATUS_SUCCESS",
    1: "STATUS_EXECUTION_FAILED",
    2: "STATUS_BAD_PARAM",
    3: "STATUS_BAD_TENSOR_DTYPE",
    4: "STATUS_BAD_TENSOR_SHAPE",
    5: "STATUS_BAD_TENSOR_STRIDES",
    6: "STATUS_MEMORY_NOT_ALLOCATED",
    7: "STATUS_INSUFFICIENT_WORKSPACE",
    8: "STATUS_BAD_DEVICE",
}


class InfiniopError(Exception):
    def __init__(self, status):
        self.status = status
        super().__init__("Error code %d (%s)" % (status, STATUS_NAMES.get(status, "?")))


def check_error(status):
    if status != 0:
        raise InfiniopError(status)


def _layout_of(dtype):
    import torch

    table = {
        torch.int8: I8, torch.int16: I16, torch.int32: I32, torch.int64: I64, torch.uint8: U8,
        torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.float64: F64,
    }
    for name, dl in (("uint16", U16), ("uint32", U32), ("uint64", U64)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = dl
    return table.get(dtype)


def create_tensor_descriptor(lib, shape, strides, layout):
    """Descriptor from plain shape / element strides (strides=None: contiguous)."""
    ndim = len(shape)
    c_shape = (ctypes.c_uint64 * max(ndim, 1))(*shape)
    c_strides = (ctypes.c_int64 * max(ndim, 1))(*strides) if strides is not None else None
    desc = infiniopTensorDescriptor_t()
    check_error(lib.infiniopCreateTensorDescriptor(ctypes.byref(desc), ndim, c_shape, c_strides, layout))
    return desc


def to_tensor(tensor, lib):
    """PyTorch tensor -> CTensor(descriptor, data pointer)."""
    dt = _layout_of(tensor.dtype)
    assert dt is not None, "unsupported dtype %s" % tensor.dtype
    desc = create_tensor_descriptor(lib, tuple(tensor.shape), tuple(tensor.stride()), dt)
    return CTensor(desc, tensor.data_ptr())


def destroy_tensor_descriptor(lib, desc):
    check_error(lib.infiniopDestroyTensorDescriptor(desc))


def create_workspace(size, torch_device):
    if size == 0:
        return None
    import torch

    return torch.zeros(size=(size,), dtype=torch.uint8, device=torch_device)


def create_handle(lib, device, id=0):
    handle = infiniopHandle_t()
    check_error(lib.infiniopCreateHandle(ctypes.byref(handle), device, id))
    return handle


def destroy_handle(lib, handle):
    check_error(lib.infiniopDestroyHandle(handle))


def rearrange_tensor(tensor, new_strides):
    """Copy `tensor` into fresh storage laid out with `new_strides` (positive,
    in elements) and return the strided view of it."""
    import torch

    shape = tuple(tensor.shape)
    if any(s <= 0 for s in new_strides):
        raise ValueError("Negative strides are not supported yet")
    extent = sum(st * (sz - 1) for st, sz in zip(new_strides, shape)) + 1
    storage = torch.zeros((extent,), dtype=tensor.dtype, device=tensor.device)
    view = torch.as_strided(storage, shape, tuple(new_strides))
    view.copy_(tensor)
    return view
