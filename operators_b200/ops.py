"""Per-operator call sequences over the C ABI.

Each `*Op` object performs the reference's create-descriptor and
workspace-size stages once (exactly the ctypes sequence of the reference's test
scripts, e.g. reference operatorspy/tests/rms_norm.py:56-79) and can then be
launched many times; the module-level functions are the one-shot forms.  All
tensors are torch tensors living on the handle's device; nothing here computes
anything in Python.  The same code drives any library that exports this ABI,
which is how the tests run the reference's own CPU build through it.
"""
import ctypes
from ctypes import POINTER, c_float, c_int, c_int64, c_uint64, c_void_p

from .data_layout import U64
from .liboperators import infiniopHandle_t, infiniopTensorDescriptor_t
from .utils import check_error, create_workspace, destroy_tensor_descriptor, to_tensor

_desc_t = c_void_p  # operator descriptors are opaque to Python


def _declare(lib):
    """Type every operator entry point once per loaded library."""
    if getattr(lib, "_b200_declared", False):
        return
    T, H, D = infiniopTensorDescriptor_t, infiniopHandle_t, _desc_t
    sigs = {
        "infiniopCreateRMSNormDescriptor": [H, POINTER(D), T, T, T, c_float],
        "infiniopGetRMSNormWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopRMSNorm": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyRMSNormDescriptor": [D],
        "infiniopCreateRoPEDescriptor": [H, POINTER(D), T, T, T, T],
        "infiniopGetRoPEWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopRoPE": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyRoPEDescriptor": [D],
        "infiniopCreateSwiGLUDescriptor": [H, POINTER(D), T, T, T],
        "infiniopSwiGLU": [D, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroySwiGLUDescriptor": [D],
        "infiniopCreateAddDescriptor": [H, POINTER(D), T, T, T],
        "infiniopAdd": [D, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyAddDescriptor": [D],
        "infiniopCreateRearrangeDescriptor": [H, POINTER(D), T, T],
        "infiniopRearrange": [D, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyRearrangeDescriptor": [D],
        "infiniopCreateAttentionDescriptor": [H, POINTER(D), T, T, T, T, T, T, c_uint64],
        "infiniopGetAttentionWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopAttention": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyAttentionDescriptor": [D],
        "infiniopCreateMatmulDescriptor": [H, POINTER(D), T, c_float, T, T, c_float],
        "infiniopGetMatmulWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopMatmul": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyMatmulDescriptor": [D],
        "infiniopCreateMLPDescriptor": [H, POINTER(D), T, T, T, T, c_float, ctypes.c_char],
        "infiniopGetMLPWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopMLP": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyMLPDescriptor": [D],
        "infiniopCreateRoPERearrangeDescriptor": [H, POINTER(D), T, T, T, T, T],
        "infiniopGetRoPERearrangeWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopRoPERearrange": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyRoPERearrangeDescriptor": [D],
        "infiniopCreateAddRMSNormDescriptor": [H, POINTER(D), T, T, T, T, T, c_float],
        "infiniopGetAddRMSNormWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopAddRMSNorm": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "infiniopDestroyAddRMSNormDescriptor": [D],
        "infiniopCreateCausalSoftmaxDescriptor": [H, POINTER(D), T],
        "infiniopGetCausalSoftmaxWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopCausalSoftmax": [D, c_void_p, c_uint64, c_void_p, c_void_p],
        "infiniopDestroyCausalSoftmaxDescriptor": [D],
        "infiniopCreateRandomSampleDescriptor": [H, POINTER(D), T, T],
        "infiniopGetRandomSampleWorkspaceSize": [D, POINTER(c_uint64)],
        "infiniopRandomSample": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_float, c_float, c_int, c_float, c_void_p],
        "infiniopDestroyRandomSampleDescriptor": [D],
        # extensions of this backend (include/infiniop_ext.h); absent from the reference library
        "infiniopGetRandomSampleBatchWorkspaceSize": [D, c_uint64, POINTER(c_uint64)],
        "infiniopRandomSampleBatch": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_int64, c_uint64, c_void_p,
                                      c_float, c_int, c_float, c_void_p],
        "infiniopRandomSampleBatchStatic": [D, c_void_p, c_void_p, c_int64, c_uint64, c_void_p, c_float, c_int, c_float,
                                            c_void_p],
        "infiniopRandomSampleShardLocal": [D, c_void_p, c_void_p, c_int64, c_uint64, c_uint64, c_int, c_float, c_void_p],
        "infiniopRandomSampleShardFinish": [H, c_void_p, c_void_p, c_int, c_uint64, c_uint64, c_void_p, c_float, c_int,
                                            c_float, c_void_p, c_void_p],
        "infiniopRandomSampleBatchTrace": [D, c_void_p, c_uint64, c_void_p, c_void_p, c_int64, c_uint64, c_void_p,
                                           c_float, c_int, c_float, c_void_p, c_void_p],
        "infiniopRandomSampleBatchPeer": [D, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_int64), c_uint64,
                                          POINTER(c_void_p), ctypes.c_uint32, ctypes.c_uint32, c_uint64, c_uint64, c_void_p,
                                          c_float, c_int, c_float, c_void_p],
        "infiniopExtPeerAlloc": [H, c_uint64, POINTER(c_void_p), c_void_p],
        "infiniopExtPeerOpen": [H, c_void_p, POINTER(c_void_p)],
        "infiniopExtPeerClose": [H, c_void_p],
        "infiniopExtPeerFree": [H, c_void_p],
        "infiniopExtPeerGatherRows": [H, c_void_p, c_int64, POINTER(c_void_p), POINTER(c_int64), POINTER(c_uint64),
                                      POINTER(c_uint64), POINTER(c_void_p), ctypes.c_uint32, ctypes.c_uint32, c_uint64,
                                      c_uint64, c_void_p],
        "infiniopExtPeerPublishResults": [H, POINTER(c_void_p), c_void_p, POINTER(c_void_p), ctypes.c_uint32,
                                          ctypes.c_uint32, c_uint64, c_uint64, c_void_p],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = c_int
    if hasattr(lib, "infiniopExtDeviceTimeouts"):
        lib.infiniopExtDeviceTimeouts.argtypes = [H, POINTER(c_uint64)]
        lib.infiniopExtDeviceTimeouts.restype = c_int
        lib.infiniopExtSetWaitLimit.argtypes = [H, ctypes.c_uint32]
        lib.infiniopExtSetWaitLimit.restype = c_int
    if hasattr(lib, "infiniopExtSelectKernel"):
        lib.infiniopExtSelectKernel.argtypes = [c_int, c_int]
        lib.infiniopExtSelectKernel.restype = c_int
    if hasattr(lib, "infiniopRandomSampleShardRecordBytes"):
        lib.infiniopRandomSampleShardRecordBytes.argtypes = []
        lib.infiniopRandomSampleShardRecordBytes.restype = c_uint64
    lib._b200_declared = True


KERNEL_FAMILIES = {"rope": 0, "random_sample": 1, "attention": 2, "matmul": 3, "long_rows": 4}


def select_kernel(lib, family, variant):
    """Forces one kernel family of an operator (tests and benchmarks): see
    infiniopExtSelectKernel in include/infiniop_ext.h.  variant 0 = the library's own choice."""
    _declare(lib)
    check_error(lib.infiniopExtSelectKernel(KERNEL_FAMILIES[family], int(variant)))


def device_timeouts(lib, handle):
    """Thread groups that gave up on a bounded wait since the library was loaded (synchronises);
    0 = every result so far is complete.  See infiniopExtDeviceTimeouts."""
    _declare(lib)
    n = c_uint64(0)
    check_error(lib.infiniopExtDeviceTimeouts(handle, ctypes.byref(n)))
    return n.value


def set_wait_limit(lib, handle, polls):
    """Polls per wait of the RoPE bulk-copy pipeline (0 = default); for the test that makes a wait run out."""
    _declare(lib)
    check_error(lib.infiniopExtSetWaitLimit(handle, int(polls)))


def _stream_ptr(stream):
    if stream is None:
        return None
    return getattr(stream, "cuda_stream", stream)


class _Op:
    """Common life cycle: descriptors of the tensors, operator descriptor, workspace."""

    _destroy = None
    _wsize = None

    def __init__(self, lib, handle):
        _declare(lib)
        self.lib, self.handle = lib, handle
        self.desc = _desc_t()
        self._tensor_descs = []
        self.workspace = None
        self.workspace_size = 0

    def _t(self, tensor, layout=None):
        ct = to_tensor(tensor, self.lib)
        if layout is not None:
            ct.descriptor.contents.dt = layout
        self._tensor_descs.append(ct.descriptor)
        return ct

    def _make_workspace(self, device):
        if self._wsize is None:
            return
        size = c_uint64(0)
        check_error(getattr(self.lib, self._wsize)(self.desc, ctypes.byref(size)))
        self.workspace_size = size.value
        self.workspace = create_workspace(size.value, device)

    def _ws_ptr(self):
        return self.workspace.data_ptr() if self.workspace is not None else None

    def destroy(self):
        if self.desc:
            check_error(getattr(self.lib, self._destroy)(self.desc))
            self.desc = _desc_t()
        for d in self._tensor_descs:
            destroy_tensor_descriptor(self.lib, d)
        self._tensor_descs = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()


class RMSNormOp(_Op):
    _destroy, _wsize = "infiniopDestroyRMSNormDescriptor", "infiniopGetRMSNormWorkspaceSize"

    def __init__(self, lib, handle, y, x, w, epsilon=1e-5):
        super().__init__(lib, handle)
        yt, xt, wt = self._t(y), self._t(x), self._t(w)
        check_error(lib.infiniopCreateRMSNormDescriptor(handle, ctypes.byref(self.desc), yt.descriptor,
                                                        xt.descriptor, wt.descriptor, epsilon))
        self._make_workspace(y.device)

    def __call__(self, y, x, w, stream=None):
        check_error(self.lib.infiniopRMSNorm(self.desc, self._ws_ptr(), self.workspace_size, y.data_ptr(),
                                             x.data_ptr(), w.data_ptr(), _stream_ptr(stream)))


class AddRMSNormOp(_Op):
    """sum = a + b, y = RMSNorm(sum) * w in one pass (an addition of this library: what the
    reference's callers get from its Add followed by its RMSNorm)."""
    _destroy, _wsize = "infiniopDestroyAddRMSNormDescriptor", "infiniopGetAddRMSNormWorkspaceSize"

    def __init__(self, lib, handle, y, total, a, b, w, epsilon=1e-5):
        super().__init__(lib, handle)
        ts = [self._t(x) for x in (y, total, a, b, w)]
        check_error(lib.infiniopCreateAddRMSNormDescriptor(handle, ctypes.byref(self.desc),
                                                           *[t.descriptor for t in ts], epsilon))
        self._make_workspace(y.device)

    def __call__(self, y, total, a, b, w, stream=None):
        check_error(self.lib.infiniopAddRMSNorm(self.desc, self._ws_ptr(), self.workspace_size, y.data_ptr(),
                                                total.data_ptr(), a.data_ptr(), b.data_ptr(), w.data_ptr(),
                                                _stream_ptr(stream)))


class RoPEOp(_Op):
    _destroy, _wsize = "infiniopDestroyRoPEDescriptor", "infiniopGetRoPEWorkspaceSize"

    def __init__(self, lib, handle, t, pos_ids, sin_table, cos_table):
        super().__init__(lib, handle)
        # position ids are u64 in the ABI; torch callers may hold them as int64
        tt, pt = self._t(t), self._t(pos_ids, U64)
        st, ct = self._t(sin_table), self._t(cos_table)
        check_error(lib.infiniopCreateRoPEDescriptor(handle, ctypes.byref(self.desc), tt.descriptor, pt.descriptor,
                                                     st.descriptor, ct.descriptor))
        self._make_workspace(t.device)

    def __call__(self, t, pos_ids, sin_table, cos_table, stream=None):
        check_error(self.lib.infiniopRoPE(self.desc, self._ws_ptr(), self.workspace_size, t.data_ptr(),
                                          pos_ids.data_ptr(), sin_table.data_ptr(), cos_table.data_ptr(),
                                          _stream_ptr(stream)))


class AttentionOp(_Op):
    """out[seq, n_q_head, dh] = attention of q[n_q_head, seq, dh] over the caches after k, v[n_kv_head, seq, dh]
    are written to their rows pos .. pos+seq (reference operatorspy/tests/attention.py; the position is part of
    the descriptor, as in the reference)."""
    _destroy, _wsize = "infiniopDestroyAttentionDescriptor", "infiniopGetAttentionWorkspaceSize"

    def __init__(self, lib, handle, out, q, k, v, k_cache, v_cache, pos):
        super().__init__(lib, handle)
        ts = [self._t(x) for x in (out, q, k, v, k_cache, v_cache)]
        check_error(lib.infiniopCreateAttentionDescriptor(handle, ctypes.byref(self.desc),
                                                          *[t.descriptor for t in ts], int(pos)))
        self._make_workspace(out.device)

    def __call__(self, out, q, k, v, k_cache, v_cache, stream=None):
        check_error(self.lib.infiniopAttention(self.desc, self._ws_ptr(), self.workspace_size, out.data_ptr(),
                                               q.data_ptr(), k.data_ptr(), v.data_ptr(), k_cache.data_ptr(),
                                               v_cache.data_ptr(), _stream_ptr(stream)))


class MatmulOp(_Op):
    """c = alpha * a @ b + beta * c on 2-D or batched 3-D tensors (reference operatorspy/tests/matmul.py)."""
    _destroy, _wsize = "infiniopDestroyMatmulDescriptor", "infiniopGetMatmulWorkspaceSize"

    def __init__(self, lib, handle, c, a, b, alpha=1.0, beta=0.0):
        super().__init__(lib, handle)
        ct, at, bt = self._t(c), self._t(a), self._t(b)
        check_error(lib.infiniopCreateMatmulDescriptor(handle, ctypes.byref(self.desc), ct.descriptor, alpha,
                                                       at.descriptor, bt.descriptor, beta))
        self._make_workspace(c.device)

    def __call__(self, c, a, b, stream=None):
        check_error(self.lib.infiniopMatmul(self.desc, self._ws_ptr(), self.workspace_size, c.data_ptr(), a.data_ptr(),
                                            b.data_ptr(), _stream_ptr(stream)))


class MLPOp(_Op):
    """y = (residual ? y : 0) + alpha * SwiGLU(x @ w12) @ w3 (reference operatorspy/tests/mlp.py)."""
    _destroy, _wsize = "infiniopDestroyMLPDescriptor", "infiniopGetMLPWorkspaceSize"

    def __init__(self, lib, handle, y, x, w12, w3, alpha=1.0, residual=True):
        super().__init__(lib, handle)
        ts = [self._t(t) for t in (y, x, w12, w3)]
        check_error(lib.infiniopCreateMLPDescriptor(handle, ctypes.byref(self.desc), *[t.descriptor for t in ts],
                                                    alpha, bytes([1 if residual else 0])))
        self._make_workspace(y.device)

    def __call__(self, y, x, w12, w3, stream=None):
        check_error(self.lib.infiniopMLP(self.desc, self._ws_ptr(), self.workspace_size, y.data_ptr(), x.data_ptr(),
                                         w12.data_ptr(), w3.data_ptr(), _stream_ptr(stream)))


class RoPERearrangeOp(_Op):
    """dst = RoPE(src) with dst a second view of the same shape (e.g. rows of the K cache); an
    addition of this library: the reference's RoPE followed by its rearrange."""
    _destroy, _wsize = "infiniopDestroyRoPERearrangeDescriptor", "infiniopGetRoPERearrangeWorkspaceSize"

    def __init__(self, lib, handle, dst, src, pos_ids, sin_table, cos_table):
        super().__init__(lib, handle)
        dt, st_, pt = self._t(dst), self._t(src), self._t(pos_ids, U64)
        sn, cs = self._t(sin_table), self._t(cos_table)
        check_error(lib.infiniopCreateRoPERearrangeDescriptor(handle, ctypes.byref(self.desc), dt.descriptor,
                                                              st_.descriptor, pt.descriptor, sn.descriptor,
                                                              cs.descriptor))
        self._make_workspace(dst.device)

    def __call__(self, dst, src, pos_ids, sin_table, cos_table, stream=None):
        check_error(self.lib.infiniopRoPERearrange(self.desc, self._ws_ptr(), self.workspace_size, dst.data_ptr(),
                                                   src.data_ptr(), pos_ids.data_ptr(), sin_table.data_ptr(),
                                                   cos_table.data_ptr(), _stream_ptr(stream)))


class SwiGLUOp(_Op):
    _destroy = "infiniopDestroySwiGLUDescriptor"

    def __init__(self, lib, handle, c, a, b):
        super().__init__(lib, handle)
        ct, at, bt = self._t(c), self._t(a), self._t(b)
        check_error(lib.infiniopCreateSwiGLUDescriptor(handle, ctypes.byref(self.desc), ct.descriptor, at.descriptor,
                                                       bt.descriptor))

    def __call__(self, c, a, b, stream=None):
        check_error(self.lib.infiniopSwiGLU(self.desc, c.data_ptr(), a.data_ptr(), b.data_ptr(), _stream_ptr(stream)))


class AddOp(_Op):
    _destroy = "infiniopDestroyAddDescriptor"

    def __init__(self, lib, handle, c, a, b):
        super().__init__(lib, handle)
        ct, at, bt = self._t(c), self._t(a), self._t(b)
        check_error(lib.infiniopCreateAddDescriptor(handle, ctypes.byref(self.desc), ct.descriptor, at.descriptor,
                                                    bt.descriptor))

    def __call__(self, c, a, b, stream=None):
        check_error(self.lib.infiniopAdd(self.desc, c.data_ptr(), a.data_ptr(), b.data_ptr(), _stream_ptr(stream)))

    def destroy(self):
        # The reference's CPU Add descriptor keeps a pointer into c's tensor
        # descriptor (reference src/ops/add/cpu/add_cpu.cc:55): destroy the
        # operator descriptor before the tensor descriptors.
        super().destroy()


class RearrangeOp(_Op):
    """dst[...] = src[...] between two views of equal shape and dtype (reference operatorspy/tests/rearrange.py)."""
    _destroy = "infiniopDestroyRearrangeDescriptor"

    def __init__(self, lib, handle, dst, src):
        super().__init__(lib, handle)
        dt, st = self._t(dst), self._t(src)
        check_error(lib.infiniopCreateRearrangeDescriptor(handle, ctypes.byref(self.desc), dt.descriptor, st.descriptor))

    def __call__(self, dst, src, stream=None):
        check_error(self.lib.infiniopRearrange(self.desc, dst.data_ptr(), src.data_ptr(), _stream_ptr(stream)))


class CausalSoftmaxOp(_Op):
    _destroy, _wsize = "infiniopDestroyCausalSoftmaxDescriptor", "infiniopGetCausalSoftmaxWorkspaceSize"

    def __init__(self, lib, handle, y):
        super().__init__(lib, handle)
        yt = self._t(y)
        check_error(lib.infiniopCreateCausalSoftmaxDescriptor(handle, ctypes.byref(self.desc), yt.descriptor))
        self._make_workspace(y.device)

    def __call__(self, y, stream=None):
        check_error(self.lib.infiniopCausalSoftmax(self.desc, self._ws_ptr(), self.workspace_size, y.data_ptr(),
                                                   _stream_ptr(stream)))


class RandomSampleOp(_Op):
    """One row of fp16 logits -> one u64 index (reference ABI), plus the batched
    extension when the library exports it."""

    _destroy, _wsize = "infiniopDestroyRandomSampleDescriptor", "infiniopGetRandomSampleWorkspaceSize"

    def __init__(self, lib, handle, result, probs):
        super().__init__(lib, handle)
        rt, pt = self._t(result, U64), self._t(probs)
        check_error(lib.infiniopCreateRandomSampleDescriptor(handle, ctypes.byref(self.desc), rt.descriptor,
                                                             pt.descriptor))
        self._make_workspace(probs.device)
        self._batch_ws = None
        self._batch_ws_size = 0

    def __call__(self, result, probs, random_val, topp, topk, temperature, stream=None):
        check_error(self.lib.infiniopRandomSample(self.desc, self._ws_ptr(), self.workspace_size, result.data_ptr(),
                                                  probs.data_ptr(), random_val, topp, topk, temperature,
                                                  _stream_ptr(stream)))

    def _ensure_batch_ws(self, rows, device):
        size = c_uint64(0)
        check_error(self.lib.infiniopGetRandomSampleBatchWorkspaceSize(self.desc, rows, ctypes.byref(size)))
        if self._batch_ws is None or self._batch_ws_size < size.value:
            self._batch_ws = create_workspace(size.value, device)
            self._batch_ws_size = size.value

    def batch(self, results, logits, random_vals, topp, topk, temperature, stream=None, trace=None):
        """results u64/int64 [rows], logits fp16 [rows, voc] (unit column stride),
        random_vals fp32 [rows], all on the device."""
        rows = logits.shape[0]
        self._ensure_batch_ws(rows, logits.device)
        args = [self.desc, self._batch_ws.data_ptr(), self._batch_ws_size, results.data_ptr(), logits.data_ptr(),
                logits.stride(0), rows, random_vals.data_ptr(), topp, topk, temperature]
        if trace is not None:
            check_error(self.lib.infiniopRandomSampleBatchTrace(*args, trace.data_ptr(), _stream_ptr(stream)))
        else:
            check_error(self.lib.infiniopRandomSampleBatch(*args, _stream_ptr(stream)))


    def batch_static(self, results, logits, random_vals, topp, topk, temperature, stream=None):
        """`batch` without a workspace: the library's built-in scratch array is
        used, nothing is allocated (see infiniopRandomSampleBatchStatic)."""
        check_error(self.lib.infiniopRandomSampleBatchStatic(
            self.desc, results.data_ptr(), logits.data_ptr(), logits.stride(0), logits.shape[0],
            random_vals.data_ptr(), topp, topk, temperature, _stream_ptr(stream)))


# ---- one-shot forms ----------------------------------------------------------

def attention(lib, handle, out, q, k, v, k_cache, v_cache, pos, stream=None):
    with AttentionOp(lib, handle, out, q, k, v, k_cache, v_cache, pos) as op:
        op(out, q, k, v, k_cache, v_cache, stream)


def matmul(lib, handle, c, a, b, alpha=1.0, beta=0.0, stream=None):
    with MatmulOp(lib, handle, c, a, b, alpha, beta) as op:
        op(c, a, b, stream)


def mlp(lib, handle, y, x, w12, w3, alpha=1.0, residual=True, stream=None):
    with MLPOp(lib, handle, y, x, w12, w3, alpha, residual) as op:
        op(y, x, w12, w3, stream)


def rope_rearrange(lib, handle, dst, src, pos_ids, sin_table, cos_table, stream=None):
    with RoPERearrangeOp(lib, handle, dst, src, pos_ids, sin_table, cos_table) as op:
        op(dst, src, pos_ids, sin_table, cos_table, stream)


def add_rms_norm(lib, handle, y, total, a, b, w, epsilon=1e-5, stream=None):
    with AddRMSNormOp(lib, handle, y, total, a, b, w, epsilon) as op:
        op(y, total, a, b, w, stream)


def rms_norm(lib, handle, y, x, w, epsilon=1e-5, stream=None):
    with RMSNormOp(lib, handle, y, x, w, epsilon) as op:
        op(y, x, w, stream)


def rope(lib, handle, t, pos_ids, sin_table, cos_table, stream=None):
    with RoPEOp(lib, handle, t, pos_ids, sin_table, cos_table) as op:
        op(t, pos_ids, sin_table, cos_table, stream)


def swiglu(lib, handle, c, a, b, stream=None):
    with SwiGLUOp(lib, handle, c, a, b) as op:
        op(c, a, b, stream)


def add(lib, handle, c, a, b, stream=None):
    with AddOp(lib, handle, c, a, b) as op:
        op(c, a, b, stream)


def rearrange(lib, handle, dst, src, stream=None):
    with RearrangeOp(lib, handle, dst, src) as op:
        op(dst, src, stream)


def causal_softmax(lib, handle, y, stream=None):
    with CausalSoftmaxOp(lib, handle, y) as op:
        op(y, stream)


def random_sample(lib, handle, result, probs, random_val, topp, topk, temperature, stream=None):
    with RandomSampleOp(lib, handle, result, probs) as op:
        op(result, probs, random_val, topp, topk, temperature, stream)


def sin_cos_table(max_seq_len, dim, theta=1e4, device="cpu"):
    """fp32 sin/cos tables [max_seq_len, dim] with pair-duplicated frequencies,
    the layout the RoPE entry point consumes (same construction as the
    reference's test helper, reference operatorspy/tests/rotary_embedding.py:54-64)."""
    import torch

    pos = torch.arange(0, max_seq_len, dtype=torch.float32, device=device)
    freqs = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device)[: dim // 2].float() / dim))
    freqs = torch.repeat_interleave(freqs, repeats=2)
    angles = torch.outer(pos, freqs)
    return torch.sin(angles), torch.cos(angles)
