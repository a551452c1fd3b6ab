"""numpy front end of the C oracle (cpu_oracle.c).

TEST INFRASTRUCTURE: the checker the CUDA kernels are compared with and the
timed CPU baseline.  Arrays are numpy; fp16 data travels as uint16 bit
patterns or float16 arrays (viewed, never converted).  Every function states
the reference file it restates in cpu_oracle.c.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    """Compile liboracle.so (and, where the reference checkout exists, the
    reference's own CPU backend into _ref/) with the Makefile next to this file."""
    so = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "cpu_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", HERE, "all"], check=True)
    return so


def build_reference():
    """Compile the reference's CPU backend from its own sources when they are
    present; returns the path of the library or None."""
    subprocess.run(["make", "-s", "-C", HERE, "ref"], check=False, capture_output=True)
    p = os.path.join(HERE, "_ref", "lib", "libinfiniop.so")
    return p if os.path.exists(p) else None


def reference_lib_dir():
    p = os.path.join(HERE, "_ref", "lib")
    return p if os.path.exists(os.path.join(p, "libinfiniop.so")) else None


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        vp, u64, i64, ci, cf = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        L.oracle_f16_to_f32.argtypes, L.oracle_f16_to_f32.restype = [ctypes.c_uint16], cf
        L.oracle_f32_to_f16.argtypes, L.oracle_f32_to_f16.restype = [cf], ctypes.c_uint16
        L.oracle_rms_norm_f16.argtypes = [vp, vp, vp, u64, u64, i64, i64, ci, cf]
        L.oracle_rope_f16.argtypes = [vp, vp, vp, vp, u64, u64, u64, i64, i64]
        L.oracle_swiglu_f16.argtypes = [vp, vp, vp, u64, u64, i64, i64, i64]
        L.oracle_add.argtypes = [vp, vp, vp, ci, u64, vp, vp, vp]
        L.oracle_rearrange.argtypes = [vp, vp, u64, u64, vp, vp, vp]
        L.oracle_causal_softmax_f16.argtypes = [vp, u64, u64, u64, i64, i64, i64]
        L.oracle_matmul_f16.argtypes, L.oracle_matmul_f16.restype = [vp, vp, vp, cf, u64, u64, u64, u64, vp, vp, vp], None
        L.oracle_matmul_f16_beta.argtypes = [vp, vp, vp, cf, cf, u64, u64, u64, u64, vp, vp, vp]
        L.oracle_matmul_f16_beta.restype = None
        L.oracle_matmul_f32.argtypes, L.oracle_matmul_f32.restype = [vp, vp, vp, cf, cf, u64, u64, u64, u64, vp, vp, vp], None
        L.oracle_set_storage.argtypes, L.oracle_set_storage.restype = [ci], None
        L.oracle_random_sample_f16.argtypes = [vp, vp, vp, ci, cf, cf, ci, cf]
        L.oracle_random_sample_workspace.argtypes, L.oracle_random_sample_workspace.restype = [ci], u64
        L.oracle_random_sample_trace.argtypes = [vp, vp, ci, ci, cf, vp, vp, vp, vp]
        for f in ("oracle_rms_norm_f16", "oracle_rope_f16", "oracle_swiglu_f16", "oracle_add",
                  "oracle_causal_softmax_f16", "oracle_random_sample_f16", "oracle_random_sample_trace"):
            getattr(L, f).restype = None
        _LIB = L
    return _LIB


class bf16_storage:
    """`with bf16_storage():` makes rms_norm / rope / swiglu / add / causal_softmax called from THIS thread read and
    write bf16 bit patterns (uint16 arrays) instead of fp16: the extension's oracle, the same restated arithmetic
    with bf16 decode and truncating encode.  The reference itself has no bf16 operator."""

    def __enter__(self):
        lib().oracle_set_storage(1)

    def __exit__(self, *exc):
        lib().oracle_set_storage(0)


def _u16(a):
    a = np.asarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return a


def _ptr(a):
    return a.ctypes.data


def _elem_strides(a):
    return [s // a.itemsize for s in a.strides]


def f32_to_f16(x):
    """Truncating fp32 -> fp16 of the reference (src/devices/cpu/common_cpu.cc:41-64)."""
    L = lib()
    x = np.asarray(x, np.float32)
    return np.array([L.oracle_f32_to_f16(float(v)) for v in x.ravel()], np.uint16).reshape(x.shape)


def f16_to_f32(h):
    L = lib()
    h = _u16(h)
    return np.array([L.oracle_f16_to_f32(int(v)) for v in h.ravel()], np.float32).reshape(h.shape)


def rms_norm(x, w, epsilon=1e-5, y=None):
    """x [n,d] fp16 (unit column stride, any row stride), w [d] fp16 or fp32 -> y fp16.
    src/ops/rms_norm/cpu/rms_norm_cpu.cc:46-86."""
    xu = _u16(x)
    n, d = xu.shape
    assert _elem_strides(xu)[1] == 1
    w = np.ascontiguousarray(w)
    w_is_f16 = w.dtype in (np.float16, np.uint16)
    if not w_is_f16:
        assert w.dtype == np.float32
    out = np.zeros((n, d), np.uint16) if y is None else _u16(y)
    lib().oracle_rms_norm_f16(_ptr(out), _ptr(xu), _ptr(w), n, d, _elem_strides(out)[0], _elem_strides(xu)[0],
                              int(w_is_f16), epsilon)
    return out.view(np.float16)


def rope(t, pos_ids, sin_table, cos_table):
    """In place on t [nt, nh, dh] fp16 (unit last stride); pos_ids uint64 [nt];
    tables fp32 [*, dh] contiguous.  src/ops/rotary_embedding/cpu/rotary_embedding_cpu.cc:16-44."""
    tu = _u16(t)
    nt, nh, dh = tu.shape
    s = _elem_strides(tu)
    assert s[2] == 1
    pos = np.ascontiguousarray(pos_ids, np.uint64)
    sin_table = np.ascontiguousarray(sin_table, np.float32)
    cos_table = np.ascontiguousarray(cos_table, np.float32)
    lib().oracle_rope_f16(_ptr(tu), _ptr(pos), _ptr(sin_table), _ptr(cos_table), nt, nh, dh, s[0], s[1])
    return t


def swiglu(a, b, c=None):
    """c = a * silu(b); 2-D fp16, unit column stride.  src/ops/swiglu/cpu/swiglu_cpu.cc:49-73."""
    au, bu = _u16(a), _u16(b)
    n, d = au.shape
    out = np.zeros((n, d), np.uint16) if c is None else _u16(c)
    assert _elem_strides(au)[1] == 1 and _elem_strides(bu)[1] == 1 and _elem_strides(out)[1] == 1
    lib().oracle_swiglu_f16(_ptr(out), _ptr(au), _ptr(bu), n, d, _elem_strides(out)[0], _elem_strides(au)[0],
                            _elem_strides(bu)[0])
    return out.view(np.float16)


def add(a, b):
    """Broadcasting add of contiguous fp16 / fp32 arrays.  src/ops/add/cpu/add_cpu.cc:18-89."""
    a = np.asarray(a, order="C")
    b = np.asarray(b, order="C")
    is_f16 = a.dtype in (np.float16, np.uint16)  # uint16: 16-bit patterns (bf16 inside `with bf16_storage()`)
    assert a.dtype == b.dtype and a.dtype in (np.float16, np.uint16, np.float32)
    shape = np.broadcast_shapes(a.shape, b.shape)
    nd = len(shape)
    out = np.zeros(shape, a.dtype)

    def adj(x):
        st = _elem_strides(x)
        res = []
        for i in range(nd):
            k = i - (nd - x.ndim)
            res.append(0 if (k < 0 or x.shape[k] != shape[i]) else st[k])
        return (ctypes.c_int64 * max(nd, 1))(*res)

    cshape = (ctypes.c_uint64 * max(nd, 1))(*shape)
    sa, sb = adj(a), adj(b)  # keep the arrays alive across the call
    lib().oracle_add(_ptr(out), _ptr(a), _ptr(b), int(is_f16), nd, ctypes.addressof(cshape),
                     ctypes.addressof(sa), ctypes.addressof(sb))
    return out


def rearrange(dst, src):
    """dst[...] = src[...]: numpy views of equal shape and itemsize with unit innermost stride (the arrays' own
    strides are used, so pass the strided views themselves).  src/ops/rearrange/cpu/rearrange_cpu.cc:70-100."""
    assert dst.shape == src.shape and dst.itemsize == src.itemsize and dst.ndim >= 1
    nd = dst.ndim
    sd, ss = _elem_strides(dst), _elem_strides(src)
    assert sd[-1] == 1 and ss[-1] == 1
    cshape = (ctypes.c_uint64 * nd)(*dst.shape)
    csd, css = (ctypes.c_int64 * nd)(*sd), (ctypes.c_int64 * nd)(*ss)
    lib().oracle_rearrange(dst.ctypes.data, src.ctypes.data, dst.itemsize, nd, ctypes.addressof(cshape),
                           ctypes.addressof(csd), ctypes.addressof(css))
    return dst


def causal_softmax(y):
    """In place on fp16 [batch, seq, total] or [seq, total].  src/ops/causal_softmax/cpu/causal_softmax_cpu.cc:52-82."""
    yu = _u16(y)
    s = _elem_strides(yu)
    if yu.ndim == 2:
        batch, sb = 1, 0
    else:
        batch, sb = yu.shape[0], s[0]
    lib().oracle_causal_softmax_f16(_ptr(yu), batch, yu.shape[-2], yu.shape[-1], sb, s[-2], s[-1])
    return y


def matmul(a, b, alpha=1.0):
    """fp16 [batch, m, k] x [batch, k, n] -> contiguous fp16 [batch, m, n] (the arrays' own strides are used).
    src/ops/matmul/cpu/matmul_cpu.cc:44-78 with beta = 0."""
    au, bu = _u16(a), _u16(b)
    assert au.ndim == 3 and bu.ndim == 3 and au.shape[0] == bu.shape[0] and au.shape[2] == bu.shape[1]
    c = np.zeros((au.shape[0], au.shape[1], bu.shape[2]), np.uint16)
    sc, sa, sb = ((ctypes.c_int64 * 3)(*_elem_strides(x)) for x in (c, au, bu))
    lib().oracle_matmul_f16(_ptr(c), _ptr(au), _ptr(bu), float(alpha), au.shape[0], au.shape[1], bu.shape[2],
                            au.shape[2], ctypes.addressof(sc), ctypes.addressof(sa), ctypes.addressof(sb))
    return c.view(np.float16)


def matmul_into(c, a, b, alpha=1.0, beta=0.0):
    """c = alpha * a @ b + beta * c in place on numpy views (2-D or batched 3-D, fp16 or fp32, the arrays' own
    strides; a and b may have batch 1 against a batched c).  src/ops/matmul/cpu/matmul_cpu.cc:44-78."""
    c3, a3, b3 = (x if x.ndim == 3 else x[None] for x in (c, a, b))
    batch, m, n = c3.shape
    k = a3.shape[2]
    assert a3.shape[1:] == (m, k) and b3.shape[1:] == (k, n) and a3.shape[0] in (1, batch) and b3.shape[0] in (1, batch)

    def strides(x):
        st = _elem_strides(x)
        if x.shape[0] == 1:
            st[0] = 0
        return (ctypes.c_int64 * 3)(*st)

    sc, sa, sb = strides(c3), strides(a3), strides(b3)
    if c.dtype == np.float32:
        assert a.dtype == np.float32 and b.dtype == np.float32
        lib().oracle_matmul_f32(_ptr(c3), _ptr(a3), _ptr(b3), float(alpha), float(beta), batch, m, n, k,
                                ctypes.addressof(sc), ctypes.addressof(sa), ctypes.addressof(sb))
    else:
        cu, au, bu = _u16(c3), _u16(a3), _u16(b3)
        lib().oracle_matmul_f16_beta(_ptr(cu), _ptr(au), _ptr(bu), float(alpha), float(beta), batch, m, n, k,
                                     ctypes.addressof(sc), ctypes.addressof(sa), ctypes.addressof(sb))
    return c


def mlp(y, x, w12, w3, alpha=1.0, residual=True):
    """The MLP composite, src/ops/mlp/operator.cc:22-122, with the operators above: gate_up = x @ w12 stored as
    fp16, act = up * silu(gate) on its column halves (gate first), y = alpha * act @ w3 (+ y).  In place on y."""
    tokens, di = x.shape[0], w12.shape[1] // 2
    gate_up = np.zeros((tokens, 2 * di), x.dtype)  # fp16, or 16-bit patterns inside `with bf16_storage()`
    matmul_into(gate_up, x, w12)
    act = swiglu(gate_up[:, di:], gate_up[:, :di])
    matmul_into(y, act, w3, alpha, 1.0 if residual else 0.0)
    return y


def attention(q, k, v, k_cache, v_cache, pos):
    """The attention composite, src/ops/attention/operator.cc:30-305, step by step with the
    operators above: k and v copied into the caches at row `pos`, q made contiguous,
    qk = matmul(q, full_k^T) * 1/sqrt(dh) with the q heads of one kv head stacked as rows,
    causal softmax in place, matmul with full_v, rows permuted to out[seq, n_q_head, dh].
    q [n_q_head, seq, dh], k and v [n_kv_head, seq, dh], caches [n_kv_head, buf_len, dh]
    (numpy fp16 views, unit innermost stride); the caches are updated in place."""
    nh, seq, dh = q.shape
    nkvh = k.shape[0]
    assert nh % nkvh == 0 and k.shape == v.shape == (nkvh, seq, dh)
    group, total = nh // nkvh, seq + pos
    rearrange(k_cache[:, pos:total, :], k)
    rearrange(v_cache[:, pos:total, :], v)
    qc = np.zeros(q.shape, np.float16)
    rearrange(qc, q)
    alpha = np.float32(1 / np.sqrt(np.float64(dh)))  # `float qk_alpha = 1 / sqrt(head_dim)`, operator.cc:136
    qk = matmul(qc.reshape(nkvh, group * seq, dh), k_cache[:, :total, :].transpose(0, 2, 1), alpha)
    qk = qk.reshape(nh, seq, total)
    causal_softmax(qk)
    temp = matmul(qk.reshape(nkvh, group * seq, total), v_cache[:, :total, :])
    out = np.zeros((seq, nh, dh), np.float16)
    rearrange(out, temp.reshape(nh, seq, dh).transpose(1, 0, 2))
    return out


def random_sample(logits, random_val, topp, topk, temperature, previous=0):
    """One row of fp16 logits -> sampled index (int).  `previous` is what the
    result slot held before the call: the reference leaves it untouched when no
    candidate satisfies the draw.  src/ops/random_sample/cpu/random_sample.cc:45-185."""
    lu = np.ascontiguousarray(_u16(logits))
    voc = lu.size
    ws = np.zeros(int(lib().oracle_random_sample_workspace(voc)), np.uint8)
    res = np.array([previous], np.uint64)
    lib().oracle_random_sample_f16(_ptr(res), _ptr(lu), _ptr(ws), voc, random_val, topp, topk, temperature)
    return int(res[0])


def random_sample_trace(logits, topk, temperature):
    """Top-k (indices, fp16 values), fp32 denominator S and truncated fp16
    probabilities of the sampling branch, plus the permuted row."""
    lu = np.ascontiguousarray(_u16(logits))
    voc = lu.size
    k = min(topk, voc)
    ws = np.zeros(int(lib().oracle_random_sample_workspace(voc)), np.uint8)
    ti, tv = np.zeros(k, np.uint64), np.zeros(k, np.uint16)
    den, tp = np.zeros(1, np.float32), np.zeros(k, np.uint16)
    lib().oracle_random_sample_trace(_ptr(lu), _ptr(ws), voc, topk, temperature, _ptr(ti), _ptr(tv), _ptr(den), _ptr(tp))
    return {"top_idx": ti, "top_val": tv.view(np.float16), "denom": den[0], "top_p": tp.view(np.float16)}
