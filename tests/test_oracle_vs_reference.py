"""The C oracle must reproduce the reference's own CPU backend bit for bit.

The reference library (compiled from its sources into oracle/_ref, see
oracle/Makefile) is called through its C ABI exactly as its test scripts do
(reference operatorspy/tests/*.py); the oracle is called on the same seeded
inputs; outputs are compared as raw bit patterns.
"""
import numpy as np
import pytest
import torch

from operators_b200 import ops
from operators_b200.utils import rearrange_tensor


def _bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("w_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(16, 2048), (5, 33), (1, 1)])
def test_rms_norm(oracle, ref_cpu, shape, w_dtype):
    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(1)
    x = (torch.rand(shape, generator=g) * 2 - 1).half()
    w = (torch.rand(shape[1], generator=g) * 2 - 1).to(w_dtype)
    y = torch.zeros(shape, dtype=torch.float16)
    ops.rms_norm(lib, handle, y, x, w, 1e-5)
    mine = oracle.rms_norm(x.numpy(), w.numpy(), 1e-5)
    assert np.array_equal(mine.view(np.uint16), _bits(y))


@pytest.mark.parametrize("shape,strides", [((7, 4, 32), None), ((3, 32, 128), (8000, 200, 1)), ((4, 1, 2), None)])
def test_rope(oracle, ref_cpu, shape, strides):
    from operators_b200 import rearrange_tensor

    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(2)
    t = torch.randn(shape, generator=g).half()
    if strides is not None:
        t = rearrange_tensor(t, strides)
    pos = torch.randperm(2 * shape[0], generator=g)[: shape[0]].to(torch.int64)
    sin, cos = ops.sin_cos_table(2 * shape[0], shape[2])
    t_np = t.numpy().copy() if strides is None else None
    expect_in = t.clone()
    ops.rope(lib, handle, t, pos, sin, cos)
    # oracle on an identically laid out copy
    if strides is None:
        mine = oracle.rope(t_np, pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
        assert np.array_equal(mine.view(np.uint16), _bits(t).reshape(shape))
    else:
        buf = rearrange_tensor(expect_in, strides)
        arr = np.lib.stride_tricks.as_strided(
            buf.numpy(), shape=shape, strides=[s * 2 for s in strides], writeable=True)
        oracle.rope(arr, pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
        assert np.array_equal(np.ascontiguousarray(arr).view(np.uint16), _bits(t).reshape(shape))


@pytest.mark.parametrize("shape,stride", [((13, 4), None), ((13, 4), 10), ((16, 5632), None), ((16, 5632), 13312)])
def test_swiglu(oracle, ref_cpu, shape, stride):
    from operators_b200 import rearrange_tensor

    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(3)
    a = torch.randn(shape, generator=g).half()
    b = (torch.randn(shape, generator=g) * 4).half()
    if stride is not None:
        a, b = rearrange_tensor(a, (stride, 1)), rearrange_tensor(b, (stride, 1))
    c = torch.zeros(shape, dtype=torch.float16)
    ops.swiglu(lib, handle, c, a, b)
    mine = oracle.swiglu(a.contiguous().numpy(), b.contiguous().numpy())
    assert np.array_equal(mine.view(np.uint16), _bits(c))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shapes", [((), (), ()), ((3, 3), (3, 3), (3, 3)), ((2, 20, 3), (2, 1, 3), (2, 20, 3)),
                                    ((4, 5, 6), (6,), (4, 5, 6)), ((2, 3, 4, 5), (2, 3, 4, 5), (2, 3, 4, 5))])
def test_add(oracle, ref_cpu, shapes, dtype):
    lib, handle = ref_cpu
    cs, as_, bs = shapes[2], shapes[0], shapes[1]
    g = torch.Generator().manual_seed(4)
    a = (torch.randn(as_, generator=g) * 100).to(dtype)
    b = torch.randn(bs, generator=g).to(dtype)
    c = torch.zeros(cs, dtype=dtype)
    ops.add(lib, handle, c, a, b)
    mine = oracle.add(a.numpy(), b.numpy())
    if dtype == torch.float16:
        assert np.array_equal(mine.view(np.uint16).reshape(cs), _bits(c).reshape(cs))
    else:
        assert np.array_equal(mine.reshape(cs), c.numpy())


# the reference's own cases (reference operatorspy/tests/rearrange.py:109-117) plus 1-D, 2-D, 4-D and fp32
REARRANGE_CASES = [
    (((2, 4, 32), None), ((2, 4, 32), (256, 64, 1)), torch.float16),
    (((32, 6, 64), (64, 2560, 1)), ((32, 6, 64), None), torch.float16),
    (((4, 6, 64), (64, 2560, 1)), ((4, 6, 64), (131072, 64, 1)), torch.float16),
    (((1, 32, 64), (2048, 64, 1)), ((1, 32, 64), (2048, 64, 1)), torch.float16),
    (((32, 1, 64), (64, 2560, 1)), ((32, 1, 64), (64, 64, 1)), torch.float16),
    (((4, 1, 64), (64, 2560, 1)), ((4, 1, 64), (64, 11264, 1)), torch.float16),
    (((77,), None), ((77,), None), torch.float16),
    (((5, 33), (40, 1)), ((5, 33), None), torch.float32),
    (((2, 3, 4, 8), None), ((2, 3, 4, 8), None), torch.float16),
]


@pytest.mark.parametrize("src_spec,dst_spec,dtype", REARRANGE_CASES)
def test_rearrange(oracle, ref_cpu, src_spec, dst_spec, dtype):
    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(9)
    x = torch.rand(src_spec[0], generator=g).to(dtype)
    y = torch.zeros(dst_spec[0], dtype=dtype)
    if src_spec[1] is not None:
        x = rearrange_tensor(x, src_spec[1])
    if dst_spec[1] is not None:
        y = rearrange_tensor(y, dst_spec[1])
    y2 = y.clone() if dst_spec[1] is None else rearrange_tensor(torch.zeros(dst_spec[0], dtype=dtype), dst_spec[1])
    ops.rearrange(lib, handle, y, x)
    oracle.rearrange(y2.numpy(), x.numpy())
    assert torch.equal(y, x) and torch.equal(y2, y)


# the reference's three attention cases (operatorspy/tests/attention.py:310-357) and two more
ATTENTION_CASES = [
    (32, 4, 5, 64, 0, 2048, (64, 2560, 1), (64, 11264, 1)),
    (32, 4, 1, 64, 3, 2048, (64, 2560, 1), (64, 11264, 1)),
    (8, 4, 2, 16, 1, 8, None, None),
    (8, 8, 3, 32, 40, 64, None, None),
    (12, 2, 1, 128, 200, 256, None, None),
]


def make_attention_inputs(nh, nkvh, seq, dh, pos, buf_len, qkv_strides, cache_strides, seed=21):
    g = torch.Generator().manual_seed(seed)
    q = (torch.rand((nh, seq, dh), generator=g) * 0.1).half()
    k = (torch.rand((nkvh, seq, dh), generator=g) * 0.1).half()
    v = (torch.rand((nkvh, seq, dh), generator=g) * 0.1).half()
    k_cache = (torch.rand((nkvh, buf_len, dh), generator=g) * 0.1).half()
    v_cache = (torch.rand((nkvh, buf_len, dh), generator=g) * 0.1).half()
    if qkv_strides is not None:
        q, k, v = (rearrange_tensor(t, qkv_strides) for t in (q, k, v))
    if cache_strides is not None:
        k_cache, v_cache = (rearrange_tensor(t, cache_strides) for t in (k_cache, v_cache))
    return q, k, v, k_cache, v_cache


@pytest.mark.parametrize("nh,nkvh,seq,dh,pos,buf_len,qkv_strides,cache_strides", ATTENTION_CASES)
def test_attention(oracle, ref_cpu, nh, nkvh, seq, dh, pos, buf_len, qkv_strides, cache_strides):
    """The composite of the reference CPU build (rearranges, two matmuls, causal softmax) and the
    oracle's step-by-step restatement write the same bits to out and to both caches."""
    lib, handle = ref_cpu
    q, k, v, k_cache, v_cache = make_attention_inputs(nh, nkvh, seq, dh, pos, buf_len, qkv_strides, cache_strides)
    kc2, vc2 = k_cache.clone(), v_cache.clone()
    if cache_strides is not None:
        kc2, vc2 = rearrange_tensor(kc2, cache_strides), rearrange_tensor(vc2, cache_strides)
    out = torch.zeros((seq, nh, dh), dtype=torch.float16)
    ops.attention(lib, handle, out, q, k, v, k_cache, v_cache, pos)
    mine = oracle.attention(q.numpy(), k.numpy(), v.numpy(), kc2.numpy(), vc2.numpy(), pos)
    assert np.array_equal(mine.view(np.uint16), _bits(out).reshape(out.shape))
    assert torch.equal(kc2, k_cache) and torch.equal(vc2, v_cache)


# the reference's own matmul cases (operatorspy/tests/matmul.py:296-308) and a few ragged / broadcast ones
MATMUL_CASES = [
    (1.0, 0.0, (1, 2048), (2048, 2048), (1, 2048), None, None, None),
    (1.0, 0.0, (2, 4, 2048), (2, 2048, 2048), (2, 4, 2048), None, None, None),
    (1.0, 0.0, (1, 2048), (2048, 2048), (1, 2048), (4096, 1), (4096, 1), (4096, 1)),
    (1.0, 1.0, (6, 2048), (2048, 2560), (6, 2560), (2048, 1), (1, 2048), (2560, 1)),
    (1.0 / 8.0, 0.0, (4, 8 * 6, 64), (4, 64, 6), (4, 8 * 6, 6), None, None, None),
    (0.5, 2.0, (37, 100), (100, 19), (37, 19), (1, 37), None, (1, 40)),
    (1.0, 0.0, (3, 9, 40), (1, 40, 24), (3, 9, 24), None, None, None),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("alpha,beta,a_shape,b_shape,c_shape,a_stride,b_stride,c_stride", MATMUL_CASES)
def test_matmul(oracle, ref_cpu, alpha, beta, a_shape, b_shape, c_shape, a_stride, b_stride, c_stride, dtype):
    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(8)
    a, b, c = (torch.rand(s, generator=g).to(dtype) for s in (a_shape, b_shape, c_shape))
    a, b, c = (t if st is None else rearrange_tensor(t, st) for t, st in ((a, a_stride), (b, b_stride), (c, c_stride)))
    mine = c.clone()
    if c_stride is not None:
        mine = rearrange_tensor(mine, c_stride)
    oracle.matmul_into(mine.numpy(), a.numpy(), b.numpy(), alpha, beta)
    ops.matmul(lib, handle, c, a, b, alpha, beta)
    assert torch.equal(mine.view(torch.int16 if dtype == torch.float16 else torch.int32),
                       c.view(torch.int16 if dtype == torch.float16 else torch.int32))


@pytest.mark.parametrize("tokens,hidden,di,alpha,residual,x_stride,w12_stride,w3_stride", [
    (4, 256, 688, 1.0, True, None, None, None), (4, 256, 688, 1.0, False, (512, 1), None, None),
    (3, 128, 344, 0.5, True, None, (1, 128), (1, 344)), (2, 4096, 11008, 1.0, True, None, None, None)])
def test_mlp(oracle, ref_cpu, tokens, hidden, di, alpha, residual, x_stride, w12_stride, w3_stride):
    """The reference composite (src/ops/mlp/operator.cc) and the oracle's restatement of its three steps write
    the same bits (shapes of operatorspy/tests/mlp.py:245-, scaled down except for the last)."""
    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(9)
    y = (torch.rand((tokens, hidden), generator=g) * 0.01).half()
    x = (torch.rand((tokens, hidden), generator=g) * 0.01).half()
    w12 = (torch.rand((hidden, 2 * di), generator=g) * 0.01).half()
    w3 = (torch.rand((di, hidden), generator=g) * 0.01).half()
    if x_stride is not None:
        x, y = rearrange_tensor(x, x_stride), rearrange_tensor(y, x_stride)
    if w12_stride is not None:
        w12, w3 = rearrange_tensor(w12, w12_stride), rearrange_tensor(w3, w3_stride)
    mine = y.clone()
    if x_stride is not None:
        mine = rearrange_tensor(mine, x_stride)
    oracle.mlp(mine.numpy(), x.numpy(), w12.numpy(), w3.numpy(), alpha, residual)
    ops.mlp(lib, handle, y, x, w12, w3, alpha, residual)
    assert torch.equal(mine.view(torch.int16), y.view(torch.int16))


@pytest.mark.parametrize("shape", [(32, 20, 512), (5, 64), (2, 7, 7), (3, 1, 9)])
def test_causal_softmax(oracle, ref_cpu, shape):
    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(5)
    y = (torch.randn(shape, generator=g) * 2).half()
    mine = oracle.causal_softmax(y.numpy().copy())
    ops.causal_softmax(lib, handle, y)
    assert np.array_equal(mine.view(np.uint16), _bits(y).reshape(shape))


@pytest.mark.parametrize("voc,u,topp,topk,temp", [
    (512, 0.92, 0.8, 3, 0.5), (4096, 0.95, 0.9, 5, 1.0), (16384, 0.85, 0.85, 10, 2.0),
    (512, 0.92, 0.0, 3, 0.5), (4096, 0.95, 0.9, 1, 1.0), (3000, 0.3, 0.9, 50, 0.8), (40, 0.5, 1.0, 64, 1.0)])
@pytest.mark.parametrize("dist", ["uniform", "normal3"])
def test_random_sample(oracle, ref_cpu, voc, u, topp, topk, temp, dist):
    lib, handle = ref_cpu
    g = torch.Generator().manual_seed(6)
    for _ in range(3):
        logits = torch.rand(voc, generator=g).half() if dist == "uniform" else (torch.randn(voc, generator=g) * 3).half()
        res = torch.zeros(1, dtype=torch.int64)
        ops.random_sample(lib, handle, res, logits, u, topp, topk, temp)
        assert oracle.random_sample(logits.numpy(), u, topp, topk, temp) == int(res[0])


def test_f32_to_f16_rule(oracle):
    """Truncation, subnormals, flush to zero and the out-of-range bit patterns
    of the reference conversion (src/devices/cpu/common_cpu.cc:41-64)."""
    cases = {1.0: 0x3C00, 1.0009765: 0x3C00, 1.00097656255: 0x3C01, -2.5: 0xC100, 65504.0: 0x7BFF, 65519.9: 0x7BFF,
             6e-8: 0x0001, 5.9e-8: 0x0000, -5.9e-8: 0x8000, float("inf"): 0x7C00, 65536.0: 0x7C00, 131072.0: 0x8000}
    for v, bits in cases.items():
        assert int(oracle.f32_to_f16(np.float32(v))) == bits, (v, hex(bits))
