"""Parity of the sm_100a kernels with the CPU oracle, through the C ABI.

Tolerances are the ones the task states: fp16 outputs within atol = rtol = 1e-3
(causal softmax 2e-3) of the reference CPU path, Add and RoPE bit-exact,
sampled indices identical for the same uniform draw.  Shapes cover the
reference's own test cases (reference operatorspy/tests/*.py) and ragged /
unaligned / strided / in-place variants.
"""
import os

import numpy as np
import pytest
import torch

from operators_b200 import ops, rearrange_tensor

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _close(got_bits, want_f16, atol, rtol):
    got = got_bits.view(np.float16).astype(np.float32)
    want = want_f16.astype(np.float32)
    err = np.abs(got - want)
    tol = atol + rtol * np.abs(want)
    assert (err <= tol).all(), "max err %g at %s" % (err.max(), np.unravel_index(err.argmax(), err.shape))
    return int((got_bits.reshape(-1) != want_f16.view(np.uint16).reshape(-1)).sum())


def _few(mismatches, total, rate):
    """Bitwise mismatches (each within tolerance) stay a small fraction."""
    return mismatches <= max(3, rate * total)


# ---- RMSNorm -----------------------------------------------------------------
@pytest.mark.parametrize("w_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape,stride", [((16, 2048), None), ((16, 2048), 4096), ((5, 33), None), ((1, 8), None),
                                          ((700, 4096), None), ((2048, 2048), None), ((3, 16384), None),
                                          ((2, 70000), None), ((9, 264), 272),
                                          # rows spread over a cluster of 2 / 4 / 8 CTAs (few rows: one vector per
                                          # thread; many rows: four), the longest register-resident row, one past it
                                          ((2, 49152), None), ((2, 65536), None), ((600, 16384), None),
                                          ((300, 32768), 32776), ((3, 200000), None), ((2, 262144), None),
                                          ((2, 262152), None), ((1, 8200), None)])
@pytest.mark.parametrize("long_rows", ["auto", "ring"])
def test_rms_norm(oracle, cuda_lib, shape, stride, w_dtype, long_rows):
    lib, handle = cuda_lib
    if long_rows == "ring" and shape[1] < 4096:
        pytest.skip("the shared-memory ring starts at rows of 4096 elements")
    g = torch.Generator().manual_seed(1)
    x = (torch.rand(shape, generator=g) * 2 - 1).half()
    w = (torch.rand(shape[1], generator=g) * 2 - 1).to(w_dtype)
    want = oracle.rms_norm(x.numpy(), w.numpy(), 1e-5)
    xd = x.to(DEV)
    yd = torch.full(shape, 7.0, dtype=torch.float16, device=DEV)
    if stride is not None:
        xd, yd = rearrange_tensor(xd, (stride, 1)), rearrange_tensor(yd, (stride, 1))
    ops.select_kernel(lib, "long_rows", 2 if long_rows == "ring" else 0)  # the ring wherever it can run, or the library's choice
    try:
        ops.rms_norm(lib, handle, yd, xd, w.to(DEV), 1e-5)
        torch.cuda.synchronize()
    finally:
        ops.select_kernel(lib, "long_rows", 0)
    mism = _close(_bits(yd).reshape(shape), want, 1e-3, 1e-3)
    # only the order of the fp32 sum of squares differs; the oracle's sequential sum over rows of 10^5 elements
    # and more is itself a few fp32 ulps off, which moves a few per cent of the outputs by one fp16 ulp
    assert _few(mism, x.numel(), 0.02 if shape[1] <= 65536 else 0.06)


# ---- fused residual add + RMSNorm (an addition of this library) ----------------------
@pytest.mark.parametrize("w_dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("in_place", [False, True])
@pytest.mark.parametrize("shape,stride", [((16, 2048), None), ((16, 2048), 4096), ((5, 33), None), ((1, 8), None),
                                          ((700, 4096), None), ((2048, 2048), None), ((3, 16384), None),
                                          ((2, 70000), None), ((9, 264), 272), ((4100, 1024), None),
                                          ((600, 8192), None), ((40, 40000), None)])
def test_add_rms_norm(oracle, cuda_lib, shape, stride, in_place, w_dtype):
    """The sum is the Add operator's, bit for bit; the normalised rows are the
    oracle's RMSNorm of that sum within the fp16 tolerance, and what this library's
    Add followed by its RMSNorm write up to the grouping of the sum of squares."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(11)
    a = (torch.rand(shape, generator=g) * 2 - 1).half()
    b = (torch.randn(shape, generator=g) * 0.5).half()
    w = (torch.rand(shape[1], generator=g) * 2 - 1).to(w_dtype)
    want_sum = oracle.add(a.numpy(), b.numpy())
    want_y = oracle.rms_norm(want_sum, w.numpy(), 1e-5)
    ad, bd, wd = a.to(DEV), b.to(DEV), w.to(DEV)
    yd = torch.full(shape, 7.0, dtype=torch.float16, device=DEV)
    sd = torch.full(shape, 9.0, dtype=torch.float16, device=DEV)
    # the two calls the fusion replaces, on contiguous copies (Add wants contiguous operands)
    s2, y2 = torch.empty_like(ad), torch.empty_like(ad)
    ops.add(lib, handle, s2, ad, bd)
    ops.rms_norm(lib, handle, y2, s2, wd, 1e-5)
    if stride is not None:
        ad, bd, yd, sd = (rearrange_tensor(t, (stride, 1)) for t in (ad, bd, yd, sd))
    if in_place:
        sd = ad
    ops.add_rms_norm(lib, handle, yd, sd, ad, bd, wd, 1e-5)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(sd).reshape(shape), want_sum.view(np.uint16).reshape(shape))
    assert np.array_equal(_bits(bd).reshape(shape), b.numpy().view(np.uint16))
    mism = _close(_bits(yd).reshape(shape), want_y, 1e-3, 1e-3)
    assert _few(mism, a.numel(), 0.02)
    # against the two calls only the grouping of the fp32 sum of squares may differ
    assert _few(int((_bits(yd).reshape(-1) != _bits(y2).reshape(-1)).sum()), a.numel(), 0.002)


def test_add_rms_norm_status_codes(cuda_lib):
    from operators_b200 import InfiniopError

    lib, handle = cuda_lib
    h = torch.zeros((4, 8), dtype=torch.float16, device=DEV)
    f = torch.zeros((4, 8), dtype=torch.float32, device=DEV)

    def status(fn):
        with pytest.raises(InfiniopError) as e:
            fn()
        return e.value.status

    assert status(lambda: ops.AddRMSNormOp(lib, handle, h, h, h, h[:2], h[0])) == 4
    assert status(lambda: ops.AddRMSNormOp(lib, handle, h, h, h, h, h[0, :4])) == 4
    assert status(lambda: ops.AddRMSNormOp(lib, handle, h, h, f, h, h[0])) == 3
    assert status(lambda: ops.AddRMSNormOp(lib, handle, h, h[:, ::2], h[:, ::2], h[:, ::2], h[0, ::2])) == 4
    assert status(lambda: ops.AddRMSNormOp(lib, handle, h[:, ::2], h[:, ::2], h[:, ::2], h[:, ::2], h[0, :4])) == 5
    with ops.AddRMSNormOp(lib, handle, h, h, h, h, h[0]) as op:  # a descriptor of one form is refused by the other call
        assert lib.infiniopRMSNorm(op.desc, None, 0, h.data_ptr(), h.data_ptr(), h.data_ptr(), None) == 2
    with ops.RMSNormOp(lib, handle, h, h, h[0]) as op:
        assert lib.infiniopAddRMSNorm(op.desc, None, 0, h.data_ptr(), h.data_ptr(), h.data_ptr(), h.data_ptr(),
                                      h.data_ptr(), None) == 2


# ---- RoPE (bit-exact) ----------------------------------------------------------
@pytest.mark.parametrize("shape,strides", [((1, 32, 128), None), ((1, 32, 64), None), ((4, 1, 32), None),
                                           ((3, 32, 128), (8000, 200, 1)), ((64, 32, 128), None),
                                           ((5, 3, 6), None), ((5, 3, 6), (37, 7, 1)), ((7, 5, 96), None),
                                           ((2, 2, 4096), None), ((9, 40, 128), (40 * 256, 256, 1)),
                                           # bulk-copy pipeline: rings reused several times, ragged token counts,
                                           # one token, more tokens than the pipeline takes (-> strided kernel)
                                           ((9000, 32, 64), None), ((1187, 32, 128), None), ((33, 8, 256), None),
                                           ((9000, 8, 64), None), ((40000, 64, 32), None), ((300, 16, 8), None)])
@pytest.mark.parametrize("stores", ["threads", "bulk"])
def test_rope(oracle, cuda_lib, shape, strides, stores):
    lib, handle = cuda_lib
    ops.select_kernel(lib, "rope", 2 if stores == "bulk" else 0)  # both forms of the bulk-copy pipeline
    g = torch.Generator().manual_seed(2)
    t = torch.randn(shape, generator=g).half()
    pos = torch.randperm(2 * shape[0], generator=g)[: shape[0]].to(torch.int64)
    sin, cos = ops.sin_cos_table(2 * shape[0], shape[2])
    want = oracle.rope(t.numpy().copy(), pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
    td = t.to(DEV)
    if strides is not None:
        td = rearrange_tensor(td, strides)
    try:
        ops.rope(lib, handle, td, pos.to(DEV), sin.to(DEV), cos.to(DEV))
        torch.cuda.synchronize()
    finally:
        ops.select_kernel(lib, "rope", 0)
    assert np.array_equal(_bits(td).reshape(shape), want.view(np.uint16))


def test_rope_pipeline_wait_limit_is_reported(oracle, cuda_lib):
    """Every wait of the bulk-copy pipeline is bounded.  With the limit set to a single poll the copies cannot
    have arrived: the groups give up, let their copies land and leave, the call still returns, and the
    timeout query reports it.  With the default limit restored the same call is complete and exact again."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(22)
    shape = (1187, 32, 128)
    t = torch.randn(shape, generator=g).half()
    pos = torch.arange(shape[0], dtype=torch.int64)
    sin, cos = ops.sin_cos_table(shape[0], shape[2])
    want = oracle.rope(t.numpy().copy(), pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
    posd, sind, cosd = pos.to(DEV), sin.to(DEV), cos.to(DEV)
    before = ops.device_timeouts(lib, handle)
    try:
        ops.set_wait_limit(lib, handle, 1)
        td = t.to(DEV)
        ops.rope(lib, handle, td, posd, sind, cosd)  # returns normally
        torch.cuda.synchronize()
        assert ops.device_timeouts(lib, handle) > before
    finally:
        ops.set_wait_limit(lib, handle, 0)
    mid = ops.device_timeouts(lib, handle)
    td = t.to(DEV)
    ops.rope(lib, handle, td, posd, sind, cosd)
    torch.cuda.synchronize()
    assert ops.device_timeouts(lib, handle) == mid
    assert np.array_equal(_bits(td).reshape(shape), want.view(np.uint16))


# ---- RoPE written into a second view, e.g. the K cache (an addition of this library; bit-exact) -------
@pytest.mark.parametrize("tokens,heads,dh,src_strides,cache_len,first", [
    (1, 8, 128, None, 64, 17), (7, 8, 128, None, 64, 50), (64, 8, 128, (40 * 128, 128, 1), 4096, 1000),
    (5, 3, 6, None, 9, 2), (5, 3, 6, (37, 7, 1), 16, 0), (300, 4, 64, None, 300, 0),
    (2048, 8, 128, (48 * 128, 128, 1), 4096, 2048), (33, 2, 256, None, 40, 3)])
def test_rope_rearrange_into_cache(oracle, cuda_lib, tokens, heads, dh, src_strides, cache_len, first):
    """k[tokens, heads, dh] (possibly a slice of a wider qkv row) is rotated and lands in
    cache[heads, cache_len, dh] at rows first .. first+tokens; k itself and every other
    byte of the cache stay as they were."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(12)
    k = torch.randn((tokens, heads, dh), generator=g).half()
    pos = torch.arange(first, first + tokens, dtype=torch.int64)
    sin, cos = ops.sin_cos_table(first + tokens, dh)
    want = oracle.rope(k.numpy().copy(), pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
    kd = k.to(DEV)
    if src_strides is not None:
        kd = rearrange_tensor(kd, src_strides)
    cache = torch.full((heads, cache_len, dh), 3.0, dtype=torch.float16, device=DEV)
    dst = cache[:, first:first + tokens, :].permute(1, 0, 2)  # [tokens, heads, dh] view of the cache rows
    ops.rope_rearrange(lib, handle, dst, kd, pos.to(DEV), sin.to(DEV), cos.to(DEV))
    torch.cuda.synchronize()
    expect = np.full((heads, cache_len, dh), np.float16(3.0)).view(np.uint16)
    expect[:, first:first + tokens, :] = want.view(np.uint16).transpose(1, 0, 2)
    assert np.array_equal(_bits(cache), expect)
    assert np.array_equal(_bits(kd).reshape(k.shape), k.numpy().view(np.uint16))
    # the two calls it replaces write the same bytes
    cache2 = torch.full((heads, cache_len, dh), 3.0, dtype=torch.float16, device=DEV)
    k2 = kd.clone()
    ops.rope(lib, handle, k2, pos.to(DEV), sin.to(DEV), cos.to(DEV))
    ops.rearrange(lib, handle, cache2[:, first:first + tokens, :].permute(1, 0, 2), k2)
    torch.cuda.synchronize()
    assert torch.equal(cache, cache2)


def test_rope_rearrange_status_codes(cuda_lib):
    from operators_b200 import InfiniopError

    lib, handle = cuda_lib
    t = torch.zeros((4, 2, 8), dtype=torch.float16, device=DEV)
    pos = torch.zeros(4, dtype=torch.int64, device=DEV)
    tab = torch.zeros((8, 8), dtype=torch.float32, device=DEV)

    def status(fn):
        with pytest.raises(InfiniopError) as e:
            fn()
        return e.value.status

    assert status(lambda: ops.RoPERearrangeOp(lib, handle, t[:3], t, pos, tab, tab)) == 4
    assert status(lambda: ops.RoPERearrangeOp(lib, handle, t.float(), t, pos, tab, tab)) == 3
    assert status(lambda: ops.RoPERearrangeOp(lib, handle, t[:, :, ::2], t[:, :, :4], pos, tab[:, :4], tab[:, :4])) == 5
    assert status(lambda: ops.RoPERearrangeOp(lib, handle, t, t, pos[:3], tab, tab)) == 4
    with ops.RoPERearrangeOp(lib, handle, t, t.clone(), pos, tab, tab) as op:
        assert lib.infiniopRoPE(op.desc, None, 0, t.data_ptr(), pos.data_ptr(), tab.data_ptr(), tab.data_ptr(), None) == 2
    with ops.RoPEOp(lib, handle, t, pos, tab, tab) as op:
        assert lib.infiniopRoPERearrange(op.desc, None, 0, t.data_ptr(), t.data_ptr(), pos.data_ptr(), tab.data_ptr(),
                                         tab.data_ptr(), None) == 2


# ---- SwiGLU ------------------------------------------------------------------
@pytest.mark.parametrize("inplace", [None, "a", "b"])
@pytest.mark.parametrize("shape,stride", [((13, 4), None), ((13, 4), 10), ((16, 5632), None), ((16, 5632), 13312),
                                          ((3, 8), None), ((257, 1024), 2048)])
def test_swiglu(oracle, cuda_lib, shape, stride, inplace):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(3)
    a = torch.randn(shape, generator=g).half()
    b = (torch.randn(shape, generator=g) * 4).half()
    want = oracle.swiglu(a.numpy(), b.numpy())
    ad, bd = a.to(DEV), b.to(DEV)
    if stride is not None:
        ad, bd = rearrange_tensor(ad, (stride, 1)), rearrange_tensor(bd, (stride, 1))
    cd = {None: torch.zeros(shape, dtype=torch.float16, device=DEV), "a": ad, "b": bd}[inplace]
    ops.swiglu(lib, handle, cd, ad, bd)
    torch.cuda.synchronize()
    mism = _close(_bits(cd).reshape(shape), want, 1e-3, 1e-3)
    assert _few(mism, a.numel(), 2e-3)  # expf differs from libm by an fp32 ulp now and then


def test_swiglu_fused_gate_up_halves(oracle, cuda_lib):
    """The MLP layout: a and b are the column halves of one [tokens, 2*di]
    buffer (reference src/ops/mlp/operator.cc:48-57,111-115)."""
    lib, handle = cuda_lib
    tokens, di = 64, 1792
    g = torch.Generator().manual_seed(33)
    gate_up = torch.randn((tokens, 2 * di), generator=g).half()
    want = oracle.swiglu(gate_up[:, di:].numpy(), gate_up[:, :di].numpy())
    gd = gate_up.to(DEV)
    cd = torch.zeros((tokens, di), dtype=torch.float16, device=DEV)
    ops.swiglu(lib, handle, cd, gd[:, di:], gd[:, :di])
    torch.cuda.synchronize()
    _close(_bits(cd).reshape(tokens, di), want, 1e-3, 1e-3)


# ---- Add (bit-exact) -------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shapes", [((), (), ()), ((3, 3), (3, 3), (3, 3)), ((2, 20, 3), (2, 1, 3), (2, 20, 3)),
                                    ((32, 20, 512), (32, 20, 512), (32, 20, 512)), ((4, 5, 6), (6,), (4, 5, 6)),
                                    ((3, 1, 7), (1, 5, 1), (3, 5, 7)), ((1000003,), (1000003,), (1000003,)),
                                    ((2, 3, 4, 5), (5,), (2, 3, 4, 5)), ((32, 64, 28, 28), (32, 64, 28, 28), (32, 64, 28, 28)),
                                    # broadcasts whose innermost axis is whole vectors (the vectorised broadcast kernel)
                                    ((64, 4096), (4096,), (64, 4096)), ((64, 1), (64, 4096), (64, 4096)),
                                    ((4, 8, 256), (4, 1, 256), (4, 8, 256)), ((16, 1, 64), (1, 8, 64), (16, 8, 64)),
                                    ((3, 5, 1, 16), (5, 7, 16), (3, 5, 7, 16)), ((2, 1, 1), (1, 3, 24), (2, 3, 24)),
                                    ((1, 40), (9, 1), (9, 40)), ((300, 8), (8,), (300, 8))])
def test_add(oracle, cuda_lib, shapes, dtype):
    lib, handle = cuda_lib
    as_, bs, cs = shapes
    g = torch.Generator().manual_seed(4)
    a = (torch.randn(as_, generator=g) * 100).to(dtype)
    b = torch.randn(bs, generator=g).to(dtype)
    want = oracle.add(a.numpy(), b.numpy()).reshape(cs)
    cd = torch.zeros(cs, dtype=dtype, device=DEV)
    ops.add(lib, handle, cd, a.to(DEV), b.to(DEV))
    torch.cuda.synchronize()
    got = cd.cpu().numpy()
    if dtype == torch.float16:
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    else:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("which", ["a", "b"])
def test_add_inplace(oracle, cuda_lib, which):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(44)
    a = torch.randn((33, 129), generator=g).half()
    b = torch.randn((33, 129), generator=g).half()
    want = oracle.add(a.numpy(), b.numpy())
    ad, bd = a.to(DEV), b.to(DEV)
    cd = ad if which == "a" else bd
    ops.add(lib, handle, cd, ad, bd)
    torch.cuda.synchronize()
    assert np.array_equal(_bits(cd).reshape(33, 129), want.view(np.uint16))


def test_add_unaligned_views(oracle, cuda_lib):
    """Contiguous tensors that start 2 bytes into an allocation."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(45)
    n = 4099
    a = torch.randn(n + 1, generator=g).half()
    b = torch.randn(n + 1, generator=g).half()
    want = oracle.add(a[1:].numpy(), b[1:].numpy())
    ad, bd, cd = a.to(DEV), b.to(DEV), torch.zeros(n + 1, dtype=torch.float16, device=DEV)
    ops.add(lib, handle, cd[1:], ad[1:], bd[1:])
    torch.cuda.synchronize()
    assert np.array_equal(_bits(cd)[1:], want.view(np.uint16))
    assert _bits(cd)[0] == 0


# ---- causal softmax --------------------------------------------------------------
@pytest.mark.parametrize("shape,strides", [((32, 20, 512), None), ((32, 20, 512), (20480, 1024, 1)), ((5, 64), None),
                                           ((2, 7, 7), None), ((3, 1, 9), None), ((2, 128, 4096), None),
                                           ((4, 33, 1000), None), ((1, 3, 20000), None), ((2, 2, 70000), None),
                                           ((8, 64, 16384), None), ((600, 1, 16384), None),
                                           # rows spread over a cluster of 2 / 4 / 8 CTAs, up to the longest
                                           # register-resident row and one vector past it
                                           ((1, 2, 40960), None), ((1, 3, 65536), None), ((8, 128, 16384), None),
                                           ((4, 40, 32768), (40 * 32776, 32776, 1)), ((2, 150, 32768), None), ((1, 2, 262144), None),
                                           ((1, 2, 262152), None), ((2, 5, 8200), None)])
@pytest.mark.parametrize("long_rows", ["auto", "ring"])
def test_causal_softmax(oracle, cuda_lib, shape, strides, long_rows):
    lib, handle = cuda_lib
    if long_rows == "ring" and shape[-1] < 4096:
        pytest.skip("the shared-memory ring starts at rows of 4096 columns")
    g = torch.Generator().manual_seed(5)
    y = (torch.randn(shape, generator=g) * 2).half()
    want = oracle.causal_softmax(y.numpy().copy())
    yd = y.to(DEV)
    if strides is not None:
        yd = rearrange_tensor(yd, strides)
    ops.select_kernel(lib, "long_rows", 2 if long_rows == "ring" else 0)
    try:
        ops.causal_softmax(lib, handle, yd)
        torch.cuda.synchronize()
    finally:
        ops.select_kernel(lib, "long_rows", 0)
    got = _bits(yd).reshape(shape)
    _close(got, want, 2e-3, 2e-3)
    # masked entries are exact zeros, as the reference's own test demands
    assert np.array_equal(got == 0, want.view(np.uint16) == 0) or (got[want.view(np.uint16) == 0] == 0).all()


# ---- random sample (index-exact) ---------------------------------------------------
REF_CASES = [(512, 0.92, 0.8, 3, 0.5), (4096, 0.95, 0.9, 5, 1.0), (16384, 0.85, 0.85, 10, 2.0),
             (512, 0.92, 0.0, 3, 0.5), (4096, 0.95, 0.9, 1, 1.0), (16384, 0.85, 0.0, 1, 2.0),
             (32000, 0.8, 0.8, 50, 1.0), (32000, 0.8, 1.0, 25, 1.0)]


@pytest.mark.parametrize("voc,u,topp,topk,temp", REF_CASES + [(40, 0.5, 1.0, 64, 1.0), (7, 0.99, 0.9, 3, 0.7),
                                                              (128256, 0.3, 0.9, 50, 0.8), (1000, 0.0, 0.5, 2, 1.5)])
@pytest.mark.parametrize("dist", ["uniform", "normal3"])
def test_random_sample_single_row_abi(oracle, cuda_lib, voc, u, topp, topk, temp, dist):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(6)
    for _ in range(2):
        logits = torch.rand(voc, generator=g).half() if dist == "uniform" else (torch.randn(voc, generator=g) * 3).half()
        want = oracle.random_sample(logits.numpy(), u, topp, topk, temp, previous=12345)
        res = torch.full((1,), 12345, dtype=torch.int64, device=DEV)
        ops.random_sample(lib, handle, res, logits.to(DEV), u, topp, topk, temp)
        torch.cuda.synchronize()
        assert int(res[0]) == want


@pytest.fixture(params=["shared", "global"])
def sampler_kernel(request, cuda_lib):
    """Both sampling kernels: the shared-memory resident pair kernel (default for
    voc <= 262144; clusters of two or four CTAs) and the global-memory kernel (any voc)."""
    ops.select_kernel(cuda_lib[0], "random_sample", 1 if request.param == "global" else 0)
    yield request.param
    ops.select_kernel(cuda_lib[0], "random_sample", 0)


@pytest.mark.parametrize("voc,rows,topp,topk,temp,dist", [
    (128256, 64, 0.9, 50, 0.8, "normal3"), (131072, 8, 0.9, 64, 1.0, "normal3"), (200000, 6, 0.9, 50, 0.8, "normal3"),
    (131073, 5, 0.9, 50, 1.0, "normal3"), (151936, 6, 0.9, 50, 1.3, "normal3"), (262144, 3, 0.9, 64, 0.8, "uniform"),
    (262145, 2, 0.9, 50, 0.8, "normal3"), (196608, 3, 0.9, 50, 1.0, "coarse"), (256000, 3, 0.9, 50, 1.0, "ascending"),
    (65536, 8, 0.9, 50, 0.8, "normal3"), (65537, 8, 0.9, 50, 1.3, "uniform"), (70000, 4, 0.9, 50, 1.0, "ascending"),
    (100000, 4, 0.95, 33, 0.6, "coarse"), (128256, 4, 0.9, 50, 1.0, "constant"), (128256, 6, 0.9, 50, 5.0, "normal3"), (32000, 96, 0.8, 50, 1.0, "uniform"), (32000, 64, 1.0, 25, 1.0, "uniform"),
    (16384, 64, 0.85, 10, 2.0, "normal3"), (5000, 200, 0.95, 64, 0.3, "normal3"), (777, 50, 0.9, 7, 1.0, "coarse"),
    (4096, 32, 0.9, 40, 1.0, "constant"), (8192, 16, 0.9, 50, 1.0, "ascending"), (8192, 16, 0.9, 50, 1.0, "descending")])
def test_random_sample_batch_with_trace(oracle, cuda_lib, sampler_kernel, voc, rows, topp, topk, temp, dist):
    """Batched extension: the denominator, the top-k order and probabilities and
    the final index all equal the oracle's, row by row."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(7)
    if dist == "uniform":
        logits = torch.rand((rows, voc), generator=g).half()
    elif dist == "normal3":
        logits = (torch.randn((rows, voc), generator=g) * 3).half()
    elif dist == "coarse":  # few distinct values: ties everywhere
        logits = torch.randint(0, 12, (rows, voc), generator=g).half()
    elif dist == "constant":
        logits = torch.full((rows, voc), 1.5).half()
    elif dist == "ascending":
        logits = (torch.arange(voc).float() / voc * 8).half().repeat(rows, 1)
    else:
        logits = (torch.arange(voc, 0, -1).float() / voc * 8).half().repeat(rows, 1)
    u = torch.rand(rows, generator=g)
    ld, ud = logits.to(DEV), u.to(DEV)
    res = torch.full((rows,), 999, dtype=torch.int64, device=DEV)
    trace = torch.zeros((rows, 145), dtype=torch.float32, device=DEV)
    with ops.RandomSampleOp(lib, handle, res[:1], ld[0]) as op:
        op.batch(res, ld, ud, topp, topk, temp, trace=trace)
        torch.cuda.synchronize()
        res2 = torch.full((rows,), 999, dtype=torch.int64, device=DEV)
        op.batch(res2, ld, ud, topp, topk, temp)  # workspace reuse, no trace
        torch.cuda.synchronize()
    tr = trace.cpu().numpy()
    k = min(topk, voc)
    bad = []
    for r in range(rows):
        row = logits[r].numpy()
        want = oracle.random_sample(row, float(u[r]), topp, topk, temp, previous=999)
        ot = oracle.random_sample_trace(row, topk, temp)
        got_idx = tr[r, 1:1 + k].view(np.uint32).astype(np.uint64)
        ok = (np.array_equal(got_idx, ot["top_idx"]) and tr[r, 0] == ot["denom"]
              and np.array_equal(tr[r, 65:65 + k], ot["top_p"].astype(np.float32))
              and int(res[r]) == want and int(res2[r]) == want)
        if not ok:
            bad.append((r, int(res[r]), want, float(tr[r, 0]), float(ot["denom"])))
    assert not bad, bad[:5]


def test_random_sample_argmax_ties(oracle, cuda_lib):
    lib, handle = cuda_lib
    logits = torch.zeros(5000).half()
    logits[[77, 4000, 123]] = 3.0
    logits[10] = -0.0
    res = torch.zeros(1, dtype=torch.int64, device=DEV)
    ops.random_sample(lib, handle, res, logits.to(DEV), 0.5, 0.0, 5, 1.0)
    torch.cuda.synchronize()
    assert int(res[0]) == 77 == oracle.random_sample(logits.numpy(), 0.5, 0.0, 5, 1.0)


@pytest.mark.parametrize("voc,rows,pitch", [(128256, 64, 128256), (32000, 33, 32000), (1, 3, 8), (7, 5, 8), (8, 4, 8),
                                            (9, 4, 16), (4097, 9, 4104), (151937, 3, 151944), (5000, 6, 5003),
                                            (262147, 2, 262152)])
@pytest.mark.parametrize("dist", ["normal3", "coarse", "neg_inf", "late_tie"])
def test_random_sample_argmax_batch(oracle, cuda_lib, voc, rows, pitch, dist):
    """Greedy decoding (top-p 0 or top-k 1): the first index of the row maximum, as the
    reference's strict-greater scan finds it; rows that end inside a 16-byte vector, rows
    whose pitch keeps them 16-byte aligned and rows whose pitch does not."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(voc + rows)
    if dist == "normal3":
        logits = (torch.randn((rows, voc), generator=g) * 3).half()
    elif dist == "coarse":
        logits = torch.randint(-3, 4, (rows, voc), generator=g).half()
    elif dist == "neg_inf":
        logits = torch.full((rows, voc), float("-inf")).half()
        if voc > 2:
            logits[1::2, voc - 1] = -7.0  # a single finite value at the ragged end of every second row
    else:  # the maximum appears in both halves of the row and as the last element
        logits = (torch.rand((rows, voc), generator=g) - 2).half()
        for r in range(rows):
            logits[r, [min(voc - 1, voc // 2 + r), voc - 1]] = 5.0
            if r % 2 and voc > 4:
                logits[r, voc // 4] = 5.0
        logits[:, 0] = -0.0
    store = torch.zeros((rows, pitch), dtype=torch.float16, device=DEV)
    store[:, :voc] = logits.to(DEV)
    ld = store[:, :voc]
    u = torch.rand(rows, generator=g).to(DEV)
    want = [oracle.random_sample(logits[r].numpy(), 0.5, 0.0, 5, 1.0) for r in range(rows)]
    for topp, topk in ((0.0, 5), (0.9, 1)):
        res = torch.full((rows,), 999, dtype=torch.int64, device=DEV)
        with ops.RandomSampleOp(lib, handle, res[:1], ld[0]) as op:
            op.batch(res, ld, u, topp, topk, 1.0)
            torch.cuda.synchronize()
        assert res.cpu().tolist() == want
    one = torch.full((1,), 999, dtype=torch.int64, device=DEV)
    ops.random_sample(lib, handle, one, ld[rows - 1], 0.5, 0.0, 5, 1.0)
    torch.cuda.synchronize()
    assert int(one[0]) == want[rows - 1]


# ---- bf16 storage (an extension: the reference has no bf16 operator; oracle = the same restated arithmetic with
# bf16 decode and truncating encode, oracle.bf16_storage) -------------------------------------------------------
def _bf16_bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _bf16_within_one_ulp(got, want):
    """Bit patterns equal, or neighbours of the same sign (one bf16 ulp apart); returns the number of mismatches."""
    got, want = got.reshape(-1).astype(np.int32), want.reshape(-1).astype(np.int32)
    diff = np.abs(got - want)
    both_zero = ((got & 0x7FFF) == 0) & ((want & 0x7FFF) == 0)
    assert ((diff <= 1) | both_zero).all(), "max pattern distance %d" % diff[~both_zero].max()
    return int(((diff != 0) & ~both_zero).sum())


def _bf16_close(got_bits, want_bits, atol, rtol):
    """|got - want| <= atol + rtol * |want| on bf16 patterns; returns the number of patterns that differ."""
    got = (got_bits.reshape(-1).astype(np.uint32) << 16).view(np.float32)
    want = (want_bits.reshape(-1).astype(np.uint32) << 16).view(np.float32)
    err = np.abs(got - want)
    assert (err <= atol + rtol * np.abs(want)).all(), "max err %g" % err.max()
    return int((got_bits.reshape(-1) != want_bits.reshape(-1)).sum())


@pytest.mark.parametrize("shapes", [((3, 3), (3, 3)), ((2, 20, 3), (2, 1, 3)), ((64, 4096), (4096,)), ((1000003,), (1000003,)),
                                    ((300, 8), (8,))])
def test_bf16_add(oracle, cuda_lib, shapes):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(40)
    a = (torch.randn(shapes[0], generator=g) * 100).bfloat16()
    b = torch.randn(shapes[1], generator=g).bfloat16()
    with oracle.bf16_storage():
        want = oracle.add(_bf16_bits(a).reshape(a.shape), _bf16_bits(b).reshape(b.shape))
    cd = torch.zeros(want.shape, dtype=torch.bfloat16, device=DEV)
    ops.add(lib, handle, cd, a.to(DEV), b.to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bf16_bits(cd).reshape(want.shape), want)


@pytest.mark.parametrize("shape,strides", [((1187, 32, 128), None), ((64, 32, 128), None), ((5, 3, 6), (37, 7, 1)),
                                           ((9, 40, 128), (40 * 256, 256, 1))])
def test_bf16_rope(oracle, cuda_lib, shape, strides):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(41)
    t = torch.randn(shape, generator=g).bfloat16()
    pos = torch.randperm(2 * shape[0], generator=g)[: shape[0]].to(torch.int64)
    sin, cos = ops.sin_cos_table(2 * shape[0], shape[2])
    want = _bf16_bits(t).reshape(shape).copy()
    with oracle.bf16_storage():
        oracle.rope(want, pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
    td = t.to(DEV)
    if strides is not None:
        td = rearrange_tensor(td, strides)
    ops.rope(lib, handle, td, pos.to(DEV), sin.to(DEV), cos.to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bf16_bits(td).reshape(shape), want)


@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(16, 2048), (5, 33), (700, 4096), (2048, 2048), (2, 70000), (2, 65536)])
def test_bf16_rms_norm(oracle, cuda_lib, shape, w_dtype):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(42)
    x = (torch.rand(shape, generator=g) * 2 - 1).bfloat16()
    w = (torch.rand(shape[1], generator=g) * 2 - 1).to(w_dtype)
    wn = _bf16_bits(w) if w_dtype == torch.bfloat16 else w.numpy()
    with oracle.bf16_storage():
        want = oracle.rms_norm(_bf16_bits(x).reshape(shape), wn, 1e-5).view(np.uint16)
    yd = torch.zeros(shape, dtype=torch.bfloat16, device=DEV)
    ops.rms_norm(lib, handle, yd, x.to(DEV), w.to(DEV), 1e-5)
    torch.cuda.synchronize()
    assert _few(_bf16_within_one_ulp(_bf16_bits(yd), want), x.numel(), 0.02)


@pytest.mark.parametrize("shape,stride", [((13, 4), None), ((16, 5632), None), ((257, 1024), 2048)])
def test_bf16_swiglu(oracle, cuda_lib, shape, stride):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(43)
    a = torch.randn(shape, generator=g).bfloat16()
    b = (torch.randn(shape, generator=g) * 4).bfloat16()
    with oracle.bf16_storage():
        want = oracle.swiglu(_bf16_bits(a).reshape(shape), _bf16_bits(b).reshape(shape)).view(np.uint16)
    ad, bd = a.to(DEV), b.to(DEV)
    if stride is not None:
        ad, bd = rearrange_tensor(ad, (stride, 1)), rearrange_tensor(bd, (stride, 1))
    cd = torch.zeros(shape, dtype=torch.bfloat16, device=DEV)
    ops.swiglu(lib, handle, cd, ad, bd)
    torch.cuda.synchronize()
    assert _few(_bf16_within_one_ulp(_bf16_bits(cd), want), a.numel(), 2e-3)


@pytest.mark.parametrize("shape", [(32, 20, 512), (5, 64), (2, 128, 4096), (4, 33, 1000), (1, 2, 40960), (2, 2, 300000)])
def test_bf16_causal_softmax(oracle, cuda_lib, shape):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(44)
    y = (torch.randn(shape, generator=g) * 2).bfloat16()
    want = _bf16_bits(y).reshape(shape).copy()
    with oracle.bf16_storage():
        oracle.causal_softmax(want)
    yd = y.to(DEV)
    ops.causal_softmax(lib, handle, yd)
    torch.cuda.synchronize()
    got = _bf16_bits(yd).reshape(shape)
    _bf16_within_one_ulp(got, want)
    assert (got[want == 0] == 0).all()  # masked entries are exact zeros


# ---- matmul (the reference's cases, operatorspy/tests/matmul.py:296-308, and the layouts either kernel serves) ----
MATMUL_CASES = [
    # alpha, beta, a_shape, b_shape, c_shape, a_stride, b_stride, c_stride
    (1.0, 0.0, (1, 2048), (2048, 2048), (1, 2048), None, None, None),
    (1.0, 0.0, (2, 4, 2048), (2, 2048, 2048), (2, 4, 2048), None, None, None),
    (1.0, 0.0, (1, 2048), (2048, 2048), (1, 2048), (4096, 1), (4096, 1), (4096, 1)),
    (1.0, 1.0, (6, 2048), (2048, 2560), (6, 2560), (2048, 1), (1, 2048), (2560, 1)),
    (1.0 / 8.0, 0.0, (4, 8 * 6, 64), (4, 64, 6), (4, 8 * 6, 6), None, None, None),
    # all four combinations of operand majors, ragged edges in m, n and k, several tiles, a column-major result
    (1.0, 0.0, (300, 136), (136, 200), (300, 200), None, (1, 136), None),
    (1.0, 0.0, (300, 136), (136, 200), (300, 200), None, None, None),
    (0.5, 0.0, (300, 136), (136, 200), (300, 200), (1, 304), (1, 136), (1, 304)),
    (1.0, 2.0, (260, 72), (72, 264), (260, 264), (1, 264), None, None),
    (1.0, 0.0, (513, 1000), (1000, 777), (513, 777), None, (1, 1000), None),
    # batched with a broadcast operand; k below one k-block; one row and one column
    (1.0, 0.0, (3, 130, 64), (1, 64, 72), (3, 130, 72), None, None, None),
    (1.0, 0.0, (40, 8), (8, 24), (40, 24), None, None, None),
    (1.0, 0.0, (1, 4096), (4096, 1), (1, 1), None, None, None),
    # decoding shapes: few rows against a wide matrix (k split over the SMs), both weight layouts
    (1.0, 0.0, (16, 4096), (4096, 3584), (16, 3584), None, None, None),
    (1.0, 1.0, (5, 3584), (3584, 4096), (5, 4096), None, (1, 3584), None),
    (1.0, 0.0, (64, 1024), (1024, 2048), (64, 2048), None, None, None),
    # layouts a TMA descriptor cannot address (odd leading dimensions, a base 2 bytes into an allocation)
    (1.0, 0.0, (33, 50), (50, 21), (33, 21), (51, 1), None, None),
]


@pytest.fixture(params=["tensor", "cuda_cores"])
def matmul_kernels(request, cuda_lib):
    """Both kernels: tcgen05 where the layout allows it, and the CUDA-core kernel that serves the rest."""
    ops.select_kernel(cuda_lib[0], "matmul", 1 if request.param == "cuda_cores" else 0)
    yield request.param
    ops.select_kernel(cuda_lib[0], "matmul", 0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("alpha,beta,a_shape,b_shape,c_shape,a_stride,b_stride,c_stride", MATMUL_CASES)
def test_matmul(oracle, cuda_lib, matmul_kernels, alpha, beta, a_shape, b_shape, c_shape, a_stride, b_stride, c_stride,
                dtype):
    """fp16 within atol = rtol = 1e-3 of the oracle (only the grouping of the fp32 sum over k differs, so most
    elements are the same bit pattern); fp32 within 1e-5 relative to the size of the sum's terms."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(8)
    a = (torch.rand(a_shape, generator=g) - 0.5).to(dtype)
    b = (torch.rand(b_shape, generator=g) - 0.5).to(dtype)
    c = (torch.rand(c_shape, generator=g) - 0.5).to(dtype)
    a, b, c = (t if st is None else rearrange_tensor(t, st) for t, st in ((a, a_stride), (b, b_stride), (c, c_stride)))
    want = c.clone()
    if c_stride is not None:
        want = rearrange_tensor(want, c_stride)
    oracle.matmul_into(want.numpy(), a.numpy(), b.numpy(), alpha, beta)
    ad, bd, cd = (t.to(DEV) for t in (a, b, c))
    ad, bd, cd = (t if st is None else rearrange_tensor(t, st) for t, st in ((ad, a_stride), (bd, b_stride), (cd, c_stride)))
    ops.matmul(lib, handle, cd, ad, bd, alpha, beta)
    torch.cuda.synchronize()
    if dtype == torch.float16:
        mism = _close(_bits(cd).reshape(c_shape), want.numpy(), 1e-3, 1e-3)
        assert _few(mism, c.numel(), 0.25)
    else:
        got, w = cd.cpu().numpy(), want.numpy()
        assert np.abs(got - w).max() <= 1e-5 * (1 + abs(beta)) * max(1.0, a_shape[-1] ** 0.5)


def test_matmul_unaligned_base_takes_the_cuda_core_kernel(oracle, cuda_lib):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(81)
    a, b = (torch.rand((40, 64), generator=g) - 0.5).half(), (torch.rand((64, 48), generator=g) - 0.5).half()
    want = np.zeros((40, 48), np.float16)
    oracle.matmul_into(want, a.numpy(), b.numpy())
    store = torch.zeros(40 * 64 + 1, dtype=torch.float16, device=DEV)
    ad = store[1:].view(40, 64)
    ad.copy_(a)
    cd = torch.zeros((40, 48), dtype=torch.float16, device=DEV)
    ops.matmul(lib, handle, cd, ad, b.to(DEV))
    torch.cuda.synchronize()
    _close(_bits(cd).reshape(40, 48), want, 1e-3, 1e-3)


def test_matmul_status_codes(cuda_lib):
    from operators_b200 import InfiniopError

    lib, handle = cuda_lib
    h = torch.zeros((8, 8), dtype=torch.float16, device=DEV)
    f = torch.zeros((8, 8), dtype=torch.float32, device=DEV)
    i = torch.zeros((8, 8), dtype=torch.int64, device=DEV)

    def status(fn):
        with pytest.raises(InfiniopError) as e:
            fn()
        return e.value.status

    assert status(lambda: ops.MatmulOp(lib, handle, i, i, i)) == 3               # dtype
    assert status(lambda: ops.MatmulOp(lib, handle, h, h[0], h)) == 4            # 1-D operand
    assert status(lambda: ops.MatmulOp(lib, handle, h, h[:, ::2], h[:4])) == 5   # no unit stride
    assert status(lambda: ops.MatmulOp(lib, handle, h, h[:, :4], h)) == 4        # k mismatch
    assert status(lambda: ops.MatmulOp(lib, handle, h, f, h)) == 3               # mixed dtypes
    b3 = torch.zeros((3, 8, 8), dtype=torch.float16, device=DEV)
    assert status(lambda: ops.MatmulOp(lib, handle, b3, b3[:2], b3)) == 2        # batch neither equal nor 1


@pytest.mark.parametrize("kernel", ["cta_pairs", "single_cta"])
def test_config_matmul_8192x4096x28672_sampled(oracle, cuda_lib, kernel):
    """[8192, 4096] x [4096, 28672] (the gate / up projection at the benchmark's SwiGLU shape) on the tensor
    cores, with 256 x 256 tiles on CTA pairs (the library's choice at this size) and with the single-CTA kernel;
    the oracle would need hours for all of it, so 24 rows x 96 columns spread over the result (first and
    last tiles included) are compared, and the two kernels' full results with each other."""
    lib, handle = cuda_lib
    ops.select_kernel(lib, "matmul", 2 if kernel == "single_cta" else 0)
    g = torch.Generator().manual_seed(82)
    a = (torch.rand((8192, 4096), generator=g) - 0.5).half()
    b = (torch.rand((4096, 28672), generator=g) - 0.5).half()
    cd = torch.zeros((8192, 28672), dtype=torch.float16, device=DEV)
    try:
        ops.matmul(lib, handle, cd, a.to(DEV), b.to(DEV))
        torch.cuda.synchronize()
    finally:
        ops.select_kernel(lib, "matmul", 0)
    rows = torch.cat([torch.arange(0, 4), torch.arange(8188, 8192), torch.randperm(8192, generator=g)[:16]])
    cols = torch.cat([torch.arange(0, 8), torch.arange(28664, 28672), torch.randperm(28672, generator=g)[:80]])
    want = np.zeros((len(rows), len(cols)), np.float16)
    oracle.matmul_into(want, a[rows].numpy(), np.ascontiguousarray(b[:, cols].numpy()))
    got = cd[rows.to(DEV)][:, cols.to(DEV)]
    _close(_bits(got).reshape(want.shape), want, 1e-3, 1e-3)
    # every element, against a float32 product of the same fp16 inputs (sums of 4096 terms of both signs)
    ref = torch.matmul(a.to(DEV).float(), b.to(DEV).float())
    err = (cd.float() - ref).abs()
    assert float((err / (1e-2 + ref.abs())).max()) < 2e-2


@pytest.mark.parametrize("w_layout", ["n_contiguous", "k_contiguous"])
@pytest.mark.parametrize("tokens,hidden,di", [(2048, 1024, 2752), (700, 512, 1384)])
def test_mlp_prefill_sized_sampled_rows(oracle, cuda_lib, tokens, hidden, di, w_layout):
    """Token counts at which both products run on CTA pairs (SwiGLU epilogue included).  MLP rows are independent,
    so the oracle runs on 20 of them."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(91)
    y = (torch.rand((tokens, hidden), generator=g) - 0.5).half()
    x = (torch.rand((tokens, hidden), generator=g) - 0.5).half()
    w12 = ((torch.rand((hidden, 2 * di), generator=g) - 0.5) * 0.1).half()
    w3 = ((torch.rand((di, hidden), generator=g) - 0.5) * 0.1).half()
    rows = torch.cat([torch.arange(0, 2), torch.arange(tokens - 2, tokens), torch.randperm(tokens, generator=g)[:16]])
    want = y[rows].numpy().copy()
    oracle.mlp(want, x[rows].numpy().copy(), w12.numpy(), w3.numpy(), 1.0, True)
    yd, xd, w12d, w3d = (t.to(DEV) for t in (y, x, w12, w3))
    if w_layout == "k_contiguous":
        w12d, w3d = rearrange_tensor(w12d, (1, hidden)), rearrange_tensor(w3d, (1, di))
    ops.mlp(lib, handle, yd, xd, w12d, w3d, 1.0, True)
    torch.cuda.synchronize()
    _close(_bits(yd[rows.to(DEV)]).reshape(want.shape), want, 1e-3, 1e-3)


# ---- MLP composite (the reference's cases, operatorspy/tests/mlp.py:245-, and prefill-sized token counts) ------
@pytest.mark.parametrize("tokens,hidden,di,alpha,residual,x_stride,w12_stride,w3_stride", [
    (4, 4096, 11008, 1.0, True, None, None, None),
    (4, 4096, 11008, 1.0, True, (8192, 1), None, None),
    (4, 4096, 11008, 1.0, True, None, (1, 4096), (1, 11008)),
    (4, 4096, 11008, 1.0, False, None, None, None),
    (4, 4096, 11008, 1.0, False, (8192, 1), None, None),
    (300, 512, 1376, 0.5, True, None, None, None),
    (300, 512, 1376, 1.0, False, None, (1, 512), (1, 1376)),
    (1, 1024, 2752, 1.0, True, None, None, None),
    (33, 264, 100, 1.0, True, None, None, None),      # intermediate size that no TMA box divides
    (7, 72, 36, 1.0, False, None, (1, 76), None)])    # a leading dimension TMA cannot address: the three-step form
def test_mlp(oracle, cuda_lib, tokens, hidden, di, alpha, residual, x_stride, w12_stride, w3_stride):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(9)
    y = (torch.rand((tokens, hidden), generator=g) - 0.5).half()
    x = (torch.rand((tokens, hidden), generator=g) - 0.5).half()
    w12 = ((torch.rand((hidden, 2 * di), generator=g) - 0.5) * 0.1).half()
    w3 = ((torch.rand((di, hidden), generator=g) - 0.5) * 0.1).half()
    want = y.numpy().copy()
    oracle.mlp(want, x.numpy(), w12.numpy(), w3.numpy(), alpha, residual)
    yd, xd, w12d, w3d = (t.to(DEV) for t in (y, x, w12, w3))
    if x_stride is not None:
        xd, yd = rearrange_tensor(xd, x_stride), rearrange_tensor(yd, x_stride)
    if w12_stride is not None:
        w12d = rearrange_tensor(w12d, w12_stride)
    if w3_stride is not None:
        w3d = rearrange_tensor(w3d, w3_stride)
    ops.mlp(lib, handle, yd, xd, w12d, w3d, alpha, residual)
    torch.cuda.synchronize()
    _close(_bits(yd).reshape(tokens, hidden), want, 1e-3, 1e-3)
    assert torch.equal(xd.cpu(), x)


# ---- bf16 matmul and MLP (an extension: the reference's are fp16 / fp32; oracle = the restated functions on bf16
# patterns, oracle.bf16_storage) ---------------------------------------------------------------------------
@pytest.mark.parametrize("alpha,beta,a_shape,b_shape,c_shape,a_stride,b_stride,c_stride",
                         [c for c in MATMUL_CASES if c[2][-2] <= 512][:8] + [(1.0, 0.0, (600, 256), (256, 384), (600, 384), None, None, None),
                                                                             (0.5, 1.0, (3, 256), (256, 1024), (3, 1024), None, (1, 256), None)])
def test_bf16_matmul(oracle, cuda_lib, matmul_kernels, alpha, beta, a_shape, b_shape, c_shape, a_stride, b_stride, c_stride):
    """Within one bf16 ulp (2^-8 of the value) of the oracle, plus 1e-5 absolute for sums that cancel: only the
    grouping of the fp32 sum over k differs, so most elements are the same pattern."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(18)
    a, b, c = ((torch.rand(sh, generator=g) - 0.5).bfloat16() for sh in (a_shape, b_shape, c_shape))
    a, b, c = (t if st is None else rearrange_tensor(t, st) for t, st in ((a, a_stride), (b, b_stride), (c, c_stride)))
    want = c.clone()
    if c_stride is not None:
        want = rearrange_tensor(want, c_stride)
    with oracle.bf16_storage():
        oracle.matmul_into(want.view(torch.int16).numpy().view(np.uint16), a.view(torch.int16).numpy().view(np.uint16),
                           b.view(torch.int16).numpy().view(np.uint16), alpha, beta)
    ad, bd, cd = (t.to(DEV) for t in (a, b, c))
    ad, bd, cd = (t if st is None else rearrange_tensor(t, st) for t, st in ((ad, a_stride), (bd, b_stride), (cd, c_stride)))
    ops.matmul(lib, handle, cd, ad, bd, alpha, beta)
    torch.cuda.synchronize()
    assert _few(_bf16_close(_bf16_bits(cd), _bf16_bits(want), 1e-5, 2.0 ** -7), c.numel(), 0.25)


@pytest.mark.parametrize("tokens,hidden,di,alpha,residual", [(16, 512, 1408, 1.0, True), (300, 512, 1376, 0.5, True),
                                                             (640, 256, 512, 1.0, False), (7, 72, 36, 1.0, False)])
def test_bf16_mlp(oracle, cuda_lib, tokens, hidden, di, alpha, residual):
    """The MLP composite on bf16 tensors: fused SwiGLU epilogue (transposed and plain orientation, CTA pairs at 640
    tokens) and the three-step form for the last shape; within two bf16 ulps of the oracle (an intermediate that
    differs by one ulp moves a few sums by one more), plus 1e-4 absolute for sums that cancel."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(19)
    y = (torch.rand((tokens, hidden), generator=g) - 0.5).bfloat16()
    x = (torch.rand((tokens, hidden), generator=g) - 0.5).bfloat16()
    w12 = ((torch.rand((hidden, 2 * di), generator=g) - 0.5) * 0.1).bfloat16()
    w3 = ((torch.rand((di, hidden), generator=g) - 0.5) * 0.1).bfloat16()
    want = _bf16_bits(y).reshape(tokens, hidden).copy()
    with oracle.bf16_storage():
        oracle.mlp(want, _bf16_bits(x).reshape(x.shape), _bf16_bits(w12).reshape(w12.shape), _bf16_bits(w3).reshape(w3.shape),
                   alpha, residual)
    yd, xd, w12d, w3d = (t.to(DEV) for t in (y, x, w12, w3))
    ops.mlp(lib, handle, yd, xd, w12d, w3d, alpha, residual)
    torch.cuda.synchronize()
    assert _few(_bf16_close(_bf16_bits(yd), want, 1e-4, 2.0 ** -6), y.numel(), 0.25)


# ---- the five configurations the benchmark quotes, at full size -----------------------------------------
def _rows_in_parallel(fn, n, parts=None):
    """Runs fn(lo, hi) on row slices from a thread pool (the oracle's C functions release the GIL and
    rows are independent), so the full-size oracle passes take a second or two."""
    import os
    from concurrent.futures import ThreadPoolExecutor

    parts = parts or min(n, os.cpu_count() or 1)
    cuts = [n * i // parts for i in range(parts + 1)]
    with ThreadPoolExecutor(parts) as pool:
        list(pool.map(lambda i: fn(cuts[i], cuts[i + 1]), range(parts)))


def test_config_rope_4096x32x128(oracle, cuda_lib):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(2)
    t = torch.randn((4096, 32, 128), generator=g).half()
    pos = torch.arange(4096, dtype=torch.int64)
    sin, cos = ops.sin_cos_table(4096, 128, theta=1e4)
    want = t.numpy().copy()
    pn, sn, cn = pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy()
    _rows_in_parallel(lambda lo, hi: oracle.rope(want[lo:hi], pn[lo:hi], sn, cn), 4096)
    td = t.to(DEV)
    ops.rope(lib, handle, td, pos.to(DEV), sin.to(DEV), cos.to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(td).reshape(t.shape), want.view(np.uint16))


def test_config_swiglu_8192x28672_halves(oracle, cuda_lib):
    lib, handle = cuda_lib
    tokens, di = 8192, 14336
    g = torch.Generator().manual_seed(3)
    gate_up = torch.randn((tokens, 2 * di), generator=g).half()
    gn = gate_up.numpy()
    want = np.zeros((tokens, di), np.float16)
    _rows_in_parallel(lambda lo, hi: oracle.swiglu(gn[lo:hi, di:], gn[lo:hi, :di], c=want[lo:hi]), tokens)
    gd = gate_up.to(DEV)
    cd = torch.zeros((tokens, di), dtype=torch.float16, device=DEV)
    ops.swiglu(lib, handle, cd, gd[:, di:], gd[:, :di])
    torch.cuda.synchronize()
    mism = _close(_bits(cd).reshape(tokens, di), want, 1e-3, 1e-3)
    assert _few(mism, tokens * di, 2e-3)
    assert torch.equal(gd.cpu(), gate_up)  # the operands are untouched


def test_config_add_8192x4096(oracle, cuda_lib):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(4)
    a, b = torch.randn((8192, 4096), generator=g).half(), torch.randn((8192, 4096), generator=g).half()
    an, bn = a.numpy(), b.numpy()
    want = np.zeros((8192, 4096), np.float16)

    def part(lo, hi):
        want[lo:hi] = oracle.add(an[lo:hi], bn[lo:hi])

    _rows_in_parallel(part, 8192)
    cd = torch.zeros((8192, 4096), dtype=torch.float16, device=DEV)
    ops.add(lib, handle, cd, a.to(DEV), b.to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(cd).reshape(8192, 4096), want.view(np.uint16))


def test_config_causal_softmax_32x512x4096(oracle, cuda_lib):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(5)
    y = (torch.randn((32, 512, 4096), generator=g) * 2).half()
    want = y.numpy().copy()
    _rows_in_parallel(lambda lo, hi: oracle.causal_softmax(want[lo:hi]), 32)
    yd = y.to(DEV)
    ops.causal_softmax(lib, handle, yd)
    torch.cuda.synchronize()
    got = _bits(yd).reshape(y.shape)
    _close(got, want, 2e-3, 2e-3)
    # row i of every head sees 3585 + i columns; everything behind is an exact zero
    col = np.arange(4096)[None, None, :]
    masked = col > (np.arange(512)[None, :, None] + 4096 - 512)
    assert (got[np.broadcast_to(masked, got.shape)] == 0).all()
    assert (want.view(np.uint16)[np.broadcast_to(masked, got.shape)] == 0).all()


def test_config_rms_norm_scaled_65536x2048(oracle, cuda_lib):
    """The benchmark's scaled RMSNorm line (the 16 x 2048 configuration itself is in test_rms_norm)."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(1)
    x = (torch.rand((65536, 2048), generator=g) * 2 - 1).half()
    w = (torch.rand(2048, generator=g) * 2 - 1).half()
    xn, wn = x.numpy(), w.numpy()
    want = np.zeros((65536, 2048), np.float16)
    _rows_in_parallel(lambda lo, hi: oracle.rms_norm(xn[lo:hi], wn, 1e-5, y=want[lo:hi]), 65536)
    yd = torch.zeros((65536, 2048), dtype=torch.float16, device=DEV)
    ops.rms_norm(lib, handle, yd, x.to(DEV), w.to(DEV), 1e-5)
    torch.cuda.synchronize()
    mism = _close(_bits(yd).reshape(65536, 2048), want, 1e-3, 1e-3)
    assert _few(mism, x.numel(), 0.02)


# ---- attention over a KV cache (the reference's composite) ---------------------------------------------
ATTENTION_CASES = [
    # the reference's own three cases (operatorspy/tests/attention.py:310-357): prefill, decode, small
    (32, 4, 5, 64, 0, 2048, (64, 2560, 1), (64, 11264, 1)),
    (32, 4, 1, 64, 3, 2048, (64, 2560, 1), (64, 11264, 1)),
    (8, 4, 2, 16, 1, 8, None, None),
    # decoding over long caches: groups of 4 and 8 q heads, one q head per kv head, one kv head for all
    (32, 8, 1, 128, 4095, 4096, None, None),
    (64, 8, 1, 128, 9000, 9001, None, None),
    (16, 16, 1, 128, 2500, 4096, None, None),
    (8, 1, 1, 64, 700, 1024, None, None),
    (2, 1, 1, 256, 300, 512, None, None),
    # head sizes that are not a power of two / not whole vectors, odd strides
    (12, 4, 1, 80, 130, 256, None, None),
    (6, 2, 3, 20, 9, 32, None, None),
    (8, 4, 2, 64, 17, 64, (67, 1000, 1), (69, 9000, 1)),
    (4, 2, 1, 8, 5, 16, None, None),
    # prefill: several row tiles per kv head, with and without a prefix in the cache
    (8, 2, 37, 64, 0, 64, None, None),
    (8, 4, 19, 128, 11, 64, (128, 8 * 128, 1), None),
    (3, 3, 70, 32, 2100, 2200, None, None),
    # the smallest cases: an empty cache, a cache exactly as long as needed, five q heads on one kv head
    (4, 4, 1, 64, 0, 4, None, None),
    (5, 1, 1, 32, 0, 1, None, None),
    (2, 1, 3, 16, 0, 3, None, None),
    (10, 2, 1, 128, 63, 64, None, None),
    # several new tokens on the tcgen05 path: prefill from an empty cache, a long prefix, speculative decoding,
    # token counts and cache lengths that are not multiples of anything
    (32, 8, 512, 128, 0, 512, None, None),
    (32, 8, 40, 128, 4096, 4136, None, None),
    (8, 2, 300, 64, 77, 400, None, None),
    (4, 4, 130, 128, 1000, 1200, None, None),
    (16, 2, 33, 256, 31, 64, None, None),
    # the same with the reference's strided layouts (q, k, v as [seq, head, dh]; caches as [token, head, dh]) and
    # with exactly one / exactly two blocks of 128 query rows
    (32, 4, 200, 64, 100, 2048, (64, 2560, 1), (64, 11264, 1)),
    (4, 2, 128, 128, 0, 128, None, None),
    (4, 1, 256, 64, 64, 320, None, None),
    # 16 .. 127 new tokens with several q heads per kv head: the heads of a group share a block of 128 query rows
    # (groups of 4, 3 and 8; the reference's strided layouts; a block that the tokens do not fill)
    (32, 8, 16, 128, 500, 600, None, None),
    (12, 4, 40, 64, 300, 400, None, None),
    (16, 2, 20, 128, 70, 128, None, None),
    (32, 4, 50, 64, 100, 2048, (64, 2560, 1), (64, 11264, 1)),
    # head sizes between the 64-element boxes of the tcgen05 kernel (the boxes read the rest as zeros)
    (12, 4, 48, 80, 200, 256, None, None),
    (4, 4, 150, 96, 30, 256, None, None),
    (8, 2, 40, 40, 1000, 1100, None, None),
    # head sizes beyond 128: all of an SM's tensor memory, one CTA per SM; with and without a cluster
    (4, 4, 140, 192, 20, 200, None, None),
    (8, 2, 40, 256, 1500, 1600, None, None),
]


ATTENTION_KERNELS = {"tensor": 0, "multiply_add": 1, "row_tiles": 2, "three_launches": 3, "one_kernel": 4}


@pytest.fixture(params=list(ATTENTION_KERNELS))
def attention_kernels(request, cuda_lib):
    """The kernel families: the library's own choice (tcgen05 products for calls with several new tokens, the
    mma.sync row-tile kernels for decoding), the multiply-add kernels that otherwise serve unaligned layouts and
    head sizes above 128, the row-tile kernels everywhere, and for several new tokens the two tcgen05 forms (scores,
    softmax and values as three launches; one kernel that keeps the scores on chip) wherever each applies.  The
    choice is read when the descriptor is created."""
    ops.select_kernel(cuda_lib[0], "attention", ATTENTION_KERNELS[request.param])
    yield request.param
    ops.select_kernel(cuda_lib[0], "attention", 0)


_attention_oracle_cache = {}


@pytest.mark.parametrize("nh,nkvh,seq,dh,pos,buf_len,qkv_strides,cache_strides", ATTENTION_CASES)
def test_attention(oracle, cuda_lib, attention_kernels, nh, nkvh, seq, dh, pos, buf_len, qkv_strides, cache_strides):
    """out within the fp16 tolerance of the oracle's composite (only the grouping of fp32 sums
    differs, so most elements are the same bit pattern); both caches byte for byte,
    rows outside pos .. pos+seq untouched."""
    lib, handle = cuda_lib
    if attention_kernels in ("three_launches", "one_kernel") and seq < (16 if nh > nkvh else 32):
        pytest.skip("fewer than 32 new tokens (16 with several q heads per kv head) never take the tcgen05 forms")
    timeouts_before = ops.device_timeouts(lib, handle)  # counts since the library was loaded
    g = torch.Generator().manual_seed(21)
    q = torch.randn((nh, seq, dh), generator=g).half()
    k = torch.randn((nkvh, seq, dh), generator=g).half()
    v = torch.randn((nkvh, seq, dh), generator=g).half()
    k_cache = torch.randn((nkvh, buf_len, dh), generator=g).half()
    v_cache = torch.randn((nkvh, buf_len, dh), generator=g).half()
    if qkv_strides is not None:
        q, k, v = (rearrange_tensor(t, qkv_strides) for t in (q, k, v))
    if cache_strides is not None:
        k_cache, v_cache = (rearrange_tensor(t, cache_strides) for t in (k_cache, v_cache))

    def dev(t):  # same strides on the device
        st = t.stride()
        return rearrange_tensor(t.to(DEV), st) if not t.is_contiguous() else t.to(DEV)

    qd, kd, vd, kcd, vcd = (dev(t) for t in (q, k, v, k_cache, v_cache))
    out = torch.full((seq, nh, dh), 7.0, dtype=torch.float16, device=DEV)
    with ops.AttentionOp(lib, handle, out, qd, kd, vd, kcd, vcd, pos) as op:
        op.workspace.fill_(0xAB)  # the workspace arrives with arbitrary contents
        op(out, qd, kd, vd, kcd, vcd)
        torch.cuda.synchronize()
        first = out.clone()
        op(out, qd, kd, vd, kcd, vcd)  # same descriptor and workspace again
        torch.cuda.synchronize()
    key = (nh, nkvh, seq, dh, pos, buf_len, qkv_strides, cache_strides)
    if key not in _attention_oracle_cache:  # the same inputs for every kernel family: one oracle pass per case
        _attention_oracle_cache[key] = (oracle.attention(q.numpy(), k.numpy(), v.numpy(), k_cache.numpy(),
                                                         v_cache.numpy(), pos), k_cache.clone(), v_cache.clone())
    want, k_cache, v_cache = _attention_oracle_cache[key]
    assert torch.equal(first, out)
    mism = _close(_bits(out).reshape(want.shape), want, 1e-3, 1e-3)
    # sums of thousands of terms of both signs: a different grouping moves the last bit of more elements than elsewhere
    assert _few(mism, want.size, 0.25)
    assert torch.equal(kcd.cpu(), k_cache) and torch.equal(vcd.cpu(), v_cache)  # the oracle updated the host caches
    assert ops.device_timeouts(lib, handle) == timeouts_before


@pytest.mark.parametrize("kernels", ["three_launches", "one_kernel"])
def test_attention_scores_at_the_top_of_the_fp16_range(oracle, cuda_lib, kernels):
    """q = k = 90.5 in every element: alpha * q.k = 65522, which the reference's truncating rule stores as the largest
    finite fp16 (65504).  The one-kernel form converts scores two at a time with a saturating instruction and
    redoes a chunk element by element when it sees that value; this is the case that takes that path (and the row
    of equal scores makes every probability 1 / visible columns)."""
    lib, handle = cuda_lib
    nh, nkvh, seq, dh, pos = 4, 2, 40, 64, 30
    g = torch.Generator().manual_seed(29)
    q = torch.full((nh, seq, dh), 90.5).half()
    k = torch.full((nkvh, seq, dh), 90.5).half()
    v = torch.randn((nkvh, seq, dh), generator=g).half()
    kc = torch.full((nkvh, pos + seq, dh), 90.5).half()
    vc = torch.randn((nkvh, pos + seq, dh), generator=g).half()
    want = oracle.attention(q.numpy(), k.numpy(), v.numpy(), kc.numpy().copy(), vc.numpy().copy(), pos)
    assert np.isfinite(want.astype(np.float32)).all()
    out = torch.zeros((seq, nh, dh), dtype=torch.float16, device=DEV)
    ops.select_kernel(lib, "attention", ATTENTION_KERNELS[kernels])
    try:
        ops.attention(lib, handle, out, q.to(DEV), k.to(DEV), v.to(DEV), kc.to(DEV), vc.to(DEV), pos)
        torch.cuda.synchronize()
    finally:
        ops.select_kernel(lib, "attention", 0)
    _close(_bits(out).reshape(want.shape), want, 1e-3, 1e-3)


@pytest.mark.parametrize("kernels", ["three_launches", "one_kernel"])
@pytest.mark.parametrize("nh,nkvh,seq,dh,pos", [(8, 2, 1024, 128, 0), (8, 4, 600, 64, 1000), (4, 1, 1536, 128, 512),
                                                (16, 4, 2048, 128, 0),
                                                # few blocks of query rows: clusters of CTAs split the cached tokens (the
                                                # first block of the first shape sees two tiles, so two of its four
                                                # CTAs have none), few new tokens over a long prefix
                                                (4, 1, 1024, 128, 0), (8, 2, 64, 128, 6000), (2, 2, 200, 64, 3000)])
def test_attention_long_prefill_against_float32(cuda_lib, nh, nkvh, seq, dh, pos, kernels):
    """Token counts at which the three-launch form runs its products on CTA pairs with the causal tile skipping
    (several 256-row blocks per head) and the one-kernel form walks dozens of tiles per block of query rows.  The
    oracle would take minutes here, so the check is against a float32 evaluation of the same composite on the GPU
    (scores, causal mask, softmax, values) with a tolerance that covers the two fp16 roundings in between; the
    smaller cases of test_attention pin the same paths to the oracle."""
    lib, handle = cuda_lib
    timeouts_before = ops.device_timeouts(lib, handle)
    ops.select_kernel(lib, "attention", ATTENTION_KERNELS[kernels])
    g = torch.Generator().manual_seed(23)
    total = pos + seq
    q = torch.randn((nh, seq, dh), generator=g).half().to(DEV)
    k = torch.randn((nkvh, seq, dh), generator=g).half().to(DEV)
    v = torch.randn((nkvh, seq, dh), generator=g).half().to(DEV)
    kc = torch.randn((nkvh, total, dh), generator=g).half().to(DEV)
    vc = torch.randn((nkvh, total, dh), generator=g).half().to(DEV)
    out = torch.zeros((seq, nh, dh), dtype=torch.float16, device=DEV)
    try:
        ops.attention(lib, handle, out, q, k, v, kc, vc, pos)
        torch.cuda.synchronize()
    finally:
        ops.select_kernel(lib, "attention", 0)
    assert ops.device_timeouts(lib, handle) == timeouts_before
    assert torch.equal(kc[:, pos:], k) and torch.equal(vc[:, pos:], v)
    group = nh // nkvh
    kf, vf = kc.float().repeat_interleave(group, 0), vc.float().repeat_interleave(group, 0)
    scores = torch.einsum("hsd,htd->hst", q.float(), kf) / dh ** 0.5
    cols, rows = torch.arange(total, device=DEV)[None, None, :], torch.arange(seq, device=DEV)[None, :, None]
    scores = scores.masked_fill(cols > rows + (total - seq), float("-inf"))
    want = torch.einsum("hst,htd->hsd", torch.softmax(scores, -1), vf).permute(1, 0, 2)
    err = (out.float() - want).abs()
    assert float(err.max()) < 4e-3 + 4e-3 * float(want.abs().max())


@pytest.mark.parametrize("seq,pos", [(1, 3000), (160, 100), (40, 3000)])
def test_attention_captures_into_a_cuda_graph(oracle, cuda_lib, seq, pos):
    """The launches of one call (decoding: two; a prompt: the cache append and the one-kernel form; a short chunk over
    a long prefix: the same as a cluster launch) neither allocate nor synchronise: captured after one eager call (one-time kernel attribute set-up), replayed on a cleared output
    and workspace."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(31)
    nh, nkvh, dh = 16, 4, 128
    q, k, v = (torch.randn(sh, generator=g).half() for sh in ((nh, seq, dh), (nkvh, seq, dh), (nkvh, seq, dh)))
    kc, vc = torch.randn((nkvh, pos + seq, dh), generator=g).half(), torch.randn((nkvh, pos + seq, dh), generator=g).half()
    qd, kd, vd, kcd, vcd = (t.to(DEV) for t in (q, k, v, kc, vc))
    out = torch.zeros((seq, nh, dh), dtype=torch.float16, device=DEV)
    with ops.AttentionOp(lib, handle, out, qd, kd, vd, kcd, vcd, pos) as op:
        op(out, qd, kd, vd, kcd, vcd)
        torch.cuda.synchronize()
        eager = out.clone()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            op(out, qd, kd, vd, kcd, vcd, torch.cuda.current_stream().cuda_stream)
        out.zero_()
        if op.workspace is not None and op.workspace.numel():
            op.workspace.fill_(0x5A)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)
    want = oracle.attention(q.numpy(), k.numpy(), v.numpy(), kc.numpy(), vc.numpy(), pos)
    assert _few(_close(_bits(out).reshape(want.shape), want, 1e-3, 1e-3), want.size, 0.25)


def test_attention_status_codes(cuda_lib):
    from operators_b200 import InfiniopError

    lib, handle = cuda_lib

    def h(*shape):
        return torch.zeros(shape, dtype=torch.float16, device=DEV)

    def status(fn):
        with pytest.raises(InfiniopError) as e:
            fn()
        return e.value.status

    out, q, k, v, kc, vc = h(2, 8, 16), h(8, 2, 16), h(4, 2, 16), h(4, 2, 16), h(4, 8, 16), h(4, 8, 16)
    assert status(lambda: ops.AttentionOp(lib, handle, out[0], q, k, v, kc, vc, 1)) == 4       # ndim
    assert status(lambda: ops.AttentionOp(lib, handle, out[:, :, ::2], q[:, :, :8], k[:, :, :8], v[:, :, :8],
                                          kc[:, :, :8], vc[:, :, :8], 1)) == 5               # out not contiguous
    assert status(lambda: ops.AttentionOp(lib, handle, out, q, k, v, kc, vc, 7)) == 2           # cache too short
    assert status(lambda: ops.AttentionOp(lib, handle, out, q, k[:3], v, kc, vc, 1)) == 2       # k and v disagree
    assert status(lambda: ops.AttentionOp(lib, handle, h(2, 6, 16), h(6, 2, 16), k, v, kc, vc, 1)) == 2  # 6 % 4 != 0
    assert status(lambda: ops.AttentionOp(lib, handle, out.float(), q, k, v, kc, vc, 1)) == 3
    with ops.AttentionOp(lib, handle, out, q, k, v, kc, vc, 1) as op:
        assert op.workspace_size > 0
        assert lib.infiniopAttention(op.desc, op.workspace.data_ptr(), op.workspace_size - 1, out.data_ptr(),
                                     q.data_ptr(), k.data_ptr(), v.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                     None) == 6                                               # workspace too small


# ---- descriptor validation: same status codes as the reference ------------------------
def test_status_codes(cuda_lib):
    import ctypes

    from operators_b200 import DeviceEnum, InfiniopError, create_handle, open_lib

    lib, handle = cuda_lib
    h16 = torch.zeros((4, 8), dtype=torch.float16, device=DEV)
    f32 = torch.zeros((4, 8), dtype=torch.float32, device=DEV)

    def status(fn):
        with pytest.raises(InfiniopError) as e:
            fn()
        return e.value.status

    assert status(lambda: ops.SwiGLUOp(lib, handle, h16, h16, h16[:2])) == 2       # BAD_PARAM (shape mismatch of a/b)
    assert status(lambda: ops.SwiGLUOp(lib, handle, f32, f32, f32)) == 3           # BAD_TENSOR_DTYPE
    assert status(lambda: ops.SwiGLUOp(lib, handle, h16.t(), h16.t(), h16.t())) == 5  # BAD_TENSOR_STRIDES
    assert status(lambda: ops.SwiGLUOp(lib, handle, h16[0], h16[0], h16[0])) == 4  # BAD_TENSOR_SHAPE
    assert status(lambda: ops.AddOp(lib, handle, h16, h16, h16[:, :3])) == 4
    assert status(lambda: ops.AddOp(lib, handle, h16, h16, f32)) == 3
    assert status(lambda: ops.AddOp(lib, handle, h16[:, ::2], h16[:, ::2], h16[:, ::2])) == 5
    assert status(lambda: ops.RMSNormOp(lib, handle, h16, h16, h16[0, :4])) == 4
    assert status(lambda: ops.CausalSoftmaxOp(lib, handle, h16[0])) == 4
    assert status(lambda: ops.CausalSoftmaxOp(lib, handle, f32)) == 3
    assert status(lambda: ops.RoPEOp(lib, handle, h16, torch.zeros(4, dtype=torch.int64, device=DEV), f32, f32)) == 4
    assert status(lambda: create_handle(lib, DeviceEnum.DEVICE_CPU)) == 8          # no CPU path in this library
    assert status(lambda: create_handle(lib, DeviceEnum.DEVICE_CUDA, 1000)) == 8
    assert status(lambda: create_handle(lib, DeviceEnum.DEVICE_CUDA, -1)) == 2
    assert lib.infiniopCreateHandle(None, 1, 0) == 6


# ---- vocabulary-sharded sampling on one GPU, the ranks played in turn ------------------------------------
SHARDED_CASES = [(128256, 64, 0.9, 50, 0.8, "normal3"), (32000, 40, 0.8, 50, 1.0, "uniform"),
                 (16384, 32, 0.85, 10, 2.0, "normal3"), (5003, 13, 0.9, 20, 1.0, "normal3")]
_sharded_oracle_cache = {}


def _sharded_inputs(oracle, voc, rows, topp, topk, temp, dist):
    key = (voc, rows, topp, topk, temp, dist)
    if key not in _sharded_oracle_cache:
        g = torch.Generator().manual_seed(8)
        logits = torch.rand((rows, voc), generator=g).half() if dist == "uniform" else (torch.randn((rows, voc), generator=g) * 3).half()
        u = torch.rand(rows, generator=g)
        want = [oracle.random_sample(logits[r].numpy(), float(u[r]), topp, topk, temp) for r in range(rows)]
        _sharded_oracle_cache[key] = (logits, u, want)
    return _sharded_oracle_cache[key]


@pytest.mark.parametrize("exchange", ["all_to_all", "all_gather"])
@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
@pytest.mark.parametrize("voc,rows,topp,topk,temp,dist", SHARDED_CASES)
def test_vocab_sharded_sampling_is_index_exact(oracle, cuda_lib, ranks, voc, rows, topp, topk, temp, dist, exchange):
    """The default mode: every rank receives whole rows through one all-to-all, samples them with the exact
    kernel and the indices are all-gathered.  EVERY row's index must be the oracle's.  The collectives are
    played by closures that hand each rank what the other ranks would send."""
    from operators_b200.sharding import VocabShardedSampler, exchange_plan, row_range, vocab_range

    lib, handle = cuda_lib
    if exchange == "all_gather" and voc % ranks != 0:
        pytest.skip("the all-gather exchange needs equal shards")
    logits, u, want = _sharded_inputs(oracle, voc, rows, topp, topk, temp, dist)
    ld, ud = logits.to(DEV), u.to(DEV)
    sent = {}
    final = None
    for r in list(range(ranks)) + [0]:  # every rank once, then rank 0 again with everybody's indices at hand
        b, e = vocab_range(voc, ranks, r)
        shard = ld[:, b:e].contiguous()

        def all_to_all(out, inp, out_splits, in_splits, r=r):
            (r0, r1), send, recv, cols = exchange_plan(rows, voc, ranks, r)
            assert list(out_splits) == recv and list(in_splits) == send and inp.numel() == sum(send)
            if exchange == "all_gather":  # every shard whole, rank after rank: [ranks][rows][columns]
                vl = voc // ranks
                out[:ranks * rows * vl].view(ranks, rows, vl).copy_(ld.view(rows, ranks, vl).permute(1, 0, 2))
                return
            off = 0
            for (cb, ce), n in zip(cols, recv):
                out[off:off + n].copy_(ld[r0:r1, cb:ce].reshape(-1))
                off += n

        def all_gather(out, inp, r=r):
            sent[r] = inp.clone()
            if len(sent) == ranks:
                for k in range(ranks):
                    out[k].copy_(sent[k])

        res = torch.full((rows,), -1, dtype=torch.int64, device=DEV)
        with ops.RandomSampleOp(lib, handle, res[:1], shard[0]) as op:
            s = VocabShardedSampler(lib, handle, op, voc, b, ranks, rank=r, all_to_all=all_to_all, all_gather=all_gather,
                                    exchange=exchange)
            s.sample(res, shard, ud, topp, topk, temp)
            torch.cuda.synchronize()
            s.destroy()
        final = res
    assert final.cpu().tolist() == want
    for r in range(ranks):  # what each rank contributed: exactly its own rows
        r0, r1 = row_range(rows, ranks, r)
        assert sent[r][:r1 - r0].cpu().tolist() == want[r0:r1]


@pytest.mark.parametrize("one_launch", [True, False], ids=["one_launch", "three_launches"])
@pytest.mark.parametrize("ranks", [1, 2, 4, 8])
@pytest.mark.parametrize("voc,rows,topp,topk,temp,dist", SHARDED_CASES)
def test_vocab_sharded_sampling_over_peer_memory_blocks(oracle, cuda_lib, ranks, voc, rows, topp, topk, temp, dist, one_launch):
    """The exact mode without collectives: every rank's shard sits in a block the others address, one kernel pulls a
    rank's rows out of all blocks, one pushes its indices into all of them.  Here the ranks are played one after the
    other on one GPU, their blocks all local; kernels that wait for each other must not run as separate launches
    on one GPU, so the flags that the absent peers would raise are set beforehand and no launch ever waits.  What is
    checked is the addressing (rows, column ranges, unequal shards), the call counter over two rounds, and that
    every block ends up with every row's index = the oracle's, with the exchange as two launches around the sampling
    kernel and folded into it (where shards are equal and whole vectors; other shapes take the three launches
    either way).  The flag protocol between real ranks runs in tests/peer_ranks.py on two GPUs."""
    from operators_b200.sharding import PeerBlocks, VocabShardedSampler, vocab_range

    lib, handle = cuda_lib
    logits, u, want = _sharded_inputs(oracle, voc, rows, topp, topk, temp, dist)
    ld, ud = logits.to(DEV), u.to(DEV)
    timeouts_before = ops.device_timeouts(lib, handle)
    blocks, samplers, keep = [], [], []
    for r in range(ranks):
        b, e = vocab_range(voc, ranks, r)
        pb = PeerBlocks(lib, handle, rows, e - b, ranks, r, DEV, local_blocks=blocks)
        op = ops.RandomSampleOp(lib, handle, pb.results[:1], pb.logits[0])
        keep.append(op)
        samplers.append(VocabShardedSampler(lib, handle, op, voc, b, ranks, rank=r, exchange="peer_memory", peer_blocks=pb,
                                            one_launch=one_launch))
    try:
        for round_no in range(2):
            for r, pb in enumerate(blocks):
                b, e = vocab_range(voc, ranks, r)
                pb.logits[:rows].copy_(ld[:, b:e])
                pb.results.fill_(-1)
                pb.flags[:32].fill_(0x3FFFFFFF)  # as if every peer had raised its flags for this and any later call
            for r, s in enumerate(samplers):
                s.sample(blocks[r].results, blocks[r].logits[:rows], ud, topp, topk, temp)
            torch.cuda.synchronize()
            for pb in blocks:
                assert pb.results[:rows].cpu().tolist() == want
                assert int(pb.flags[32].item()) == round_no + 1  # the call counter the kernels keep in the block
        assert ops.device_timeouts(lib, handle) == timeouts_before
    finally:
        torch.cuda.synchronize()
        for s in samplers:
            s.destroy()
        for op in keep:
            op.destroy()
        for pb in blocks:
            pb.destroy()


@pytest.mark.parametrize("one_launch", [True, False], ids=["one_launch", "three_launches"])
def test_peer_memory_wait_runs_out_when_a_rank_never_shows_up(cuda_lib, one_launch):
    """Failure detection without a fault: of two ranks only rank 0 samples, so the words rank 1 would raise never
    arrive.  Every wait gives up after its clock budget (about a second), the call has returned STATUS_SUCCESS
    long before, the context stays usable, and infiniopExtDeviceTimeouts reports the waits that ran out.  (The
    one-launch form then samples from what the shards hold; the gather kernel of the three-launch form leaves the
    columns of a peer it gave up on unwritten.)"""
    import time

    from operators_b200.sharding import PeerBlocks, VocabShardedSampler, vocab_range

    lib, handle = cuda_lib
    voc, rows, ranks = 4096, 2, 2
    g = torch.Generator().manual_seed(5)
    ld = (torch.randn((rows, voc), generator=g) * 3).half().to(DEV)
    ud = torch.rand(rows, generator=g).to(DEV)
    before = ops.device_timeouts(lib, handle)
    blocks = []
    for r in range(ranks):
        b, e = vocab_range(voc, ranks, r)
        pb = PeerBlocks(lib, handle, rows, e - b, ranks, r, DEV, local_blocks=blocks)  # appends itself to `blocks`
        pb.logits[:rows].copy_(ld[:, b:e])
    op = ops.RandomSampleOp(lib, handle, blocks[0].results[:1], blocks[0].logits[0])
    s = VocabShardedSampler(lib, handle, op, voc, 0, ranks, rank=0, exchange="peer_memory", peer_blocks=blocks[0],
                            one_launch=one_launch)
    whole = torch.zeros(rows, dtype=torch.int64, device=DEV)
    ref = ops.RandomSampleOp(lib, handle, whole[:1], ld[0])
    try:
        ref.batch(whole, ld, ud, 0.9, 50, 0.8)
        t0 = time.time()
        s.sample(blocks[0].results, blocks[0].logits[:rows], ud, 0.9, 50, 0.8)  # returns at once
        issued = time.time() - t0
        torch.cuda.synchronize()
        waited = time.time() - t0
        assert issued < 0.5 and 0.5 < waited < 20.0
        assert ops.device_timeouts(lib, handle) > before
        if one_launch:  # rank 0 owns row 0; the one-launch form reads the shards after its wait, and the data was there
            assert int(blocks[0].results[0].item()) == int(whole[0].item())
        y = torch.ones(8, device=DEV) * 2  # the context still works
        assert float(y.sum().item()) == 16.0
    finally:
        torch.cuda.synchronize()
        s.destroy()
        op.destroy()
        ref.destroy()
        for pb in blocks:
            pb.destroy()


def test_random_sample_batch_peer_status_codes(cuda_lib):
    """The one-launch form states its conditions as status codes (the caller then takes the three launches): no
    rows, the greedy branch, shards that are not whole 16-byte vectors, shards that do not add up to the row."""
    import ctypes

    from operators_b200.sharding import PeerBlocks

    lib, handle = cuda_lib
    rows, voc = 4, 4096
    blocks = []
    pb = PeerBlocks(lib, handle, rows, voc, 1, 0, DEV, local_blocks=blocks)
    op = ops.RandomSampleOp(lib, handle, pb.results[:1], pb.logits[0])
    u = torch.rand(rows, device=DEV)
    one = lambda v: (ctypes.c_void_p * 1)(v)  # noqa: E731
    shards, flags, res = one(pb.ptr + pb.logits_off), one(pb.ptr), one(pb.ptr + pb.results_off)
    strides = (ctypes.c_int64 * 1)(voc)

    def call(nrows=rows, cols=voc, topp=0.9, topk=50, temp=0.8, stride=None):
        st = strides if stride is None else (ctypes.c_int64 * 1)(stride)
        return lib.infiniopRandomSampleBatchPeer(op.desc, res, shards, st, cols, flags, 1, 0, 0, nrows, u.data_ptr(), topp, topk,
                                                 temp, None)

    try:
        assert call() == 0
        torch.cuda.synchronize()
        bad_param = 2  # STATUS_BAD_PARAM
        assert call(nrows=0) == bad_param
        assert call(topp=0.0) == bad_param and call(topk=1) == bad_param and call(temp=0.0) == bad_param
        assert call(cols=voc - 8) == bad_param      # shards do not add up to the descriptor's row
        assert call(stride=voc + 4) == bad_param    # rows that do not start on 16-byte boundaries
        assert lib.infiniopRandomSampleBatchPeer(op.desc, res, shards, strides, voc, flags, 17, 0, 0, rows, u.data_ptr(), 0.9, 50,
                                                 0.8, None) == bad_param
    finally:
        torch.cuda.synchronize()
        op.destroy()
        pb.destroy()


def test_vocab_sharded_sampling_over_peer_memory_two_gpus():
    """Two real ranks on two GPUs: CUDA IPC blocks, the flag protocol, three rounds, indices against the unsharded
    sampler; tests/peer_ranks.py is the program both ranks run."""
    import subprocess
    import sys

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), "peer_ranks.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", script],
                       capture_output=True, text=True, timeout=300, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0 and "peer ranks ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("ranks", [1, 2, 8])
@pytest.mark.parametrize("voc,rows,topp,topk,temp,dist", SHARDED_CASES[:3])
def test_vocab_sharded_sampling_fast_mode(oracle, cuda_lib, ranks, voc, rows, topp, topk, temp, dist):
    """Fast mode: stage 1 per shard, records concatenated in rank order (what the all-gather
    delivers), stage 2.  The top-k and its tie order must be the oracle's in every
    row; the index may differ in rare rows because the sharded denominator is the
    correctly rounded sum, not the reference's sequential fp32 sum."""
    from operators_b200.sharding import VocabShardedSampler, vocab_range

    lib, handle = cuda_lib
    logits, u, want = _sharded_inputs(oracle, voc, rows, topp, topk, temp, dist)
    ld, ud = logits.to(DEV), u.to(DEV)
    res = torch.full((rows,), -1, dtype=torch.int64, device=DEV)
    shards, samplers, keep = [], [], []
    for r in range(ranks):
        b, e = vocab_range(voc, ranks, r)
        shard = ld[:, b:e]
        op = ops.RandomSampleOp(lib, handle, res[:1], shard[0])
        keep.append(op)
        shards.append((shard, b))
        samplers.append(VocabShardedSampler(lib, handle, op, voc, b, ranks, all_gather=lambda out, inp: None, mode="fast",
                                            rank=r))
    # play stage 1 of every rank, then hand rank 0 the gathered buffer
    locals_ = []
    for (shard, b), s in zip(shards, samplers):
        local, gathered, status = s._buffers(rows, shard.device)
        from operators_b200.utils import check_error
        check_error(lib.infiniopRandomSampleShardLocal(s.op.desc, local.data_ptr(), shard.data_ptr(), shard.stride(0), rows,
                                                       b, topk, temp, None))
        locals_.append(local)
    all_records = torch.stack(locals_)

    def fake_gather(out, inp):
        out.copy_(all_records)

    samplers[0]._gather = fake_gather
    samplers[0].sample(res, shards[0][0], ud, topp, topk, temp)
    torch.cuda.synchronize()
    same = sum(int(int(res[r]) == want[r]) for r in range(rows))
    assert same >= rows - max(1, rows // 20), (same, rows)
    # candidates gathered from the shards contain the oracle's top-k, in index order per shard
    rec = all_records.cpu().numpy().view(np.uint32)
    for r in range(0, rows, 7):
        top = set(int(i) for i in oracle.random_sample_trace(logits[r].numpy(), topk, temp)["top_idx"])
        have = set()
        for k in range(ranks):
            cnt = int(rec[k, r, 0])
            idx = rec[k, r, 8:8 + 2 * cnt:2]
            assert (np.diff(idx.astype(np.int64)) > 0).all()
            have |= set(int(i) for i in idx)
        assert top <= have
    for op in keep:
        op.destroy()


def test_vocab_sharded_fast_mode_mismatch_rate(cuda_lib):
    """How often the fast mode's index differs from the exact kernel's (which the tests above pin to the
    oracle): 10240 rows of 128256 logits ~ N(0, 3), T 0.8, top-k 50, top-p 0.9, eight shards.  The rate is
    printed (run with -s to see it) and bounded."""
    from operators_b200.sharding import VocabShardedSampler, vocab_range
    from operators_b200.utils import check_error

    lib, handle = cuda_lib
    voc, ranks, chunk, chunks = 128256, 8, 512, 20
    g = torch.Generator(device=DEV).manual_seed(99)
    differ = total = 0
    for _ in range(chunks):
        ld = (torch.randn((chunk, voc), generator=g, device=DEV) * 3).half()
        ud = torch.rand(chunk, generator=g, device=DEV)
        exact = torch.full((chunk,), -1, dtype=torch.int64, device=DEV)
        fast = torch.full((chunk,), -1, dtype=torch.int64, device=DEV)
        with ops.RandomSampleOp(lib, handle, exact[:1], ld[0]) as op:
            op.batch(exact, ld, ud, 0.9, 50, 0.8)
        locals_, keep, first = [], [], None
        for r in range(ranks):
            b, e = vocab_range(voc, ranks, r)
            shard = ld[:, b:e]
            op = ops.RandomSampleOp(lib, handle, fast[:1], shard[0])
            keep.append(op)
            s = VocabShardedSampler(lib, handle, op, voc, b, ranks, mode="fast", rank=r, all_gather=lambda out, inp: None)
            local, _, _ = s._buffers(chunk, DEV)
            check_error(lib.infiniopRandomSampleShardLocal(op.desc, local.data_ptr(), shard.data_ptr(), shard.stride(0),
                                                           chunk, b, 50, 0.8, None))
            locals_.append(local)
            first = first or (s, shard)
        records = torch.stack(locals_)
        first[0]._gather = lambda out, inp: out.copy_(records)
        first[0].sample(fast, first[1], ud, 0.9, 50, 0.8)
        torch.cuda.synchronize()
        differ += int((fast != exact).sum())
        total += chunk
        for op in keep:
            op.destroy()
    print("fast-mode rows whose index differs from the exact kernel's: %d of %d (%.4f %%)" % (differ, total, 100.0 * differ / total))
    assert differ <= total // 100


def test_vocab_sharded_overflow_is_reported(cuda_lib):
    from operators_b200.sharding import VocabShardedSampler

    lib, handle = cuda_lib
    logits = torch.full((4, 4096), 1.0, dtype=torch.float16, device=DEV)  # every element ties with every other
    res = torch.zeros(4, dtype=torch.int64, device=DEV)
    with ops.RandomSampleOp(lib, handle, res[:1], logits[0]) as op:
        s = VocabShardedSampler(lib, handle, op, 4096, 0, 1, mode="fast")
        with pytest.raises(RuntimeError):
            s.sample(res, logits, torch.rand(4, device=DEV), 0.9, 20, 1.0)


# ---- host buffers through the three-stream staging ---------------------------------
def test_staged_pipeline_host_buffers(oracle, cuda_lib):
    """Add (out of place) and RoPE (in place) fed from pinned host tensors through StagedPipeline,
    three passes in a row with fresh host inputs each time: every pass must return that pass's
    results (the event chain keeps uploads from overtaking the previous pass's downloads)."""
    from operators_b200.staging import Stage, StagedPipeline

    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(77)
    n_tok, nh, dh = 257, 4, 64
    a_h = torch.zeros((1 << 16,), dtype=torch.float16).pin_memory()
    b_h = torch.zeros_like(a_h).pin_memory()
    c_h = torch.zeros_like(a_h).pin_memory()
    t_h = torch.zeros((n_tok, nh, dh), dtype=torch.float16).pin_memory()
    t_out = torch.zeros_like(t_h).pin_memory()
    pos = torch.arange(n_tok, dtype=torch.int64)
    sin, cos = ops.sin_cos_table(n_tok, dh)
    a_d, b_d, c_d, t_d = (x.to(DEV) for x in (a_h, b_h, c_h, t_h))
    pos_d, sin_d, cos_d = pos.to(DEV), sin.to(DEV), cos.to(DEV)
    add_op = ops.AddOp(lib, handle, c_d, a_d, b_d)
    rope_op = ops.RoPEOp(lib, handle, t_d, pos_d, sin_d, cos_d)
    pipe = StagedPipeline([
        Stage("add", [(a_d, a_h), (b_d, b_h)], lambda s: add_op(c_d, a_d, b_d, s), [(c_d, c_h)]),
        Stage("rope", [(t_d, t_h)], lambda s: rope_op(t_d, pos_d, sin_d, cos_d, s), [(t_d, t_out)]),
    ], DEV)
    for it in range(3):
        a = torch.randn(a_h.shape, generator=g).half()
        b = torch.randn(a_h.shape, generator=g).half()
        t = torch.randn(t_h.shape, generator=g).half()
        pipe.synchronize()  # the host buffers are read asynchronously: refill them only when idle
        a_h.copy_(a), b_h.copy_(b), t_h.copy_(t)
        pipe.run()
        pipe.synchronize()
        want_c = oracle.add(a.numpy(), b.numpy())
        want_t = oracle.rope(t.numpy().copy(), pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
        assert np.array_equal(c_h.numpy().view(np.uint16), want_c.view(np.uint16)), it
        assert np.array_equal(t_out.numpy().view(np.uint16), want_t.view(np.uint16)), it
    # back-to-back passes without waiting in between: the last pass's results are the ones left
    pipe.run()
    pipe.run()
    pipe.synchronize()
    assert np.array_equal(t_out.numpy().view(np.uint16), want_t.view(np.uint16))


# ---- rearrange -------------------------------------------------------------------
REARRANGE_GPU_CASES = [
    # the reference's own cases (reference operatorspy/tests/rearrange.py:109-117)
    (((2, 4, 32), None), ((2, 4, 32), (256, 64, 1)), torch.float16),
    (((32, 6, 64), (64, 2560, 1)), ((32, 6, 64), None), torch.float16),
    (((4, 6, 64), (64, 2560, 1)), ((4, 6, 64), (131072, 64, 1)), torch.float16),
    (((1, 32, 64), (2048, 64, 1)), ((1, 32, 64), (2048, 64, 1)), torch.float16),
    (((32, 1, 64), (64, 2560, 1)), ((32, 1, 64), (64, 64, 1)), torch.float16),
    (((4, 1, 64), (64, 2560, 1)), ((4, 1, 64), (64, 11264, 1)), torch.float16),
    # other ranks, element sizes and alignments
    (((77,), None), ((77,), None), torch.float16),
    (((5, 33), (40, 1)), ((5, 33), None), torch.float32),
    (((3, 7), (9, 1)), ((3, 7), (11, 1)), torch.uint8),
    (((2, 3, 4, 8), None), ((2, 3, 4, 8), (200, 50, 10, 1)), torch.float16),
    (((2, 3, 4, 5, 6), (1000, 300, 70, 12, 1)), ((2, 3, 4, 5, 6), None), torch.float64),
    # KV-cache write: 32 heads x 128 of 64 new tokens into a [heads, max_seq, 128] cache, and a decode-sized q
    (((64, 32, 128), None), ((64, 32, 128), (128, 4096 * 128, 1)), torch.float16),
    (((1024, 32, 128), (128, 1024 * 128, 1)), ((1024, 32, 128), None), torch.float16),
]


@pytest.mark.parametrize("src_spec,dst_spec,dtype", REARRANGE_GPU_CASES)
def test_rearrange(oracle, cuda_lib, src_spec, dst_spec, dtype):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(9)
    x = (torch.rand(src_spec[0], generator=g) * 200).to(dtype)
    if src_spec[1] is not None:
        x = rearrange_tensor(x, src_spec[1])
    make_dst = lambda: (torch.full(dst_spec[0], 7, dtype=dtype) if dst_spec[1] is None
                        else rearrange_tensor(torch.full(dst_spec[0], 7, dtype=dtype), dst_spec[1]))
    want = make_dst()
    oracle.rearrange(want.numpy(), x.numpy())
    storage = lambda t: torch.as_strided(t, (sum(st * (sz - 1) for st, sz in zip(t.stride(), t.shape)) + 1,), (1,))
    xd_store, yd_store = storage(x).to(DEV), storage(make_dst()).to(DEV)
    xd = torch.as_strided(xd_store, x.shape, x.stride())
    yd = torch.as_strided(yd_store, want.shape, want.stride())
    ops.rearrange(lib, handle, yd, xd)
    torch.cuda.synchronize()
    # the whole destination storage: the copied rows and the untouched gaps between them
    assert torch.equal(yd_store.cpu(), storage(want))


def test_rearrange_unaligned_base_and_status(cuda_lib):
    lib, handle = cuda_lib
    src = torch.arange(4 * 64 + 1, dtype=torch.float16, device=DEV)
    dst = torch.zeros(4 * 80 + 1, dtype=torch.float16, device=DEV)
    xs, yd = torch.as_strided(src, (4, 64), (64, 1), 1), torch.as_strided(dst, (4, 64), (80, 1), 1)
    ops.rearrange(lib, handle, yd, xs)
    torch.cuda.synchronize()
    assert torch.equal(yd.cpu(), xs.cpu()) and dst[0].item() == 0 and dst[65:81].abs().sum().item() == 0
    bad = [
        (torch.zeros((4, 8), dtype=torch.float16, device=DEV), torch.zeros((4, 8), dtype=torch.float32, device=DEV), 3),
        (torch.zeros((4, 8), dtype=torch.float16, device=DEV), torch.zeros((4, 9), dtype=torch.float16, device=DEV), 4),
        (torch.zeros((4, 8), dtype=torch.float16, device=DEV), torch.zeros((2, 4, 8), dtype=torch.float16, device=DEV), 4),
        (torch.zeros((4, 8), dtype=torch.float16, device=DEV),
         torch.as_strided(torch.zeros(64, dtype=torch.float16, device=DEV), (4, 8), (16, 2)), 5),
    ]
    for d, s, code in bad:
        with pytest.raises(Exception) as e:
            ops.rearrange(lib, handle, d, s)
        assert str(code) in str(e.value)


# ---- stream capture ------------------------------------------------------------------
def test_entry_points_capture_into_a_cuda_graph(oracle, cuda_lib):
    """bench.py times a CUDA graph of the step: the compute entry points must neither allocate nor
    synchronise.  SwiGLU, Add, RoPE, causal softmax and batched sampling are captured on a side stream
    (after one eager call each, which performs the one-time per-device kernel attribute set-up), the graph is
    replayed on fresh inputs, and the results are those of the oracle."""
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(123)
    a = torch.randn((64, 256), generator=g).half()
    b = torch.randn((64, 256), generator=g).half()
    t = torch.randn((40, 8, 64), generator=g).half()
    pos = torch.arange(40, dtype=torch.int64)
    sin, cos = ops.sin_cos_table(40, 64)
    y = (torch.randn((3, 16, 64), generator=g) * 2).half()
    logits = (torch.randn((4, 5000), generator=g) * 3).half()
    u = torch.rand(4, generator=g)
    ad, bd, td, yd, ld, ud = (x.to(DEV) for x in (a, b, t, y, logits, u))
    posd, sind, cosd = pos.to(DEV), sin.to(DEV), cos.to(DEV)
    cd, sd = torch.zeros_like(ad), torch.zeros_like(ad)
    res = torch.zeros(4, dtype=torch.int64, device=DEV)
    swi, add = ops.SwiGLUOp(lib, handle, sd, ad, bd), ops.AddOp(lib, handle, cd, ad, bd)
    rope, sm = ops.RoPEOp(lib, handle, td, posd, sind, cosd), ops.CausalSoftmaxOp(lib, handle, yd)
    rs = ops.RandomSampleOp(lib, handle, res[:1], ld[0])

    def step(s):
        swi(sd, ad, bd, s)
        add(cd, ad, bd, s)
        rope(td, posd, sind, cosd, s)
        sm(yd, s)
        rs.batch(res, ld, ud, 0.9, 20, 0.8, s)

    step(None)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step(torch.cuda.current_stream().cuda_stream)
    # fresh contents in the captured buffers, then two replays of the in-place operators' inputs
    td.copy_(t.to(DEV))
    yd.copy_(y.to(DEV))
    cd.zero_(), sd.zero_(), res.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(_bits(cd).reshape(64, 256), oracle.add(a.numpy(), b.numpy()).view(np.uint16))
    want_t = oracle.rope(t.numpy().copy(), pos.numpy().astype(np.uint64), sin.numpy(), cos.numpy())
    assert np.array_equal(_bits(td).reshape(40, 8, 64), want_t.view(np.uint16))
    got_s, want_s = sd.cpu().float().numpy(), oracle.swiglu(a.numpy(), b.numpy()).astype(np.float32)
    assert np.allclose(got_s, want_s, atol=1e-3, rtol=1e-3)
    got_y, want_y = yd.cpu().float().numpy(), oracle.causal_softmax(y.numpy().copy()).astype(np.float32)
    assert np.allclose(got_y, want_y, atol=2e-3, rtol=2e-3)
    for r in range(4):
        assert int(res[r]) == oracle.random_sample(logits[r].numpy(), float(u[r]), 0.9, 20, 0.8)
