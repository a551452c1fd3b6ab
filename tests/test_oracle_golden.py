"""The C oracle against golden vectors produced by the reference's own CPU
backend (tests/golden/make_golden.py): bit-identical outputs on every operator.
Runs anywhere: needs neither the reference sources nor a GPU."""
import os

import numpy as np
import pytest

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hot_path_golden.npz"))


@pytest.mark.parametrize("w", ["f16", "f32"])
def test_rms_norm(oracle, w):
    wv = G["rms_w_" + w]
    got = oracle.rms_norm(G["rms_x"], wv.view(np.float16) if w == "f16" else wv, 1e-5)
    assert np.array_equal(got.view(np.uint16), G["rms_y_" + w])


def test_rope(oracle):
    t = G["rope_in"].copy()
    oracle.rope(t, G["rope_pos"], G["rope_sin"], G["rope_cos"])
    assert np.array_equal(t, G["rope_out"])


@pytest.mark.parametrize("tag", ["small", "wide"])
def test_swiglu(oracle, tag):
    got = oracle.swiglu(G["swiglu_a_" + tag], G["swiglu_b_" + tag])
    assert np.array_equal(got.view(np.uint16), G["swiglu_c_" + tag])


def test_add(oracle):
    got = oracle.add(G["add16_a"].view(np.float16), G["add16_b"].view(np.float16))
    assert np.array_equal(got.view(np.uint16), G["add16_c"])
    got = oracle.add(G["add32_a"], G["add32_b"])
    assert np.array_equal(got.view(np.uint32), G["add32_c"].view(np.uint32))


def test_rearrange(oracle):
    for tag in ("a", "b"):
        shape, s_src, s_dst = (tuple(int(v) for v in row) for row in G["rearrange_meta_" + tag])
        src_store = G["rearrange_src_" + tag].copy()
        dst_store = np.zeros_like(G["rearrange_dst_" + tag])
        view = lambda store, strides: np.lib.stride_tricks.as_strided(store, shape, tuple(2 * st for st in strides))
        oracle.rearrange(view(dst_store, s_dst), view(src_store, s_src))
        assert np.array_equal(dst_store, G["rearrange_dst_" + tag]), tag


def test_causal_softmax(oracle):
    y = G["softmax_in"].copy()
    oracle.causal_softmax(y)
    assert np.array_equal(y, G["softmax_out"])
    assert (G["softmax_out"][:, 0, 493:] == 0).all()  # row 0 of [.., 20, 512] sees 493 columns


def test_random_sample(oracle):
    off = 0
    for (voc, u, topp, topk, temp), want in zip(G["rs_params"], G["rs_idx"]):
        voc, topk = int(voc), int(topk)
        row = G["rs_rows"][off:off + voc]
        off += voc
        assert oracle.random_sample(row, float(np.float32(u)), float(np.float32(topp)), topk, float(np.float32(temp))) == want
    assert off == G["rs_rows"].size


@pytest.mark.parametrize("tag", ["decode", "prefill"])
def test_attention(oracle, tag):
    nh, nkvh, seq, dh, pos, buf = (int(x) for x in G["attn_meta_" + tag])
    f16 = lambda name, shape: G["attn_%s_%s" % (name, tag)].copy().view(np.float16).reshape(shape)
    q, k, v = f16("q", (nh, seq, dh)), f16("k", (nkvh, seq, dh)), f16("v", (nkvh, seq, dh))
    kc, vc = f16("kc_in", (nkvh, buf, dh)), f16("vc_in", (nkvh, buf, dh))
    got = oracle.attention(q, k, v, kc, vc, pos)
    assert np.array_equal(got.view(np.uint16).reshape(-1), G["attn_out_" + tag].reshape(-1))
    assert np.array_equal(kc.view(np.uint16).reshape(-1), G["attn_kc_out_" + tag].reshape(-1))
    assert np.array_equal(vc.view(np.uint16).reshape(-1), G["attn_vc_out_" + tag].reshape(-1))
