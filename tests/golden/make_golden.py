"""Generate tests/golden/hot_path_golden.npz from the REFERENCE's own CPU backend.

Run in a checkout that has the reference sources (they are compiled into
oracle/_ref by `make -C oracle ref`); the reference library is then driven
through its C ABI exactly like its test scripts drive it
(reference operatorspy/tests/*.py), on small seeded inputs.  The stored outputs
are what tests/test_oracle_golden.py holds the C oracle to on machines that
have neither the reference sources nor oracle/_ref.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from operators_b200 import DeviceEnum, create_handle, open_lib, ops, rearrange_tensor  # noqa: E402
from oracle import cpu_oracle  # noqa: E402


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    d = cpu_oracle.build_reference()
    assert d, "reference sources not available: cannot regenerate golden vectors"
    lib = open_lib(os.path.dirname(d))
    h = create_handle(lib, DeviceEnum.DEVICE_CPU)
    g = torch.Generator().manual_seed(20241125)
    out = {}

    # RMSNorm (reference test shape (16, 2048), fp16 and fp32 weight)
    x = (torch.rand((16, 2048), generator=g) * 2 - 1).half()
    for name, w in (("f16", (torch.rand(2048, generator=g) * 2 - 1).half()), ("f32", torch.rand(2048, generator=g) * 2 - 1)):
        y = torch.zeros_like(x)
        ops.rms_norm(lib, h, y, x, w, 1e-5)
        out["rms_x"] = bits(x)
        out["rms_w_" + name] = bits(w) if w.dtype == torch.float16 else w.numpy().copy()
        out["rms_y_" + name] = bits(y)

    # RoPE (7 tokens, 4 heads, dh 32; shuffled positions; theta 1e4)
    t = torch.randn((7, 4, 32), generator=g).half()
    pos = torch.randperm(14, generator=g)[:7].to(torch.int64)
    sin, cos = ops.sin_cos_table(14, 32)
    out["rope_in"], out["rope_pos"] = bits(t), pos.numpy().astype(np.uint64)
    out["rope_sin"], out["rope_cos"] = sin.numpy().copy(), cos.numpy().copy()
    ops.rope(lib, h, t, pos, sin, cos)
    out["rope_out"] = bits(t)

    # SwiGLU (reference shape (13, 4) and 4 rows of its (16, 5632)); b spans the exp range
    for tag, shape in (("small", (13, 4)), ("wide", (4, 5632))):
        a = torch.randn(shape, generator=g).half()
        b = (torch.randn(shape, generator=g) * 6).half()
        c = torch.zeros(shape, dtype=torch.float16)
        ops.swiglu(lib, h, c, a, b)
        out["swiglu_a_" + tag], out["swiglu_b_" + tag], out["swiglu_c_" + tag] = bits(a), bits(b), bits(c)

    # Add with broadcasting, fp16 and fp32
    a = (torch.randn((2, 20, 3), generator=g) * 100).half()
    b = torch.randn((2, 1, 3), generator=g).half()
    c = torch.zeros((2, 20, 3), dtype=torch.float16)
    ops.add(lib, h, c, a, b)
    out["add16_a"], out["add16_b"], out["add16_c"] = bits(a), bits(b), bits(c)
    a32, b32 = torch.randn((4, 5, 6), generator=g), torch.randn((6,), generator=g)
    c32 = torch.zeros((4, 5, 6))
    ops.add(lib, h, c32, a32, b32)
    out["add32_a"], out["add32_b"], out["add32_c"] = a32.numpy().copy(), b32.numpy().copy(), c32.numpy().copy()

    # causal softmax (reference shape (32, 20, 512) cut to 2 heads)
    y = (torch.randn((2, 20, 512), generator=g) * 2).half()
    out["softmax_in"] = bits(y)
    ops.causal_softmax(lib, h, y)
    out["softmax_out"] = bits(y)

    # random sample: the reference's own parameter sets on uniform and normal rows
    cases = [(512, 0.92, 0.8, 3, 0.5), (4096, 0.95, 0.9, 5, 1.0), (16384, 0.85, 0.85, 10, 2.0), (512, 0.92, 0.0, 3, 0.5),
             (4096, 0.95, 0.9, 1, 1.0), (16384, 0.85, 0.0, 1, 2.0), (32000, 0.8, 0.8, 50, 1.0), (32000, 0.8, 1.0, 25, 1.0)]
    rs_params, rs_rows, rs_idx = [], [], []
    for voc, u, topp, topk, temp in cases:
        for dist in (("uniform", "normal3") if voc <= 4096 else ("uniform",)):
            row = torch.rand(voc, generator=g).half() if dist == "uniform" else (torch.randn(voc, generator=g) * 3).half()
            res = torch.zeros(1, dtype=torch.int64)
            ops.random_sample(lib, h, res, row, u, topp, topk, temp)
            rs_params.append((voc, u, topp, topk, temp))
            rs_rows.append(bits(row))
            rs_idx.append(int(res[0]))
    out["rs_params"] = np.array(rs_params, np.float64)
    out["rs_rows"] = np.concatenate(rs_rows)
    out["rs_idx"] = np.array(rs_idx, np.int64)

    # rearrange (two of the reference's own cases, reference operatorspy/tests/rearrange.py:111-112): the
    # source view's whole storage, and the destination storage the reference leaves (gaps stay zero)
    from operators_b200 import rearrange_tensor

    for tag, shape, s_src, s_dst in (("a", (2, 4, 32), None, (256, 64, 1)), ("b", (32, 6, 64), (64, 2560, 1), None)):
        x = torch.rand(shape, generator=g).half()
        y = torch.zeros(shape, dtype=torch.float16)
        if s_src is not None:
            x = rearrange_tensor(x, s_src)
        if s_dst is not None:
            y = rearrange_tensor(y, s_dst)
        ops.rearrange(lib, h, y, x)
        storage = lambda t: torch.as_strided(t, (sum(st * (sz - 1) for st, sz in zip(t.stride(), t.shape)) + 1,), (1,))
        out["rearrange_src_" + tag], out["rearrange_dst_" + tag] = bits(storage(x)), bits(storage(y))
        out["rearrange_meta_" + tag] = np.array([shape, x.stride(), y.stride()], np.int64)

    # attention composite (reference operatorspy/tests/attention.py): one decoding token over a prefix in the
    # cache, and a short prefill; contiguous tensors.  Inputs, the output and both caches after the call.
    for tag, nh, nkvh, seq, dh, pos, buf in (("decode", 8, 2, 1, 32, 37, 64), ("prefill", 6, 3, 4, 16, 0, 8)):
        q = torch.randn((nh, seq, dh), generator=g).half()
        k = torch.randn((nkvh, seq, dh), generator=g).half()
        v = torch.randn((nkvh, seq, dh), generator=g).half()
        kc = torch.randn((nkvh, buf, dh), generator=g).half()
        vc = torch.randn((nkvh, buf, dh), generator=g).half()
        for name, t in (("q", q), ("k", k), ("v", v), ("kc_in", kc), ("vc_in", vc)):
            out["attn_%s_%s" % (name, tag)] = bits(t)
        res = torch.zeros((seq, nh, dh), dtype=torch.float16)
        ops.attention(lib, h, res, q, k, v, kc, vc, pos)
        out["attn_out_" + tag], out["attn_kc_out_" + tag], out["attn_vc_out_" + tag] = bits(res), bits(kc), bits(vc)
        out["attn_meta_" + tag] = np.array([nh, nkvh, seq, dh, pos, buf], np.int64)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hot_path_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
