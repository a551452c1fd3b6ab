"""The C-ABI library loads without a GPU and exports every symbol the headers
declare; struct layouts match what the reference's ctypes wrapper assumes
(reference operatorspy/liboperators.py:14-36, operatorspy/data_layout.py:5-26)."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


@pytest.fixture(scope="module")
def lib():
    from operators_b200 import build, open_lib

    build.build()
    return open_lib(os.path.join(ROOT, "operators_b200", "lib"))


def _declared():
    names = set()
    for h in ("infiniop.h", "infiniop_ext.h"):
        names |= set(re.findall(r"\b(infiniop[A-Z]\w+)\s*\(", open(os.path.join(INC, h)).read()))
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    declared = _declared()
    assert len(declared) >= 36
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, missing


def test_reference_symbol_set(lib):
    """The symbols the reference exports for these operators (reference include/ops/*/*.h,
    include/handle/handle_export.h, include/tensor/tensor_descriptor.h)."""
    ref = ["infiniopCreateHandle", "infiniopDestroyHandle", "infiniopCreateTensorDescriptor",
           "infiniopDestroyTensorDescriptor"]
    for op, ws in (("RMSNorm", True), ("RoPE", True), ("SwiGLU", False), ("Add", False), ("CausalSoftmax", True),
                   ("RandomSample", True), ("Rearrange", False), ("Attention", True)):
        ref += ["infiniopCreate%sDescriptor" % op, "infiniop%s" % op, "infiniopDestroy%sDescriptor" % op]
        if ws:
            ref.append("infiniopGet%sWorkspaceSize" % op)
    assert not [n for n in ref if not hasattr(lib, n)]


def test_layouts_match_the_reference_wrapper():
    from operators_b200 import BF16, F16, F32, U64, DataLayout
    from operators_b200.liboperators import Handle, TensorDescriptor

    assert ctypes.sizeof(DataLayout) == 4
    assert (F16.bits(), BF16.bits(), F32.bits(), U64.bits()) == (0x050A0501, 0x08070501, 0x08170901, 0x00401001)
    assert ctypes.sizeof(TensorDescriptor) == 32 and TensorDescriptor.ndim.offset == 8
    assert TensorDescriptor.shape.offset == 16 and TensorDescriptor.pattern.offset == 24
    assert ctypes.sizeof(Handle) == 4


def test_headers_compile_as_c_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "infini_operators.h"\n#include "ops/rms_norm/rms_norm.h"\n#include "infiniop_ext.h"\n'
                   "int main(void){ return (sizeof(DataLayout)==4 && sizeof(struct TensorDescriptor)==32 && "
                   "STATUS_BAD_DEVICE==8 && DevNvGpu==1) ? 0 : 1; }\n")
    for cc, extra in (("gcc", []), ("g++", ["-x", "c++"])):
        exe = tmp_path / ("t_" + cc)
        subprocess.run([cc, "-I", INC] + extra + [str(src), "-o", str(exe)], check=True)
        assert subprocess.run([str(exe)]).returncode == 0


def test_tensor_descriptor_without_gpu(lib):
    """Descriptor creation is host-only: default strides are row-major, ndim 0 is legal
    (reference src/tensor/tensor_descriptor.cc:4-19)."""
    from operators_b200 import F16, create_tensor_descriptor, destroy_tensor_descriptor

    d = create_tensor_descriptor(lib, (3, 4, 5), None, F16)
    assert [d.contents.pattern[i] for i in range(3)] == [20, 5, 1]
    assert [d.contents.shape[i] for i in range(3)] == [3, 4, 5] and d.contents.ndim == 3
    destroy_tensor_descriptor(lib, d)
    d0 = create_tensor_descriptor(lib, (), None, F16)
    assert d0.contents.ndim == 0
    destroy_tensor_descriptor(lib, d0)


def test_handle_errors_without_compute(lib):
    """NULL out-pointer, negative id and non-GPU devices are refused with the
    reference's codes (reference src/devices/handle.cc:17-22,45); no kernel runs."""
    from operators_b200.liboperators import infiniopHandle_t

    h = infiniopHandle_t()
    assert lib.infiniopCreateHandle(None, 1, 0) == 6
    assert lib.infiniopCreateHandle(ctypes.byref(h), 1, -1) == 2
    assert lib.infiniopCreateHandle(ctypes.byref(h), 0, 0) == 8  # DevCpu: this library has no CPU path
    assert lib.infiniopCreateHandle(ctypes.byref(h), 2, 0) == 8


def test_fastdiv_exact(tmp_path):
    """The multiply-high divider used for flat-index -> (row, column) is exact for every 32-bit numerator."""
    src = tmp_path / "fd.cc"
    src.write_text(r'''
#include "fastdiv.h"
#include <cstdio>
#include <cstdint>
int main() {
    const uint32_t ds[] = {1, 2, 3, 5, 7, 8, 13, 255, 256, 641, 1792, 4096, 14336, 65535, 65536, 1000003, 0x7fffffffu, 0x80000000u, 0xfffffffeu, 0xffffffffu};
    uint64_t lcg = 12345;
    for (uint32_t d : ds) {
        b200::FastDiv f(d);
        for (int i = 0; i < 400000; ++i) {
            lcg = lcg * 6364136223846793005ull + 1442695040888963407ull;
            uint32_t n = (i < 8) ? (0xffffffffu - i) : (uint32_t)(lcg >> 32);
            if (i >= 8 && i < 5000) n = (uint32_t)(((uint64_t)(i / 3)) * d + (i % 3) - 1);   // around multiples of d
            uint32_t q, r; f.divmod(n, q, r);
            if (q != n / d || r != n % d) { printf("FAIL d=%u n=%u q=%u r=%u\n", d, n, q, r); return 1; }
        }
    }
    return 0;
}
''')
    exe = tmp_path / "fd"
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "operators_b200", "csrc"), str(src), "-o", str(exe)],
                   check=True)
    assert subprocess.run([str(exe)]).returncode == 0
