import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (C restatement of the reference CPU backend)."""
    from oracle import cpu_oracle

    cpu_oracle.lib()
    return cpu_oracle


@pytest.fixture(scope="session")
def ref_cpu():
    """(lib, handle) of the reference's own CPU backend compiled from its
    sources, driven through the same ctypes wrapper as the CUDA library.
    Built on demand where the reference checkout exists; skipped otherwise."""
    from oracle import cpu_oracle
    from operators_b200 import DeviceEnum, create_handle, open_lib

    if cpu_oracle.reference_lib_dir() is None:
        cpu_oracle.build_reference()
    d = cpu_oracle.reference_lib_dir()
    if d is None:
        pytest.skip("reference CPU backend not built (no reference checkout on this machine)")
    lib = open_lib(d)
    return lib, create_handle(lib, DeviceEnum.DEVICE_CPU)


@pytest.fixture(scope="session")
def cuda_lib():
    """(lib, handle) of the sm_100a library on cuda:0.  Fails (does not skip)
    when the library is missing: there is no other implementation to test."""
    import torch

    from operators_b200 import DeviceEnum, create_handle, open_lib

    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    lib = open_lib(os.path.join(ROOT, "operators_b200", "lib"))
    return lib, create_handle(lib, DeviceEnum.DEVICE_CUDA, 0)
