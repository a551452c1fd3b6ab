"""The sampling entry point that allocates nothing.

Collected last on purpose (file name): a run that stops at the first failure
has then already run every other test.

Serving loops that own all device memory through their own arena, or plug-ins
that only get input and output pointers, cannot lend the sampler a workspace.
infiniopRandomSampleBatchStatic keeps the per-row working copies in an array
built into the library instead.  The array is used by the global-memory
sampling kernel (rows of more than 262144 logits, or any row when that kernel
is asked for), so the tests below make that kernel run: each calls the entry
point through the C ABI twice in a row (the array keeps the previous call's
contents, so the second call starts from a dirty array with a stale tail) and
requires exactly the indices of the workspace-based entry point and of the CPU
oracle.
"""
import pytest
import torch

from operators_b200 import InfiniopError, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _two_calls(oracle, lib, handle, voc, calls):
    g = torch.Generator().manual_seed(2024)
    with ops.RandomSampleOp(lib, handle, torch.zeros(1, dtype=torch.int64, device=DEV),
                            torch.zeros(voc, dtype=torch.float16, device=DEV)) as op:
        for rows, dist, (topp, topk, temp) in calls:
            logits = (torch.randn((rows, voc), generator=g) * 3).half() if dist == "normal3" else \
                torch.rand((rows, voc), generator=g).half()
            u = torch.rand(rows, generator=g)
            ld, ud = logits.to(DEV), u.to(DEV)
            want = torch.full((rows,), -1, dtype=torch.int64, device=DEV)
            got = torch.full((rows,), -1, dtype=torch.int64, device=DEV)
            op.batch(want, ld, ud, topp, topk, temp)
            op.batch_static(got, ld, ud, topp, topk, temp)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
            cpu = [oracle.random_sample(logits[r].numpy(), float(u[r]), topp, topk, temp) for r in range(rows)]
            assert got.cpu().tolist() == cpu


def test_static_scratch_long_rows(oracle, cuda_lib):
    """Rows too long for the shared-memory kernel: the working copies live in the built-in array."""
    lib, handle = cuda_lib
    _two_calls(oracle, lib, handle, 300000, [(8, "normal3", (0.9, 50, 0.8)), (5, "uniform", (0.8, 25, 1.0))])


def test_static_scratch_global_kernel_at_the_benchmark_shape(oracle, cuda_lib):
    """64 x 128256 through the kernel that uses the array (asked for explicitly), then fewer rows of other values."""
    lib, handle = cuda_lib
    ops.select_kernel(lib, "random_sample", 1)
    try:
        _two_calls(oracle, lib, handle, 128256, [(64, "normal3", (0.9, 50, 0.8)), (48, "uniform", (0.8, 25, 1.0))])
    finally:
        ops.select_kernel(lib, "random_sample", 0)


def test_static_scratch_size_limit(cuda_lib):
    lib, handle = cuda_lib
    # 60 rows of 300000 logits need ~36 MB of working copies > 32 MiB
    logits = torch.zeros((60, 300000), dtype=torch.float16, device=DEV)
    u = torch.zeros(60, device=DEV)
    out = torch.zeros(60, dtype=torch.int64, device=DEV)
    with ops.RandomSampleOp(lib, handle, out[:1], logits[0]) as op:
        with pytest.raises(InfiniopError) as e:
            op.batch_static(out, logits, u, 0.9, 50, 0.8)
        assert e.value.status == 7  # STATUS_INSUFFICIENT_WORKSPACE
    # rows that are sampled out of shared memory use no scratch: no limit on their number
    logits = torch.zeros((200, 128256), dtype=torch.float16, device=DEV)
    logits[:, 77] = 9.0
    u = torch.zeros(200, device=DEV)
    out = torch.full((200,), -1, dtype=torch.int64, device=DEV)
    with ops.RandomSampleOp(lib, handle, out[:1], logits[0]) as op:
        op.batch_static(out, logits, u, 0.9, 50, 0.8)
        torch.cuda.synchronize()
    assert (out == 77).all()
