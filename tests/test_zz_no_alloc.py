"""The sampling entry point that allocates nothing.

Collected last on purpose (file name): a run that stops at the first failure
has then already run every other test.

Serving loops that own all device memory through their own arena, or plug-ins
that only get input and output pointers, cannot lend the sampler a workspace.
infiniopRandomSampleBatchStatic keeps the per-row working copies in an array
built into the library instead.  Here it is called through the C ABI twice in a
row (the array keeps the previous call's contents, so the second call starts
from a dirty array) and must return exactly the indices of the workspace-based
entry point, which the parity tests pin to the CPU oracle.
"""
import pytest
import torch

from operators_b200 import InfiniopError, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_static_scratch_sampling_matches_workspace_sampling(cuda_lib):
    lib, handle = cuda_lib
    g = torch.Generator().manual_seed(2024)
    first = (torch.randn((64, 128256), generator=g) * 3).half().to(DEV)
    second = torch.rand((48, 128256), generator=g).half().to(DEV)  # other values, fewer rows: stale tail in the array
    u1, u2 = torch.rand(64, generator=g).to(DEV), torch.rand(48, generator=g).to(DEV)
    with ops.RandomSampleOp(lib, handle, torch.zeros(1, dtype=torch.int64, device=DEV), first[0]) as op:
        for logits, u, (topp, topk, temp) in ((first, u1, (0.9, 50, 0.8)), (second, u2, (0.8, 25, 1.0))):
            rows = logits.shape[0]
            want = torch.full((rows,), -1, dtype=torch.int64, device=DEV)
            got = torch.full((rows,), -1, dtype=torch.int64, device=DEV)
            op.batch(want, logits, u, topp, topk, temp)
            op.batch_static(got, logits, u, topp, topk, temp)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
            assert int(got.min()) >= 0 and int(got.max()) < 128256


def test_static_scratch_rejects_oversized_requests(cuda_lib):
    lib, handle = cuda_lib
    logits = torch.zeros((200, 128256), dtype=torch.float16, device=DEV)  # 200 rows need ~51 MB > 32 MiB
    u = torch.zeros(200, device=DEV)
    out = torch.zeros(200, dtype=torch.int64, device=DEV)
    with ops.RandomSampleOp(lib, handle, out[:1], logits[0]) as op:
        with pytest.raises(InfiniopError) as e:
            op.batch_static(out, logits, u, 0.9, 50, 0.8)
        assert e.value.status == 7  # STATUS_INSUFFICIENT_WORKSPACE
