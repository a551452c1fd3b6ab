"""Run by tests/test_gpu_parity.py::test_vocab_sharded_sampling_over_peer_memory_two_gpus under torchrun, one process
per GPU: vocabulary-sharded exact sampling with the rows exchanged over peer memory (CUDA IPC blocks, flag
protocol of operators_b200/csrc/peer_exchange.cu), several rounds, every rank's indices compared with the unsharded
sampler on the same logits.  Prints "peer ranks ok" on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from operators_b200 import DeviceEnum, create_handle, open_lib, ops  # noqa: E402
from operators_b200.sharding import PeerBlocks, VocabShardedSampler, vocab_range  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("gloo")  # plumbing only: the handles and the closing barrier; the data path is peer memory
    lib = open_lib(os.path.join(ROOT, "operators_b200", "lib"))
    handle = create_handle(lib, DeviceEnum.DEVICE_CUDA, local)
    before = ops.device_timeouts(lib, handle)
    bad = 0
    # equal shards (the exchange inside the sampling kernel, then as launches of its own), uneven rows, uneven shards
    for voc, rows, one_launch in ((128256, 64, True), (128256, 64, False), (32000, 13, True), (4099, 5, True), (4096, 1, True)):
        g = torch.Generator().manual_seed(100 + voc)
        b, e = vocab_range(voc, world, rank)
        pb = PeerBlocks(lib, handle, rows, e - b, world, rank, dev)
        whole = torch.empty((rows, voc), dtype=torch.float16, device=dev)
        want = torch.zeros(rows, dtype=torch.int64, device=dev)
        op = ops.RandomSampleOp(lib, handle, pb.results[:1], pb.logits[0])
        ref = ops.RandomSampleOp(lib, handle, want[:1], whole[0])
        s = VocabShardedSampler(lib, handle, op, voc, b, world, rank=rank, exchange="peer_memory", peer_blocks=pb,
                                one_launch=one_launch)
        for _ in range(3):
            logits = (torch.randn((rows, voc), generator=g) * 3).half()  # the same on every rank
            u = torch.rand(rows, generator=g)
            whole.copy_(logits)
            ud = u.to(dev)
            ref.batch(want, whole, ud, 0.9, 50, 0.8)
            pb.logits[:rows].copy_(whole[:, b:e])
            s.sample(pb.results, pb.logits[:rows], ud, 0.9, 50, 0.8)
            torch.cuda.synchronize()
            bad += int((pb.results[:rows] != want).sum().item())
        dist.barrier()  # nobody frees a block that a peer may still read
        s.destroy()
        op.destroy()
        ref.destroy()
        pb.destroy()
    timeouts = ops.device_timeouts(lib, handle) - before
    total = torch.tensor([bad, timeouts])
    dist.all_reduce(total)
    dist.destroy_process_group()
    if int(total[0]) or int(total[1]):
        print("peer ranks FAILED: %d wrong indices, %d waits that ran out" % (int(total[0]), int(total[1])))
        sys.exit(1)
    if rank == 0:
        print("peer ranks ok")


if __name__ == "__main__":
    main()
