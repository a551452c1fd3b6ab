"""Multi-GPU use of the hot path: one process per GPU, `torch.distributed` for
the plumbing.

The reference has no multi-device code; what is here is new and sits on top of
the unchanged single-device C ABI:

* Row-parallel operators (RMSNorm, RoPE, SwiGLU, Add; causal softmax over its
  leading axis) need no communication: `row_range` / `shard_rows` give each rank
  a contiguous slice and the rank builds its descriptors for that slice.
* `VocabShardedSampler` samples from logits whose vocabulary axis is split over
  the ranks (the layout a tensor-parallel LM head leaves them in): a local
  candidate kernel on every rank, ONE all-gather of ~1 KB per row per rank, a
  finishing kernel.  The gathered records are in local memory before any kernel
  reads them; nothing here loads from a peer's memory.
"""

from .ops import _declare, _stream_ptr
from .utils import check_error


def row_range(n_rows, world_size, rank):
    """[begin, end) of the rows rank `rank` owns: contiguous, sizes differ by at most one."""
    base, extra = divmod(n_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_rows(tensor, world_size, rank, dim=0):
    """The rank's slice of `tensor` along `dim` (a view; strides are kept, so the
    same descriptor strides apply with a smaller extent)."""
    begin, end = row_range(tensor.shape[dim], world_size, rank)
    return tensor.narrow(dim, begin, end - begin)


def vocab_range(voc_total, world_size, rank):
    """Columns of the vocabulary rank `rank` holds."""
    return row_range(voc_total, world_size, rank)


class VocabShardedSampler:
    """Sampling branch of random sample (topp > 0, 2 <= topk <= 64) over
    vocabulary shards.  `all_gather(out, inp)` defaults to
    torch.distributed.all_gather_into_tensor on `group`."""

    def __init__(self, lib, handle, sample_op, voc_total, shard_offset, world_size, group=None, all_gather=None):
        _declare(lib)
        self.lib, self.handle, self.op = lib, handle, sample_op
        self.voc_total, self.shard_offset, self.world = int(voc_total), int(shard_offset), int(world_size)
        self.group = group
        self.record_bytes = int(lib.infiniopRandomSampleShardRecordBytes())
        self._gather = all_gather
        self._bufs = {}

    def _buffers(self, rows, device):
        import torch

        key = (rows, str(device))
        if key not in self._bufs:
            words = self.record_bytes // 4
            self._bufs[key] = (torch.zeros((rows, words), dtype=torch.int32, device=device),
                               torch.zeros((self.world, rows, words), dtype=torch.int32, device=device),
                               torch.zeros(1, dtype=torch.int32, device=device))
        return self._bufs[key]

    def sample(self, results, local_logits, random_vals, topp, topk, temperature, stream=None, check=True):
        """local_logits fp16 [rows, voc_local] (this rank's columns), random_vals
        fp32 [rows] and results int64/uint64 [rows] on the device; every rank gets
        the same results."""
        rows = local_logits.shape[0]
        local, gathered, status = self._buffers(rows, local_logits.device)
        sp = _stream_ptr(stream)
        check_error(self.lib.infiniopRandomSampleShardLocal(
            self.op.desc, local.data_ptr(), local_logits.data_ptr(), local_logits.stride(0), rows, self.shard_offset,
            topk, temperature, sp))
        if self._gather is not None:
            self._gather(gathered, local)
        elif self.world > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(gathered.view(-1), local.view(-1), group=self.group)
        else:
            gathered[0].copy_(local)
        status.zero_()
        check_error(self.lib.infiniopRandomSampleShardFinish(
            self.handle, results.data_ptr(), gathered.data_ptr(), self.world, rows, self.voc_total,
            random_vals.data_ptr(), topp, topk, temperature, status.data_ptr(), sp))
        if check and int(status.item()) != 0:
            raise RuntimeError("vocabulary-sharded sampling: a shard held more than 128 tied candidates in some row; "
                               "gather the logits and use the unsharded entry point for this batch")
        return results
