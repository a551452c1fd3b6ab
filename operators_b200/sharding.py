"""Multi-GPU use of the hot path: one process per GPU, `torch.distributed` for
the plumbing.

The reference has no multi-device code; what is here is new and sits on top of
the unchanged single-device C ABI:

* Row-parallel operators (RMSNorm, RoPE, SwiGLU, Add; causal softmax over its
  leading axis) need no communication: `row_range` / `shard_rows` give each rank
  a contiguous slice and the rank builds its descriptors for that slice.
* `VocabShardedSampler` samples from logits whose vocabulary axis is split over
  the ranks (the layout a tensor-parallel LM head leaves them in).  Its default
  mode is index-exact: one all-to-all hands every rank whole rows, the exact
  batched kernel samples them, one all-gather returns the indices.  Its fast mode
  exchanges ~1 KB of candidates per row per rank in ONE all-gather.  With the
  collectives, received data is in local memory before any kernel reads it.
* `PeerBlocks` + `exchange="peer_memory"`: the exact mode without a collective
  library.  Every rank's shard, results and flags live in one block that the
  other ranks opened through CUDA IPC; two small kernels of this library pull a
  rank's rows from the peers' shards and push its indices to every peer, with
  plain loads and stores over NVLink and bounded flag waits.
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


def exchange_plan(rows, voc_total, world_size, rank):
    """Who sends what when every rank holds all rows of its vocabulary shard and rank r is to own whole rows
    row_range(rows, world_size, r): (my row range, element counts this rank sends to each peer, element counts
    it receives from each peer, the shards' column ranges)."""
    cols = [vocab_range(voc_total, world_size, r) for r in range(world_size)]
    my_cols = cols[rank][1] - cols[rank][0]
    owned = [row_range(rows, world_size, r) for r in range(world_size)]
    mine = owned[rank][1] - owned[rank][0]
    send = [(e - b) * my_cols for b, e in owned]
    recv = [mine * (e - b) for b, e in cols]
    return owned[rank], send, recv, cols


def assemble_rows(received, n_rows, cols, out=None):
    """The flat buffer an all-to-all delivers (peer after peer: [n_rows, that peer's columns]) re-laid as
    [n_rows, voc_total]."""
    import torch

    voc_total = cols[-1][1]
    if out is None:
        out = torch.empty((n_rows, voc_total), dtype=received.dtype, device=received.device)
    off = 0
    for b, e in cols:
        n = n_rows * (e - b)
        out[:, b:e].copy_(received[off:off + n].view(n_rows, e - b))
        off += n
    return out


class _DeviceArray:
    """A raw device pointer as something torch.as_tensor accepts."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 3, "strides": None}


class PeerBlocks:
    """One block of device memory per rank that every other rank of the node can address: 256 bytes of flags (the
    library's), `max_rows` int64 results, and this rank's fp16 logits shard [max_rows, shard_cols].

    Collective: every rank of `group` constructs it at the same point (the IPC handles travel through
    all_gather_object).  `local_blocks` replaces the exchange in tests that play several ranks in one process: a
    list that every played rank appends its own block to before any of them samples."""

    FLAG_BYTES = 256

    def __init__(self, lib, handle, max_rows, shard_cols, world_size, rank, device, group=None, local_blocks=None):
        import ctypes

        import torch

        _declare(lib)
        self.lib, self.handle, self.world, self.rank = lib, handle, int(world_size), int(rank)
        self.max_rows, self.shard_cols = int(max_rows), int(shard_cols)
        self.results_off = self.FLAG_BYTES
        self.logits_off = self.results_off + (self.max_rows * 8 + 255) // 256 * 256
        self.nbytes = self.logits_off + self.max_rows * self.shard_cols * 2
        ptr, ipc = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        with torch.cuda.device(device):
            status = lib.infiniopExtPeerAlloc(handle, self.nbytes, ctypes.byref(ptr), ipc)
        self.ptr, self._opened, self.device = (int(ptr.value) if status == 0 else None), [], device
        if local_blocks is not None:
            check_error(status)
            local_blocks.append(self)
            self._local_blocks, self.bases = local_blocks, None
        else:
            # Every rank takes part in both exchanges whatever happened to it, and all ranks come to the same decision:
            # either every block is allocated and opened everywhere, or every rank frees what it has and raises.
            self._local_blocks = None
            handles = [bytes(ipc) if status == 0 else None]
            if self.world > 1:
                import torch.distributed as dist

                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(ipc) if status == 0 else None, group=group)
            self.bases, opened_all = [], all(h is not None for h in handles)
            for r in range(self.world if opened_all else 0):
                if r == self.rank:
                    self.bases.append(self.ptr)
                    continue
                other = ctypes.c_void_p()
                raw = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                with torch.cuda.device(device):
                    if lib.infiniopExtPeerOpen(handle, raw, ctypes.byref(other)) != 0:
                        opened_all = False
                        break
                self._opened.append(int(other.value))
                self.bases.append(int(other.value))
            decisions = [opened_all]
            if self.world > 1:
                decisions = [None] * self.world
                dist.all_gather_object(decisions, opened_all, group=group)
            if not all(decisions):
                self.results = self.logits = self.flags = None
                self.destroy()
                raise RuntimeError("peer memory blocks could not be allocated and opened on every rank")
        self.results = torch.as_tensor(_DeviceArray(self.ptr + self.results_off, (self.max_rows,), "<i8"), device=device)
        self.logits = torch.as_tensor(_DeviceArray(self.ptr + self.logits_off, (self.max_rows, self.shard_cols), "<f2"),
                                      device=device)
        self.flags = torch.as_tensor(_DeviceArray(self.ptr, (self.FLAG_BYTES // 4,), "<i4"), device=device)

    def base_of(self, r):
        if self._local_blocks is not None:
            return self._local_blocks[r].ptr
        return self.bases[r]

    def destroy(self):
        import torch

        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for other in self._opened:
                self.lib.infiniopExtPeerClose(self.handle, other)
            if self.ptr is not None:
                self.lib.infiniopExtPeerFree(self.handle, self.ptr)
        self.ptr, self._opened, self.results, self.logits, self.flags = None, [], None, None, None


class VocabShardedSampler:
    """Sampling branch of random sample (topp > 0, 2 <= topk <= 64) over vocabulary shards; every rank gets
    the same results.

    mode "exact" (default): the sampled index is the unsharded entry point's, i.e. the reference CPU path's,
    for every row.  The reference's softmax denominator is a sequential fp32 sum over the whole row, which no
    per-shard partial can reproduce, so the rows are redistributed instead: rank r gets the whole rows
    row_range(rows, world, r), the exact batched kernel samples them, the indices go back to every rank.  How the rows
    travel (`exchange`): "auto" shares one block per rank over CUDA IPC at the first call and lets the sampling
    kernel itself read the peers' shards and store the indices to every rank (PeerBlocks; one launch, no
    collective); where the blocks cannot be shared on every rank it uses "all_gather" (from four ranks with equal
    shards) or "all_to_all", one NCCL collective in and one all-gather of 8 bytes per row out.  The set-up allocates
    and exchanges handles, so the first call (and the first with more rows than any before) belongs outside stream
    capture; later calls launch kernels only.

    mode "fast": a local candidate kernel on every rank, ONE all-gather of ~1 KB per row per rank, a finishing
    kernel.  Top-k set, tie order and numerators are the reference's; the denominator is the correctly rounded
    sum instead of the sequential one, so a small fraction of rows picks a neighbouring candidate.

    `stream`, when given, must be a torch.cuda.Stream: the collectives and the library's kernels are all issued
    on it.  `all_gather(out, inp)` / `all_to_all(out, inp, out_splits, in_splits)` replace the
    torch.distributed calls on `group` (tests play several ranks in one process with them)."""

    def __init__(self, lib, handle, sample_op, voc_total, shard_offset, world_size, group=None, all_gather=None,
                 mode="exact", rank=None, all_to_all=None, exchange="auto", peer_blocks=None, one_launch=True):
        _declare(lib)
        assert mode in ("exact", "fast") and exchange in ("auto", "all_to_all", "all_gather", "peer_memory")
        # "peer_memory": no collective at all.  `peer_blocks` (PeerBlocks, built collectively beforehand) holds every
        # rank's shard where the others can read it; the caller writes its logits into peer_blocks.logits[:rows]
        # (sample() copies them there when it is handed another tensor) and two kernels of the library move rows
        # in and indices out.  All ranks then read their results from peer_blocks.results as well.
        assert (exchange == "peer_memory") == (peer_blocks is not None)
        self.peer = peer_blocks
        # peer memory: fold the exchange into the sampling kernel where its conditions hold (equal shards of a multiple
        # of 8 columns, rows of at most 262144 logits); False keeps the three launches (gather, sample, publish)
        self.one_launch = one_launch
        # How the exact mode moves the rows: "all_to_all" sends every rank only the rows it will own;
        # "all_gather" hands every rank all shards (world_size times the bytes, but one collective whose latency
        # does not grow with the number of peers the way the send / receive pairs of an all-to-all do) and lets it
        # pick its rows.  It needs equal shards; "auto" takes it from four ranks up.
        equal = int(voc_total) % int(world_size) == 0
        # "auto" with real ranks: peer memory, set up at the first call (collective; the blocks are sized for that
        # call's rows and made anew when a later call has more); when the blocks cannot be shared on every rank, the
        # collective exchanges below.  destroy() is then collective as well (nobody frees a block a peer may read).
        self._auto_peer = (exchange == "auto" and mode == "exact" and int(world_size) > 1 and all_to_all is None
                           and all_gather is None)
        self._own_peer = False
        if exchange == "auto":
            exchange = "all_gather" if (int(world_size) >= 4 and equal and all_to_all is None) else "all_to_all"
        if exchange == "all_gather" and not equal:
            exchange = "all_to_all"
        self.exchange = exchange
        self.lib, self.handle, self.op = lib, handle, sample_op
        self.voc_total, self.shard_offset, self.world = int(voc_total), int(shard_offset), int(world_size)
        self.group, self.mode = group, mode
        self.record_bytes = int(lib.infiniopRandomSampleShardRecordBytes())
        self._gather, self._a2a = all_gather, all_to_all
        if rank is None:
            rank = 0
            if self.world > 1 and all_to_all is None:
                import torch.distributed as dist

                rank = dist.get_rank(group)
        self.rank = int(rank)
        self._bufs = {}
        self._exact = {}
        self.last_events = None

    def destroy(self):
        for entry in self._exact.values():
            entry[3].destroy()
            if entry[4] is not None:
                entry[4].destroy()
        self._exact = {}
        self._drop_own_peer()

    def _drop_own_peer(self):
        if self._own_peer and self.peer is not None:
            import torch
            import torch.distributed as dist

            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            self.peer.destroy()
            self.peer, self._own_peer = None, False
            self._bufs = {k: v for k, v in self._bufs.items() if not (isinstance(k, tuple) and k[0] == "tables")}

    def _auto_peer_setup(self, rows, device):
        """First exact call of an "auto" sampler with real ranks (and any later call with more rows): try to share
        blocks over CUDA IPC; every rank comes to the same decision (PeerBlocks), so either all switch to peer memory
        or all keep the collective exchange."""
        if self.peer is not None and self._own_peer and rows > self.peer.max_rows:
            self._drop_own_peer()
            for entry in self._exact.values():  # buffers sized for the other exchange
                entry[3].destroy()
                if entry[4] is not None:
                    entry[4].destroy()
            self._exact = {}
        if self.peer is None:
            b, e = vocab_range(self.voc_total, self.world, self.rank)
            try:
                self.peer = PeerBlocks(self.lib, self.handle, rows, e - b, self.world, self.rank, device, group=self.group)
                self._own_peer, self._fallback_exchange, self.exchange = True, self.exchange, "peer_memory"
            except RuntimeError:
                self._auto_peer = False

    def _buffers(self, rows, device):
        import torch

        key = (rows, str(device))
        if key not in self._bufs:
            words = self.record_bytes // 4
            self._bufs[key] = (torch.zeros((rows, words), dtype=torch.int32, device=device),
                               torch.zeros((self.world, rows, words), dtype=torch.int32, device=device),
                               torch.zeros(1, dtype=torch.int32, device=device))
        return self._bufs[key]

    def _exact_buffers(self, rows, device):
        import torch

        from .ops import RandomSampleOp

        key = (rows, str(device))
        if key not in self._exact:
            (r0, r1), _, recv, _ = exchange_plan(rows, self.voc_total, self.world, self.rank)
            most = max(e - b for b, e in (row_range(rows, self.world, r) for r in range(self.world)))
            n_recv = rows * self.voc_total if self.exchange == "all_gather" else sum(recv)
            if self.exchange == "peer_memory":
                n_recv = 1
            received = torch.empty(max(1, n_recv), dtype=torch.float16, device=device)
            full = torch.empty((max(1, r1 - r0), self.voc_total), dtype=torch.float16, device=device)
            picked = torch.zeros((self.world, most), dtype=torch.int64, device=device)
            op = RandomSampleOp(self.lib, self.handle, picked[0, :1], full[0])
            op._ensure_batch_ws(max(1, r1 - r0), device)
            op_copy = full_view = received_view = None
            mine = r1 - r0
            if mine and self.voc_total % self.world == 0 and received.is_cuda and self.exchange != "peer_memory":
                from .ops import RearrangeOp

                vl = self.voc_total // self.world
                full_view = full[:mine].view(mine, self.world, vl).permute(1, 0, 2)  # [shard, row, cols] view of the rows
                if self.exchange == "all_gather":  # every shard arrives whole: [shard][all rows][cols]; this rank's rows of each
                    received_view = received[:self.world * rows * vl].view(self.world, rows, vl)[:, r0:r1, :]
                else:
                    received_view = received[:self.world * mine * vl].view(self.world, mine, vl)
                op_copy = RearrangeOp(self.lib, self.handle, full_view, received_view)
            self._exact[key] = (received, full, picked, op, op_copy, full_view, received_view)
        return self._exact[key]

    def sample(self, results, local_logits, random_vals, topp, topk, temperature, stream=None, check=True,
               timed=False):
        """local_logits fp16 [rows, voc_local] (this rank's columns), random_vals fp32 [rows] and results
        int64/uint64 [rows] on the device.  timed=True records CUDA events between the stages in
        self.last_events (names and events, in issue order)."""
        import contextlib

        import torch

        ctx = torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()
        events = []

        def mark(name):
            if timed:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append((name, ev))

        with ctx:
            sp = _stream_ptr(torch.cuda.current_stream(local_logits.device)) if local_logits.is_cuda else None
            mark("start")
            if self.mode == "exact":
                self._sample_exact(results, local_logits, random_vals, topp, topk, temperature, sp, mark)
            else:
                self._sample_fast(results, local_logits, random_vals, topp, topk, temperature, sp, check, mark)
        self.last_events = events
        return results

    def _sample_exact(self, results, local_logits, random_vals, topp, topk, temperature, sp, mark):
        import torch

        rows = local_logits.shape[0]
        if self._auto_peer and local_logits.is_cuda and (self.peer is None or rows > self.peer.max_rows):
            self._auto_peer_setup(rows, local_logits.device)
        (r0, r1), send, recv, cols = exchange_plan(rows, self.voc_total, self.world, self.rank)
        mine = r1 - r0
        received, full, picked, op, op_copy, full_view, received_view = self._exact_buffers(rows, local_logits.device)
        if self.exchange == "peer_memory":
            self._sample_peer(results, local_logits, random_vals, topp, topk, temperature, sp, mark, rows, r0, r1,
                              cols, full, picked, op)
            return
        src = local_logits if local_logits.is_contiguous() else local_logits.contiguous()
        if self._a2a is not None:
            self._a2a(received, src.view(-1), recv, send)
        elif self.world > 1:
            import torch.distributed as dist

            if self.exchange == "all_gather":
                dist.all_gather_into_tensor(received[:self.world * src.numel()], src.view(-1), group=self.group)
            else:
                dist.all_to_all_single(received[:sum(recv)], src.view(-1), recv, send, group=self.group)
        else:
            received[:src.numel()].copy_(src.view(-1))
        mark("exchange")
        if mine:
            if op_copy is not None:  # equal shards: [shard][row][cols] -> [row][shard][cols] in one strided copy
                op_copy(full_view, received_view, stream=sp)
            else:
                assemble_rows(received, mine, cols, out=full)
            mark("assemble")
            op.batch(picked[self.rank, :mine], full[:mine], random_vals[r0:r1], topp, topk, temperature, stream=sp)
        mark("sample")
        even = rows % self.world == 0
        if self._gather is not None:
            self._gather(picked, picked[self.rank])
        elif self.world > 1:
            import torch.distributed as dist

            if even and results.is_contiguous():  # equal row counts: the indices are gathered straight into `results`
                dist.all_gather_into_tensor(results.view(torch.int64), picked[self.rank, :mine], group=self.group)
                mark("all_gather")
                mark("finish")
                return
            dist.all_gather_into_tensor(picked.view(-1), picked[self.rank], group=self.group)
        mark("all_gather")
        if even:
            results.view(torch.int64).copy_(picked.view(-1))
        else:
            for r in range(self.world):
                b, e = row_range(rows, self.world, r)
                results.view(torch.int64)[b:e].copy_(picked[r, :e - b])
        mark("finish")

    def _peer_tables(self, rows, cols):
        import ctypes

        key = ("tables", rows)
        if key not in self._bufs:
            pb, w = self.peer, self.world
            assert rows <= pb.max_rows and pb.shard_cols == cols[self.rank][1] - cols[self.rank][0]
            widths = [e - b for b, e in cols]
            shards = (ctypes.c_void_p * w)(*[pb.base_of(r) + pb.logits_off for r in range(w)])
            strides = (ctypes.c_int64 * w)(*widths)  # every rank's shard is [max_rows, its columns], dense
            col0 = (ctypes.c_uint64 * w)(*[b for b, _ in cols])
            ncols = (ctypes.c_uint64 * w)(*widths)
            flags = (ctypes.c_void_p * w)(*[pb.base_of(r) for r in range(w)])
            res = (ctypes.c_void_p * w)(*[pb.base_of(r) + pb.results_off for r in range(w)])
            self._bufs[key] = (shards, strides, col0, ncols, flags, res)
        return self._bufs[key]

    def _sample_peer(self, results, local_logits, random_vals, topp, topk, temperature, sp, mark, rows, r0, r1, cols,
                     full, picked, op):
        import torch

        pb, mine = self.peer, r1 - r0
        shards, strides, col0, ncols, flags, res = self._peer_tables(rows, cols)
        if local_logits.data_ptr() != pb.logits.data_ptr():
            pb.logits[:rows].copy_(local_logits)
        vl = pb.shard_cols
        one_launch = (self.one_launch and mine > 0 and vl * self.world == self.voc_total and vl % 8 == 0
                      and self.voc_total <= 262144 and topp > 0 and 2 <= topk <= 64)
        if one_launch:
            # the exchange inside the sampling kernel: peers' shards read by its own loads, indices stored to every rank
            check_error(self.lib.infiniopRandomSampleBatchPeer(
                op.desc, res, shards, strides, vl, flags, self.world, self.rank, r0, mine,
                random_vals[r0:r1].data_ptr(), topp, topk, temperature, sp))
            mark("sample")
            if results.data_ptr() != pb.results.data_ptr():
                results.view(torch.int64).copy_(pb.results[:rows])
            mark("finish")
            return
        check_error(self.lib.infiniopExtPeerGatherRows(
            self.handle, full.data_ptr(), full.stride(0), shards, strides, col0, ncols, flags, self.world, self.rank,
            r0, mine, sp))
        mark("exchange")
        if mine:
            op.batch(picked[self.rank, :mine], full[:mine], random_vals[r0:r1], topp, topk, temperature, stream=sp)
        mark("sample")
        check_error(self.lib.infiniopExtPeerPublishResults(
            self.handle, res, picked[self.rank].data_ptr(), flags, self.world, self.rank, r0, mine, sp))
        mark("publish")
        if results.data_ptr() != pb.results.data_ptr():
            results.view(torch.int64).copy_(pb.results[:rows])
        mark("finish")

    def _sample_fast(self, results, local_logits, random_vals, topp, topk, temperature, sp, check, mark):
        rows = local_logits.shape[0]
        local, gathered, status = self._buffers(rows, local_logits.device)
        check_error(self.lib.infiniopRandomSampleShardLocal(
            self.op.desc, local.data_ptr(), local_logits.data_ptr(), local_logits.stride(0), rows, self.shard_offset,
            topk, temperature, sp))
        mark("local")
        if self._gather is not None:
            self._gather(gathered, local)
        elif self.world > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(gathered.view(-1), local.view(-1), group=self.group)
        else:
            gathered[0].copy_(local)
        mark("all_gather")
        status.zero_()
        check_error(self.lib.infiniopRandomSampleShardFinish(
            self.handle, results.data_ptr(), gathered.data_ptr(), self.world, rows, self.voc_total,
            random_vals.data_ptr(), topp, topk, temperature, status.data_ptr(), sp))
        mark("finish")
        if check and int(status.item()) != 0:
            raise RuntimeError("vocabulary-sharded sampling: a shard held more than 128 tied candidates in some row; "
                               "gather the logits and use the unsharded entry point for this batch")
