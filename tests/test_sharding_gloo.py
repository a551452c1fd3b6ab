"""Multi-rank host logic on CPU ranks (gloo, world size 2): row sharding of the
row-parallel operators, and the record / all-gather / merge protocol of
vocabulary-sharded sampling.  Device kernels are replaced by their CPU
restatements (the oracle for the operators, tests/shard_protocol_cpu.py for the
two sampling stages); what is under test is the partitioning, the record
layout, the gather order and the merge, which are the same on GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from operators_b200.sharding import assemble_rows, exchange_plan, row_range, shard_rows, vocab_range
    from oracle import cpu_oracle as oracle
    from shard_protocol_cpu import finish_numpy, pack_record_numpy

    ok = True
    # --- row-parallel operator: every rank works on its slice, the gathered result equals the unsharded one
    g = torch.Generator().manual_seed(11)
    gate_up = torch.randn((36, 2 * 64), generator=g).half()
    full = oracle.swiglu(gate_up[:, 64:].numpy(), gate_up[:, :64].numpy())
    mine = shard_rows(gate_up, world, rank)
    part = torch.from_numpy(oracle.swiglu(mine[:, 64:].numpy(), mine[:, :64].numpy()).view(np.uint16).astype(np.int32))
    sizes = [row_range(36, world, r) for r in range(world)]
    parts = [torch.zeros((e - b, 64), dtype=torch.int32) for b, e in sizes]
    dist.all_gather(parts, part)
    ok &= np.array_equal(torch.cat(parts).numpy().astype(np.uint16), full.view(np.uint16))
    ok &= sizes[0][0] == 0 and sizes[-1][1] == 36 and all(sizes[i][1] == sizes[i + 1][0] for i in range(world - 1))

    # --- vocabulary-sharded sampling: local records -> all_gather -> merge on every rank
    rows, voc, topk, topp, temp, words = 12, 6000, 20, 0.9, 0.8, 8 + 2 * 128
    logits = (torch.randn((rows, voc), generator=g) * 3).half()
    logits[3] = (torch.randint(0, 500, (voc,), generator=g).float() / 64).half()  # ties inside the top-k
    logits[5] = torch.randint(0, 6, (voc,), generator=g).half()  # more tied candidates than a record holds
    u = torch.rand(rows, generator=g)
    b, e = vocab_range(voc, world, rank)
    local = np.stack([pack_record_numpy(logits[r, b:e].numpy(), b, topk, temp, words) for r in range(rows)])
    gathered = [torch.zeros((rows, words), dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(local.view(np.int32)))
    G = np.stack([t.numpy().view(np.uint32) for t in gathered])
    got = [finish_numpy(G, r, float(u[r]), topp, topk, temp, voc) for r in range(rows)]
    want = [oracle.random_sample(logits[r].numpy(), float(u[r]), topp, topk, temp) for r in range(rows)]
    # same top-k order as the oracle in every row (the denominators differ in the last bits, see the kernel's header)
    ok &= got[5] == "overflow"
    fine = [r for r in range(rows) if r != 5]
    same_topk = all(
        np.array_equal(np.array(_topk_order(G, r, topk), np.uint64), oracle.random_sample_trace(logits[r].numpy(), topk, temp)["top_idx"])
        for r in fine)
    ok &= same_topk
    ok &= sum(int(got[r] == want[r]) for r in fine) >= len(fine) - 1
    # every rank computed the same answer
    mine_t = torch.tensor([(-1 if (x is None or x == "overflow") else x) for x in got])
    both = [torch.zeros_like(mine_t) for _ in range(world)]
    dist.all_gather(both, mine_t)
    ok &= all(torch.equal(both[0], t) for t in both)
    # --- index-exact mode: one all-to-all hands every rank whole rows, the oracle samples them (the exact kernel's
    # stand-in), one all-gather returns the indices: every row's index is the unsharded answer
    rows2, voc2 = 7, 5003  # neither divides by the world size
    logits2 = (torch.randn((rows2, voc2), generator=g) * 3).half()
    u2 = torch.rand(rows2, generator=g)
    (r0, r1), send, recv, cols = exchange_plan(rows2, voc2, world, rank)
    mine_cols = logits2[:, cols[rank][0]:cols[rank][1]].contiguous()
    received = torch.zeros(sum(recv), dtype=torch.int32)  # gloo's all-to-all takes no 16-bit types: bit patterns as int32
    dist.all_to_all_single(received, mine_cols.view(torch.int16).view(-1).to(torch.int32), recv, send)
    full = assemble_rows(received, r1 - r0, cols).to(torch.int16).view(torch.float16)
    ok &= torch.equal(full, logits2[r0:r1])
    most = max(e - b for b, e in (row_range(rows2, world, r) for r in range(world)))
    picked = torch.full((most,), -1, dtype=torch.int64)
    for i in range(r1 - r0):
        picked[i] = oracle.random_sample(full[i].numpy(), float(u2[r0 + i]), topp, topk, temp)
    everybody = [torch.zeros_like(picked) for _ in range(world)]
    dist.all_gather(everybody, picked)
    got2 = []
    for r in range(world):
        b2, e2 = row_range(rows2, world, r)
        got2 += everybody[r][:e2 - b2].tolist()
    ok &= got2 == [oracle.random_sample(logits2[r].numpy(), float(u2[r]), topp, topk, temp) for r in range(rows2)]
    open(os.path.join(out_dir, "ok_%d" % rank), "w").write("1" if ok else "0")
    dist.destroy_process_group()


def _topk_order(G, row, topk):
    buf = []
    for r in range(G.shape[0]):
        rec = G[r, row]
        for c in range(int(rec[0])):
            carried = (int(rec[9 + 2 * c]), int(rec[8 + 2 * c]))
            for s in range(len(buf)):
                if buf[s][0] < carried[0]:
                    buf[s], carried = carried, buf[s]
            if len(buf) < topk:
                buf.append(carried)
    return [i for _, i in buf]


@pytest.mark.timeout(300)
def test_two_cpu_ranks(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / ("ok_%d" % r)).read() == "1"


def test_row_range_partitions():
    from operators_b200.sharding import row_range

    for n in (0, 1, 7, 16, 8192, 128256):
        for w in (1, 2, 3, 4, 8):
            edges = [row_range(n, w, r) for r in range(w)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            assert all(edges[i][1] == edges[i + 1][0] for i in range(w - 1))
            assert max(e - b for b, e in edges) - min(e - b for b, e in edges) <= 1
