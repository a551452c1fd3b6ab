"""numpy restatement of the vocabulary-sharded sampling protocol (record layout,
gather order, merge) used by the CPU tests of the multi-rank host logic.  Test
infrastructure only: the shipped path runs the two CUDA stages of
operators_b200/csrc/random_sample_sharded.cu."""
def pack_record_numpy(local_logits_row, shard_offset, topk, temperature, record_words):
    """numpy restatement of the stage-1 record for one row (used by the CPU tests
    of the gather / merge logic): [count, max key, sum lo, sum hi, 0,0,0,0, (idx, key)*]."""
    import numpy as np

    h = np.asarray(local_logits_row).view(np.uint16).astype(np.uint32)
    mag = h & 0x7FFF
    keys = np.where(h & 0x8000, 0x8000 - mag, 0x8000 + mag).astype(np.uint32)
    k = min(topk, keys.size)
    kth = np.sort(keys)[-k]
    cand = np.nonzero(keys >= kth)[0]
    vals = np.asarray(local_logits_row).view(np.float16).astype(np.float64)
    m = vals.max()
    s = np.exp((vals - m) / temperature).sum()
    rec = np.zeros(record_words, np.uint32)
    rec[0] = cand.size if cand.size <= (record_words - 8) // 2 else 0xFFFFFFFF
    rec[1] = keys.max()
    rec[2:4] = np.array([s], np.float64).view(np.uint32)
    if rec[0] != 0xFFFFFFFF:
        rec[8:8 + 2 * cand.size:2] = (cand + shard_offset).astype(np.uint32)
        rec[9:9 + 2 * cand.size:2] = keys[cand]
    return rec


def finish_numpy(gathered, row, random_val, topp, topk, temperature, voc_total):
    """numpy restatement of the stage-2 merge for one row of `gathered`
    [ranks, rows, words]: returns the sampled index (or None when no candidate
    satisfies the draw)."""
    import numpy as np

    def val(key):
        key = int(key)
        hbits = key - 0x8000 if key >= 0x8000 else (0x8000 | (0x8000 - key))
        return np.array([hbits], np.uint16).view(np.float16).astype(np.float32)[0]

    def trunc16(x):
        b = np.array([x], np.float32).view(np.uint32)[0]
        sign, e, man = (b >> 16) & 0x8000, int((b >> 23) & 0xFF) - 127, b & 0x7FFFFF
        if e >= -14:
            hb = sign | ((e + 15) << 10) | (man >> 13)
        elif e >= -24:
            hb = sign | (((man | 0x800000) >> (-14 - e)) >> 13)
        else:
            hb = sign
        return np.array([hb], np.uint16).view(np.float16).astype(np.float32)[0]

    ranks = gathered.shape[0]
    k = min(topk, voc_total)
    if any(int(gathered[r, row, 0]) == 0xFFFFFFFF for r in range(ranks)):
        return "overflow"  # the CUDA stage raises its status flag in this case
    mkey = max(int(gathered[r, row, 1]) for r in range(ranks))
    M = val(mkey)
    S = 0.0
    buf = []  # (key, idx), sorted with the strict-greater insertion cascade
    for r in range(ranks):
        rec = gathered[r, row].view(np.uint32)
        sr = rec[2:4].view(np.float64)[0]
        dx = np.float32(np.float32(val(rec[1]) - M) / np.float32(temperature))
        S += sr * np.exp(np.float64(dx))
        for c in range(int(rec[0])):
            carried = (int(rec[9 + 2 * c]), int(rec[8 + 2 * c]))
            for s in range(len(buf)):
                if buf[s][0] < carried[0]:
                    buf[s], carried = carried, buf[s]
            if len(buf) < k:
                buf.append(carried)
    Sf = np.float32(S)
    p = []
    for key, _ in buf[:k]:
        x = np.float32(np.float32(val(key) - M) / np.float32(temperature))
        p.append(trunc16(np.float32(np.float32(np.exp(np.float64(x))) / Sf)))
    acc, end = np.float32(0), 0
    for end in range(k):
        acc = np.float32(acc + p[end])
        if acc >= np.float32(topp):
            break
    end = end + 1 if end < k - 1 else k
    tot = np.float32(0)
    for i in range(end):
        tot = np.float32(tot + p[i])
    rr = np.float32(np.float32(random_val) * tot)
    run = np.float32(0)
    for i in range(end):
        run = np.float32(run + p[i])
        if rr < run:
            return buf[i][1]
    return None
