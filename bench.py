#!/usr/bin/env python
"""Benchmark of the decode hot path: RMSNorm, RoPE, SwiGLU, Add, causal softmax
and random sample at the configurations of BASELINE.json.

One "step" runs the six operators once, each on its BASELINE.json configuration
(seeded synthetic inputs of those shapes and value distributions).  The metric
is achieved HBM bandwidth: algorithmic bytes of the step / time, reported for
the whole step (`value`) and per operator (`ops`), plus tokens/s for sampling.

  python bench.py [--gpus N] [--steps K] [--warmup W]        this library (sm_100a kernels)
  python bench.py --impl reference [...]                      the reference CPU backend on the host cores

Under torchrun (N > 1) every rank runs the same step on its own GPU and its
own rows (weak scaling, no data-path collective); time = max over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# ---- BASELINE.json configurations ---------------------------------------------------
RMS_N, RMS_D = 16, 2048
ROPE_T, ROPE_H, ROPE_DH = 4096, 32, 128
SWI_T, SWI_DI = 8192, 14336
ADD_T, ADD_D = 8192, 4096
SM_H, SM_Q, SM_KV = 32, 512, 4096
RS_B, RS_V = 64, 128256
RS_TEMP, RS_TOPK, RS_TOPP = 0.8, 50, 0.9

# Algorithmic bytes per operator launch: every input element read once, every
# output element written once (for causal softmax only the visible part is read).
ALGO_BYTES = {
    "rms_norm": 2 * RMS_N * RMS_D * 2 + RMS_D * 2,
    "rope": 2 * ROPE_T * ROPE_H * ROPE_DH * 2 + ROPE_T * 8 + 2 * ROPE_T * ROPE_DH * 4,
    "swiglu": 3 * SWI_T * SWI_DI * 2,
    "add": 3 * ADD_T * ADD_D * 2,
    "causal_softmax": SM_H * sum((SM_KV - SM_Q + i + 1) for i in range(SM_Q)) * 2 + SM_H * SM_Q * SM_KV * 2,
    "random_sample": RS_B * RS_V * 2 + RS_B * 4 + RS_B * 8,
}
OPS = list(ALGO_BYTES)
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

def ncu_traffic_bytes(profile):
    """DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel, from the
    line `dram_traffic_bytes_per_launch: N` of the committed ncu summary profiles/<profile>; None when absent."""
    import re

    try:
        text = open(os.path.join(ROOT, "profiles", profile)).read()
    except OSError:
        return None
    m = re.search(r"dram_traffic_bytes_per_launch:\s*(\d+)", text)
    return int(m.group(1)) if m else None


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def measured_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def make_inputs(seed, rows_fraction=1.0, only=None):
    """Seeded CPU tensors of the six configurations (fp32 draws cast to fp16).
    `only` names one operator: the other operators then get one-row stand-ins."""
    import torch

    g = torch.Generator().manual_seed(seed)

    def frac(n, op=None):
        if only is not None and op != only:
            return 1
        return max(1, int(round(n * rows_fraction)))

    d = {}
    d["rms_x"] = (torch.rand((frac(RMS_N, "rms_norm"), RMS_D), generator=g) * 2 - 1).half()
    d["rms_w"] = (torch.rand(RMS_D, generator=g) * 2 - 1).half()
    nt = frac(ROPE_T, "rope")
    d["rope_t"] = torch.randn((nt, ROPE_H, ROPE_DH), generator=g).half()
    d["rope_pos"] = torch.arange(nt, dtype=torch.int64)
    from operators_b200.ops import sin_cos_table

    d["rope_sin"], d["rope_cos"] = sin_cos_table(ROPE_T, ROPE_DH, 1e4)
    # 235M-element normal draws dominate set-up time: draw once in fp32 chunks
    gu = torch.empty((frac(SWI_T, "swiglu"), 2 * SWI_DI), dtype=torch.float16)
    step = 512
    for r in range(0, gu.shape[0], step):
        gu[r:r + step] = torch.randn((min(step, gu.shape[0] - r), 2 * SWI_DI), generator=g).half()
    d["gate_up"] = gu
    d["add_a"] = torch.randn((frac(ADD_T, "add"), ADD_D), generator=g).half()
    d["add_b"] = torch.randn((frac(ADD_T, "add"), ADD_D), generator=g).half()
    d["att"] = (torch.randn((frac(SM_H, "causal_softmax"), SM_Q, SM_KV), generator=g) * 2).half()
    nb = frac(RS_B, "random_sample")
    d["logits"] = (torch.randn((nb, RS_V), generator=g) * 3).half()
    d["u"] = torch.rand(nb, generator=g)
    return d


def sample_bytes(inputs):
    """Algorithmic bytes of a step over `inputs` (which may hold a row sample)."""
    b = {}
    n = inputs["rms_x"].shape[0]
    b["rms_norm"] = 2 * n * RMS_D * 2 + RMS_D * 2
    nt = inputs["rope_t"].shape[0]
    b["rope"] = 2 * nt * ROPE_H * ROPE_DH * 2 + nt * 8 + 2 * nt * ROPE_DH * 4
    b["swiglu"] = 3 * inputs["gate_up"].shape[0] * SWI_DI * 2
    b["add"] = 3 * inputs["add_a"].shape[0] * ADD_D * 2
    h = inputs["att"].shape[0]
    b["causal_softmax"] = h * sum((SM_KV - SM_Q + i + 1) for i in range(SM_Q)) * 2 + h * SM_Q * SM_KV * 2
    nb = inputs["logits"].shape[0]
    b["random_sample"] = nb * RS_V * 2 + nb * 4 + nb * 8
    return b


# ---- clocks ---------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons of one GPU, polled through NVML (read-only
    queries) from a host thread while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, torch_index):
        self.samples, self.reason_bits, self.stop_flag, self.thread = [], 0, False, None
        self.handle, self.max_mhz = None, None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(torch_index).uuid)
                if not uuid.startswith("GPU-"):
                    uuid = "GPU-" + uuid
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(torch_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.handle = None

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
            except Exception:
                break
            time.sleep(0.001)

    def start(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm = sorted(self.samples)
        reasons = sorted(k for k, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(sm)}


def pin_to_gpu_numa_node(torch, local):
    """Moves this process onto the CPUs of the NUMA node the GPU hangs off (read from sysfs), so that the pinned
    staging buffers allocated afterwards are first touched there.  Returns what was done, for the JSON line."""
    try:
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
    except OSError:
        nodes = []
    if len(nodes) <= 1:
        return "host exposes one NUMA node: all ranks stage through it"
    try:
        props = torch.cuda.get_device_properties(local)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bdf).read().strip())
        if node < 0:
            return "GPU %s reports no NUMA node; affinity left as it was" % bdf
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return "node %d of GPU %s has no CPU this process may use; affinity left as it was" % (node, bdf)
        os.sched_setaffinity(0, allowed)
        return "rank pinned to NUMA node %d (%d CPUs) of GPU %s" % (node, len(allowed), bdf)
    except Exception as exc:  # noqa: BLE001
        return "NUMA node of the GPU not found (%s); affinity left as it was" % exc


# ---- this library ------------------------------------------------------------------------
class DecodeStep:
    """The six operators bound to device buffers; run() launches one step."""

    def __init__(self, lib, handle, dev, inputs):
        import torch

        from operators_b200 import ops

        self.torch, self.dev = torch, dev
        t = {k: (v.to(dev) if v is not None else None) for k, v in inputs.items()}
        self.t = t
        t["rms_y"] = torch.zeros_like(t["rms_x"])
        di = SWI_DI
        t["swi_b"], t["swi_a"] = t["gate_up"][:, :di], t["gate_up"][:, di:]  # gate half -> silu, up half -> multiplier
        t["swi_c"] = torch.zeros((t["gate_up"].shape[0], di), dtype=torch.float16, device=dev)
        t["add_c"] = torch.zeros_like(t["add_a"])
        t["rs_out"] = torch.zeros(t["logits"].shape[0], dtype=torch.int64, device=dev)
        self.rms = ops.RMSNormOp(lib, handle, t["rms_y"], t["rms_x"], t["rms_w"], 1e-5)
        self.rope = ops.RoPEOp(lib, handle, t["rope_t"], t["rope_pos"], t["rope_sin"], t["rope_cos"])
        self.swi = ops.SwiGLUOp(lib, handle, t["swi_c"], t["swi_a"], t["swi_b"])
        self.add = ops.AddOp(lib, handle, t["add_c"], t["add_a"], t["add_b"])
        self.sm = ops.CausalSoftmaxOp(lib, handle, t["att"])
        self.rs = ops.RandomSampleOp(lib, handle, t["rs_out"][:1], t["logits"][0])
        self.launches_per_step = 6

    def calls(self):
        t = self.t
        return [
            ("rms_norm", lambda s: self.rms(t["rms_y"], t["rms_x"], t["rms_w"], s)),
            ("rope", lambda s: self.rope(t["rope_t"], t["rope_pos"], t["rope_sin"], t["rope_cos"], s)),
            ("swiglu", lambda s: self.swi(t["swi_c"], t["swi_a"], t["swi_b"], s)),
            ("add", lambda s: self.add(t["add_c"], t["add_a"], t["add_b"], s)),
            ("causal_softmax", lambda s: self.sm(t["att"], s)),
            ("random_sample", lambda s: self.rs.batch(t["rs_out"], t["logits"], t["u"], RS_TOPP, RS_TOPK, RS_TEMP, s)),
        ]


def only_rearrange(lib, handle, dev, steps, warmup):
    """Not part of the step: the permute on the way out of attention, for ncu captures."""
    import torch

    from operators_b200 import ops as _ops

    src = torch.randn((ROPE_T, ROPE_H, ROPE_DH), device=dev).half()
    dst = torch.as_strided(torch.empty(ROPE_T * ROPE_H * ROPE_DH, device=dev, dtype=torch.float16),
                           (ROPE_T, ROPE_H, ROPE_DH), (ROPE_DH, ROPE_T * ROPE_DH, 1))  # [heads, tokens, dh] storage
    op = _ops.RearrangeOp(lib, handle, dst, src)
    for _ in range(warmup):
        op(dst, src)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        op(dst, src)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    nbytes = 2 * src.numel() * 2
    return {"only": "rearrange", "shape": list(src.shape), "ms": round(ms, 5),
            "gbs": round(nbytes / ms / 1e6, 1),
            "note": "back-to-back launches of one operator; not a bench value"}


def only_add_rms_norm(lib, handle, dev, steps, warmup):
    """Not part of the step: the fused residual form beside the two calls it replaces."""
    import torch

    from operators_b200 import ops as _ops

    shape = (ADD_T, ADD_D)
    a = torch.randn(shape, device=dev).half()
    b = torch.randn(shape, device=dev).half()
    w = torch.rand(shape[1], device=dev).half()
    total, y = torch.empty_like(a), torch.empty_like(a)
    fused = _ops.AddRMSNormOp(lib, handle, y, total, a, b, w)
    add_op, norm_op = _ops.AddOp(lib, handle, total, a, b), _ops.RMSNormOp(lib, handle, y, total, w)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / steps

    ms_fused = timed(lambda: fused(y, total, a, b, w))
    ms_pair = timed(lambda: (add_op(total, a, b), norm_op(y, total, w)))
    nbytes = 4 * a.numel() * 2 + w.numel() * 2  # a, b read; sum, y written (268 MB per launch: larger than L2)
    return {"only": "add_rms_norm", "shape": list(shape), "ms": round(ms_fused, 5),
            "gbs": round(nbytes / ms_fused / 1e6, 1), "ms_add_then_rms_norm": round(ms_pair, 5),
            "note": "back-to-back launches of one operator; not a bench value"}


def only_rope_rearrange(lib, handle, dev, steps, warmup):
    """Not part of the step: K rotated into the cache beside the two calls it replaces."""
    import torch

    from operators_b200 import ops as _ops

    tokens, kv_heads, dh, cache_len = 4 * ROPE_T, 8, ROPE_DH, 4 * ROPE_T
    qkv = torch.randn((tokens, (ROPE_H + 2 * kv_heads) * dh), device=dev).half()
    k = qkv[:, ROPE_H * dh:(ROPE_H + kv_heads) * dh].view(tokens, kv_heads, dh)  # the K slice of a qkv row
    pos = torch.arange(tokens, device=dev, dtype=torch.int64)
    sin, cos = _ops.sin_cos_table(tokens, dh, device=dev)
    cache = torch.zeros((kv_heads, cache_len, dh), device=dev, dtype=torch.float16)
    dst = cache.permute(1, 0, 2)
    fused = _ops.RoPERearrangeOp(lib, handle, dst, k, pos, sin, cos)
    rope_op, copy_op = _ops.RoPEOp(lib, handle, k, pos, sin, cos), _ops.RearrangeOp(lib, handle, dst, k)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            fn()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / steps

    ms_fused = timed(lambda: fused(dst, k, pos, sin, cos))
    ms_pair = timed(lambda: (rope_op(k, pos, sin, cos), copy_op(dst, k)))
    nbytes = 2 * k.numel() * 2 + 2 * sin.numel() * 4 + pos.numel() * 8
    return {"only": "rope_rearrange", "shape": list(k.shape), "ms": round(ms_fused, 5),
            "gbs": round(nbytes / ms_fused / 1e6, 1), "ms_rope_then_rearrange": round(ms_pair, 5),
            "note": "back-to-back launches of one operator on L2-sized data; not a bench value"}


def only_attention(lib, handle, dev, steps, warmup):
    """Not part of the step: one decoding token over a long KV cache."""
    import torch

    from operators_b200 import ops as _ops

    nh, nkvh, dh, pos = 32, 8, ROPE_DH, 65535  # 268 MB of K and V rows per call: larger than L2
    q = torch.randn((nh, 1, dh), device=dev).half()
    k = torch.randn((nkvh, 1, dh), device=dev).half()
    v = torch.randn((nkvh, 1, dh), device=dev).half()
    k_cache = torch.randn((nkvh, pos + 1, dh), device=dev).half()
    v_cache = torch.randn((nkvh, pos + 1, dh), device=dev).half()
    out = torch.empty((1, nh, dh), device=dev, dtype=torch.float16)
    op = _ops.AttentionOp(lib, handle, out, q, k, v, k_cache, v_cache, pos)
    for _ in range(warmup):
        op(out, q, k, v, k_cache, v_cache)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        op(out, q, k, v, k_cache, v_cache)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    nbytes = 2 * nkvh * (pos + 1) * dh * 2
    return {"only": "attention", "q_heads": nh, "kv_heads": nkvh, "head_dim": dh, "cached_tokens": pos + 1,
            "ms": round(ms, 5), "gbs": round(nbytes / ms / 1e6, 1), "launches_per_call": 2,
            "note": "back-to-back calls of one operator; bytes = K and V rows read once; not a bench value"}


PREFILL_CASE = {"new_tokens": None, "cached_tokens": 0}  # --new-tokens / --cached-tokens: one case only (ncu captures)


def only_attention_prefill(lib, handle, dev, steps, warmup):
    """Not part of the step: attention for a prompt (new tokens into an empty cache) and for a chunk of a prompt over a
    cached prefix, 32 q / 8 kv heads, dh 128.  FLOPs count the visible part of the two products."""
    import torch

    from operators_b200 import ops as _ops

    nh, nkvh, dh = 32, 8, ROPE_DH
    peak = measured_tflops()
    cases = {}
    for seq, pos in ((512, 0), (2048, 0), (4096, 0), (512, 32768), (64, 8192)):
        if PREFILL_CASE["new_tokens"] is not None and (PREFILL_CASE["new_tokens"], PREFILL_CASE["cached_tokens"]) != (seq, pos):
            continue
        total = pos + seq
        q = torch.randn((nh, seq, dh), device=dev).half()
        k = torch.randn((nkvh, seq, dh), device=dev).half()
        v = torch.randn((nkvh, seq, dh), device=dev).half()
        k_cache = torch.randn((nkvh, total, dh), device=dev).half()
        v_cache = torch.randn((nkvh, total, dh), device=dev).half()
        out = torch.empty((seq, nh, dh), device=dev, dtype=torch.float16)
        op = _ops.AttentionOp(lib, handle, out, q, k, v, k_cache, v_cache, pos)
        ms = _timed_calls(torch, lambda: op(out, q, k, v, k_cache, v_cache), steps, warmup)
        op.destroy()
        flops = 4.0 * nh * dh * (seq * pos + seq * (seq + 1) / 2)
        name = "%d_new_tokens" % seq if pos == 0 else "%d_new_over_%d_cached" % (seq, pos)
        cases[name] = {"ms": round(ms, 5), "tflops": round(flops / ms / 1e9, 1),
                       "frac_of_measured_bf16": round(flops / ms / 1e9 / peak[0], 3) if peak[0] else None}
        del q, k, v, k_cache, v_cache, out
    return {"only": "attention_prefill", "q_heads": nh, "kv_heads": nkvh, "head_dim": dh, "cases": cases,
            "peak_tflops": {"value": peak[0], "source": peak[1]},
            "note": "back-to-back calls: cache append + one kernel that keeps the scores on chip (--select-kernel "
                    "attention=3: scores, softmax and values as three launches); the exponentials (two per visible "
                    "score: the reference's rounding needs the row sum before any probability), not the tensor "
                    "pipe, bound the one kernel; not a bench value"}


def _timed_calls(torch, fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / steps


SHARDED_MODES = ("exact", "exact_all_to_all", "exact_all_gather", "exact_peer_memory", "fast")
MATMUL_CASE = {"tokens": None, "weights": None}  # --tokens / --weights: one case only (ncu captures)


def only_matmul(lib, handle, dev, steps, warmup):
    """Not part of the step: the gate / up projection of the SwiGLU configuration, [tokens, 4096] x [4096, 28672],
    for a prefill-sized and two decoding token counts, weights in both layouts.  Prefill shapes are judged in
    TFLOP/s against the measured cuBLAS bf16 peak, decoding shapes in GB/s against the measured copy bandwidth
    (the 235 MB weight matrix is read once; it is larger than L2)."""
    import torch

    from operators_b200 import ops as _ops

    hidden, n = ADD_D, 2 * SWI_DI
    peak_tf, tf_kind = measured_tflops()
    peak_bw, bw_kind = measured_peak()
    w_kn = torch.randn((hidden, n), device=dev).half() * 0.02       # [k, n] row-major: n contiguous
    w_nk = (torch.randn((n, hidden), device=dev).half() * 0.02).t()  # [k, n] view of a [n, k] weight: k contiguous
    out = {"only": "matmul", "k": hidden, "n": n, "cases": [],
           "note": "back-to-back calls of one operator; not a bench value"}
    for tokens in (SWI_T, 16, 1):
        if MATMUL_CASE["tokens"] not in (None, tokens):
            continue
        a = torch.randn((tokens, hidden), device=dev).half()
        c = torch.empty((tokens, n), device=dev, dtype=torch.float16)
        for name, w in (("k_contiguous", w_nk), ("n_contiguous", w_kn)):
            if MATMUL_CASE["weights"] not in (None, name):
                continue
            op = _ops.MatmulOp(lib, handle, c, a, w)
            ms = _timed_calls(torch, lambda: op(c, a, w), max(3, steps // (4 if tokens > 64 else 1)), warmup)
            op.destroy()
            flops, nbytes = 2.0 * tokens * hidden * n, 2.0 * (tokens * hidden + hidden * n + tokens * n)
            case = {"tokens": tokens, "weights": name, "ms": round(ms, 5), "tflops": round(flops / ms / 1e9, 1),
                    "gbs": round(nbytes / ms / 1e6, 1)}
            if tokens > 64:
                case["frac_of_%s_bf16_peak" % tf_kind] = round(flops / ms / 1e9 / peak_tf, 4)
            else:
                case["frac_of_%s_hbm_peak" % bw_kind] = round(nbytes / ms / 1e6 / peak_bw, 4)
            out["cases"].append(case)
        del a, c
    return out


def only_mlp(lib, handle, dev, steps, warmup):
    """Not part of the step: the MLP composite at hidden 4096, intermediate 14336 (SwiGLU runs as the epilogue of
    the first product: the [tokens, 2 x 14336] tensor of the SwiGLU configuration never reaches HBM)."""
    import torch

    from operators_b200 import ops as _ops

    hidden, di = ADD_D, SWI_DI
    w12 = torch.randn((hidden, 2 * di), device=dev).half() * 0.02
    w3 = torch.randn((di, hidden), device=dev).half() * 0.02
    out = {"only": "mlp", "hidden": hidden, "intermediate": di, "cases": [],
           "note": "back-to-back calls of one operator; not a bench value"}
    for tokens in (SWI_T, 16):
        x = torch.randn((tokens, hidden), device=dev).half() * 0.1
        y = torch.randn((tokens, hidden), device=dev).half()
        op = _ops.MLPOp(lib, handle, y, x, w12, w3, 1.0, True)
        ms = _timed_calls(torch, lambda: op(y, x, w12, w3), max(3, steps // (4 if tokens > 64 else 1)), warmup)
        op.destroy()
        flops, wbytes = 2.0 * tokens * hidden * 3 * di, 2.0 * 3 * hidden * di
        out["cases"].append({"tokens": tokens, "ms": round(ms, 5), "tflops": round(flops / ms / 1e9, 1),
                             "weight_gbs": round(wbytes / ms / 1e6, 1)})
        del x, y
    return out


NEXT_ROWS = {"matmul": only_matmul, "mlp": only_mlp, "rearrange": only_rearrange, "add_rms_norm": only_add_rms_norm, "rope_rearrange": only_rope_rearrange,
             "attention": only_attention, "attention_prefill": only_attention_prefill}


def run_b200(args):
    import torch

    from operators_b200 import DeviceEnum, create_handle, open_lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU path in this library"
    torch.cuda.set_device(local)
    dev = "cuda:%d" % local
    if world > 1:
        import torch.distributed as dist

        import datetime

        # a collective that a peer never joins ends with an error after five minutes instead of hanging the box
        dist.init_process_group("nccl", device_id=torch.device(dev), timeout=datetime.timedelta(minutes=5))
    lib = open_lib(os.path.join(ROOT, "operators_b200", "lib"))
    handle = create_handle(lib, DeviceEnum.DEVICE_CUDA, local)
    for item in args.select_kernel:
        from operators_b200 import ops as _sel

        family, _, variant = item.partition("=")
        _sel.select_kernel(lib, family, int(variant))

    if args.only in NEXT_ROWS:  # operators either side of the step, one at a time (for ncu captures and tuning)
        print(json.dumps(NEXT_ROWS[args.only](lib, handle, dev, args.steps, args.warmup)))
        return
    inputs = make_inputs(1000 + rank, only=args.only)
    step = DecodeStep(lib, handle, dev, inputs)
    calls = step.calls()
    if args.only:  # profiling runs: a single operator, nothing else launched
        calls = [c for c in calls if c[0] == args.only]
        step.launches_per_step = 1
        for _ in range(args.warmup):
            calls[0][1](None)
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            calls[0][1](None)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / args.steps
        print(json.dumps({"only": args.only, "ms": round(ms, 5), "gbs": round(ALGO_BYTES[args.only] / ms / 1e6, 1),
                          "note": "back-to-back launches of one operator; not a bench value"}))
        return
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream
    from operators_b200 import ops as _ops_mod

    device_timeouts_before = _ops_mod.device_timeouts(lib, handle)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        for _, fn in calls:
            fn(sptr)
    barrier()

    # One step captured into a CUDA graph (the entry points neither allocate nor synchronise, so they can be
    # captured as they are); the timed region replays it K times.  Plain launches if capture is unavailable.
    graph = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(stream)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _, fn in calls:
                    fn(torch.cuda.current_stream().cuda_stream)
            stream.wait_stream(side)
            g.replay()
            torch.cuda.synchronize()
            graph = g
        except Exception as exc:  # noqa: BLE001
            print("bench: CUDA graph capture failed (%s); timing plain launches" % exc, file=sys.stderr)
            torch.cuda.synchronize()
    barrier()

    # ---- timed region: exactly K steps between two device events, nothing else on the stream ----
    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    for k in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            for _, fn in calls:
                fn(sptr)
    t_end.record(stream)
    barrier()
    ms_per_step = t_begin.elapsed_time(t_end) / args.steps

    # ---- sustained: the same step replayed for at least a second (the K timed steps above last milliseconds and
    # say nothing about the power-capped state); clocks sampled over this second alone ----
    sustained = None
    if args.sustain_seconds > 0:
        n_sus = max(args.steps, int(args.sustain_seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)
        sus_clocks = ClockSampler(local)
        barrier()
        sus_clocks.start()
        s_begin, s_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_begin.record(stream)
        for k in range(n_sus):
            if graph is not None:
                graph.replay()
            else:
                for _, fn in calls:
                    fn(sptr)
        s_end.record(stream)
        barrier()
        sus_clk = sus_clocks.stop()
        sus_ms = s_begin.elapsed_time(s_end) / n_sus
        sustained = (sus_ms, n_sus, sus_clk)

    # ---- the same K steps again with an event after every operator: the per-operator breakdown ----
    # (an event between two launches costs about a microsecond of device time, so these sum to a little more
    # than ms_per_step; `value` comes from the run above)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(calls) + 1)] for _ in range(args.steps)]
    for k in range(args.steps):
        ev[k][0].record(stream)
        for i, (_, fn) in enumerate(calls):
            fn(sptr)
            ev[k][i + 1].record(stream)
    barrier()
    clk = clocks.stop()  # sampled over both passes: the same kernels under the same load
    per_op_all = {name: sorted(ev[k][i].elapsed_time(ev[k][i + 1]) for k in range(args.steps))
                  for i, (name, _) in enumerate(calls)}
    per_op_ms = {name: sum(v) / len(v) for name, v in per_op_all.items()}

    # ---- RMSNorm at a size that can load the memory system (the configuration above is 135 KB: launch latency) ----
    # rank 0 only, outside every timed region above; 36 launches over three rotating [65536, 2048] buffers
    rms_scaled = None
    if rank == 0:
        from operators_b200 import ops as _ops

        n_big, d_big, rot = 65536, 2048, 3
        xs = [torch.randn((n_big, d_big), device=dev).half() for _ in range(rot)]
        ys = [torch.empty_like(x) for x in xs]
        big = _ops.RMSNormOp(lib, handle, ys[0], xs[0], step.t["rms_w"], 1e-5)
        for i in range(rot):
            big(ys[i], xs[i], step.t["rms_w"], sptr)
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record(stream)
        for _ in range(12):
            for i in range(rot):
                big(ys[i], xs[i], step.t["rms_w"], sptr)
        b1.record(stream)
        torch.cuda.synchronize()
        big_ms = b0.elapsed_time(b1) / (12 * rot)
        big_bytes = 2 * n_big * d_big * 2 + d_big * 2
        rms_scaled = {"shape": [n_big, d_big], "bytes": big_bytes, "ms": round(big_ms, 5),
            "gbs": round(big_bytes / big_ms / 1e6, 1)}
        big.destroy()
        del xs, ys
    # ---- RoPE at four times the tokens (the configuration's 67 MB pass in a few microseconds more than launch ramp
    # and tail; this size shows the kernel's own rate) ----
    rope_scaled = None
    if rank == 0:
        from operators_b200 import ops as _ops

        t_big, rot = 4 * ROPE_T, 3
        ts = [torch.randn((t_big, ROPE_H, ROPE_DH), device=dev).half() for _ in range(rot)]
        pos_big = torch.arange(t_big, dtype=torch.int64, device=dev)
        sin_big, cos_big = _ops.sin_cos_table(t_big, ROPE_DH)
        sin_big, cos_big = sin_big.to(dev), cos_big.to(dev)
        rbig = _ops.RoPEOp(lib, handle, ts[0], pos_big, sin_big, cos_big)
        for i in range(rot):
            rbig(ts[i], pos_big, sin_big, cos_big, sptr)
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record(stream)
        for _ in range(12):
            for i in range(rot):
                rbig(ts[i], pos_big, sin_big, cos_big, sptr)
        b1.record(stream)
        torch.cuda.synchronize()
        r_ms = b0.elapsed_time(b1) / (12 * rot)
        r_bytes = 2 * t_big * ROPE_H * ROPE_DH * 2 + t_big * 8 + 2 * t_big * ROPE_DH * 4
        rope_scaled = {"shape": [t_big, ROPE_H, ROPE_DH], "bytes": r_bytes, "ms": round(r_ms, 5),
                       "gbs": round(r_bytes / r_ms / 1e6, 1)}
        rbig.destroy()
        del ts
        # what a plain device copy of the configuration's bytes takes under the same conditions (back-to-back
        # launches over three rotating buffers): 33.5 MB in, 33.5 MB out are a few microseconds of HBM time, so ramp
        # and tail weigh as much as the transfer; the copy is the yardstick for what 67 MB can reach at all
        srcs = [torch.randn((ROPE_T, ROPE_H, ROPE_DH), device=dev).half() for _ in range(3)]
        dsts = [torch.empty_like(x) for x in srcs]
        for i in range(3):
            dsts[i].copy_(srcs[i])
        torch.cuda.synchronize()
        b0.record(stream)
        for _ in range(12):
            for i in range(3):
                dsts[i].copy_(srcs[i])
        b1.record(stream)
        torch.cuda.synchronize()
        rope_scaled["copy_of_config_bytes_ms"] = round(b0.elapsed_time(b1) / 36, 5)
        rcfg = _ops.RoPEOp(lib, handle, srcs[0], step.t["rope_pos"], step.t["rope_sin"], step.t["rope_cos"])
        b0.record(stream)
        for _ in range(12):
            for i in range(3):
                rcfg(srcs[i], step.t["rope_pos"], step.t["rope_sin"], step.t["rope_cos"], sptr)
        b1.record(stream)
        torch.cuda.synchronize()
        rope_scaled["config_back_to_back_ms"] = round(b0.elapsed_time(b1) / 36, 5)
        rcfg.destroy()
        del srcs, dsts
    barrier()

    # ---- end to end: host buffers in, host results out, every step ----
    numa = pin_to_gpu_numa_node(torch, local)  # before the pinned buffers are allocated and first touched
    host_in = {k: inputs[k].pin_memory() for k in
               ("rms_x", "rms_w", "rope_t", "rope_pos", "rope_sin", "rope_cos", "gate_up", "add_a", "add_b", "att",
                "logits", "u")}
    out_names = ["rms_y", "rope_t", "swi_c", "add_c", "att", "rs_out"]
    host_out = {k: torch.empty_like(step.t[k], device="cpu").pin_memory() for k in out_names}
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = sum(v.numel() * v.element_size() for v in host_out.values())

    # Uploads, launches and downloads run on three streams chained by events (operators_b200/staging.py): the
    # upload of the next operator's inputs overlaps the download of the previous one's results, every byte
    # still crosses the link every step.
    from operators_b200.staging import Stage, StagedPipeline

    io = {"rms_norm": (("rms_x", "rms_w"), ("rms_y",)), "rope": (("rope_t", "rope_pos", "rope_sin", "rope_cos"), ("rope_t",)),
          "swiglu": (("gate_up",), ("swi_c",)), "add": (("add_a", "add_b"), ("add_c",)),
          "causal_softmax": (("att",), ("att",)), "random_sample": (("logits", "u"), ("rs_out",))}
    assert sorted(k for ins, _ in io.values() for k in ins) == sorted(host_in) and \
        sorted(k for _, outs in io.values() for k in outs) == sorted(out_names)
    pipe = StagedPipeline([Stage(name, [(step.t[k], host_in[k]) for k in io[name][0]], fn,
                                 [(step.t[k], host_out[k]) for k in io[name][1]]) for name, fn in calls], dev)
    assert pipe.h2d_bytes == h2d and pipe.d2h_bytes == d2h

    e2e_steps = max(2, min(args.steps, 5))
    pipe.run()
    pipe.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    pipe.fork(stream)
    for _ in range(e2e_steps):
        pipe.run()
    pipe.join(stream)
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # ---- N > 1: ONE configuration split over the ranks (strong scaling) ----
    # rows for RMSNorm (scaled shape) / RoPE / SwiGLU / Add, heads for causal softmax; no collective.  Every rank
    # times its slice, the slowest rank counts; the full-size time beside it is this rank's own from the pass above.
    strong = None
    sharded = None
    if world > 1:
        import torch.distributed as dist

        from operators_b200 import ops as _ops
        from operators_b200.sharding import PeerBlocks, VocabShardedSampler, shard_rows, vocab_range

        t = step.t
        sl = {k: shard_rows(t[k], world, rank) for k in ("rope_t", "rope_pos", "gate_up", "swi_c", "add_a", "add_b", "add_c", "att")}
        s_ops = [
            ("rope", _ops.RoPEOp(lib, handle, sl["rope_t"], sl["rope_pos"], t["rope_sin"], t["rope_cos"]),
             lambda op: op(sl["rope_t"], sl["rope_pos"], t["rope_sin"], t["rope_cos"], sptr)),
            ("swiglu", _ops.SwiGLUOp(lib, handle, sl["swi_c"], sl["gate_up"][:, SWI_DI:], sl["gate_up"][:, :SWI_DI]),
             lambda op: op(sl["swi_c"], sl["gate_up"][:, SWI_DI:], sl["gate_up"][:, :SWI_DI], sptr)),
            ("add", _ops.AddOp(lib, handle, sl["add_c"], sl["add_a"], sl["add_b"]),
             lambda op: op(sl["add_c"], sl["add_a"], sl["add_b"], sptr)),
            ("causal_softmax", _ops.CausalSoftmaxOp(lib, handle, sl["att"]), lambda op: op(sl["att"], sptr)),
        ]
        strong_ms = {}
        for name, op, call in s_ops:
            for _ in range(3):
                call(op)
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            for _ in range(args.steps):
                call(op)
            a1.record(stream)
            barrier()
            strong_ms[name] = a0.elapsed_time(a1) / args.steps
            op.destroy()
        strong = strong_ms

        # ---- vocabulary-sharded sampling: index-exact mode (all-to-all of rows, exact kernel, all-gather of the
        # indices) and fast mode (local candidates, one all-gather, finishing kernel), with a stage breakdown ----
        gsh = torch.Generator().manual_seed(77)  # the same logits on every rank, each keeps its columns
        full = (torch.randn((RS_B, RS_V), generator=gsh) * 3).half()
        ush = torch.rand(RS_B, generator=gsh).to(dev)
        b0, e0 = vocab_range(RS_V, world, rank)
        shard_own = full[:, b0:e0].contiguous().to(dev)
        out_own = torch.zeros(RS_B, dtype=torch.int64, device=dev)
        sop = _ops.RandomSampleOp(lib, handle, out_own[:1], shard_own[0])
        sharded = {}
        exact_indices = None
        for mode in SHARDED_MODES:
            exch = mode[6:] if mode.startswith("exact_") else "auto"
            out, shard, pb = out_own, shard_own, None
            if exch == "peer_memory":  # shard and results live in the block the peers address: no copy on the way
                pb = PeerBlocks(lib, handle, RS_B, e0 - b0, world, rank, dev)
                pb.logits.copy_(shard_own)
                out, shard = pb.results, pb.logits
            sampler = VocabShardedSampler(lib, handle, sop, RS_V, b0, world, mode=mode[:5].rstrip("_"), rank=rank,
                                          exchange=exch, peer_blocks=pb)
            for _ in range(3):
                sampler.sample(out, shard, ush, RS_TOPP, RS_TOPK, RS_TEMP, check=False)
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record(stream)
            for _ in range(args.steps):
                sampler.sample(out, shard, ush, RS_TOPP, RS_TOPK, RS_TEMP, check=False)
            s1.record(stream)
            barrier()
            res = {"ms": s0.elapsed_time(s1) / args.steps}
            # the stages one by one (events between them; a few runs, mean)
            acc = {}
            for _ in range(5):
                sampler.sample(out, shard, ush, RS_TOPP, RS_TOPK, RS_TEMP, check=False, timed=True)
                torch.cuda.synchronize()
                evs = sampler.last_events
                for (_, ea), (nb, eb) in zip(evs, evs[1:]):
                    acc[nb] = acc.get(nb, 0.0) + ea.elapsed_time(eb) / 5
            res["stages_ms"] = acc
            # the whole call as one CUDA graph (collectives included), when the capture works on every rank;
            # only on request: a process that still holds a graph with captured NCCL kernels can block in
            # destroy_process_group, so the graph is dropped before the group is
            res["ms_graph"] = None
            gr = None
            res["exchange"] = sampler.exchange if mode != "fast" else None
            # (the peer-memory mode holds no NCCL kernel, so its graph is always timed)
            if not (args.sharded_graph or exch == "peer_memory"):
                if mode == "exact":
                    exact_indices = out.cpu().tolist()
                    res["indices"] = exact_indices
                elif mode.startswith("exact_"):
                    res["same_indices_as_exact"] = out.cpu().tolist() == exact_indices
                sharded[mode] = res
                sampler.destroy()
                if pb is not None:
                    barrier()  # nobody frees a block that a peer may still read
                    pb.destroy()
                continue
            try:
                side = torch.cuda.Stream()
                side.wait_stream(stream)
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=side):
                    sampler.sample(out, shard, ush, RS_TOPP, RS_TOPK, RS_TEMP, check=False)
                stream.wait_stream(side)
            except Exception as exc:  # noqa: BLE001
                res["graph_error"] = str(exc)[:200]
                gr = None
            torch.cuda.synchronize()
            captured = torch.tensor([1 if gr is not None else 0], device=dev)
            dist.all_reduce(captured, op=dist.ReduceOp.MIN)  # replay only when every rank holds a graph
            if int(captured.item()) == 1:
                gr.replay()
                barrier()
                g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                g0.record(stream)
                for _ in range(args.steps):
                    gr.replay()
                g1.record(stream)
                barrier()
                res["ms_graph"] = g0.elapsed_time(g1) / args.steps
            del gr
            torch.cuda.synchronize()
            if mode == "exact":
                exact_indices = out.cpu().tolist()
                res["indices"] = exact_indices
            elif mode.startswith("exact_"):
                res["same_indices_as_exact"] = out.cpu().tolist() == exact_indices
            sharded[mode] = res
            sampler.destroy()
            if pb is not None:
                barrier()
                pb.destroy()
        sharded_ms = sharded["exact"]["ms"]
    else:
        sharded_ms = None

    device_timeouts_after = _ops_mod.device_timeouts(lib, handle)

    # ---- max over ranks ----
    extra_names, extra_vals = [], []
    if sustained is not None:
        extra_names.append("sustained"), extra_vals.append(sustained[0])
    if strong is not None:
        for k, v in strong.items():
            extra_names.append("strong." + k), extra_vals.append(v)
    if sharded is not None:
        for mode, res in sharded.items():
            extra_names.append("sharded.%s.ms" % mode), extra_vals.append(res["ms"])
            extra_names.append("sharded.%s.ms_graph" % mode), extra_vals.append(res["ms_graph"] or 0.0)
            for k, v in res["stages_ms"].items():
                extra_names.append("sharded.%s.stage.%s" % (mode, k)), extra_vals.append(v)
    vals = torch.tensor([ms_per_step, e2e_ms, sharded_ms or 0.0] + [per_op_ms[o] for o in OPS] + extra_vals,
                        dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    vals = vals.cpu().tolist()
    ms_per_step, e2e_ms, sharded_ms = vals[0], vals[1], vals[2]
    own_per_op_ms = dict(per_op_ms)  # this rank's full-size times, the baseline of the strong-scaling speed-ups
    per_op_ms = dict(zip(OPS, vals[3:3 + len(OPS)]))
    extra = dict(zip(extra_names, vals[3 + len(OPS):]))

    step_bytes = sum(ALGO_BYTES.values())
    peak, peak_kind = measured_peak()
    ops_out = {}
    for o in OPS:
        gbs = ALGO_BYTES[o] * world / (per_op_ms[o] * 1e-3) / 1e9
        ops_out[o] = {"bytes": ALGO_BYTES[o], "ms": round(per_op_ms[o], 5),
                      "ms_median": round(per_op_all[o][len(per_op_all[o]) // 2], 5), "ms_best": round(per_op_all[o][0], 5),
            "gbs": round(gbs, 1),
                      "frac_of_%s_peak" % peak_kind: round(gbs / world / peak, 4),
                      "frac_of_8TBs": round(gbs / world / NOMINAL_HBM_GBS, 4)}
    ops_out["random_sample"]["tokens_per_s"] = round(RS_B * world / (per_op_ms["random_sample"] * 1e-3), 1)
    if rms_scaled is not None:
        rms_scaled["frac_of_measured_peak"] = round(rms_scaled["gbs"] / peak, 4)
        ops_out["rms_norm"]["scaled"] = rms_scaled
    if rope_scaled is not None:
        rope_scaled["frac_of_measured_peak"] = round(rope_scaled["gbs"] / peak, 4)
        ops_out["rope"]["scaled"] = rope_scaled

    line = {
        "metric": "achieved_hbm_gbs_decode_hot_path",
        "value": round(step_bytes * world / (ms_per_step * 1e-3) / 1e9, 1),
        "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f32/f64 arithmetic", "data": "synthetic (seeded, BASELINE.json shapes and distributions)",
        "config": {"workload": "six-operator decode step at BASELINE.json configs: rms_norm[16,2048] rope[4096,32,128] "
                               "swiglu[8192,2x14336] add[8192,4096] causal_softmax[32,512,4096] "
                               "random_sample[64,128256] T0.8 k50 p0.9",
                   "bytes_per_step": step_bytes, "sharding": "rows per GPU fixed (weak), no collective",
                   "l2": "step working set 1.25 GB > 126 MB L2; every operator's buffers were last touched a full step earlier",
                   "random_sample": "batched extension entry, one launch for 64 rows",
                   "launch": ("one step captured in a CUDA graph, replayed K times" if graph is not None
                              else "plain launches on one stream")},
        "ops": ops_out,
        "sample_tokens_per_s": ops_out["random_sample"]["tokens_per_s"],
        "e2e": {"value": round(step_bytes * world / (e2e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms, 3), "numa": numa},
        "gpu_launches": step.launches_per_step * args.steps,
        "clocks": clk,
    }
    if sustained is not None:
        sus_ms = extra["sustained"]
        line["sustained"] = {"value": round(step_bytes * world / (sus_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                             "ms_per_step": round(sus_ms, 4), "steps": sustained[1],
                             "seconds": round(sus_ms * sustained[1] / 1e3, 2), "clocks": sustained[2]}
    line["device_timeouts"] = device_timeouts_after - device_timeouts_before
    if world > 1:
        # strong scaling: the SAME configuration split over the ranks (rows; heads for causal softmax), slowest rank
        split = {}
        for o in ("rope", "swiglu", "add", "causal_softmax"):
            ms = extra["strong." + o]
            split[o] = {"ms_split": round(ms, 5), "ms_one_gpu": round(own_per_op_ms[o], 5),
                        "speedup": round(own_per_op_ms[o] / ms, 2),
                        "gbs": round(ALGO_BYTES[o] / (ms * 1e-3) / 1e9, 1)}
        line["strong_scaling"] = {
            "what": "each BASELINE.json configuration split over %d GPUs (token rows; heads for causal softmax), no "
                    "collective; ms_split = slowest rank; ms_one_gpu = the whole configuration on rank 0's GPU in the "
                    "same run.  RMSNorm [16, 2048] (8 KB per GPU at 8 GPUs) and slices that take under ~10 us are "
                    "launch latency, not bandwidth" % world,
            "ops": split}
        rs = {}
        for mode in SHARDED_MODES:
            rs[mode] = {"ms": round(extra["sharded.%s.ms" % mode], 4), "exchange": sharded[mode].get("exchange"),
                        "ms_graph": round(extra["sharded.%s.ms_graph" % mode], 4) or None,
                        "tokens_per_s": round(RS_B / (extra["sharded.%s.ms" % mode] * 1e-3), 1),
                        "stages_ms": {k.split(".stage.")[1]: round(v, 4) for k, v in extra.items()
                                      if k.startswith("sharded.%s.stage." % mode)}}
            if "graph_error" in sharded[mode]:
                rs[mode]["graph_error"] = sharded[mode]["graph_error"]
            if "same_indices_as_exact" in sharded[mode]:
                rs[mode]["same_indices_as_exact"] = sharded[mode]["same_indices_as_exact"]
        rs["exact"]["what"] = ("64 rows, vocabulary 128256 split over %d GPUs; default mode, index-exact, every rank "
                               "samples %d whole rows.  exchange 'peer_memory' (the default where the ranks can share "
                               "memory over CUDA IPC): the caller's shard is copied into the rank's block, the sampling "
                               "kernel reads the peers' shards and stores the indices to every rank, the results are "
                               "copied out.  exact_all_to_all / exact_all_gather force the NCCL exchanges (all-to-all: %d "
                               "bytes received per rank; all-gather of all shards: %d bytes; then one all-gather of the "
                               "indices)" %
                               (world, RS_B // world, RS_B // world * RS_V * 2 * (world - 1) // world,
                                RS_B * RS_V * 2 * (world - 1) // world))
        rs["exact_peer_memory"]["what"] = ("the same exchange with the logits produced in and the results read from "
                                           "the rank's block (no copies): ONE launch per rank, whose CTAs wait for the "
                                           "peers' flag words, read their %d rows out of the peers' shards over NVLink "
                                           "(plain loads), store the indices to every peer and run the closing flag "
                                           "round; every wait bounded" % (RS_B // world))
        rs["fast"]["what"] = ("local candidate kernel, one NCCL all-gather of %d bytes per rank, finishing kernel; "
                              "denominator correctly rounded instead of sequential" % (RS_B * 1056))
        rs["one_gpu_unsharded_ms"] = round(own_per_op_ms["random_sample"], 4)
        line["random_sample_vocab_sharded"] = rs
    sw_ms = per_op_ms["swiglu"]
    ach = ALGO_BYTES["swiglu"] / (sw_ms * 1e-3) / 1e9
    line["roofline"] = {"kernel": "swiglu_vec8_kernel", "bound": "hbm", "achieved": round(ach, 1), "peak": peak,
                        "peak_kind": "of " + peak_kind, "unit": "GB/s", "frac": round(ach / peak, 4),
                        "traffic": ncu_traffic_bytes("swiglu_vec8_kernel_8192x14336.md")}
    if world == 1 and not args.only:
        # the operators built either side of the step (not part of `value`): each timed alone after the step's runs
        line["next_rows"] = {name: fn(lib, handle, dev, 20, 3) for name, fn in NEXT_ROWS.items()}
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_seconds=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


# ---- the reference CPU backend on the host cores --------------------------------------------
def _cpu_backend():
    """(kind, lib, handle): the reference's own CPU build when it was compiled
    into oracle/_ref, else None (the oracle port is then used)."""
    from operators_b200 import DeviceEnum, create_handle, open_lib
    from oracle import cpu_oracle

    d = cpu_oracle.reference_lib_dir()
    if d is None:
        return "port", None, None
    lib = open_lib(d)
    return "reference", lib, create_handle(lib, DeviceEnum.DEVICE_CPU)


def cpu_step(kind, lib, handle, inputs, threads):
    """One step of the CPU path over `inputs`, rows split over `threads` host
    threads (the reference functions are single-threaded; rows are independent).
    Returns seconds."""
    import numpy as np
    import torch

    from operators_b200 import ops
    from oracle import cpu_oracle

    def chunks(n):
        t = min(threads, n)
        edges = [n * i // t for i in range(t + 1)]
        return [(edges[i], edges[i + 1]) for i in range(t) if edges[i + 1] > edges[i]]

    jobs = []
    x, w = inputs["rms_x"], inputs["rms_w"]
    y = torch.zeros_like(x)
    tt, pos, sin, cos = inputs["rope_t"].clone(), inputs["rope_pos"], inputs["rope_sin"], inputs["rope_cos"]
    gu = inputs["gate_up"]
    c = torch.zeros((gu.shape[0], SWI_DI), dtype=torch.float16)
    a, b = inputs["add_a"], inputs["add_b"]
    s = torch.zeros_like(a)
    att = inputs["att"].clone()
    logits, u = inputs["logits"], inputs["u"]
    res = torch.zeros(logits.shape[0], dtype=torch.int64)

    if kind == "reference":
        for lo, hi in chunks(x.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: ops.rms_norm(lib, handle, y[lo:hi], x[lo:hi], w, 1e-5))
        for lo, hi in chunks(tt.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: ops.rope(lib, handle, tt[lo:hi], pos[lo:hi], sin, cos))
        for lo, hi in chunks(gu.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: ops.swiglu(lib, handle, c[lo:hi], gu[lo:hi, SWI_DI:], gu[lo:hi, :SWI_DI]))
        for lo, hi in chunks(a.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: ops.add(lib, handle, s[lo:hi], a[lo:hi], b[lo:hi]))
        for lo, hi in chunks(att.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: ops.causal_softmax(lib, handle, att[lo:hi]))
        for r in range(logits.shape[0]):
            jobs.append(lambda r=r: ops.random_sample(lib, handle, res[r:r + 1], logits[r], float(u[r]), RS_TOPP,
                                                      RS_TOPK, RS_TEMP))
    else:
        xn, wn, tn = x.numpy(), w.numpy(), tt.numpy()
        for lo, hi in chunks(x.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: cpu_oracle.rms_norm(xn[lo:hi], wn, 1e-5))
        for lo, hi in chunks(tt.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: cpu_oracle.rope(tn[lo:hi], pos.numpy()[lo:hi].astype(np.uint64),
                                                             sin.numpy(), cos.numpy()))
        gn = gu.numpy()
        for lo, hi in chunks(gu.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: cpu_oracle.swiglu(gn[lo:hi, SWI_DI:], gn[lo:hi, :SWI_DI]))
        an, bn = a.numpy(), b.numpy()
        for lo, hi in chunks(a.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: cpu_oracle.add(an[lo:hi], bn[lo:hi]))
        attn = att.numpy()
        for lo, hi in chunks(att.shape[0]):
            jobs.append(lambda lo=lo, hi=hi: cpu_oracle.causal_softmax(attn[lo:hi]))
        ln = logits.numpy()
        for r in range(logits.shape[0]):
            jobs.append(lambda r=r: cpu_oracle.random_sample(ln[r], float(u[r]), RS_TOPP, RS_TOPK, RS_TEMP))

    from concurrent.futures import ThreadPoolExecutor

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as pool:  # ctypes calls release the GIL
        list(pool.map(lambda j: j(), jobs))
    return time.perf_counter() - t0


def _host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_baseline(sample_seconds=20.0):
    """The CPU path on a bounded row sample of the same step (about
    `sample_seconds` of CPU work), all host threads."""
    kind, lib, handle = _cpu_backend()
    threads = _host_threads()
    # one full step costs roughly 7 core-seconds; pick the row fraction for the budget
    fraction = max(1.0 / 64, min(1.0, sample_seconds / 7.0))
    inputs = make_inputs(1000, rows_fraction=fraction)
    cpu_step(kind, lib, handle, inputs, threads)  # untimed: pages and thread pool warm
    reps = 3
    secs = sum(cpu_step(kind, lib, handle, inputs, threads) for _ in range(reps)) / reps
    nbytes = sum(sample_bytes(inputs).values())
    # the reference as shipped is single-threaded: the same step over an eighth of the rows on one thread
    small = make_inputs(1000, rows_fraction=0.125)
    secs1 = cpu_step(kind, lib, handle, small, 1)
    nbytes1 = sum(sample_bytes(small).values())
    return {"value": round(nbytes / secs / 1e9, 3), "unit": "GB/s", "cores": threads, "kind": kind,
            "sample": "mean of %d steps over %.3g of the rows of every operator (%d bytes per step, %.2f s per step on %d "
                      "threads)" % (reps, fraction, nbytes, secs, threads),
            "one_core": {"value": round(nbytes1 / secs1 / 1e9, 3), "unit": "GB/s",
                         "sample": "one step over 0.125 of the rows (%d bytes) in %.2f s on 1 thread" % (nbytes1, secs1)}}


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, lib, handle = _cpu_backend()
    threads = _host_threads()
    # bounded sample: a quarter of the rows of every operator per step
    fraction = 0.25 if threads >= 8 else 1.0 / 16
    inputs = make_inputs(1000, rows_fraction=fraction)
    nbytes = sum(sample_bytes(inputs).values())
    for _ in range(args.warmup):
        cpu_step(kind, lib, handle, inputs, threads)
    secs = [cpu_step(kind, lib, handle, inputs, threads) for _ in range(args.steps)]
    per = sum(secs) / len(secs)
    value = round(nbytes / per / 1e9, 3)
    sample = "each step = %.3g of the rows of every operator (%d algorithmic bytes)" % (fraction, nbytes)
    line = {
        "impl": "reference",
        "metric": "achieved_hbm_gbs_decode_hot_path", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(per * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 storage, f32/f64 arithmetic", "data": "synthetic (seeded, BASELINE.json shapes and distributions)",
        "config": {"workload": "six-operator decode step at BASELINE.json configs (row sample)", "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU leg (profiling runs)")
    ap.add_argument("--sustain-seconds", type=float, default=1.0,
                    help="replay the step for this long after the timed K steps and report it as `sustained`")
    ap.add_argument("--sharded-graph", action="store_true",
                    help="N > 1: also time vocabulary-sharded sampling replayed as one CUDA graph (NCCL calls captured)")
    ap.add_argument("--no-graph", action="store_true", help="time plain launches instead of a CUDA graph of the step")
    ap.add_argument("--only", choices=OPS + list(NEXT_ROWS),
                    help="launch a single operator at its configuration (for ncu captures)")
    ap.add_argument("--select-kernel", action="append", default=[], metavar="FAMILY=VARIANT",
                    help="force a kernel family for this run (infiniopExtSelectKernel), e.g. rope=2; for comparisons")
    ap.add_argument("--tokens", type=int, choices=[SWI_T, 16, 1], help="with --only matmul: this token count only")
    ap.add_argument("--weights", choices=["k_contiguous", "n_contiguous"], help="with --only matmul: this weight layout only")
    ap.add_argument("--new-tokens", type=int, choices=[64, 512, 2048, 4096], help="with --only attention_prefill: this case only")
    ap.add_argument("--cached-tokens", type=int, choices=[0, 8192, 32768], default=0,
                    help="with --only attention_prefill --new-tokens: the case with this many tokens already cached")
    args = ap.parse_args()
    MATMUL_CASE["tokens"], MATMUL_CASE["weights"] = args.tokens, args.weights
    PREFILL_CASE["new_tokens"], PREFILL_CASE["cached_tokens"] = args.new_tokens, args.cached_tokens
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
