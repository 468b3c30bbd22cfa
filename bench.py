#!/usr/bin/env python
"""Benchmark of the B200 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One process per GPU (for N > 1 launch with torch.distributed.run; rank, local
rank and world size come from the environment).  A step is one pass of the
workload over one batch of seeded synthetic input.  W warm-up steps, then exactly
K steps timed with CUDA events on the launching stream between a barrier +
synchronize on both sides; the time is the max over ranks; rank 0 prints ONE
JSON line.

Workloads (default `all`: prefill is the headline line, the others ride along under
"others", each with its own roofline, e2e and cpu_baseline)
  prefill      causal prefill, batch 8, 32 heads, seq 4096, D 128, bf16.  Tensor-bound.
               N > 1: every rank its own (batch, head) units (weak).
  decode       GQA decode, batch 64, 32 q / 8 kv heads, D 128, 8192 cached keys, bf16.
               HBM-bound.  N > 1: every rank its own (batch, kv-head) units (weak).
  segops       segmented wave64 reduce + inclusive-scan sweep over 2^26 elements per
               dtype: reduce {f32,f64,i32,i64} x {sum,max,min}, reduce {f16,bf16} sum
               (fp32 accumulation), scan-sum {f32,f64,i32,i64,f16,bf16}.  HBM-bound.
               N > 1: every rank sweeps its own 2^26-element shard (weak scaling).
  decode_long  the 131072-key decode with the KV sequence split across the ranks and the
               (O, lse) partials exchanged once per step (strong scaling; N = 1 holds the
               whole sequence).  At N > 1 both forms of the exchange are timed.
  runtime      the 22-layer Llama-style decoder: 512-token prompt + 128 greedy tokens,
               2 sequences per GPU.
  fa_steps     the FA2 build-order steps at the reference's validation shape (batch 1,
               8 heads, seq 512, D 64): four steps in fp16, three in fp32.
  wave_api     the device-level wave API in the reference's own terms: LayerNorm / softmax
               rows on the primitives vs the portable shuffle loop, and the register-resident
               reduce loop (elements per second).  Secondary, labelled.

--impl reference times the CPU statement of the same path (the oracle) on the
host cores, on a bounded sample, in the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_peaks():
    """Measured roofline denominators (driver-written file), else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------
# clocks: sampled DURING the timed region through NVML (read-only)
# --------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period: float = 0.0):       # 0: back-to-back NVML queries (each takes about a millisecond)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for b, name in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(name)
            except Exception:
                pass
            if self.period > 0:
                time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------
# workload: segmented reduce / scan sweep
# --------------------------------------------------------------------------------------
class SegopsSweep:
    name = "segops"
    metric = "segmented wave64 reduce+scan sweep throughput (algorithmic bytes)"
    unit = "GB/s"
    dtype = "f32,f64,i32,i64 (+f16,bf16 with f32 accumulation)"
    N = 1 << 26

    KINDS = ["f32", "f64", "i32", "i64", "f16", "bf16"]
    SIZE = {"f32": 4, "f64": 8, "i32": 4, "i64": 8, "f16": 2, "bf16": 2}

    def __init__(self, n=None):
        self.n = n or self.N
        self.cases = []   # (label, fn, kind, op, bytes)
        for kind in ("f32", "f64", "i32", "i64"):
            for op in ("sum", "max", "min"):
                self.cases.append((f"reduce_{op}<{kind}>", "reduce", kind, op, self.n * self.SIZE[kind] + self.n // 64 * self.SIZE[kind]))
        for kind in ("f16", "bf16"):
            self.cases.append((f"reduce_sum<{kind}>", "reduce", kind, "sum", self.n * 2 + self.n // 64 * 4))
        for kind in self.KINDS:
            self.cases.append((f"scan_inclusive_sum<{kind}>", "scan", kind, "sum", 2 * self.n * self.SIZE[kind]))
        self.bytes_per_step = sum(c[4] for c in self.cases)

    def config(self, world):
        return {"workload": "segmented wave64 reduce + inclusive-scan sweep (BASELINE config 2)",
                "elements_per_dtype_per_gpu": self.n, "segment": 64,
                "launches_per_step": len(self.cases),
                "sharding": f"segments x{world}, no collective",
                "l2": "inputs larger than L2; successive launches read different buffers",
                "inputs": "f32/f64 N(0,1); i32/i64 U[-1000,1000]; f16/bf16 N(0,1) rounded; seeded"}

    # host inputs (pinned) -- seeded; rank shifts the seed so shards differ
    def make_host(self, torch, rank, pinned=True):
        import numpy as np
        rng = np.random.default_rng(0xB200 + 2 + 1000 * rank)
        host = {}
        for kind in self.KINDS:
            if kind in ("i32", "i64"):
                a = rng.integers(-1000, 1001, self.n, dtype=np.int32 if kind == "i32" else np.int64)
                t = torch.from_numpy(a)
            else:
                a = rng.standard_normal(self.n, dtype=np.float32)
                t = torch.from_numpy(a)
                if kind == "f64":
                    t = t.double()
                elif kind == "f16":
                    t = t.half()
                elif kind == "bf16":
                    t = t.bfloat16()
            host[kind] = t.pin_memory() if pinned else t
        return host

    def setup(self, torch, pkg, device, rank):
        self.torch, self.pkg = torch, pkg
        self.host = self.make_host(torch, rank)
        self.dev = {k: v.to(device, non_blocking=True) for k, v in self.host.items()}
        self.dev_alt = {k: v.flip(0).contiguous() for k, v in self.dev.items()}     # second buffers for launch_case
        self.out = []
        for label, fn, kind, op, _ in self.cases:
            x = self.dev[kind]
            if fn == "reduce":
                odt = torch.float32 if kind in ("f16", "bf16") else x.dtype
                self.out.append(torch.empty(self.n // 64, dtype=odt, device=device))
            else:
                self.out.append(torch.empty_like(x))
        torch.cuda.synchronize()

    def step(self, events=None):
        """One sweep with inputs resident in HBM.  events: list that receives one
        CUDA event after every launch (plus one before the first)."""
        torch, pkg = self.torch, self.pkg
        for i, (label, fn, kind, op, _) in enumerate(self.cases):
            if fn == "reduce":
                pkg.segreduce(self.dev[kind], op, out=self.out[i])
            else:
                pkg.segscan(self.dev[kind], op, out=self.out[i])
            if events is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                events.append(e)

    def launch_case(self, i, rep):
        """Kernel i alone; successive reps read different input buffers (each larger than L2/2,
        together larger than L2)."""
        label, fn, kind, op, _ = self.cases[i]
        x = (self.dev if rep % 2 == 0 else self.dev_alt)[kind]
        if fn == "reduce":
            self.pkg.segreduce(x, op, out=self.out[i])
        else:
            self.pkg.segscan(x, op, out=self.out[i])

    def setup_e2e(self):
        """The same sweep through the package's host-buffer entry point: one chunk per dtype,
        uploads, kernels and downloads of successive chunks overlapped on three streams."""
        import importlib
        hp = importlib.import_module(self.pkg.__name__ + ".hostpipe")
        jobs = [(kind, fn, op) for (_l, fn, kind, op, _b) in self.cases]
        self.pipe, self.e2e_results = hp.segops_sweep_host(self.pkg, self.host, jobs)

    def step_e2e(self, compute=True):
        self.pipe.run(compute=compute)

    cpu_sample = 1 << 24
    cpu_sample_text = "the same sweep over 2^24 elements per dtype (1/4 of the workload)"

    def e2e_bytes(self):
        return self.pipe.bytes()

    e2e_note = "host-buffer sweep (hostpipe.segops_sweep_host): per-dtype chunks, H2D / kernels / D2H on three streams"

    # CPU statement of the same sweep on a bounded sample
    def cpu_run(self, orc, n, threads, reps=1):
        import numpy as np
        rng = np.random.default_rng(0xB200 + 2)
        f32 = rng.standard_normal(n, dtype=np.float32)
        data = {"f32": f32, "f64": f32.astype(np.float64),
                "i32": rng.integers(-1000, 1001, n, dtype=np.int32), "i64": rng.integers(-1000, 1001, n, dtype=np.int64),
                "f16": orc.f32_to_f16_bits(f32), "bf16": orc.f32_to_bf16_bits(f32)}
        t0 = time.perf_counter()
        for _ in range(reps):
            for label, fn, kind, op, _b in self.cases:
                o = orc.OPS[op]
                if kind in ("f16", "bf16"):
                    if fn == "reduce":
                        orc.shfl_reduce_narrow(o, data[kind], kind == "bf16", threads=threads)
                    else:
                        orc.shfl_scan_narrow(o, data[kind], kind == "bf16", threads=threads)
                elif fn == "reduce":
                    orc.seq_reduce(o, data[kind], threads=threads)
                else:
                    orc.seq_scan(o, data[kind], threads=threads)
        dt = (time.perf_counter() - t0) / reps
        scale = n / self.n
        return self.bytes_per_step * scale / dt / 1e9, dt


# --------------------------------------------------------------------------------------
# workload: GQA decode (BASELINE config 4)
# --------------------------------------------------------------------------------------
class DecodeGQA:
    name = "decode"
    metric = "GQA decode attention throughput (algorithmic K/V/q/o bytes)"
    unit = "GB/s"
    dtype = "bf16 (fp32 softmax and accumulation)"
    B, NQH, NKVH, D, N = 64, 32, 8, 128, 8192

    def __init__(self, n=None):
        if n:
            self.N = n
        self.bytes_per_step = 2 * self.B * self.NKVH * self.N * self.D * 2 + 2 * self.B * self.NQH * self.D * 2
        self.cases = [("decode_mma_kernel (+ combine)", None, None, None, self.bytes_per_step)]

    def config(self, world):
        return {"workload": "GQA decode (BASELINE config 4)", "batch_per_gpu": self.B, "q_heads": self.NQH, "kv_heads": self.NKVH,
                "head_dim": self.D, "kv_len": self.N, "sharding": f"(batch, kv-head) x{world}, no collective",
                "l2": "K/V (2 GiB) larger than L2", "e2e": "q H2D + o D2H every step; the KV cache is resident state",
                "inputs": "q, K, V ~ N(0,1) rounded to bf16, seeded"}

    def setup(self, torch, pkg, device, rank):
        self.torch, self.pkg = torch, pkg
        g = torch.Generator(device=device); g.manual_seed(0xB204 + 1000 * rank)
        self.q = torch.randn(self.B, self.NQH, self.D, device=device, generator=g).bfloat16()
        self.K = torch.randn(self.B, self.NKVH, self.N, self.D, device=device, generator=g).bfloat16()
        self.V = torch.randn(self.B, self.NKVH, self.N, self.D, device=device, generator=g).bfloat16()
        self.o = torch.empty_like(self.q)
        self.ws = pkg.decode_workspace(self.q, self.K)
        self.q_host = self.q.cpu().pin_memory()
        self.o_host = torch.empty(self.o.shape, dtype=self.o.dtype).pin_memory()
        torch.cuda.synchronize()

    def step(self, events=None):
        self.pkg.decode(self.q, self.K, self.V, out=self.o, workspace=self.ws)
        if events is not None:
            e = self.torch.cuda.Event(enable_timing=True); e.record(); events.append(e)

    def step_e2e(self):
        self.q.copy_(self.q_host, non_blocking=True)
        self.step()
        self.o_host.copy_(self.o, non_blocking=True)

    def e2e_bytes(self):
        return self.q_host.numel() * 2, self.o_host.numel() * 2

    def extra_fields(self):
        """The reference's own decode table: batch 1, D 128, GQA 32q / 8kv, fp16, N = 256 .. 8192 keys; us per launch
        (median of 20, one event pair each) next to the reference's MI300X time."""
        torch, pkg = self.torch, self.pkg
        ref_us = {256: 18.1, 512: 32.2, 1024: 60.4, 2048: 118.7, 4096: 384.5, 8192: 803.4}
        out = {}
        for n, r in ref_us.items():
            g = torch.Generator(device=self.q.device); g.manual_seed(0xB204 + n)
            q = torch.randn(1, 32, 128, device=self.q.device, generator=g).half()
            K = torch.randn(1, 8, n, 128, device=self.q.device, generator=g).half()
            V = torch.randn(1, 8, n, 128, device=self.q.device, generator=g).half()
            o = torch.empty_like(q)
            ws = pkg.decode_workspace(q, K)
            for _ in range(3):
                pkg.decode(q, K, V, out=o, workspace=ws)
            ts = []
            for _ in range(20):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); pkg.decode(q, K, V, out=o, workspace=ws); b.record()
                ts.append((a, b))
            torch.cuda.synchronize()
            us = sorted(a.elapsed_time(b) for a, b in ts)[10] * 1e3
            e = {"us_per_call_from_python": round(us, 1), "reference_mi300x_us": r}
            # a launch of this size is shorter than a Python call: the device time is that of 20 calls captured in
            # one CUDA graph and replayed (the reference times a C++ loop of launches)
            try:
                side = torch.cuda.Stream(device=self.q.device)
                side.wait_stream(torch.cuda.current_stream())
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph, stream=side):
                        for _ in range(20):
                            pkg.decode(q, K, V, out=o, workspace=ws)
                    graph.replay()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(side)
                    for _ in range(5):
                        graph.replay()
                    b.record(side)
                b.synchronize()
                e["us"] = round(a.elapsed_time(b) * 1e3 / 100, 2)
                torch.cuda.current_stream().wait_stream(side)
                del graph
            except Exception as ex:                                   # capture not possible: keep the per-call figure
                e["us"] = e["us_per_call_from_python"]; e["graph"] = f"unavailable: {type(ex).__name__}"
            out[f"batch1_gqa32q8kv_d128_n{n}"] = e
        return {"reference_shapes": out}

    def cpu_run(self, orc, n, threads, reps=1):
        """n = sequences of the batch (full kv length)."""
        import numpy as np
        rng = np.random.default_rng(0xB204)
        q = rng.standard_normal((n, self.NQH, self.D), dtype=np.float32)
        K = rng.standard_normal((n, self.NKVH, self.N, self.D), dtype=np.float32)
        V = rng.standard_normal((n, self.NKVH, self.N, self.D), dtype=np.float32)
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.cpu_decode(q, K, V, self.D, self.N, self.NQH, self.NKVH, batch=n, threads=threads)
        dt = (time.perf_counter() - t0) / reps
        return self.bytes_per_step * (n / self.B) / dt / 1e9, dt

    cpu_sample = 8
    cpu_sample_text = "8 of the 64 sequences at full KV length"


# --------------------------------------------------------------------------------------
# workload: causal prefill (BASELINE config 3)
# --------------------------------------------------------------------------------------
class PrefillCausal:
    name = "prefill"
    metric = "FA2 causal prefill attention throughput"
    unit = "TFLOP/s"
    dtype = "bf16 (fp32 softmax and accumulation)"
    B, H, S, D = 8, 32, 4096, 128
    bound = "tensor"

    def __init__(self, n=None):
        if n:
            self.S = n
        # the reference's FLOP convention for causal attention: 2 GEMMs x 2 flops, half the square
        # (research/flash-attention-mi300x/fa_robust.hip:266-268)
        self.flops_per_step = 2.0 * 2.0 * self.B * self.H * self.S * self.S * self.D * 0.5
        self.bytes_per_step = self.flops_per_step        # "units" the generic code divides by time
        self.cases = [("prefill_tc_kernel", None, None, None, self.flops_per_step)]

    def config(self, world):
        return {"workload": "FA2 causal prefill (BASELINE config 3)", "batch_per_gpu": self.B, "heads": self.H, "seq_len": self.S,
                "head_dim": self.D, "causal": True, "sharding": f"(batch, head) x{world}, no collective",
                "flops": "2*2*B*H*S*S*D/2 (the reference's convention)",
                "l2": "Q,K,V,O (4 x 268 MB) larger than L2", "inputs": "Q, K, V ~ N(0,1)*0.5 rounded to bf16, seeded"}

    def setup(self, torch, pkg, device, rank):
        self.torch, self.pkg = torch, pkg
        g = torch.Generator(device=device); g.manual_seed(0xB203 + 1000 * rank)
        shape = (self.B, self.H, self.S, self.D)
        self.Q = (torch.randn(shape, device=device, generator=g) * 0.5).bfloat16()
        self.K = (torch.randn(shape, device=device, generator=g) * 0.5).bfloat16()
        self.V = (torch.randn(shape, device=device, generator=g) * 0.5).bfloat16()
        self.O = torch.empty_like(self.Q)
        self.host = [t.cpu().pin_memory() for t in (self.Q, self.K, self.V)]
        self.O_host = torch.empty(shape, dtype=torch.bfloat16).pin_memory()
        torch.cuda.synchronize()

    def step(self, events=None):
        self.pkg.prefill(self.Q, self.K, self.V, causal=True, out=self.O)
        if events is not None:
            e = self.torch.cuda.Event(enable_timing=True); e.record(); events.append(e)

    def setup_e2e(self):
        import importlib
        hp = importlib.import_module(self.pkg.__name__ + ".hostpipe")
        self.pipe, self.O_host = hp.prefill_host(self.pkg, self.host[0], self.host[1], self.host[2], causal=True, Oh=self.O_host)

    def step_e2e(self, compute=True):
        self.pipe.run(compute=compute)

    def e2e_bytes(self):
        return self.pipe.bytes()

    e2e_note = "host-buffer prefill (hostpipe.prefill_host): one chunk per sequence, H2D / kernel / D2H on three streams"

    def extra_fields(self):
        """The same kernel off the headline shape (device-resident, 10 launches each after 3 warm-ups): non-causal,
        twice the sequence length, and head dimension 64 (the runtime's shape)."""
        torch, pkg = self.torch, self.pkg
        out = {}
        for label, (B, H, S, D, causal) in (("non_causal_s4096_d128", (8, 32, 4096, 128, False)),
                                             ("causal_s8192_d128", (4, 32, 8192, 128, True)),
                                             ("causal_s4096_d64", (8, 32, 4096, 64, True)),
                                             ("causal_s512_d64_gqa_32q_4kv", (16, 32, 512, 64, True))):
            g = torch.Generator(device=self.Q.device); g.manual_seed(0xB203 + S + D)
            hkv = 4 if "gqa" in label else H
            q = (torch.randn(B, H, S, D, device=self.Q.device, generator=g) * 0.5).bfloat16()
            k = (torch.randn(B, hkv, S, D, device=self.Q.device, generator=g) * 0.5).bfloat16()
            v = (torch.randn(B, hkv, S, D, device=self.Q.device, generator=g) * 0.5).bfloat16()
            o = torch.empty_like(q)
            for _ in range(3):
                pkg.prefill(q, k, v, causal=causal, out=o)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                pkg.prefill(q, k, v, causal=causal, out=o)
            b.record(); b.synchronize()
            ms = a.elapsed_time(b) / 10
            out[label] = {"ms": round(ms, 4), "TFLOP/s": round(4.0 * B * H * S * S * D * (0.5 if causal else 1.0) / ms / 1e9, 1)}
            del q, k, v, o
        # the shapes of the reference's own prefill tables (batch 1, D 128, fp16): MHA 8 heads non-causal and GQA 32q/8kv
        # causal at 512 .. 4096 tokens; us per launch (median of 20, one event pair each), next to the reference's MI300X time
        ref_us = {("mha8_full", 512): 103.7, ("mha8_full", 4096): 6015.1,
                  ("gqa32q8kv_causal", 512): 389.5, ("gqa32q8kv_causal", 1024): 1051.9, ("gqa32q8kv_causal", 2048): 3407.9, ("gqa32q8kv_causal", 4096): 11829.4}
        ref = {}
        for kind, H, hkv, causal in (("mha8_full", 8, 8, False), ("gqa32q8kv_causal", 32, 8, True)):
            for S in (512, 1024, 2048, 4096):
                g = torch.Generator(device=self.Q.device); g.manual_seed(0xB203 + S + H)
                q = (torch.randn(1, H, S, 128, device=self.Q.device, generator=g) * 0.5).half()
                k = (torch.randn(1, hkv, S, 128, device=self.Q.device, generator=g) * 0.5).half()
                v = (torch.randn(1, hkv, S, 128, device=self.Q.device, generator=g) * 0.5).half()
                o = torch.empty_like(q)
                for _ in range(3):
                    pkg.prefill(q, k, v, causal=causal, out=o)
                ts = []
                for _ in range(20):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(); pkg.prefill(q, k, v, causal=causal, out=o); b.record()
                    ts.append((a, b))
                torch.cuda.synchronize()
                us = sorted(a.elapsed_time(b) for a, b in ts)[10] * 1e3
                e = {"us": round(us, 1), "TFLOP/s": round(4.0 * H * S * S * 128 * (0.5 if causal else 1.0) / us / 1e6, 1)}
                if (kind, S) in ref_us:
                    e["reference_mi300x_us"] = ref_us[(kind, S)]
                ref[f"{kind}_s{S}"] = e
        return {"other_shapes": out, "reference_shapes": ref}

    def cpu_run(self, orc, n, threads, reps=1):
        """n = (batch, head) units at full sequence length."""
        import numpy as np
        rng = np.random.default_rng(0xB203)
        q = (rng.standard_normal((n, self.S, self.D), dtype=np.float32) * 0.5)
        k = (rng.standard_normal((n, self.S, self.D), dtype=np.float32) * 0.5)
        v = (rng.standard_normal((n, self.S, self.D), dtype=np.float32) * 0.5)
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.cpu_prefill(q, k, v, self.D, self.S, self.S, n, n, 1, 1, threads=threads)
        dt = (time.perf_counter() - t0) / reps
        return self.flops_per_step * (n / (self.B * self.H)) / dt / 1e12, dt

    cpu_sample = 16
    cpu_sample_text = "16 of the 256 (batch, head) units at full sequence length"


# --------------------------------------------------------------------------------------
# workload: long-context decode, KV sequence sharded across the GPUs (strong scaling)
# --------------------------------------------------------------------------------------
class DecodeLong:
    name = "decode_long"
    metric = "long-context GQA decode attention throughput (algorithmic K/V/q/o bytes)"
    unit = "GB/s"
    dtype = "bf16 (fp32 softmax and accumulation)"
    scaling = "strong"
    B, NQH, NKVH, D, N = 64, 32, 8, 128, 131072
    exchange = "auto"                     # --exchange: peer stores fused into the kernels, or NCCL all-gather
    used_exchange = "none"

    def __init__(self, n=None):
        if n:
            self.N = n
        self.total_bytes = 2 * self.B * self.NKVH * self.N * self.D * 2 + 2 * self.B * self.NQH * self.D * 2
        self.cases = [("decode_mma_kernel + combine (+ all-gather, lse merge)", None, None, None, self.total_bytes)]

    def config(self, world):
        return {"workload": "long-context GQA decode (BASELINE config 4, 131072-token variant)", "batch": self.B,
                "q_heads": self.NQH, "kv_heads": self.NKVH, "head_dim": self.D, "kv_len": self.N,
                "sharding": (f"KV sequence in {world} contiguous chunks; (O, lse) ({self.B * self.NQH * (self.D + 1) * 4} B per "
                             f"rank) exchanged by " + ("peer stores from the combine kernel + flag wait in the merge kernel"
                                                       if self.used_exchange == "peer" else "one NCCL all-gather")
                             + ", local lse merge") if world > 1
                            else "single GPU holds the whole KV sequence; no collective",
                "exchange": self.used_exchange,
                "l2": "K/V shard larger than L2", "e2e": "q H2D + o D2H every step; the KV cache is resident state",
                "inputs": "q, K, V ~ N(0,1) rounded to bf16, seeded"}

    def setup(self, torch, pkg, device, rank):
        import torch.distributed as dist
        import importlib
        sharding = importlib.import_module(pkg.__name__ + ".sharding")
        self.torch, self.pkg = torch, pkg
        world = dist.get_world_size() if dist.is_initialized() else 1
        self.world = world
        self.bytes_per_step = self.total_bytes / world        # the generic code multiplies by world
        self.off, self.len = sharding.kv_shard(self.N, rank, world)
        g = torch.Generator(device=device); g.manual_seed(0xB214)          # same q on every rank
        self.q = torch.randn(self.B, self.NQH, self.D, device=device, generator=g).bfloat16()
        g.manual_seed(0xB214 + 1 + rank)
        self.K = torch.empty(self.B, self.NKVH, max(self.len, 1), self.D, device=device, dtype=torch.bfloat16)
        self.V = torch.empty_like(self.K)
        for b in range(self.B):                                            # per sequence: bounds the fp32 temporaries
            self.K[b] = torch.randn(self.K.shape[1:], device=device, generator=g).bfloat16()
            self.V[b] = torch.randn(self.K.shape[1:], device=device, generator=g).bfloat16()
        self.dec = sharding.LongContextDecoder(pkg, dist if world > 1 else None, self.B, self.NQH, self.D,
                                               torch.bfloat16, device, exchange=self.exchange)
        self.used_exchange = self.dec.exchange
        self.q_host = self.q.cpu().pin_memory()
        self.o_host = torch.empty(self.q.shape, dtype=torch.bfloat16).pin_memory()
        torch.cuda.synchronize()

    def step(self, events=None):
        self.dec.step(self.q, self.K, self.V, n_keys=self.len)
        if events is not None:
            e = self.torch.cuda.Event(enable_timing=True); e.record(); events.append(e)

    def step_e2e(self):
        self.q.copy_(self.q_host, non_blocking=True)
        self.step()
        self.o_host.copy_(self.dec.out, non_blocking=True)

    def time_other_exchange(self, steps, barrier, max_over_ranks):
        """N > 1: the same steps with the OTHER form of the (O, lse) exchange (NCCL all-gather when the timed
        region used peer stores, and the reverse), so that one run records both.  Returns (name, ms per step)."""
        import torch.distributed as dist
        import importlib
        torch = self.torch
        if self.world == 1:
            return None
        other = "nccl" if self.used_exchange == "peer" else "peer"
        sharding = importlib.import_module(self.pkg.__name__ + ".sharding")
        try:
            dec = sharding.LongContextDecoder(self.pkg, dist, self.B, self.NQH, self.D, torch.bfloat16, self.q.device, exchange=other)
        except Exception as exc:                                  # no symmetric memory on this box: only NCCL exists
            return {"exchange": other, "unavailable": str(exc)[:120]}
        for _ in range(3):
            dec.step(self.q, self.K, self.V, n_keys=self.len)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            dec.step(self.q, self.K, self.V, n_keys=self.len)
        b.record()
        barrier()
        ms = max_over_ranks(a.elapsed_time(b)) / steps
        dec.check()
        same = bool(torch.equal(dec.out, self.dec.out))
        return {"exchange": other, "ms_per_step": ms, "GB/s": self.total_bytes / (ms * 1e-3) / 1e9, "same_bits_as_timed_exchange": same}

    def parity(self):
        """Outside the timed region: rank 0's output for two sampled sequences against a single-launch decode over
        the whole KV sequence of those sequences, gathered from the ranks' shards -- what a single GPU would have
        computed.  The only check the concurrent multi-GPU exchange can get (max |delta|, bf16 outputs)."""
        import torch.distributed as dist
        torch = self.torch
        seqs = [0, self.B - 1]
        if self.world == 1:
            return None
        rank = dist.get_rank()
        Ks = [torch.empty((len(seqs),) + tuple(self.K.shape[1:]), dtype=self.K.dtype, device=self.K.device) for _ in range(self.world)]
        Vs = [torch.empty_like(Ks[0]) for _ in range(self.world)]
        dist.all_gather(Ks, self.K[seqs].contiguous())
        dist.all_gather(Vs, self.V[seqs].contiguous())
        out = None
        if rank == 0:
            Kf, Vf = torch.cat(Ks, dim=2)[:, :, :self.N].contiguous(), torch.cat(Vs, dim=2)[:, :, :self.N].contiguous()
            ref = self.pkg.decode(self.q[seqs].contiguous(), Kf, Vf)
            out = float((ref.float() - self.dec.out[seqs].float()).abs().max().item())
        del Ks, Vs
        return out

    def e2e_bytes(self):
        return self.q_host.numel() * 2, self.o_host.numel() * 2

    def cpu_run(self, orc, n, threads, reps=1):
        """n = sequences; KV length 8192 (1/16 of the workload's) to bound host memory and time."""
        import numpy as np
        N = 8192
        rng = np.random.default_rng(0xB214)
        q = rng.standard_normal((n, self.NQH, self.D), dtype=np.float32)
        K = rng.standard_normal((n, self.NKVH, N, self.D), dtype=np.float32)
        V = rng.standard_normal((n, self.NKVH, N, self.D), dtype=np.float32)
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.cpu_decode(q, K, V, self.D, N, self.NQH, self.NKVH, batch=n, threads=threads)
        dt = (time.perf_counter() - t0) / reps
        return (2 * n * self.NKVH * N * self.D * 2 + 2 * n * self.NQH * self.D * 2) / dt / 1e9, dt

    cpu_sample = 8
    cpu_sample_text = "8 sequences x 8192 keys (1/128 of the workload's K/V bytes)"


# --------------------------------------------------------------------------------------
# workload: the small Llama-style decoder in the runtime (BASELINE config 5)
# --------------------------------------------------------------------------------------
class RuntimeLlama:
    name = "runtime"
    metric = "greedy generation throughput of the runtime (generated tokens/s; prompt 512 + 128 new tokens)"
    unit = "tokens/s"
    dtype = "bf16 weights and activations, fp32 hidden state and accumulation"
    CFG = dict(n_layers=22, hidden=2048, n_heads=32, n_kv_heads=4, head_dim=64, ffn_dim=5632, vocab_size=32000, rope_theta=10000.0)
    B, T, NEW = 2, 512, 128                    # 16 sequences over 8 GPUs = 2 per GPU

    def __init__(self, n=None):
        if n:
            self.NEW = n
        self.bytes_per_step = float(self.B * self.NEW)          # "units" per step = generated tokens
        self.cases = [("generate (prefill 512 + decode)", None, None, None, self.bytes_per_step)]
        c = self.CFG
        qd, kvd = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
        per_layer = (qd + 2 * kvd) * c["hidden"] + c["hidden"] * qd + 3 * c["ffn_dim"] * c["hidden"]
        self.weight_bytes = 2 * (c["n_layers"] * per_layer + c["vocab_size"] * c["hidden"])   # read every decode step

    def config(self, world):
        return {"workload": "small Llama-style decoder in the runtime (BASELINE config 5)", **self.CFG,
                "batch_per_gpu": self.B, "prompt_tokens": self.T, "new_tokens": self.NEW,
                "sharding": f"sequences x{world} (2 per GPU), weights replicated, no collective",
                "weights": "random-init bf16 ~ N(0, 0.02), norm weights 1 (no checkpoint available offline)",
                "inputs": "uniform random token ids, seeded"}

    def setup(self, torch, pkg, device, rank):
        import numpy as np
        self.torch, self.pkg = torch, pkg
        c = self.CFG
        g = torch.Generator(device=device); g.manual_seed(0xB205)        # the same model on every rank
        H, F, D = c["hidden"], c["ffn_dim"], c["head_dim"]
        qd, kvd = c["n_heads"] * D, c["n_kv_heads"] * D

        def w(*shape):
            return (torch.randn(shape, device=device, generator=g) * 0.02).bfloat16()

        ones = torch.ones(H, device=device, dtype=torch.bfloat16)
        layers = [{"Wq": w(qd, H), "Wk": w(kvd, H), "Wv": w(kvd, H), "Wo": w(H, qd), "Wgate": w(F, H), "Wup": w(F, H),
                   "Wdown": w(H, F), "norm_attn": ones, "norm_mlp": ones} for _ in range(c["n_layers"])]
        weights = {"embed_tokens": w(c["vocab_size"], H), "lm_head": w(c["vocab_size"], H), "final_norm": ones, "layers": layers}
        self.sess = pkg.Session(c, weights, self.T + self.NEW, self.B)
        self.ids = np.random.default_rng(0xB205 + rank).integers(0, c["vocab_size"], (self.B, self.T)).astype(np.int32)
        self.timings = []
        torch.cuda.synchronize()

    def step(self, events=None):
        toks, tm = self.sess.generate(self.ids, self.NEW)
        self.timings.append(tm)
        if events is not None:
            e = self.torch.cuda.Event(enable_timing=True); e.record(); events.append(e)

    step_e2e = step                               # generate() takes host ids and returns host tokens

    def e2e_bytes(self):
        return self.ids.nbytes, self.B * self.NEW * 4

    def extra(self):
        import statistics as st
        tt = [t[0] for t in self.timings[-5:]]; dd = [t[1] for t in self.timings[-5:]]
        ms_tok = st.median(dd) / max(1, self.NEW - 1)
        kv_bytes = 2 * self.CFG["n_layers"] * self.B * self.CFG["n_kv_heads"] * (self.T + self.NEW // 2) * self.CFG["head_dim"] * 2
        return {"ttft_ms": st.median(tt), "decode_ms_per_token": ms_tok,
                "decode_step_bytes": self.weight_bytes + kv_bytes,
                "decode_hbm_GBs": (self.weight_bytes + kv_bytes) / (ms_tok * 1e-3) / 1e9,
                "gemm_calls_total": self.sess.gemm_calls}

    def cpu_run(self, orc, n, threads, reps=1):
        """n = new tokens; one sequence, prompt 64 (bounded: the CPU statement needs seconds per prompt token block).
        One random layer's matrices serve all 22 layers: the arithmetic per token is the full model's, and drawing
        1.1e9 normals on the host would cost more than the run it feeds."""
        import numpy as np
        from oracle import runtime_ref as rr
        if not hasattr(self, "_cpu_w"):
            one = rr.make_weights(dict(self.CFG, n_layers=1), seed=5, kind="bf16", std=0.02)
            one["layers"] = one["layers"] * self.CFG["n_layers"]
            self._cpu_w = one
        ids = np.random.default_rng(1).integers(0, self.CFG["vocab_size"], (1, 64))
        t0 = time.perf_counter()
        for _ in range(reps):
            rr.RefSession(self.CFG, self._cpu_w, 64 + n, 1, "bf16").generate(ids, n)
        dt = (time.perf_counter() - t0) / reps
        return n / dt, dt

    cpu_sample = 8
    cpu_sample_text = "1 sequence, prompt 64 tokens + 8 new tokens (numpy restatement of the reference Session)"


# --------------------------------------------------------------------------------------
# workload: the FA2 build-order steps at the reference's validation shape (BASELINE config 1)
# --------------------------------------------------------------------------------------
class FaSteps:
    name = "fa_steps"
    metric = "FA2 build-order steps at the validation shape (batch 1, 8 heads, seq 512, D 64): aggregate throughput of the 7 kernels"
    unit = "TFLOP/s"
    dtype = "fp16 and fp32 I/O (fp32 softmax and accumulation)"
    bound = "tensor"
    B, H, S, D = 1, 8, 512, 64
    FLOPS = 4.0 * 1 * 8 * 512 * 512 * 64                         # 536 870 912, the reference's count (fa_naive.hip:336-337)

    def __init__(self, n=None):
        self.cases = [(f"fa_{st}<{dt}>", st, dt, None, self.FLOPS)
                      for dt, steps in (("f16", ("naive", "dpp", "dme", "mfma2")), ("f32", ("naive", "dpp", "dme"))) for st in steps]
        self.flops_per_step = self.FLOPS * len(self.cases)
        self.bytes_per_step = self.flops_per_step

    def config(self, world):
        return {"workload": "FA2 forward steps naive/dpp/dme/mfma2 (BASELINE config 1)", "batch": self.B, "heads": self.H, "seq_len": self.S,
                "head_dim": self.D, "causal": False, "tiles": "Br 16, Bc 64", "launches_per_step": len(self.cases),
                "sharding": f"replicas x{world}, no collective", "flops": "4*B*H*S*S*D per kernel (the reference's convention)",
                "l2": "working set 4 MiB (smaller than L2 by the config's definition): a 256 MB buffer is written between timed launches",
                "protocol": "per kernel: 20 warm-up + 200 timed launches, one event pair per launch, L2 flushed in between; median and p99",
                "inputs": "fp16: N(0,0.5) rounded, seeded; fp32: uniform[-1,1], seeded"}

    def setup(self, torch, pkg, device, rank):
        self.torch, self.pkg = torch, pkg
        g = torch.Generator(device=device); g.manual_seed(0xB201)
        shape = (self.B, self.H, self.S, self.D)
        self.x16 = [(torch.randn(shape, device=device, generator=g) * 0.5).half() for _ in range(3)]
        self.x32 = [torch.rand(shape, device=device, generator=g) * 2 - 1 for _ in range(3)]
        self.o16, self.o32 = torch.empty_like(self.x16[0]), torch.empty_like(self.x32[0])
        self.h32 = [t.cpu().pin_memory() for t in self.x32]
        self.oh = torch.empty(shape, dtype=torch.float32).pin_memory()
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        torch.cuda.synchronize()

    def launch(self, i):
        _l, st, dt, _o, _f = self.cases[i]
        if dt == "f16":
            self.pkg.fa_step(st, *self.x16, out=self.o16)
        else:
            self.pkg.fa_step(st, *self.x32, out=self.o32)

    def step(self, events=None):
        for i in range(len(self.cases)):
            self.launch(i)
            if events is not None:
                e = self.torch.cuda.Event(enable_timing=True); e.record(); events.append(e)

    def step_e2e(self):
        """fp32 Q, K, V from pinned host memory, the three fp32 steps, O back."""
        for d, h in zip(self.x32, self.h32):
            d.copy_(h, non_blocking=True)
        for i, c in enumerate(self.cases):
            if c[2] == "f32":
                self.launch(i)
        self.oh.copy_(self.o32, non_blocking=True)

    e2e_units = 3 * FLOPS

    def e2e_bytes(self):
        return 3 * self.x32[0].numel() * 4, self.o32.numel() * 4

    def per_kernel(self):
        """The reference's protocol per kernel (research/wave-primitives/benchmarks/bench_common.hpp:86-119):
        20 warm-up + 200 timed launches; here each timed launch has its own event pair and L2 is flushed before it."""
        torch = self.torch
        out = []
        for i, c in enumerate(self.cases):
            for _ in range(20):
                self.launch(i)
            ts = []
            for _ in range(200):
                self.flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); self.launch(i); b.record()
                ts.append((a, b))
            torch.cuda.synchronize()
            us = sorted(a.elapsed_time(b) * 1e3 for a, b in ts)
            med, p99 = us[len(us) // 2], us[int(len(us) * 0.99) - 1]
            out.append({"kernel": c[0], "us": round(med, 2), "us_p99": round(p99, 2), "TFLOP/s": round(self.FLOPS / (med * 1e-6) / 1e12, 3)})
        return out

    def cpu_run(self, orc, n, threads, reps=1):
        import numpy as np
        rng = np.random.default_rng(0xB201)
        q, k, v = (rng.uniform(-1, 1, (self.B, self.H, self.S, self.D)).astype(np.float32) for _ in range(3))
        t0 = time.perf_counter()
        for _ in range(reps * n):
            orc.cpu_prefill(q, k, v, self.D, self.S, self.S, self.H, self.H, self.B, 0, threads=threads)
        dt = (time.perf_counter() - t0) / (reps * n)
        return self.FLOPS / dt / 1e12, dt

    cpu_sample = 8
    cpu_sample_text = "the full shape (8 heads over the host threads), 8 passes"


# --------------------------------------------------------------------------------------
# workload: the device-level wave API in the reference's own terms (secondary, labelled)
# --------------------------------------------------------------------------------------
class WaveApi:
    name = "wave_api"
    metric = "LayerNorm + softmax rows on the wave primitives (one warp per row; algorithmic bytes), with the register-resident reduce loop as context"
    unit = "GB/s"
    dtype = "f32 (loop: f32, f64, i32)"
    BYTES = 65536 * 512 * 4                                          # one operand; rows x cols = 2^25 floats at either width

    def __init__(self, n=None):
        self.cases = [(f"{which}<{cols} cols, {backend}>", which, cols, backend, 2 * self.BYTES)
                      for which in ("layernorm", "softmax") for cols in (64, 512) for backend in ("primitives", "portable")]
        self.bytes_per_step = sum(c[4] for c in self.cases)

    def config(self, world):
        return {"workload": "device-level wave API: LayerNorm / softmax rows (bench_layernorm.hip, bench_softmax.hip of the reference) "
                            "and its register-resident reduce loop (bench_reduce_dpp_types.hip)",
                "rows": {"64": self.BYTES // 256, "512": self.BYTES // 2048}, "launches_per_step": len(self.cases),
                "sharding": f"replicas x{world}, no collective",
                "l2": "a 256 MB buffer is written between timed launches of the per-kernel timing; in/out are 134 MB each",
                "loop": "4736 waves x 64 values x 4096 repetitions per launch, no memory traffic inside the loop; Gelem/s",
                "context": "the reference quotes its primitives in these terms (elements per second of the reduce loop on MI300X); "
                           "an HBM roofline does not apply to the loop",
                "inputs": "N(0,1)*3, seeded"}

    def setup(self, torch, pkg, device, rank):
        self.torch, self.pkg = torch, pkg
        g = torch.Generator(device=device); g.manual_seed(0xB206)
        n = self.BYTES // 4
        self.x = {64: torch.randn(n // 64, 64, device=device, generator=g) * 3, 512: torch.randn(n // 512, 512, device=device, generator=g) * 3}
        self.gb = {c: (torch.randn(c, device=device, generator=g), torch.randn(c, device=device, generator=g)) for c in (64, 512)}
        self.out = {c: torch.empty_like(self.x[c]) for c in (64, 512)}
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        self.xh = self.x[512].cpu().pin_memory()
        self.oh = torch.empty(self.x[512].shape, dtype=torch.float32).pin_memory()
        torch.cuda.synchronize()

    def launch(self, i):
        _l, which, cols, backend, _b = self.cases[i]
        g, b = self.gb[cols]
        self.pkg.row_op(which, self.x[cols], g, b, backend, out=self.out[cols])

    def step(self, events=None):
        for i in range(len(self.cases)):
            self.launch(i)

    def step_e2e(self):
        self.x[512].copy_(self.xh, non_blocking=True)
        self.launch(2)                                              # layernorm, 512 columns, primitives
        self.oh.copy_(self.out[512], non_blocking=True)

    e2e_units = 2 * BYTES

    def e2e_bytes(self):
        return self.BYTES, self.BYTES

    def per_kernel(self):
        torch = self.torch
        res = []
        for i, c in enumerate(self.cases):
            for _ in range(5):
                self.launch(i)
            ts = []
            for _ in range(30):
                self.flush.fill_(1)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); self.launch(i); b.record()
                ts.append((a, b))
            torch.cuda.synchronize()
            us = sorted(a.elapsed_time(b) * 1e3 for a, b in ts)[len(ts) // 2]
            res.append({"kernel": c[0], "us": round(us, 2), "bytes": c[4], "GB/s": round(c[4] / (us * 1e-6) / 1e9, 1)})
        return res

    def extra_fields(self):
        """The reduce loop, primitives against the portable shuffle loop: Gelem/s (median of 20 launches)."""
        torch, pkg = self.torch, self.pkg
        waves, reps = 4736, 4096
        out = {}
        for dt, name in ((torch.float32, "f32"), (torch.int32, "i32"), (torch.float64, "f64")):
            x = (torch.arange(64 * waves, device=self.x[64].device) % 64).to(dt)
            o = torch.empty(waves, dtype=dt, device=x.device)
            for op in ("sum", "max"):
                for backend in ("primitives", "portable"):
                    for _ in range(3):
                        pkg.wave_reduce_loop(x, op, reps, backend, out=o)
                    ts = []
                    for _ in range(20):
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record(); pkg.wave_reduce_loop(x, op, reps, backend, out=o); b.record()
                        ts.append((a, b))
                    torch.cuda.synchronize()
                    ms = sorted(a.elapsed_time(b) for a, b in ts)[10]
                    out[f"reduce_{op}<{name}> {backend}"] = round(64.0 * waves * reps / (ms * 1e-3) / 1e9, 1)
        for dt, name in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
            x = (torch.arange(64 * waves, device=self.x[64].device) % 7).to(dt)
            o = torch.empty(waves, dtype=dt, device=x.device)
            for backend, label in (("primitives", "fp32 accumulation (primitives)"), ("portable", "16-bit accumulation (portable)")):
                for _ in range(3):
                    pkg.wave_reduce_loop(x, "sum", reps, backend, out=o)
                ts = []
                for _ in range(20):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(); pkg.wave_reduce_loop(x, "sum", reps, backend, out=o); b.record()
                    ts.append((a, b))
                torch.cuda.synchronize()
                ms = sorted(a.elapsed_time(b) for a, b in ts)[10]
                out[f"reduce_sum<{name}> {label}"] = round(64.0 * waves * reps / (ms * 1e-3) / 1e9, 1)
        scan = {}
        for dt, name in ((torch.float32, "f32"), (torch.int32, "i32"), (torch.float64, "f64")):
            x = ((torch.arange(64 * waves, device=self.x[64].device) % 3) - 1).to(dt)
            o = torch.empty_like(x)
            for backend in ("primitives", "portable"):
                for _ in range(3):
                    pkg.wave_scan_loop(x, reps, backend, out=o)
                ts = []
                for _ in range(20):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(); pkg.wave_scan_loop(x, reps, backend, out=o); b.record()
                    ts.append((a, b))
                torch.cuda.synchronize()
                ms = sorted(a.elapsed_time(b) for a, b in ts)[10]
                scan[f"scan_inclusive_sum<{name}> {backend}"] = round(64.0 * waves * reps / (ms * 1e-3) / 1e9, 1)
        return {"wave_reduce_loop_Gelem_per_s": out, "wave_scan_loop_Gelem_per_s": scan}

    def cpu_run(self, orc, n, threads, reps=1):
        """n = thousands of rows of 512 columns: numpy LayerNorm + softmax (the CPU statement of the two row kernels)."""
        import numpy as np
        x = (np.random.default_rng(6).standard_normal((n * 1024, 512)) * 3).astype(np.float32)
        t0 = time.perf_counter()
        for _ in range(reps):
            m = x.mean(axis=1, keepdims=True); v = ((x - m) ** 2).mean(axis=1, keepdims=True)
            _ = (x - m) / np.sqrt(v + 1e-5)
            e = np.exp(x - x.max(axis=1, keepdims=True)); _ = e / e.sum(axis=1, keepdims=True)
        dt = (time.perf_counter() - t0) / reps
        return 2 * 2 * x.nbytes / dt / 1e9, dt

    cpu_sample = 16
    cpu_sample_text = "16384 rows of 512 columns, LayerNorm + softmax in numpy (one thread)"


WORKLOADS = {"wave_api": WaveApi, "fa_steps": FaSteps, "segops": SegopsSweep, "decode": DecodeGQA, "prefill": PrefillCausal, "decode_long": DecodeLong,
             "runtime": RuntimeLlama}
ALL_ORDER = ["prefill", "decode", "segops", "decode_long", "runtime", "fa_steps", "wave_api"]   # `--workload all`: the first is the headline


def make_workload(name, elements=None):
    return WORKLOADS[name](elements) if elements else WORKLOADS[name]()


# --------------------------------------------------------------------------------------
def load_traffic():
    """Measured DRAM traffic per launch of the dominant kernels: a small tracked data file kept beside the
    profiler summaries it was read from (each entry names its summary and how it scales)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except OSError:
        return {}


def traffic_for(label, units_bytes, table):
    """Bytes of DRAM traffic per launch for a kernel label, or None when no capture covers it."""
    try:
        if label.startswith("reduce_") and "f16" not in label and "bf16" not in label:
            t = table["segreduce"]
            n_in = units_bytes * 64 / 65                          # units = n*size + n/64*size
            return int(n_in * t["read_factor"] + (units_bytes - n_in) * t["result_factor"])
        if label.startswith("scan_inclusive_sum<f16") or label.startswith("scan_inclusive_sum<bf16"):
            return int(table["segscan_16bit"]["bytes_at_2p26"] * units_bytes / (2 * (1 << 26) * 2))
        if label.startswith("scan_"):
            t = table["segscan"]
            return int(units_bytes / 2 * (t["read_factor"] + t["write_factor"]))
        if label.startswith("decode_mma_kernel"):
            return int(table["decode_mma_kernel"]["bytes"]) if units_bytes == 2148532224 else None
        if label.startswith("prefill_tc_kernel"):
            return int(table["prefill_tc_kernel"]["bytes"])
    except (KeyError, TypeError):
        pass
    return None


def cpu_line(wl, orc, steps, budget_s=120.0):
    """The CPU statement of the workload (oracle) on the host cores: median over `steps`
    runs of a bounded sample."""
    threads = orc.hardware_threads()
    wl.cpu_run(orc, max(1, wl.cpu_sample // 8), threads)
    vals, t_all = [], time.perf_counter()
    for _ in range(max(1, steps)):
        vals.append(wl.cpu_run(orc, wl.cpu_sample, threads))
        if time.perf_counter() - t_all > budget_s:
            break
    v = statistics.median(x[0] for x in vals)
    dt = statistics.median(x[1] for x in vals)
    return v, dt, len(vals), threads


def reference_arm(args, names, rank, world, emit):
    """`--impl reference`: the CPU statement of the path on the host cores; rank 0 only."""
    if rank != 0:
        return
    import oracle as orc
    lines = []
    for name in names:
        wl = make_workload(name, args.elements)
        v, dt, n, threads = cpu_line(wl, orc, min(args.steps, 5), budget_s=100.0 / len(names))
        lines.append({"impl": "reference", "metric": wl.metric, "value": v, "unit": wl.unit, "n_gpus": args.gpus,
                      "steps": n, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                      "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None, "dtype": wl.dtype,
                      "data": "synthetic (seeded)", "config": wl.config(world),
                      "cpu_baseline": {"value": v, "unit": wl.unit, "cores": threads, "kind": "port",
                                       "sample": f"{wl.cpu_sample_text} per step; independent units split over {threads} host threads"},
                      "e2e": {"value": v, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    line = lines[0]
    if len(lines) > 1:
        line["others"] = lines[1:]
    emit(line)


def measure(wl, args, ctx):
    """W warm-up steps, K timed steps (device-resident), the end-to-end run, the CPU baseline.
    Returns the JSON-ready dict (on every rank; rank 0 prints)."""
    torch, dist, pkg = ctx["torch"], ctx["dist"], ctx["pkg"]
    device, rank, world, local_rank = ctx["device"], ctx["rank"], ctx["world"], ctx["local_rank"]
    peaks, traffic = ctx["peaks"], ctx["traffic"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    wl.setup(torch, pkg, device, rank)
    steps = args.steps if wl.name != "runtime" else max(2, min(args.steps, 5))     # a runtime step is a whole generation
    warm = max(args.warmup, 3) if wl.name != "runtime" else 3
    for _ in range(warm):
        wl.step()
    barrier()

    # ---- device-resident timing: K steps between two events -----------------------------
    launches0 = pkg.launch_count()
    with ClockSampler(local_rank) as clk:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            wl.step()
        t1.record()
        barrier()
    launches = pkg.launch_count() - launches0
    my_ms = t0.elapsed_time(t1)
    ms_per_step = max_over_ranks(my_ms) / steps
    ms_by_rank = None
    if world > 1:                                             # every rank's own time: a straggler GPU shows here
        mine = torch.tensor([my_ms / steps], dtype=torch.float64, device=device)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        ms_by_rank = [round(float(x.item()), 4) for x in allr]
    tensor_bound = getattr(wl, "bound", "hbm") == "tensor"
    unit_scale = 1e12 if tensor_bound else (1.0 if wl.unit == "tokens/s" else 1e9)
    peak = peaks["bf16_tflops"] if tensor_bound else peaks["hbm_gbs"]
    value = world * wl.bytes_per_step / (ms_per_step * 1e-3) / unit_scale

    # ---- per-kernel durations ------------------------------------------------------------
    # One kernel per step: its average launch duration over the timed region itself.  Several kernels per
    # step (the sweep): each one alone, 20 launches back to back between two events, alternating between two
    # input buffers so that no launch finds its input in L2 -- the kernel's own average launch duration.
    ncase = len(wl.cases)
    kernels = []
    strong = getattr(wl, "scaling", "weak") == "strong"
    if hasattr(wl, "per_kernel"):
        kernels = wl.per_kernel()
        for k in kernels:
            k["frac"] = round(k[wl.unit] / peak, 5)
    elif hasattr(wl, "launch_case"):
        reps = 20
        for i, (label, fn, kind, op, units) in enumerate(wl.cases):
            for r in range(4):
                wl.launch_case(i, r)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for r in range(reps):
                wl.launch_case(i, r)
            b.record()
            b.synchronize()
            us = max(a.elapsed_time(b) / reps * 1e3, 1e-3)
            rate = units / (us * 1e-6) / unit_scale
            kernels.append({"kernel": label, "us": round(us, 2), "bytes": units, wl.unit: round(rate, 1), "frac": round(rate / peak, 4)})
    else:
        label, _f, _k, _o, units = wl.cases[0]
        units = units / world if strong else units
        us = ms_per_step * 1e3
        rate = units / (us * 1e-6) / unit_scale
        kernels.append({"kernel": label, "us": round(us, 2), "flops" if tensor_bound else "bytes": units,
                        wl.unit: round(rate, 1), "frac": round(rate / peak, 4)})
    # the roofline names the kernel FURTHEST below its roof
    low = min(kernels, key=lambda k: k["frac"])
    roofline = {"bound": "tensor" if tensor_bound else "hbm", "kernel": low["kernel"],
                "achieved": low[wl.unit], "peak": peak, "unit": wl.unit, "frac": low["frac"],
                "peak_source": f"{peaks['source']} " + ("cuBLAS bf16 burst" if tensor_bound else "copy bandwidth"),
                "timing": ("CUDA events around back-to-back launches of this kernel alone (inputs alternate between buffers larger than L2)"
                           if hasattr(wl, "launch_case") else
                           "one CUDA event pair per launch, L2 flushed before each" if hasattr(wl, "per_kernel") else
                           "CUDA events around the timed region / launches in it"),
                "lowest_of": len(kernels),
                "traffic": traffic_for(low["kernel"], low.get("bytes", low.get("flops", 0)), traffic)}
    if len(kernels) > 8:                                           # keep the record short: the extremes, not all twenty
        ks = sorted(kernels, key=lambda k: k["frac"])
        kernels = ks[:4] + ks[-2:]

    # ---- end to end: host buffers in, host results out, every step ----------------------
    e2e_steps = args.e2e_steps or max(3, min(steps, 10))
    if hasattr(wl, "setup_e2e"):
        wl.setup_e2e()
    wl.step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        wl.step_e2e()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    h2d, d2h = wl.e2e_bytes()
    e2e_units = getattr(wl, "e2e_units", wl.bytes_per_step)
    e2e = {"value": world * e2e_units / (e2e_ms * 1e-3) / unit_scale, "unit": wl.unit, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps}
    if hasattr(wl, "e2e_note"):
        e2e["how"] = wl.e2e_note
    if hasattr(wl, "setup_e2e"):
        # the same bytes moved with no kernel launched: what the copies alone cost on this box at this N
        wl.step_e2e(compute=False)
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(e2e_steps):
            wl.step_e2e(compute=False)
        f1.record()
        barrier()
        e2e["e2e_floor_ms"] = max_over_ranks(f0.elapsed_time(f1)) / e2e_steps

    # ---- CPU baseline (rank 0, N = 1 only) ----------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle as orc
        v, dt, n, threads = cpu_line(wl, orc, 3, budget_s=12.0)
        cpu = {"value": v, "unit": wl.unit, "cores": threads, "kind": "port",
               "sample": f"{wl.cpu_sample_text}, median of {n} runs of {dt:.2f} s; independent units split over {threads} host threads"}

    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms_per_step, "ms_per_step_by_rank": ms_by_rank, "higher_is_better": True,
            "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic (seeded)", "config": None, "clocks": clk.summary(), "e2e": e2e,
            "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu, "kernels": kernels}
    if hasattr(wl, "extra"):
        ex = wl.extra()
        line["roofline"] = {"bound": "hbm", "kernel": "decode step (weights + KV cache streamed once per token)",
                            "achieved": round(ex["decode_hbm_GBs"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": round(ex["decode_hbm_GBs"] / peaks["hbm_gbs"], 4),
                            "peak_source": f"{peaks['source']} copy bandwidth", "traffic": None}
        line["kernels"] = [ex]
    if hasattr(wl, "extra_fields"):
        line.update(wl.extra_fields())
    if hasattr(wl, "time_other_exchange"):
        other = wl.time_other_exchange(steps, barrier, max_over_ranks)
        if other is not None:
            line["other_exchange"] = other
        par = wl.parity()
        if par is not None or world > 1:
            line["parity_max_abs"] = par
            line["parity_how"] = "rank 0, sequences 0 and 63: sharded result vs one decode launch over the gathered KV sequence (bf16 outputs)"
    line["config"] = wl.config(world)
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="all",
                    help="all = prefill (headline) with the others reported under 'others'; or one name, or a comma-separated "
                         "list of names (the first is the headline): " + ", ".join(sorted(WORKLOADS)))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=None, help="steps of the host-buffer (end-to-end) measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="decode_long at N>1: how the (O, lse) partials cross the GPUs in the timed region")
    ap.add_argument("--elements", type=int, default=None,
                    help="problem size override (elements per dtype / kv length / seq length); "
                         "smaller cases are for profiler captures only")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    names = ALL_ORDER if args.workload == "all" else [w.strip() for w in args.workload.split(",") if w.strip()]
    for w in names:
        if w not in WORKLOADS:
            ap.error(f"unknown workload {w!r}")
    # stdout must carry exactly ONE JSON line: libraries that chat on file descriptor 1
    # (NCCL prints its version there) are pointed at stderr; the line goes to the saved descriptor.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference":
        reference_arm(args, names, rank, world, emit)
        return

    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    pkg = ge.load_package()
    pkg.lib()                                   # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    ctx = {"torch": torch, "dist": dist, "pkg": pkg, "device": device, "rank": rank, "world": world,
           "local_rank": local_rank, "peaks": load_peaks(), "traffic": load_traffic()}
    lines = []
    for name in names:
        wl = make_workload(name, args.elements)
        if hasattr(wl, "exchange"):
            wl.exchange = args.exchange
        lines.append(measure(wl, args, ctx))
        if hasattr(wl, "dec"):
            wl.dec.check()                      # a bounded wait of the peer exchange that ran out is an error
        del wl
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    if rank == 0:
        line = lines[0]
        if len(lines) > 1:
            line["others"] = lines[1:]
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
