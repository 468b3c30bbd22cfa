#!/usr/bin/env python
"""Benchmark of the B200 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One process per GPU (for N > 1 launch with torch.distributed.run; rank, local
rank and world size come from the environment).  A step is one pass of the
workload over one batch of seeded synthetic input.  W warm-up steps, then exactly
K steps timed with CUDA events on the launching stream between a barrier +
synchronize on both sides; the time is the max over ranks; rank 0 prints ONE
JSON line.

Workloads (default `all`: segops is the headline line, decode and prefill ride along
under "others", each with its own roofline, e2e and cpu_baseline)
  segops       segmented wave64 reduce + inclusive-scan sweep over 2^26 elements per
               dtype: reduce {f32,f64,i32,i64} x {sum,max,min}, reduce {f16,bf16} sum
               (fp32 accumulation), scan-sum {f32,f64,i32,i64,f16,bf16}.  HBM-bound.
               N > 1: every rank sweeps its own 2^26-element shard (weak scaling).
  decode       GQA decode, batch 64, 32 q / 8 kv heads, D 128, 8192 cached keys, bf16.
               HBM-bound.  N > 1: every rank its own (batch, kv-head) units (weak).
  prefill      causal prefill, batch 8, 32 heads, seq 4096, D 128, bf16.  Tensor-bound.
               N > 1: every rank its own (batch, head) units (weak).
  decode_long  the 131072-key decode with the KV sequence split across the ranks and
               one NCCL all-gather of (O, lse) per step (strong scaling).

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

    def __init__(self, index: int, period: float = 0.01):
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
        self.host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in self.out]
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

    def step_e2e(self):
        """The same sweep through the public API from HOST buffers: H2D of every
        input from pinned memory, the launches, D2H of every result."""
        for k, h in self.host.items():
            self.dev[k].copy_(h, non_blocking=True)
        self.step()
        for o, h in zip(self.out, self.host_out):
            h.copy_(o, non_blocking=True)

    cpu_sample = 1 << 24
    cpu_sample_text = "the same sweep over 2^24 elements per dtype (1/4 of the workload)"

    def e2e_bytes(self):
        h2d = sum(v.numel() * v.element_size() for v in self.host.values())
        d2h = sum(v.numel() * v.element_size() for v in self.host_out)
        return h2d, d2h

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

    def step_e2e(self):
        for d, h in zip((self.Q, self.K, self.V), self.host):
            d.copy_(h, non_blocking=True)
        self.step()
        self.O_host.copy_(self.O, non_blocking=True)

    def e2e_bytes(self):
        return 3 * self.Q.numel() * 2, self.O.numel() * 2

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
        """n = new tokens; one sequence, prompt 64 (bounded: the CPU statement needs seconds per prompt token block)."""
        import numpy as np
        from oracle import runtime_ref as rr
        if not hasattr(self, "_cpu_w"):
            self._cpu_w = rr.make_weights(self.CFG, seed=5, kind="bf16", std=0.02)
        ids = np.random.default_rng(1).integers(0, self.CFG["vocab_size"], (1, 64))
        t0 = time.perf_counter()
        for _ in range(reps):
            rr.RefSession(self.CFG, self._cpu_w, 64 + n, 1, "bf16").generate(ids, n)
        dt = (time.perf_counter() - t0) / reps
        return n / dt, dt

    cpu_sample = 8
    cpu_sample_text = "1 sequence, prompt 64 tokens + 8 new tokens (numpy restatement of the reference Session)"


WORKLOADS = {"segops": SegopsSweep, "decode": DecodeGQA, "prefill": PrefillCausal, "decode_long": DecodeLong,
             "runtime": RuntimeLlama}
ALL_ORDER = ["segops", "decode", "prefill"]          # `--workload all`: the first is the headline


def make_workload(name, elements=None):
    return WORKLOADS[name](elements) if elements else WORKLOADS[name]()


# --------------------------------------------------------------------------------------
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
        v, dt, n, threads = cpu_line(wl, orc, args.steps, budget_s=120.0 / len(names))
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
    peaks = ctx["peaks"]

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
    warm = max(args.warmup, 3)
    for _ in range(warm):
        wl.step()
    barrier()

    # ---- device-resident timing: K steps between two events -----------------------------
    launches0 = pkg.launch_count()
    with ClockSampler(local_rank) as clk:
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            wl.step()
        t1.record()
        barrier()
    launches = pkg.launch_count() - launches0
    ms_per_step = max_over_ranks(t0.elapsed_time(t1)) / args.steps
    tensor_bound = getattr(wl, "bound", "hbm") == "tensor"
    unit_scale = 1e12 if tensor_bound else (1.0 if wl.unit == "tokens/s" else 1e9)
    peak = peaks["bf16_tflops"] if tensor_bound else peaks["hbm_gbs"]
    value = world * wl.bytes_per_step / (ms_per_step * 1e-3) / unit_scale

    # ---- per-kernel durations ------------------------------------------------------------
    # (a) inside the step: the same steps again with one event after every launch (each event
    #     costs ~3 us of stream time, and a launch is charged for write-backs its predecessor left
    #     in L2); (b) where the workload has several kernels, each one alone: `reps` launches back
    #     to back between two events, alternating between two input buffers so that no launch finds
    #     its input in L2 -- the kernel's own average launch duration.
    ncase = len(wl.cases)
    if ncase == 1:
        # one kernel per step: its average launch duration over the timed region itself
        isteps, per = 1, [ms_per_step]
    else:
        isteps = max(1, min(args.steps, 10))
        events = [torch.cuda.Event(enable_timing=True)]
        events[0].record()
        for _ in range(isteps):
            wl.step(events)
        barrier()
        per = [0.0] * ncase
        for s_ in range(isteps):
            for i in range(ncase):
                per[i] += events[s_ * ncase + i].elapsed_time(events[s_ * ncase + i + 1])
    alone = None
    if hasattr(wl, "launch_case"):
        reps, alone = 20, []
        for i in range(ncase):
            for r in range(4):
                wl.launch_case(i, r)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for r in range(reps):
                wl.launch_case(i, r)
            b.record()
            b.synchronize()
            alone.append(a.elapsed_time(b) / reps)
    kernels = []
    for i, (label, fn, kind, op, units) in enumerate(wl.cases):
        units = units / world if getattr(wl, "scaling", "weak") == "strong" else units
        us_step = max(per[i] / isteps * 1e3, 1e-3)
        us = max(alone[i] * 1e3, 1e-3) if alone is not None else us_step
        rate = units / (us * 1e-6) / unit_scale
        k = {"kernel": label, "us": round(us, 2), "flops" if tensor_bound else "bytes": units,
             wl.unit: round(rate, 1), "frac": round(rate / peak, 4)}
        if alone is not None:
            k["us_inside_step"] = round(us_step, 2)
        kernels.append(k)
    dom = max(range(ncase), key=lambda i: per[i])
    roofline = {"bound": "tensor" if tensor_bound else "hbm", "kernel": kernels[dom]["kernel"],
                "achieved": kernels[dom][wl.unit], "peak": peak, "unit": wl.unit, "frac": kernels[dom]["frac"],
                "peak_source": f"{peaks['source']} " + ("cuBLAS bf16 burst" if tensor_bound else "copy bandwidth"),
                "timing": ("CUDA events around 20 back-to-back launches of this kernel on alternating input buffers"
                           if alone is not None else "CUDA events around the timed region / launches in it"),
                "traffic": TRAFFIC.get(kernels[dom]["kernel"])}

    # ---- end to end: host buffers in, host results out, every step ----------------------
    e2e_steps = args.e2e_steps or max(3, min(args.steps, 10))
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
    e2e = {"value": world * wl.bytes_per_step / (e2e_ms * 1e-3) / unit_scale, "unit": wl.unit, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps}

    # ---- CPU baseline (rank 0, N = 1 only) ----------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle as orc
        v, dt, n, threads = cpu_line(wl, orc, 3, budget_s=30.0)
        cpu = {"value": v, "unit": wl.unit, "cores": threads, "kind": "port",
               "sample": f"{wl.cpu_sample_text}, median of {n} runs of {dt:.2f} s; independent units split over {threads} host threads"}

    if hasattr(wl, "extra"):
        ex = wl.extra()
        roofline = {"bound": "hbm", "kernel": "decode step (weights + KV cache streamed once per token)",
                    "achieved": round(ex["decode_hbm_GBs"], 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(ex["decode_hbm_GBs"] / peaks["hbm_gbs"], 4),
                    "peak_source": f"{peaks['source']} copy bandwidth", "traffic": None}
        kernels = [ex]
    return {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic (seeded)", "config": wl.config(world), "clocks": clk.summary(), "e2e": e2e,
            "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu, "kernels": kernels}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="all", choices=sorted(WORKLOADS) + ["all"],
                    help="all = segops (headline) with decode and prefill reported under 'others'")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=None, help="steps of the host-buffer (end-to-end) measurement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="auto", choices=["auto", "peer", "nccl"],
                    help="decode_long at N>1: how the (O, lse) partials cross the GPUs")
    ap.add_argument("--elements", type=int, default=None,
                    help="problem size override (elements per dtype / kv length / seq length); "
                         "smaller cases are for profiler captures only")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    names = ALL_ORDER if args.workload == "all" else [args.workload]
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
           "local_rank": local_rank, "peaks": load_peaks()}
    lines = []
    for name in names:
        wl = make_workload(name, args.elements)
        if hasattr(wl, "exchange"):
            wl.exchange = args.exchange
        lines.append(measure(wl, args, ctx))
        if hasattr(wl, "dec"):
            wl.dec.check()                      # a bounded wait of the peer exchange that ran out is an error
        del wl
        torch.cuda.empty_cache()
    if rank == 0:
        line = lines[0]
        if len(lines) > 1:
            line["others"] = lines[1:]
        emit(line)
    if world > 1:
        dist.destroy_process_group()


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/, scaled from the captured case to a full launch by the units
# processed (traffic of these streaming kernels is proportional to them).
def _seg_traffic():
    t = {}
    for kind, size in (("f32", 4), ("i32", 4), ("f64", 8), ("i64", 8)):
        for op in ("sum", "max", "min"):                      # profiles/segreduce_f32_sum_2p25.md: read 1.00x, results 3x
            t[f"reduce_{op}<{kind}>"] = (1 << 26) * size + 3 * (1 << 20) * size
        # profiles/segscan_f64_sum_2p25.md: read 1.00x; 78 % of the output reached DRAM before the launch ended
        t[f"scan_inclusive_sum<{kind}>"] = int((1 << 26) * size * (1.0 + 0.784))
    for kind in ("f16", "bf16"):                                  # profiles/segscan_lane_16bit_sum_2p26.md: 215 MB of 268 MB
        t[f"scan_inclusive_sum<{kind}>"] = 215_000_000
    return t


TRAFFIC = _seg_traffic()
# profiles/decode_mma_bf16_d128_n8192_full.md and profiles/prefill_tc_bf16_d128_s4096_full.md: full-size captures
TRAFFIC["decode_mma_kernel (+ combine)"] = int(7.130e12 * 301.984e-6)
TRAFFIC["prefill_tc_kernel"] = int(793.7e9 * 1.332064e-3)

if __name__ == "__main__":
    main()
