"""numpy front end of the CPU oracle (oracle/oracle.cpp) and, when present, of the
reference's own CPU functions compiled by oracle/build_ref.py.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline / reference arm.  The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(HERE, "oracle.cpp")
_SO = os.path.join(HERE, "liboracle.so")
_FLAGS = ["-O2", "-std=c++17", "-ffp-contract=off", "-shared", "-fPIC", "-pthread"]

SUM, MAX, MIN = 0, 1, 2
OPS = {"sum": SUM, "max": MAX, "min": MIN}


def build(force: bool = False) -> str:
    """Compile oracle.cpp into liboracle.so (skipped when up to date)."""
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.run(["g++", *_FLAGS, _SRC, "-o", _SO], check=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_shfl_reduce_f32.restype = C.c_float
        _lib.orc_hardware_threads.restype = C.c_int
    return _lib


def hardware_threads() -> int:
    return int(lib().orc_hardware_threads())


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- 16-bit conversions (bit patterns as uint16) ------------------------------------
def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x); out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16(_p(x), _p(out), C.c_size_t(x.size)); return out


def f16_bits_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16); out = np.empty(h.shape, np.float32)
    lib().orc_f16_to_f32(_p(h), _p(out), C.c_size_t(h.size)); return out


def f32_to_bf16_bits(x) -> np.ndarray:
    x = _f32(x); out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), C.c_size_t(x.size)); return out


def bf16_bits_to_f32(h) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16); out = np.empty(h.shape, np.float32)
    lib().orc_bf16_to_f32(_p(h), _p(out), C.c_size_t(h.size)); return out


def round_to(x, kind: str) -> np.ndarray:
    """x rounded to fp16 / bf16 and widened back to fp32 ("f32" leaves it)."""
    if kind == "f16":
        return f16_bits_to_f32(f32_to_f16_bits(x))
    if kind == "bf16":
        return bf16_bits_to_f32(f32_to_bf16_bits(x))
    return _f32(x)


# ---- generators -----------------------------------------------------------------------
def gen_normal_mt19937(seed: int, mean: float, std: float, n: int) -> np.ndarray:
    """n draws of std::normal_distribution<float>(mean, std) on std::mt19937(seed)."""
    out = np.empty(n, np.float32)
    lib().orc_gen_normal_mt19937(C.c_uint32(seed), C.c_float(mean), C.c_float(std), _p(out), C.c_size_t(n))
    return out


def gen_qkv_mt19937(seed: int, std: float, q_elems: int, kv_elems: int):
    """The reference's recipe: one stream, Q then K then V."""
    a = gen_normal_mt19937(seed, 0.0, std, q_elems + 2 * kv_elems)
    return a[:q_elems].copy(), a[q_elems:q_elems + kv_elems].copy(), a[q_elems + kv_elems:].copy()


def gen_decode_dme_case(seed: int, skip: int, D: int, N: int, nQH: int, nKVH: int, max_seq: int):
    """q, cacheK, cacheV (fp16 bit patterns) of one validate_decode_dme config, and
    the number of draws it consumed."""
    q = np.empty(nQH * D, np.uint16)
    ck = np.empty(nKVH * max_seq * D, np.uint16)
    cv = np.empty(nKVH * max_seq * D, np.uint16)
    lib().orc_gen_decode_dme_case(C.c_uint32(seed), C.c_size_t(skip), D, N, nQH, nKVH, max_seq, _p(q), _p(ck), _p(cv))
    return q, ck, cv, nQH * D + 2 * nKVH * N * D


_SEG = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.int32): "i32", np.dtype(np.int64): "i64"}


# ---- segmented reduce / scan ------------------------------------------------------------
def dpp_reduce(op: int, x: np.ndarray, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x); assert x.size % 64 == 0
    out = np.empty(x.size // 64, x.dtype)
    getattr(lib(), "orc_dpp_reduce_" + _SEG[x.dtype])(op, _p(x), _p(out), C.c_size_t(out.size), threads)
    return out


def dpp_scan(op: int, x: np.ndarray, exclusive: bool = False, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x); assert x.size % 64 == 0
    out = np.empty_like(x)
    getattr(lib(), "orc_dpp_scan_" + _SEG[x.dtype])(op, _p(x), _p(out), C.c_size_t(x.size // 64), int(exclusive), threads)
    return out


def seq_reduce(op: int, x: np.ndarray, threads: int = 1) -> np.ndarray:
    """Plain sequential loop per segment (the reference's CPU-side check)."""
    x = np.ascontiguousarray(x); assert x.size % 64 == 0
    out = np.empty(x.size // 64, x.dtype)
    getattr(lib(), "orc_seq_reduce_" + _SEG[x.dtype])(op, _p(x), _p(out), C.c_size_t(out.size), threads)
    return out


def seq_scan(op: int, x: np.ndarray, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x); assert x.size % 64 == 0
    out = np.empty_like(x)
    getattr(lib(), "orc_seq_scan_" + _SEG[x.dtype])(op, _p(x), _p(out), C.c_size_t(x.size // 64), threads)
    return out


def shfl_reduce_narrow(op: int, bits: np.ndarray, bf16: bool, threads: int = 1):
    """(fp32 result before rounding, result rounded to the input type as bits)."""
    bits = np.ascontiguousarray(bits, np.uint16); assert bits.size % 64 == 0
    f = np.empty(bits.size // 64, np.float32); nrw = np.empty(bits.size // 64, np.uint16)
    lib().orc_shfl_reduce_narrow(op, int(bf16), _p(bits), _p(f), _p(nrw), C.c_size_t(f.size), threads)
    return f, nrw


def shfl_scan_narrow(op: int, bits: np.ndarray, bf16: bool, threads: int = 1) -> np.ndarray:
    bits = np.ascontiguousarray(bits, np.uint16); assert bits.size % 64 == 0
    out = np.empty_like(bits)
    lib().orc_shfl_scan_narrow(op, int(bf16), _p(bits), _p(out), C.c_size_t(bits.size // 64), threads)
    return out


def shfl_reduce_f32(op: int, x64) -> float:
    x64 = _f32(x64); assert x64.size == 64
    return float(lib().orc_shfl_reduce_f32(op, _p(x64)))


# ---- attention ------------------------------------------------------------------------
def cpu_prefill(Q, K, V, D, seqQ, seqK, nQH, nKVH, batch, causal, threads: int = 1) -> np.ndarray:
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    assert Q.size == batch * nQH * seqQ * D and K.size == batch * nKVH * seqK * D == V.size
    O = np.zeros(Q.size, np.float32)
    lib().orc_cpu_prefill(_p(Q), _p(K), _p(V), _p(O), D, seqQ, seqK, nQH, nKVH, batch, int(causal), threads)
    return O.reshape(batch, nQH, seqQ, D)


def cpu_prefill_units(Q, K, V, D, seqQ, seqK, nQH, nKVH, batch, causal, units, threads: int = 1) -> np.ndarray:
    """Only the (batch*nQH + head) units listed; other rows of the result stay 0."""
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    u = np.ascontiguousarray(units, np.int32)
    O = np.zeros(Q.size, np.float32)
    lib().orc_cpu_prefill_units(_p(Q), _p(K), _p(V), _p(O), D, seqQ, seqK, nQH, nKVH, int(causal), _p(u), int(u.size), threads)
    return O.reshape(batch, nQH, seqQ, D)


def cpu_attention_ref_heads(Q, K, V, n_units, seq_len, d, scale, threads: int = 1) -> np.ndarray:
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    O = np.zeros(Q.size, np.float32)
    lib().orc_cpu_attention_ref_heads(_p(Q), _p(K), _p(V), _p(O), n_units, seq_len, d, C.c_float(scale), threads)
    return O.reshape(n_units, seq_len, d)


def cpu_decode(q, K, V, D, N, nQH, nKVH, stride_kv=None, batch: int = 1, kv_batch_stride=None, threads: int = 1) -> np.ndarray:
    q, K, V = _f32(q), _f32(K), _f32(V)
    stride_kv = N if stride_kv is None else stride_kv
    kv_batch_stride = nKVH * stride_kv * D if kv_batch_stride is None else kv_batch_stride
    o = np.zeros(batch * nQH * D, np.float32)
    lib().orc_cpu_decode(_p(q), _p(K), _p(V), _p(o), D, N, nQH, nKVH, C.c_longlong(stride_kv), batch,
                         C.c_longlong(kv_batch_stride), threads)
    return o.reshape(batch, nQH, D)


def merge_partials(O_parts, m_parts, l_parts) -> np.ndarray:
    O_parts, m_parts, l_parts = _f32(O_parts), _f32(m_parts), _f32(l_parts)
    parts, rows, D = O_parts.shape
    out = np.empty((rows, D), np.float32)
    lib().orc_merge_partials(_p(O_parts), _p(m_parts), _p(l_parts), _p(out), parts, C.c_size_t(rows), D)
    return out


def merge_lse(O_parts, lse_parts):
    O_parts, lse_parts = _f32(O_parts), _f32(lse_parts)
    parts, rows, D = O_parts.shape
    out = np.empty((rows, D), np.float32); lse = np.empty(rows, np.float32)
    lib().orc_merge_lse(_p(O_parts), _p(lse_parts), _p(out), _p(lse), parts, C.c_size_t(rows), D)
    return out, lse


# ---- the reference's own CPU functions (oracle/_ref) --------------------------------------
_ref = None


def ref_lib():
    """libref_cpu.so built from the reference tree by oracle/build_ref.py, or None."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libref_cpu.so")
        if not os.path.exists(path):
            return None
        _ref = C.CDLL(path)
    return _ref


def ref_call(name: str, Q, K, V, out_size: int, *ints, scale=None) -> np.ndarray:
    r = ref_lib()
    Q, K, V = _f32(Q), _f32(K), _f32(V)
    O = np.zeros(out_size, np.float32)
    args = [_p(Q), _p(K), _p(V), _p(O), *[int(i) for i in ints]]
    if scale is not None:
        args.append(C.c_float(scale))
    getattr(r, name)(*args)
    return O
