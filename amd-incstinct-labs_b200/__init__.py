"""B200 (sm_100a) implementation of the reference's wave reduce/scan primitives and
FA2 attention kernels: Python host layer over the C ABI of libb200p.so.

The library is hand-written CUDA (csrc/) behind `extern "C"` entry points
(include/b200p.h).  This module only loads it with ctypes and offers thin
wrappers that take torch CUDA tensors (torch is used for device memory and
streams, nothing else).  There is no CPU fallback: importing works anywhere
(so that symbols can be inspected), but every compute call raises unless the
library is present and the tensors live on a CUDA device.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "lib", "libb200p.so")

F32, F64, I32, I64, F16, BF16 = 0, 1, 2, 3, 4, 5
SUM, MAX, MIN = 0, 1, 2
OPS = {"sum": SUM, "max": MAX, "min": MIN}

# every symbol include/b200p.h declares: (name, restype, argtypes)
_vp, _sz, _i, _ll = C.c_void_p, C.c_size_t, C.c_int, C.c_longlong
SYMBOLS = {
    "b200p_version": (C.c_char_p, []),
    "b200p_strerror": (C.c_char_p, [_i]),
    "b200p_launch_count": (C.c_ulonglong, []),
    "b200p_set_tuning": (_i, [C.c_char_p, _i]),
    "b200p_segreduce": (_i, [_i, _i, _vp, _vp, _sz, _vp]),
    "b200p_segreduce_narrow": (_i, [_i, _i, _vp, _vp, _sz, _vp]),
    "b200p_segscan_inclusive": (_i, [_i, _i, _vp, _vp, _sz, _vp]),
    "b200p_segscan_exclusive_sum": (_i, [_i, _vp, _vp, _sz, _vp]),
    "b200p_wave_probe": (_i, [_i, _i, _i, _vp, _vp, _vp]),
    "b200p_wave_probe_n": (_i, [_i, _i, _i, _vp, _vp, _i, _vp]),
    "b200p_wave_vote_probe": (_i, [_vp, _vp, _vp]),
    "b200p_api_probe": (_i, [_i, _vp, _vp, _i, _i, _vp]),
    "b200p_wave_reduce_loop": (_i, [_i, _i, _i, _vp, _vp, _i, _i, _vp]),
    "b200p_wave_scan_loop": (_i, [_i, _i, _vp, _vp, _i, _i, _vp]),
    "b200p_row_op": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _i, C.c_float, _vp]),
    "b200p_fa_rows_f32": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, C.c_float, _vp]),
    "b200p_model_read_meta": (_i, [C.c_char_p, _vp, _vp, _vp]),
    "b200p_model_load": (_vp, [C.c_char_p, _vp]),
    "b200p_model_weights_of": (_vp, [_vp]),
    "b200p_model_free": (None, [_vp]),
    "b200p_attn_decode_workspace_bytes": (_sz, [_vp]),
    "b200p_attn_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200p_attn_decode_dyn": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "b200p_attn_decode_partial": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200p_attn_merge_lse": (_i, [_vp, _vp, _i, _i, _i, _ll, _ll, _i, _vp, _vp]),
    "b200p_attn_decode_push": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _i, _vp]),
    "b200p_attn_merge_lse_wait": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, C.c_ulonglong, _vp]),
    "b200p_attn_workspace_status": (_i, [_vp, _vp]),
    "b200p_attn_decode_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "b200p_attn_decode_noalloc_max_bytes": (_sz, []),
    "b200p_attn_prefill": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "b200p_attn_prefill_strided": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "b200p_attn_prefill_debug": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "b200p_device_status": (_i, [_i]),
    "b200p_session_create": (_vp, [_vp, _i, _i, _vp]),
    "b200p_session_destroy": (None, [_vp]),
    "b200p_session_generate": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp]),
    "b200p_session_prefill_logits": (_i, [_vp, _vp, _i, _vp, _vp]),
    "b200p_session_step_logits": (_i, [_vp, _vp, _vp, _vp]),
    "b200p_skinny_gemm": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, C.c_float, _vp]),
    "b200p_session_kv_len": (_i, [_vp]),
    "b200p_session_gemm_calls": (C.c_ulonglong, [_vp]),
    "b200p_session_blas_calls": (C.c_ulonglong, [_vp]),
    "b200p_gemm_16": (_i, [_i, _i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp]),
    "b200p_session_graph_replays": (C.c_ulonglong, [_vp]),
    "b200p_session_mega_launches": (C.c_ulonglong, [_vp]),
    "b200p_fa_step": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, C.c_float, _vp]),
}


MAX_PEERS = 16


class PeerExchange(C.Structure):
    """struct b200p_peer_exchange: every rank's receive buffer and flag array as
    addressable from this GPU, plus this rank's local CTA counter."""
    _fields_ = [("rank", _i), ("world", _i), ("slots", _vp * MAX_PEERS), ("flags", _vp * MAX_PEERS), ("counter", _vp)]


def peer_exchange(rank: int, world: int, slot_ptrs, flag_ptrs, counter_ptr: int) -> PeerExchange:
    if not (1 <= world <= MAX_PEERS) or len(slot_ptrs) != world or len(flag_ptrs) != world:
        raise ValueError(f"world must be 1..{MAX_PEERS} with one slot and flag pointer per rank")
    px = PeerExchange()
    px.rank, px.world, px.counter = rank, world, counter_ptr
    for g in range(world):
        px.slots[g], px.flags[g] = int(slot_ptrs[g]), int(flag_ptrs[g])
    return px


class PrefillCfg(C.Structure):
    """struct b200p_prefill_cfg == cdna3::attn::PrefillCfg."""
    _fields_ = [("D", _i), ("seqQ", _i), ("seqK", _i), ("nQHeads", _i), ("nKVHeads", _i), ("batch", _i), ("causal", _i)]


class DecodeArgs(C.Structure):
    """struct b200p_decode_args (include/b200p.h)."""
    _fields_ = [("D", _i), ("N", _i), ("nQHeads", _i), ("nKVHeads", _i), ("stride_kv", _i), ("batch", _i),
                ("dtype", _i), ("kv_batch_stride", _ll), ("key_offset", _ll), ("q_batch_stride", _ll),
                ("o_batch_stride", _ll)]


class B200PError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().b200p_strerror(status).decode() if _lib is not None else "library not loaded"
        super().__init__(f"{where}: status {status} ({msg})")


_lib = None


def lib() -> C.CDLL:
    """libb200p.so, loaded once.  Raises if it has not been built (python
    amd-incstinct-labs_b200/build.py, or __graft_entry__.build())."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build the CUDA library first; there is no fallback path")
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(h, name)          # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        _lib = h
    return _lib


def _check(status: int, where: str) -> None:
    if status != 0:
        raise B200PError(status, where)


def launch_count() -> int:
    return int(lib().b200p_launch_count())


def set_tuning(key: str, value: int) -> int:
    return int(lib().b200p_set_tuning(key.encode(), int(value)))


def _dtype_code(t) -> int:
    import torch
    return {torch.float32: F32, torch.float64: F64, torch.int32: I32, torch.int64: I64,
            torch.float16: F16, torch.bfloat16: BF16}[t.dtype]


def _stream(t) -> int:
    import torch
    return torch.cuda.current_stream(t.device).cuda_stream


def _dev(t, name: str):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: there is no CPU path")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


# ---- segmented wave reduce / scan (wave::dpp::reduce_* / scan_*) ------------------------
def segreduce(x, op: str = "sum", out=None, narrow: bool = False):
    """Reduce every run of 64 consecutive elements of `x` (1-D) with `op`.
    f16/bf16 inputs accumulate in fp32 and return fp32, or the input type with
    narrow=True (what the reference's overloads return)."""
    import torch
    _dev(x, "x")
    code = _dtype_code(x)
    nseg = x.numel() // 64
    if narrow:
        out_dtype = x.dtype
    else:
        out_dtype = torch.float32 if code in (F16, BF16) else x.dtype
    if out is None:
        out = torch.empty(nseg, dtype=out_dtype, device=x.device)
    fn = lib().b200p_segreduce_narrow if narrow else lib().b200p_segreduce
    _check(fn(OPS[op], code, x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)), "segreduce")
    return out


def segscan(x, op: str = "sum", out=None, exclusive: bool = False):
    """Inclusive (or exclusive-sum) scan of every run of 64 consecutive elements."""
    import torch
    _dev(x, "x")
    if out is None:
        out = torch.empty_like(x)
    if exclusive:
        _check(lib().b200p_segscan_exclusive_sum(_dtype_code(x), x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)),
               "segscan_exclusive_sum")
    else:
        _check(lib().b200p_segscan_inclusive(OPS[op], _dtype_code(x), x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)),
               "segscan_inclusive")
    return out


def wave_probe(x, fn: str = "reduce", op: str = "sum"):
    """Waves of 64 values (x.numel() a multiple of 64) through the device-level pair-per-lane
    API, one warp per wave."""
    import torch
    _dev(x, "x")
    assert x.numel() % 64 == 0
    out = torch.empty_like(x)
    code = {"reduce": 0, "scan": 1, "scan_exclusive": 2}[fn]
    _check(lib().b200p_wave_probe_n(code, OPS[op], _dtype_code(x), x.data_ptr(), out.data_ptr(), x.numel() // 64, _stream(x)),
           "wave_probe")
    return out


def wave_vote_probe(x64):
    """One wave of 64 int32 values through the vote / bitwise wrappers (predicate: value > 0).
    Returns [ballot64, any, all, popcount, reduce_and, reduce_or, ballot32 of the first elements, lane_mask_lt(5)]."""
    import torch
    _dev(x64, "x64")
    assert x64.numel() == 64 and x64.dtype == torch.int32
    out = torch.zeros(8, dtype=torch.int64, device=x64.device)
    _check(lib().b200p_wave_vote_probe(x64.data_ptr(), out.data_ptr(), _stream(x64)), "wave_vote_probe")
    return out


def api_probe(which: int, x, rows: int, tiles: int = 1, out_elems: int = None):
    """Kernels written against <cdna3/cdna3.hpp> and <cdna3/examples/fused_softmax.hpp> (see b200p_api_probe)."""
    import torch
    _dev(x, "x")
    n = out_elems if out_elems is not None else x.numel()
    out = torch.empty(n, dtype=torch.float32, device=x.device)
    _check(lib().b200p_api_probe(which, x.data_ptr(), out.data_ptr(), rows, tiles, _stream(x)), "api_probe")
    return out


# ---- decode attention (cdna3::attn::decode / decode_dme) ----------------------------------
def _decode_args(q, K, N, key_offset):
    """q [batch, nQH, D] (or [nQH, D]); K/V [batch, nKVH, stride_kv, D] (or [nKVH, stride_kv, D])."""
    if q.dim() == 2:
        q = q.unsqueeze(0)
    if K.dim() == 3:
        K = K.unsqueeze(0)
    batch, nQH, D = q.shape
    _, nKVH, stride_kv, _ = K.shape
    N = stride_kv - key_offset if N is None else N
    a = DecodeArgs(D, N, nQH, nKVH, stride_kv, batch, _dtype_code(q), K.stride(0), key_offset, q.stride(0), 0)
    return a, batch, nQH, D


def decode_workspace(q, K, N=None, key_offset: int = 0):
    """Scratch tensor of the size the decode launch needs for these shapes."""
    import torch
    a, *_ = _decode_args(q, K, N, key_offset)
    nbytes = int(lib().b200p_attn_decode_workspace_bytes(C.byref(a)))
    if nbytes == 0:
        raise B200PError(-6, "decode_workspace")
    return torch.empty(nbytes, dtype=torch.uint8, device=q.device)


def decode(q, K, V, N=None, out=None, workspace=None, key_offset: int = 0):
    """One query token per sequence against N cached keys.  K/V may be the packed
    [.., N, D] tensors of cdna3::attn::decode or the strided cache [.., max_seq, D]
    of cdna3::attn::decode_dme (then pass N)."""
    import torch
    for t, n in ((q, "q"), (K, "K"), (V, "V")):
        _dev(t, n)
    a, batch, nQH, D = _decode_args(q, K, N, key_offset)
    ws = decode_workspace(q, K, N, key_offset) if workspace is None else workspace
    if out is None:
        out = torch.empty_like(q)
    _check(lib().b200p_attn_decode(q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), C.byref(a),
                                   ws.data_ptr(), ws.numel(), _stream(q)), "attn_decode")
    return out


def decode_noalloc(q, K, V, N=None, out=None, key_offset: int = 0):
    """decode() for hosts that cannot lend scratch memory: the split-KV partials go to
    a fixed 8 MiB array inside the library, so nothing is allocated by the call (pass
    `out` to keep this wrapper from allocating the result either).  Shapes that need
    more scratch raise B200PError(-10).  Calls share that array: do not let two of
    them overlap on the GPU."""
    import torch
    for t, n in ((q, "q"), (K, "K"), (V, "V")):
        _dev(t, n)
    a, batch, nQH, D = _decode_args(q, K, N, key_offset)
    if out is None:
        out = torch.empty_like(q)
    _check(lib().b200p_attn_decode_noalloc(q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), C.byref(a),
                                           _stream(q)), "attn_decode_noalloc")
    return out


def decode_dyn(q, K, V, n_dev, n_add: int = 0, N=None, workspace=None, out=None):
    """decode() attending to min(n_dev[0] + n_add, N) keys, the count read on the device
    (n_dev: int32 CUDA tensor); N (default: the K tensor's key extent) is only the bound."""
    import torch
    for t, n in ((q, "q"), (K, "K"), (V, "V"), (n_dev, "n_dev")):
        _dev(t, n)
    if n_dev.dtype != torch.int32:
        raise ValueError("n_dev must be int32")
    a, batch, nQH, D = _decode_args(q, K, N, 0)
    ws = decode_workspace(q, K, N, 0) if workspace is None else workspace
    if out is None:
        out = torch.empty((batch, nQH, D), dtype=q.dtype, device=q.device)
    _check(lib().b200p_attn_decode_dyn(q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), C.byref(a),
                                       n_dev.data_ptr(), int(n_add), ws.data_ptr(), ws.numel(), _stream(q)), "attn_decode_dyn")
    return out


def decode_partial(q, K, V, N=None, workspace=None, key_offset: int = 0, out=None, lse=None):
    """Attention over a shard of the KV sequence: (O normalised over the shard as fp32
    [batch, nQH, D], lse [batch, nQH]) for merge_lse."""
    import torch
    for t, n in ((q, "q"), (K, "K"), (V, "V")):
        _dev(t, n)
    a, batch, nQH, D = _decode_args(q, K, N, key_offset)
    ws = decode_workspace(q, K, N, key_offset) if workspace is None else workspace
    if out is None:
        out = torch.empty((batch, nQH, D), dtype=torch.float32, device=q.device)
    if lse is None:
        lse = torch.empty((batch, nQH), dtype=torch.float32, device=q.device)
    _check(lib().b200p_attn_decode_partial(q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                           C.byref(a), ws.data_ptr(), ws.numel(), _stream(q)), "attn_decode_partial")
    return out, lse


def decode_push(q, K, V, px: PeerExchange, seq: int, N=None, workspace=None, key_offset: int = 0):
    """Attention over this rank's KV shard, its (O, lse) stored into every rank's receive
    buffer through the peer pointers of `px`, then flag word [rank] of every rank set to seq."""
    for t, n in ((q, "q"), (K, "K"), (V, "V")):
        _dev(t, n)
    a, batch, nQH, D = _decode_args(q, K, N, key_offset)
    ws = decode_workspace(q, K, N, key_offset) if workspace is None else workspace
    _check(lib().b200p_attn_decode_push(q.data_ptr(), K.data_ptr(), V.data_ptr(), C.byref(a), ws.data_ptr(), ws.numel(),
                                        C.byref(px), int(seq), _stream(q)), "attn_decode_push")


def merge_lse_wait(px: PeerExchange, seq: int, rows: int, D: int, out, status, wait_ns: int = 0):
    """Bounded wait for all ranks' flag words to reach seq, then the lse merge of this step's
    partials from the local receive buffer into out [rows.., D].  status: int32 device tensor
    (zeroed by the caller); 1 afterwards means a wait ran out."""
    _dev(out, "out"); _dev(status, "status")
    _check(lib().b200p_attn_merge_lse_wait(C.byref(px), int(seq), rows, D, _dtype_code(out), out.data_ptr(),
                                           status.data_ptr(), int(wait_ns), _stream(out)), "attn_merge_lse_wait")
    return out


def merge_lse(o_parts, lse_parts, dtype, out=None):
    """o_parts [parts, rows.., D] fp32, lse_parts [parts, rows..] -> [rows.., D] in dtype."""
    import torch
    _dev(o_parts, "o_parts"); _dev(lse_parts, "lse_parts")
    parts, D = o_parts.shape[0], o_parts.shape[-1]
    rows = lse_parts[0].numel()
    if out is None:
        out = torch.empty(o_parts.shape[1:], dtype=dtype, device=o_parts.device)
    _check(lib().b200p_attn_merge_lse(o_parts.data_ptr(), lse_parts.data_ptr(), parts, rows, D, 0, 0, _dtype_code(out),
                                      out.data_ptr(), _stream(o_parts)), "attn_merge_lse")
    return out


def merge_lse_packed(gathered, rows: int, D: int, out):
    """gathered [parts, rows*(D+1)] fp32: each part is a rank's O [rows, D] followed by its
    lse [rows] (the buffer one all-gather of decode_partial's packed output produces)."""
    _dev(gathered, "gathered")
    parts = gathered.shape[0]
    stride = rows * (D + 1)
    base = gathered.data_ptr()
    _check(lib().b200p_attn_merge_lse(base, base + rows * D * 4, parts, rows, D, stride, stride, _dtype_code(out),
                                      out.data_ptr(), _stream(gathered)), "attn_merge_lse")
    return out


def workspace_status(workspace) -> int:
    """0, or B200P_E_TIMEOUT if a kernel using this workspace abandoned a bounded wait (synchronises)."""
    return int(lib().b200p_attn_workspace_status(workspace.data_ptr(), _stream(workspace)))


# ---- prefill attention (cdna3::attn::prefill) ----------------------------------------------
def prefill(Q, K, V, causal: bool = False, out=None, raw_scores=None):
    """Q [batch, nQH, seqQ, D], K/V [batch, nKVH, seqK, D] (fp16 or bf16) -> O like Q."""
    import torch
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        _dev(t, n)
    batch, nQH, seqQ, D = Q.shape
    _, nKVH, seqK, _ = K.shape
    cfg = PrefillCfg(D, seqQ, seqK, nQH, nKVH, batch, int(causal))
    if out is None:
        out = torch.empty_like(Q)
    if raw_scores is None:
        st = lib().b200p_attn_prefill(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), C.byref(cfg),
                                      _dtype_code(Q), _stream(Q))
    else:
        st = lib().b200p_attn_prefill_debug(Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), C.byref(cfg),
                                            _dtype_code(Q), raw_scores.data_ptr(), _stream(Q))
    _check(st, "attn_prefill")
    return out


class AttnStrides(C.Structure):
    """struct b200p_attn_strides: (token, head, sequence) element strides of Q, K, V, O."""
    _fields_ = [(n, _ll) for n in ("q_seq", "q_head", "q_batch", "k_seq", "k_head", "k_batch",
                                   "v_seq", "v_head", "v_batch", "o_seq", "o_head", "o_batch")]


def prefill_strided(Q, K, V, O, causal: bool = False):
    """prefill() on 4-D views [batch, heads, seq, D] with arbitrary (8-element aligned)
    strides, e.g. a permuted token-major projection or a slice of a KV cache; D contiguous."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (O, "O")):
        if not t.is_cuda:
            raise ValueError(f"{n} must be a CUDA tensor: there is no CPU path")
        if t.stride(3) != 1:
            raise ValueError(f"{n}: the head dimension must be contiguous")
    batch, nQH, seqQ, D = Q.shape
    _, nKVH, seqK, _ = K.shape
    cfg = PrefillCfg(D, seqQ, seqK, nQH, nKVH, batch, int(causal))
    st = AttnStrides(Q.stride(2), Q.stride(1), Q.stride(0), K.stride(2), K.stride(1), K.stride(0),
                     V.stride(2), V.stride(1), V.stride(0), O.stride(2), O.stride(1), O.stride(0))
    _check(lib().b200p_attn_prefill_strided(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), C.byref(cfg),
                                            _dtype_code(Q), C.byref(st), _stream(Q)), "attn_prefill_strided")
    return O


def device_status(clear: bool = True) -> int:
    """0, or B200P_E_TIMEOUT if a kernel abandoned a bounded wait (synchronises the device)."""
    return int(lib().b200p_device_status(int(clear)))


FA_STEPS = {"naive": 0, "dpp": 1, "dme": 2, "mfma2": 3}


def fa_step(step: str, Q, K, V, scale: float = 0.0, out=None):
    """One of the reference's FA2 build-order steps (fa_naive / fa_dpp / fa_dme / fa_mfma2).
    Q,K,V [batch, heads, seq, D] in fp16, bf16 or (steps naive/dpp/dme) fp32."""
    import torch
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        _dev(t, n)
    batch, heads, sq, D = Q.shape
    sk = K.shape[2]
    if out is None:
        out = torch.empty_like(Q)
    _check(lib().b200p_fa_step(FA_STEPS[step], _dtype_code(Q), Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(),
                               batch, heads, sq, sk, D, float(scale), _stream(Q)), "fa_step")
    return out


def wave_reduce_loop(x, op: str, reps: int, backend: str = "primitives", out=None):
    """The reference's register-resident reduce benchmark loop over x.numel() / 64 waves (a multiple of 8);
    backend "primitives" (wave::dpp::reduce_*) or "portable" (shuffle-down loop).  Returns one value per wave."""
    import torch
    _dev(x, "x")
    waves = x.numel() // 64
    if out is None:
        out = torch.empty(waves, dtype=x.dtype, device=x.device)
    _check(lib().b200p_wave_reduce_loop(OPS[op], _dtype_code(x), {"primitives": 0, "portable": 1}[backend], x.data_ptr(),
                                        out.data_ptr(), waves, int(reps), _stream(x)), "wave_reduce_loop")
    return out


def wave_scan_loop(x, reps: int, backend: str = "primitives", out=None):
    """The reference's register-resident scan benchmark loop over x.numel() / 64 waves (a multiple of 8): `reps`
    inclusive prefix sums per wave, the total fed back.  Returns the waves' final state (same shape as x)."""
    import torch
    _dev(x, "x")
    waves = x.numel() // 64
    if out is None:
        out = torch.empty_like(x)
    _check(lib().b200p_wave_scan_loop(_dtype_code(x), {"primitives": 0, "portable": 1}[backend], x.data_ptr(), out.data_ptr(),
                                      waves, int(reps), _stream(x)), "wave_scan_loop")
    return out


def row_op(which: str, x, gamma=None, beta=None, backend: str = "primitives", eps: float = 1e-5, out=None):
    """LayerNorm ("layernorm", needs gamma and beta) or softmax ("softmax") over the rows of x [rows, 64 | 512] fp32,
    one warp per row, on the wave primitives or on the portable shuffle loop."""
    import torch
    _dev(x, "x")
    rows, cols = x.shape
    if out is None:
        out = torch.empty_like(x)
    _check(lib().b200p_row_op({"layernorm": 0, "softmax": 1}[which], {"primitives": 0, "portable": 1}[backend], cols, x.data_ptr(),
                              gamma.data_ptr() if gamma is not None else None, beta.data_ptr() if beta is not None else None,
                              out.data_ptr(), rows, float(eps), _stream(x)), "row_op")
    return out


def fa_rows_f32(variant: str, bc: int, Q, K, V, scale: float = 0.0, out=None):
    """The reference's fp32-I/O kernels (one query row per block, bc keys per tile, any seq_len):
    variant "naive" or "dpp"; Q,K,V [batch, heads, seq, D] fp32."""
    import torch
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        _dev(t, n)
    batch, heads, seq, D = Q.shape
    if out is None:
        out = torch.empty_like(Q)
    _check(lib().b200p_fa_rows_f32({"naive": 0, "dpp": 1}[variant], bc, Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(),
                                   batch, heads, seq, D, float(scale), _stream(Q)), "fa_rows_f32")
    return out


# ---- the small LLM runtime (cdna3::runtime::Session) --------------------------------------------
class ModelConfig(C.Structure):
    """struct b200p_model_config == cdna3::runtime::ModelConfig."""
    _fields_ = [("n_layers", _i), ("hidden", _i), ("n_heads", _i), ("n_kv_heads", _i), ("head_dim", _i),
                ("ffn_dim", _i), ("vocab_size", _i), ("rope_theta", C.c_float)]


_LAYER_FIELDS = ("Wq", "Wk", "Wv", "Wo", "bq", "bk", "bv", "Wgate", "Wup", "Wdown", "norm_attn", "norm_mlp")


class LayerWeights(C.Structure):
    _fields_ = [(n, _vp) for n in _LAYER_FIELDS]


class ModelWeights(C.Structure):
    _fields_ = [("cfg", ModelConfig), ("dtype", _i), ("embed_tokens", _vp), ("lm_head", _vp), ("final_norm", _vp),
                ("layers", C.POINTER(LayerWeights))]


def skinny_gemm(W, out, x16=None, x32=None, norm_w=None, epilogue: str = "store16", eps: float = 1e-6):
    """The decode step's projection kernel: out = X . W^T for at most 16 rows of X.
    X is x16 [M, K] (16-bit) or RMSNorm(x32 [M, K]) * norm_w; epilogue one of
    store16 / store32 / acc32 (out += Y) / silu16 (W = [gate; up], out = SiLU(gate) * up)."""
    epi = {"store16": 0, "acc32": 1, "store32": 2, "silu16": 3}[epilogue]
    _dev(W, "W"); _dev(out, "out")
    N, K = W.shape
    if epi == 3:
        N //= 2
    if x16 is not None:
        if not x16.is_cuda or x16.stride(1) != 1:
            raise ValueError("x16 must be a CUDA tensor with contiguous rows: there is no CPU path")
        M, pro, ldx = x16.shape[0], 0, x16.stride(0)
    else:
        _dev(x32, "x32"); _dev(norm_w, "norm_w")
        M, pro, ldx = x32.shape[0], 1, 0
    _check(lib().b200p_skinny_gemm(_dtype_code(W), pro, epi, W.data_ptr(), x16.data_ptr() if x16 is not None else None,
                                   x32.data_ptr() if x32 is not None else None, norm_w.data_ptr() if norm_w is not None else None,
                                   out.data_ptr(), M, N, K, ldx, out.stride(0), eps, _stream(W)), "skinny_gemm")
    return out


def read_model_meta(model_dir: str):
    """meta.json of a model directory in the reference's export format -> (config dict, qkv_bias, dtype code).
    Host only."""
    mc, bias, dt = ModelConfig(), _i(0), _i(0)
    _check(lib().b200p_model_read_meta(os.fsencode(model_dir), C.byref(mc), C.byref(bias), C.byref(dt)), "model_read_meta")
    return {n: getattr(mc, n) for n, _ in ModelConfig._fields_}, bool(bias.value), dt.value


class Model:
    """A model directory (meta.json + per-tensor .bin files, cdna3::runtime::ModelLoader) loaded into
    device memory the object owns."""

    def __init__(self, model_dir: str):
        st = _i(0)
        self._h = lib().b200p_model_load(os.fsencode(model_dir), C.byref(st))
        if not self._h:
            raise B200PError(st.value, "model_load")
        self.weights = C.cast(lib().b200p_model_weights_of(self._h), C.POINTER(ModelWeights)).contents
        self.cfg = {n: getattr(self.weights.cfg, n) for n, _ in ModelConfig._fields_}

    def close(self):
        if getattr(self, "_h", None):
            lib().b200p_model_free(self._h)
            self._h = None

    __del__ = close


def gemm_16(A, W, out, epilogue: str = "store16"):
    """out[M, N] = A[M, K] . W[N, K]^T on the tensor cores; epilogue store16 / store32 / acc32 (out += product) /
    silu16 (W = [gate; up] with 2N rows, out = SiLU(gate) * up).  A, W 16-bit CUDA tensors with contiguous rows."""
    epi = {"store16": 0, "acc32": 1, "store32": 2, "silu16": 3}[epilogue]
    for t, n in ((A, "A"), (W, "W"), (out, "out")):
        if not t.is_cuda or t.stride(-1) != 1:
            raise ValueError(f"{n} must be a CUDA tensor with contiguous rows: there is no CPU path")
    M, K = A.shape
    N = W.shape[0] // (2 if epi == 3 else 1)
    _check(lib().b200p_gemm_16(_dtype_code(A), epi, A.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K,
                               A.stride(0), W.stride(0), out.stride(0), _stream(A)), "gemm_16")
    return out


class Session:
    """Greedy-decoding session over caller-owned weights.

    weights: {"embed_tokens", "lm_head", "final_norm": tensors, "layers": [ {Wq, Wk, Wv, Wo, Wgate, Wup, Wdown,
    norm_attn, norm_mlp[, bq, bk, bv]} ... ]}, all CUDA tensors of one 16-bit dtype, nn.Linear layout [out, in].
    cfg: dict with the ModelConfig fields.  The session keeps the tensors alive."""

    @classmethod
    def from_model(cls, model: "Model", max_seq: int, batch: int):
        """Session over a Model loaded from disk (Session(model_dir, max_seq) of the reference)."""
        import torch
        self = cls.__new__(cls)
        self._weights = model                       # keeps the device memory alive
        self.cfg, self.batch, self.max_seq = dict(model.cfg), batch, max_seq
        st = _i(0)
        self._h = lib().b200p_session_create(C.byref(model.weights), max_seq, batch, C.byref(st))
        if not self._h:
            raise B200PError(st.value, "session_create")
        self._device = torch.device("cuda", torch.cuda.current_device())
        return self

    def __init__(self, cfg: dict, weights: dict, max_seq: int, batch: int):
        self._weights = weights
        self.cfg, self.batch, self.max_seq = dict(cfg), batch, max_seq
        layers = (LayerWeights * cfg["n_layers"])()
        for i, lw in enumerate(weights["layers"]):
            for n in _LAYER_FIELDS:
                t = lw.get(n)
                setattr(layers[i], n, _dev(t, n).data_ptr() if t is not None else None)
        self._layers = layers
        mc = ModelConfig(cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"],
                         cfg["ffn_dim"], cfg["vocab_size"], float(cfg.get("rope_theta", 10000.0)))
        mw = ModelWeights(mc, _dtype_code(weights["embed_tokens"]), _dev(weights["embed_tokens"], "embed_tokens").data_ptr(),
                          _dev(weights["lm_head"], "lm_head").data_ptr(), _dev(weights["final_norm"], "final_norm").data_ptr(),
                          layers)
        st = _i(0)
        self._h = lib().b200p_session_create(C.byref(mw), max_seq, batch, C.byref(st))
        if not self._h:
            raise B200PError(st.value, "session_create")
        self._device = weights["embed_tokens"].device

    def close(self):
        if getattr(self, "_h", None) and lib is not None:        # `lib` is gone when the interpreter is shutting down
            lib().b200p_session_destroy(self._h)
            self._h = None

    __del__ = close

    def _ids(self, ids):
        import numpy as np
        a = np.ascontiguousarray(ids, dtype=np.int32)
        return a

    def generate(self, input_ids, max_new_tokens: int):
        """input_ids [batch, T] (host ints) -> (tokens [batch, max_new_tokens] numpy int32,
        (ttft_ms, decode_ms))."""
        import numpy as np
        import torch
        a = self._ids(input_ids).reshape(self.batch, -1)
        out = np.zeros((self.batch, max_new_tokens), np.int32)
        tm = (C.c_float * 2)()
        _check(lib().b200p_session_generate(self._h, a.ctypes.data, a.shape[1], max_new_tokens, out.ctypes.data, tm,
                                            torch.cuda.current_stream(self._device).cuda_stream), "session_generate")
        return out, (tm[0], tm[1])

    def prefill_logits(self, input_ids):
        import numpy as np
        import torch
        a = self._ids(input_ids).reshape(self.batch, -1)
        out = np.zeros((self.batch, self.cfg["vocab_size"]), np.float32)
        _check(lib().b200p_session_prefill_logits(self._h, a.ctypes.data, a.shape[1], out.ctypes.data,
                                                  torch.cuda.current_stream(self._device).cuda_stream), "session_prefill_logits")
        return out

    def step_logits(self, token_ids):
        import numpy as np
        import torch
        a = self._ids(token_ids).reshape(self.batch)
        out = np.zeros((self.batch, self.cfg["vocab_size"]), np.float32)
        _check(lib().b200p_session_step_logits(self._h, a.ctypes.data, out.ctypes.data,
                                               torch.cuda.current_stream(self._device).cuda_stream), "session_step_logits")
        return out

    @property
    def kv_len(self) -> int:
        return int(lib().b200p_session_kv_len(self._h))

    @property
    def gemm_calls(self) -> int:
        return int(lib().b200p_session_gemm_calls(self._h))

    @property
    def blas_calls(self) -> int:
        return int(lib().b200p_session_blas_calls(self._h))

    @property
    def graph_replays(self) -> int:
        return int(lib().b200p_session_graph_replays(self._h))

    @property
    def mega_launches(self) -> int:
        """Launches of the persistent decode kernel (all decode steps of a generate() call in one)."""
        return int(lib().b200p_session_mega_launches(self._h))
