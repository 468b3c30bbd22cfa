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
}


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


def wave_probe(x64, fn: str = "reduce", op: str = "sum"):
    """One wave64 through the device-level pair-per-lane API."""
    import torch
    _dev(x64, "x64")
    assert x64.numel() == 64
    out = torch.empty_like(x64)
    code = {"reduce": 0, "scan": 1, "scan_exclusive": 2}[fn]
    _check(lib().b200p_wave_probe(code, OPS[op], _dtype_code(x64), x64.data_ptr(), out.data_ptr(), _stream(x64)), "wave_probe")
    return out
