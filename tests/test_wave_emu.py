"""The cross-lane logic of include/wave_primitives/wave64.cuh, executed on a host
warp shim (32 lockstep threads, tests/emu/), against the oracle's emulation of
the reference's DPP / shuffle association.  Bit-exact.  No GPU."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
FN_REDUCE, FN_SCAN_DPP, FN_SCAN_FAST, FN_SCAN_KS64, FN_SCAN_EXCL = 0, 1, 2, 3, 4
DT = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 2, np.dtype(np.int64): 3}


@pytest.fixture(scope="module")
def emu():
    so = os.path.join(HERE, "emu", "libwave64_emu.so")
    src = os.path.join(HERE, "emu", "wave64_emu.cpp")
    hdr = os.path.join(ROOT, "include", "wave_primitives", "wave64.cuh")
    shim = os.path.join(HERE, "emu", "warp_shim.hpp")
    if not os.path.exists(so) or os.path.getmtime(so) < max(map(os.path.getmtime, (src, hdr, shim))):
        subprocess.run(["g++", "-O1", "-std=c++20", "-pthread", "-shared", "-fPIC", "-ffp-contract=off",
                        "-I" + os.path.join(ROOT, "include"),
                        '-DWAVE64_HOST_EMULATION="../../tests/emu/warp_shim.hpp"', src, "-o", so], check=True)
    return C.CDLL(so)


def data(dt, n, seed):
    rng = np.random.default_rng(seed)
    if np.issubdtype(dt, np.integer):
        return rng.integers(-1000, 1001, n).astype(dt)
    return rng.standard_normal(n).astype(dt)


def run(emu, fn, op, x, vec):
    out = np.empty_like(x)
    assert emu.emu_run(fn, op, DT[x.dtype], vec, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)) == 0
    return out


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32, np.int64])
@pytest.mark.parametrize("vec", [2, 4, 8, 16])
@pytest.mark.parametrize("op", [orc.SUM, orc.MAX, orc.MIN])
def test_segment_reduce(emu, dt, vec, op):
    x = data(dt, 32 * vec, 10 + vec)
    got = run(emu, FN_REDUCE, op, x, vec).reshape(-1, 64)
    ref = orc.dpp_reduce(op, x)
    assert np.array_equal(got, np.repeat(ref[:, None], 64, axis=1))     # every lane, bit-exact


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32, np.int64])
@pytest.mark.parametrize("vec", [2, 4, 8, 16])
@pytest.mark.parametrize("op", [orc.SUM, orc.MAX, orc.MIN])
def test_segment_scan_dpp_order(emu, dt, vec, op):
    x = data(dt, 32 * vec, 20 + vec)
    assert np.array_equal(run(emu, FN_SCAN_DPP, op, x, vec), orc.dpp_scan(op, x))
    if op == orc.SUM:
        assert np.array_equal(run(emu, FN_SCAN_EXCL, op, x, vec), orc.dpp_scan(op, x, exclusive=True))


@pytest.mark.parametrize("dt", [np.int32, np.int64])
@pytest.mark.parametrize("vec", [2, 4, 8, 16])
@pytest.mark.parametrize("op", [orc.SUM, orc.MAX, orc.MIN])
def test_segment_scan_fast_ints(emu, dt, vec, op):
    x = data(dt, 32 * vec, 30 + vec)
    assert np.array_equal(run(emu, FN_SCAN_FAST, op, x, vec), orc.dpp_scan(op, x))


@pytest.mark.parametrize("vec", [2, 4, 8, 16])
def test_scan_fast_float_within_tolerance(emu, vec):
    x = data(np.float32, 32 * vec, 40 + vec)
    got = run(emu, FN_SCAN_FAST, orc.SUM, x, vec).reshape(-1, 64)
    seg = x.reshape(-1, 64).astype(np.float64)
    assert (np.abs(got - np.cumsum(seg, axis=1)) <= 1e-6 * np.abs(seg).sum(axis=1)[:, None]).all()


@pytest.mark.parametrize("vec", [2, 4, 8, 16])
@pytest.mark.parametrize("op", [orc.SUM, orc.MAX, orc.MIN])
def test_kogge_stone_64_is_portable_scan(emu, vec, op):
    """row_scan_kogge_stone<VEC,64> on floats == the reference's Hillis-Steele scan of
    16-bit inputs accumulated in fp32 (wave_scan.hpp:52-74), checked through fp16."""
    x = orc.round_to(data(np.float32, 32 * vec, 50 + vec), "f16")
    got = orc.f32_to_f16_bits(run(emu, FN_SCAN_KS64, op, x, vec))
    ref = orc.shfl_scan_narrow(op, orc.f32_to_f16_bits(x), bf16=False)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("op", [orc.SUM, orc.MAX, orc.MIN])
def test_lane_serial_kogge_stone_is_portable_scan(emu, op, kind):
    """lane_scan_kogge_stone<64> (one lane holds the whole segment, as the 16-bit array scan does)
    gives the bits of the reference's fp32 Hillis-Steele scan over 64 lanes (wave_scan.hpp:52-74)."""
    bf = kind == "bf16"
    x = orc.round_to(data(np.float32, 32 * 64, 90 + op), kind)
    out = np.empty_like(x)
    assert emu.emu_lane_scan(op, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)) == 0
    bits = orc.f32_to_bf16_bits(x) if bf else orc.f32_to_f16_bits(x)
    got = orc.f32_to_bf16_bits(out) if bf else orc.f32_to_f16_bits(out)
    assert np.array_equal(got, orc.shfl_scan_narrow(op, bits, bf16=bf))


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32, np.int64])
def test_pair_api_known_answers(emu, dt):
    """The public wave::dpp:: pair API on the reference's probe vectors
    (probe_scan_dpp.hip:13-47, bench_reduce_dpp_types.hip:53-82)."""
    def pair(fn2, op, x):
        out = np.empty_like(x)
        assert emu.emu_pair(fn2, op, DT[x.dtype], x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)) == 0
        return out
    lane = np.arange(64).astype(dt); ones = np.ones(64, dt)
    assert np.array_equal(pair(0, orc.SUM, lane), np.full(64, 2016, dt))
    assert np.array_equal(pair(0, orc.MAX, lane), np.full(64, 63, dt))
    assert np.array_equal(pair(0, orc.MIN, lane), np.zeros(64, dt))
    assert np.array_equal(pair(1, orc.SUM, ones), (np.arange(64) + 1).astype(dt))
    assert np.array_equal(pair(1, orc.MAX, lane), lane)
    assert np.array_equal(pair(1, orc.MIN, lane), np.zeros(64, dt))
    assert np.array_equal(pair(2, orc.SUM, ones), lane)
