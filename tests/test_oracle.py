"""The CPU oracle against every known-answer vector the reference's tests hold for
the wave primitives, plus self-consistency of its helpers.  No GPU."""
import numpy as np
import pytest

import oracle as orc

TYPES = [np.float32, np.float64, np.int32, np.int64]


# research/wave-primitives/benchmarks/bench_reduce_dpp_types.hip:53-82 --
# values i % 64 -> sum 2016, max 63, min 0, for f32/f64/i32/i64.
@pytest.mark.parametrize("dt", TYPES)
def test_reduce_lanes_0_63(dt):
    x = (np.arange(64 * 5) % 64).astype(dt)
    assert np.array_equal(orc.dpp_reduce(orc.SUM, x), np.full(5, 2016, dt))
    assert np.array_equal(orc.dpp_reduce(orc.MAX, x), np.full(5, 63, dt))
    assert np.array_equal(orc.dpp_reduce(orc.MIN, x), np.full(5, 0, dt))


# research/wave-primitives/tests/probe_scan_dpp.hip:13-47 -- ones -> i+1; v=lane -> max i,
# min 0; exclusive ones -> i; lane-by-lane, exact, four types.
@pytest.mark.parametrize("dt", TYPES)
def test_scan_probe_vectors(dt):
    ones = np.ones(64, dt)
    lane = np.arange(64).astype(dt)
    assert np.array_equal(orc.dpp_scan(orc.SUM, ones), (np.arange(64) + 1).astype(dt))
    assert np.array_equal(orc.dpp_scan(orc.MAX, lane), lane)
    assert np.array_equal(orc.dpp_scan(orc.MIN, lane), np.zeros(64, dt))
    assert np.array_equal(orc.dpp_scan(orc.SUM, ones, exclusive=True), np.arange(64).astype(dt))


# research/wave-primitives/tests/test_correctness.hip:130-224 -- portable API:
# sum of lane ids = W(W-1)/2, max = W-1, min of 1..64 = 1, scans of ones.
def test_portable_api_vectors():
    lane = np.arange(64, dtype=np.float32)
    assert orc.shfl_reduce_f32(orc.SUM, lane) == 2016.0
    assert orc.shfl_reduce_f32(orc.MAX, lane) == 63.0
    assert orc.shfl_reduce_f32(orc.MIN, lane + 1) == 1.0
    ones_h = orc.f32_to_f16_bits(np.ones(64, np.float32))
    inc = orc.f16_bits_to_f32(orc.shfl_scan_narrow(orc.SUM, ones_h, bf16=False))
    assert np.array_equal(inc, np.arange(1, 65, dtype=np.float32))
    ones_b = orc.f32_to_bf16_bits(np.ones(64, np.float32))
    inc = orc.bf16_bits_to_f32(orc.shfl_scan_narrow(orc.SUM, ones_b, bf16=True))
    assert np.array_equal(inc, np.arange(1, 65, dtype=np.float32))


# research/wave-primitives/benchmarks/bench_all_types.hip:95-127 -- 64 x fp16(0.1) summed
# in fp32: the reference records an error of 0.0016 against 6.4
# (research/wave-primitives/results/2026-06-05_h3_h4_multitype_mi300x.txt:15).
def test_fp16_accumulation_known_answer():
    h = orc.f32_to_f16_bits(np.full(64, 0.1, np.float32))
    f, narrow = orc.shfl_reduce_narrow(orc.SUM, h, bf16=False)
    exact = 64 * float(np.float16(0.1))
    assert f[0] == np.float32(exact)            # 64 equal values sum exactly in fp32
    assert abs(f[0] - 6.4) < 0.002 and abs(abs(f[0] - 6.4) - 0.0016) < 2e-4
    assert orc.f16_bits_to_f32(narrow)[0] == np.float32(np.float16(exact))


def test_f16_conversion_matches_numpy():
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 70000.0, -70000.0, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  2.0 ** -14, 2.0 ** -14 * 0.9999, np.inf, -np.inf, 1.0009765625, 1.00048828125], np.float32),
    ])
    with np.errstate(over="ignore"):
        ref = x.astype(np.float16)
    got = orc.f32_to_f16_bits(x)
    assert np.array_equal(got, ref.view(np.uint16))
    allh = np.arange(65536, dtype=np.uint16)
    back = orc.f16_bits_to_f32(allh)
    exp = allh.view(np.float16).astype(np.float32)
    ok = np.isnan(exp) | (back == exp)
    assert ok.all()
    assert np.array_equal(np.signbit(back), np.signbit(exp))


def test_bf16_conversion_round_to_nearest_even():
    import torch
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(50000) * 10.0 ** rng.integers(-20, 20, 50000)).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.f32_to_bf16_bits(x), ref)
    assert np.array_equal(orc.bf16_bits_to_f32(ref), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_reduce_sum_is_balanced_adjacent_tree(dt):
    """dpp_reduce's association is the balanced tree over adjacent pairs."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal(64 * 300).astype(dt)
    t = x.reshape(-1, 64).copy()
    while t.shape[1] > 1:
        t = (t[:, 1::2] + t[:, 0::2]).astype(dt)
    assert np.array_equal(orc.dpp_reduce(orc.SUM, x), t[:, 0])


@pytest.mark.parametrize("dt", TYPES)
def test_reduce_scan_vs_numpy(dt):
    rng = np.random.default_rng(4)
    if np.issubdtype(dt, np.integer):
        x = rng.integers(-1000, 1001, 64 * 257).astype(dt)
    else:
        x = rng.standard_normal(64 * 257).astype(dt)
    seg = x.reshape(-1, 64)
    assert np.array_equal(orc.dpp_reduce(orc.MAX, x), seg.max(axis=1))
    assert np.array_equal(orc.dpp_reduce(orc.MIN, x), seg.min(axis=1))
    assert np.array_equal(orc.dpp_scan(orc.MAX, x).reshape(-1, 64), np.maximum.accumulate(seg, axis=1))
    assert np.array_equal(orc.dpp_scan(orc.MIN, x).reshape(-1, 64), np.minimum.accumulate(seg, axis=1))
    ref_sum = seg.astype(np.float64).sum(axis=1) if not np.issubdtype(dt, np.integer) else seg.sum(axis=1)
    ref_scan = np.cumsum(seg.astype(np.float64), axis=1) if not np.issubdtype(dt, np.integer) else np.cumsum(seg, axis=1)
    got_sum, got_scan = orc.dpp_reduce(orc.SUM, x), orc.dpp_scan(orc.SUM, x).reshape(-1, 64)
    if np.issubdtype(dt, np.integer):
        assert np.array_equal(got_sum, ref_sum) and np.array_equal(got_scan, ref_scan)
        ex = orc.dpp_scan(orc.SUM, x, exclusive=True).reshape(-1, 64)
        assert np.array_equal(ex[:, 1:], ref_scan[:, :-1]) and not ex[:, 0].any()
    else:
        bound = 1e-6 * np.abs(seg).astype(np.float64).sum(axis=1)
        assert (np.abs(got_sum - ref_sum) <= bound).all()
        assert (np.abs(got_scan - ref_scan) <= bound[:, None]).all()


def test_int_sum_wraps():
    x = np.full(64, 2 ** 30, np.int32)
    assert orc.dpp_reduce(orc.SUM, x)[0] == np.int32((64 * 2 ** 30) % 2 ** 32)
    assert orc.dpp_scan(orc.SUM, x)[3] == np.int32(-(2 ** 32) + 4 * 2 ** 30) or orc.dpp_scan(orc.SUM, x)[3] == 0


def test_merge_forms_agree():
    """Split-KV merge on (O, m, l) equals the merge on normalised (O/l, lse)."""
    rng = np.random.default_rng(5)
    parts, rows, D = 5, 37, 64
    O = rng.standard_normal((parts, rows, D)).astype(np.float32)
    m = rng.standard_normal((parts, rows)).astype(np.float32) * 3
    l = rng.uniform(0.5, 50.0, (parts, rows)).astype(np.float32)
    a = orc.merge_partials(O, m, l)
    b, lse = orc.merge_lse(O / l[..., None], m + np.log(l))
    assert np.abs(a - b).max() < 1e-5
    ref_lse = np.log(np.sum(l.astype(np.float64) * np.exp(m.astype(np.float64)), axis=0))
    assert np.abs(lse - ref_lse).max() < 1e-5


def test_threads_do_not_change_results():
    rng = np.random.default_rng(6)
    x = rng.standard_normal(64 * 10000).astype(np.float32)
    assert np.array_equal(orc.dpp_reduce(orc.SUM, x, threads=1), orc.dpp_reduce(orc.SUM, x, threads=4))
    q, k, v = orc.gen_qkv_mt19937(42, 0.5, 2 * 4 * 32 * 64, 2 * 2 * 32 * 64)
    a = orc.cpu_prefill(q, k, v, 64, 32, 32, 4, 2, 2, 1, threads=1)
    b = orc.cpu_prefill(q, k, v, 64, 32, 32, 4, 2, 2, 1, threads=4)
    assert np.array_equal(a, b)
