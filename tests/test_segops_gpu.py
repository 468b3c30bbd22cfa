"""Parity of the CUDA segmented reduce/scan (through the C ABI) with the oracle.
Everything is bit-exact: integers, max/min, fp32/fp64 sums and scans in the reference's DPP
association, 16-bit sums and scans in the fp32 shuffle association its 16-bit overloads use."""
import numpy as np
import pytest

import oracle as orc

pytestmark = pytest.mark.gpu

NP = {"f32": np.float32, "f64": np.float64, "i32": np.int32, "i64": np.int64}
SIZES = [64, 64 * 3, 64 * 31, 64 * 1025, 64 * 40000 + 64]


def gen(kind, n, seed):
    rng = np.random.default_rng(seed)
    if kind in ("i32", "i64"):
        return rng.integers(-1000, 1001, n).astype(NP[kind])      # uniform in [-1000, 1000]
    return rng.standard_normal(n).astype(NP.get(kind, np.float32))


def to_dev(torch, a):
    return torch.from_numpy(a).cuda()


def narrow_dev(torch, bits, kind):
    t = torch.from_numpy(bits.view(np.int16)).cuda()
    return t.view(torch.float16 if kind == "f16" else torch.bfloat16)


def narrow_bits(torch, t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("vec_bytes", [16, 32])
@pytest.mark.parametrize("kind", ["f32", "f64", "i32", "i64"])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_reduce_bit_exact(b200p, torch_cuda, kind, op, vec_bytes):
    torch = torch_cuda
    b200p.set_tuning("seg_vec_bytes", vec_bytes)
    try:
        for n in SIZES:
            x = gen(kind, n, n % 1000 + 1)
            got = b200p.segreduce(to_dev(torch, x), op).cpu().numpy()
            assert np.array_equal(got, orc.dpp_reduce(orc.OPS[op], x, threads=8)), (kind, op, n)
    finally:
        b200p.set_tuning("seg_vec_bytes", -1)


@pytest.mark.parametrize("vec_bytes", [16, 32])
@pytest.mark.parametrize("kind", ["f32", "f64", "i32", "i64"])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_scan_bit_exact(b200p, torch_cuda, kind, op, vec_bytes):
    torch = torch_cuda
    b200p.set_tuning("seg_vec_bytes", vec_bytes)
    try:
        for n in SIZES:
            x = gen(kind, n, n % 1000 + 2)
            got = b200p.segscan(to_dev(torch, x), op).cpu().numpy()
            assert np.array_equal(got, orc.dpp_scan(orc.OPS[op], x, threads=8)), (kind, op, n)
            if op == "sum":
                got = b200p.segscan(to_dev(torch, x), exclusive=True).cpu().numpy()
                assert np.array_equal(got, orc.dpp_scan(orc.SUM, x, exclusive=True, threads=8)), (kind, n)
    finally:
        b200p.set_tuning("seg_vec_bytes", -1)


@pytest.mark.parametrize("kind", ["f32", "f64"])
def test_scan_fast_mode_within_tolerance(b200p, torch_cuda, kind):
    torch = torch_cuda
    b200p.set_tuning("scan_fp_exact", 0)
    try:
        x = gen(kind, 64 * 5000, 77)
        got = b200p.segscan(to_dev(torch, x), "sum").cpu().numpy().reshape(-1, 64)
        seg = x.reshape(-1, 64).astype(np.float64)
        # tolerance: 1e-6 relative to sum|x| of the segment (plain relative error is
        # meaningless for N(0,1) data, whose partial sums cancel)
        assert (np.abs(got - np.cumsum(seg, axis=1)) <= 1e-6 * np.abs(seg).sum(axis=1)[:, None]).all()
    finally:
        b200p.set_tuning("scan_fp_exact", -1)


@pytest.mark.parametrize("vec_bytes", [16, 32])
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_reduce_16bit_fp32_accumulation(b200p, torch_cuda, kind, vec_bytes):
    torch = torch_cuda
    bf = kind == "bf16"
    b200p.set_tuning("seg_vec_bytes", vec_bytes)
    try:
        for n in SIZES:
            f = gen("f32", n, n % 1000 + 3)
            bits = orc.f32_to_bf16_bits(f) if bf else orc.f32_to_f16_bits(f)
            xr = (orc.bf16_bits_to_f32(bits) if bf else orc.f16_bits_to_f32(bits)).reshape(-1, 64).astype(np.float64)
            xd = narrow_dev(torch, bits, kind)
            for op in ("max", "min"):
                ref_f, ref_n = orc.shfl_reduce_narrow(orc.OPS[op], bits, bf, threads=8)
                assert np.array_equal(b200p.segreduce(xd, op).cpu().numpy(), ref_f)
                assert np.array_equal(narrow_bits(torch, b200p.segreduce(xd, op, narrow=True)), ref_n)
            # sum: the reference's fp32 shfl_down association (elements i and i + 32 first), bit for bit
            ref_f, ref_n = orc.shfl_reduce_narrow(orc.SUM, bits, bf, threads=8)
            got = b200p.segreduce(xd, "sum").cpu().numpy()
            assert np.array_equal(got, ref_f), (kind, n)
            assert np.array_equal(narrow_bits(torch, b200p.segreduce(xd, "sum", narrow=True)), ref_n), (kind, n)
            # and, as north-star asks of every fp reduce, within 1e-6 * sum|x| of the float64 value
            assert (np.abs(got.astype(np.float64) - xr.sum(axis=1)) <= 1e-6 * np.abs(xr).sum(axis=1)).all()
    finally:
        b200p.set_tuning("seg_vec_bytes", -1)


@pytest.mark.parametrize("lane_form", [1, 0], ids=["segment-per-lane", "four-lanes"])
@pytest.mark.parametrize("vec_bytes", [16, 32])
@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_scan_16bit_bit_exact(b200p, torch_cuda, kind, op, vec_bytes, lane_form):
    """Both forms of the 16-bit scan (a whole segment per lane, the default, and a segment
    spread over four lanes) give the reference's fp32 Hillis-Steele result bit for bit."""
    torch = torch_cuda
    bf = kind == "bf16"
    b200p.set_tuning("seg_vec_bytes", vec_bytes)
    b200p.set_tuning("scan16_lane", lane_form)
    try:
        for n in SIZES:
            f = gen("f32", n, n % 1000 + 4)
            bits = orc.f32_to_bf16_bits(f) if bf else orc.f32_to_f16_bits(f)
            got = narrow_bits(torch, b200p.segscan(narrow_dev(torch, bits, kind), op))
            assert np.array_equal(got, orc.shfl_scan_narrow(orc.OPS[op], bits, bf, threads=8)), (kind, op, n)
    finally:
        b200p.set_tuning("seg_vec_bytes", -1)
        b200p.set_tuning("scan16_lane", -1)


def test_wave_probe_known_answers(b200p, torch_cuda):
    """The reference's probe vectors through the device-level pair API:
    bench_reduce_dpp_types.hip:53-82 and probe_scan_dpp.hip:13-47."""
    torch = torch_cuda
    for dt in (torch.float32, torch.float64, torch.int32, torch.int64):
        lane = torch.arange(64, device="cuda").to(dt)
        ones = torch.ones(64, device="cuda", dtype=dt)
        assert (b200p.wave_probe(lane, "reduce", "sum") == 2016).all()
        assert (b200p.wave_probe(lane, "reduce", "max") == 63).all()
        assert (b200p.wave_probe(lane, "reduce", "min") == 0).all()
        assert torch.equal(b200p.wave_probe(ones, "scan", "sum"), lane + 1)
        assert torch.equal(b200p.wave_probe(lane, "scan", "max"), lane)
        assert (b200p.wave_probe(lane, "scan", "min") == 0).all()
        assert torch.equal(b200p.wave_probe(ones, "scan_exclusive", "sum"), lane)
    # 64 x fp16(0.1) with fp32 accumulation (bench_all_types.hip:95-127)
    h = torch.full((64,), 0.1, device="cuda", dtype=torch.float16)
    r = b200p.wave_probe(h, "reduce", "sum")
    assert float(r[0]) == float(np.float16(64 * float(np.float16(0.1))))
    b = torch.ones(64, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(b200p.wave_probe(b, "scan", "sum").float(), torch.arange(1, 65, device="cuda").float())


@pytest.mark.parametrize("kind", ["f32", "f64", "i32", "i64"])
def test_pair_per_lane_api_on_random_data(b200p, torch_cuda, kind):
    """The drop-in device API itself -- wave::dpp::reduce_*(a, b), scan_*(a, b): lane l holds elements 2l
    and 2l+1 of the wave; the only place redux.sync is used -- on seeded N(0,1) / U[-1000,1000] data,
    4099 waves, bit-exact against the DPP-order oracle (wave_reduce_dpp.hpp:106-113, wave_scan_dpp.hpp:70-87)."""
    torch = torch_cuda
    x = gen(kind, 64 * 4099, 31)
    xd = to_dev(torch, x)
    for op in ("sum", "max", "min"):
        got = b200p.wave_probe(xd, "reduce", op).cpu().numpy().reshape(-1, 64)
        ref = orc.dpp_reduce(orc.OPS[op], x, threads=8)
        assert np.array_equal(got, np.repeat(ref[:, None], 64, axis=1)), (kind, op)       # every lane holds the result
        assert np.array_equal(b200p.wave_probe(xd, "scan", op).cpu().numpy(), orc.dpp_scan(orc.OPS[op], x, threads=8)), (kind, op)
    assert np.array_equal(b200p.wave_probe(xd, "scan_exclusive", "sum").cpu().numpy(), orc.dpp_scan(orc.SUM, x, exclusive=True, threads=8))


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_pair_per_lane_api_16bit_on_random_data(b200p, torch_cuda, kind):
    """wave::reduce_sum/max/min(__half | bf16 pair) and scan_inclusive_sum: fp32 inside, the reference's
    shuffle association (wave_reduce.hpp:48-119, wave_scan.hpp:52-74), rounded to the input type."""
    torch = torch_cuda
    bf = kind == "bf16"
    f = gen("f32", 64 * 2053, 32)
    bits = orc.f32_to_bf16_bits(f) if bf else orc.f32_to_f16_bits(f)
    xd = narrow_dev(torch, bits, kind)
    for op in ("sum", "max", "min"):
        _, ref_n = orc.shfl_reduce_narrow(orc.OPS[op], bits, bf, threads=8)
        got = narrow_bits(torch, b200p.wave_probe(xd, "reduce", op)).reshape(-1, 64)
        assert np.array_equal(got, np.repeat(ref_n[:, None], 64, axis=1)), (kind, op)
    got = narrow_bits(torch, b200p.wave_probe(xd, "scan", "sum"))
    assert np.array_equal(got, orc.shfl_scan_narrow(orc.SUM, bits, bf, threads=8))


def test_vote_and_bitwise_wrappers(b200p, torch_cuda):
    """ballot / any / all / popcount / reduce_and / reduce_or on a pair per lane
    (research/wave-primitives/tests/test_correctness.hip:226-256: even lanes vote -> mask 0x5555...)."""
    torch = torch_cuda
    lane = torch.arange(64, device="cuda", dtype=torch.int32)
    even = ((lane % 2) == 0).int()                               # elements 0, 2, 4, ... vote
    r = b200p.wave_vote_probe(even).cpu().numpy().astype(np.uint64)
    assert r[0] == np.uint64(0x5555555555555555) and r[1] == 1 and r[2] == 0 and r[3] == 32
    assert r[6] == np.uint64(0xFFFFFFFF) and r[7] == np.uint64(0b11111)
    rng = np.random.default_rng(3)
    v = rng.integers(-5, 1 << 20, 64).astype(np.int32)
    r = b200p.wave_vote_probe(torch.from_numpy(v).cuda()).cpu().numpy().astype(np.uint64)
    want = sum(1 << i for i in range(64) if v[i] > 0)
    assert int(r[0]) == want and int(r[3]) == bin(want).count("1")
    assert int(r[4]) == int(np.bitwise_and.reduce(v.view(np.uint32))) and int(r[5]) == int(np.bitwise_or.reduce(v.view(np.uint32)))
    ones = torch.ones(64, device="cuda", dtype=torch.int32)
    r = b200p.wave_vote_probe(ones).cpu().numpy()
    assert r[1] == 1 and r[2] == 1 and r[3] == 64


def test_misaligned_input_takes_16_byte_path(b200p, torch_cuda):
    torch = torch_cuda
    x = gen("f32", 64 * 999 + 4, 5)
    xd = to_dev(torch, x)[4:]                       # 16-byte aligned, not 32
    assert xd.data_ptr() % 32 == 16
    assert np.array_equal(b200p.segreduce(xd, "sum").cpu().numpy(), orc.dpp_reduce(orc.SUM, x[4:]))
    assert np.array_equal(b200p.segscan(xd, "sum").cpu().numpy(), orc.dpp_scan(orc.SUM, x[4:]))
    with pytest.raises(b200p.B200PError) as e:
        b200p.segreduce(to_dev(torch, x)[1:64 * 999 + 1], "sum")
    assert e.value.status == -5
    with pytest.raises(b200p.B200PError) as e:
        b200p.segreduce(to_dev(torch, x)[:100], "sum")
    assert e.value.status == -4
    assert b200p.segreduce(to_dev(torch, x)[:0], "sum").numel() == 0


def test_full_size_sweep_properties(b200p, torch_cuda):
    """2^26 elements: f32 sum against the oracle in full, then size-independent
    properties: scan's last element == reduce (bitwise, same tree? no: within
    tolerance), scan(max) is non-decreasing, exclusive == inclusive shifted,
    integer linearity reduce(a+b) == reduce(a)+reduce(b), three runs identical."""
    torch = torch_cuda
    n = 1 << 26
    x = gen("f32", n, 2026)
    xd = to_dev(torch, x)
    r = b200p.segreduce(xd, "sum")
    assert np.array_equal(r.cpu().numpy(), orc.dpp_reduce(orc.SUM, x, threads=8))
    for _ in range(2):
        assert torch.equal(b200p.segreduce(xd, "sum"), r)
    inc = b200p.segscan(xd, "sum")
    exc = b200p.segscan(xd, exclusive=True)
    a = inc.view(-1, 64); e = exc.view(-1, 64)
    assert torch.equal(e[:, 1:], a[:, :-1]) and not e[:, 0].any()
    seg_abs = xd.view(-1, 64).abs().double().sum(dim=1)
    assert ((a[:, -1].double() - r.double()).abs() <= 1e-6 * seg_abs).all()
    mx = b200p.segscan(xd, "max").view(-1, 64)
    assert (mx[:, 1:] >= mx[:, :-1]).all() and torch.equal(mx[:, -1], b200p.segreduce(xd, "max"))
    del inc, exc, mx, a, e
    ia = torch.randint(-1000, 1001, (n,), device="cuda", dtype=torch.int64)
    ib = torch.randint(-1000, 1001, (n,), device="cuda", dtype=torch.int64)
    assert torch.equal(b200p.segreduce(ia + ib, "sum"), b200p.segreduce(ia, "sum") + b200p.segreduce(ib, "sum"))
    assert torch.equal(b200p.segreduce(ia, "sum"), ia.view(-1, 64).sum(dim=1))
    assert torch.equal(b200p.segscan(ia, "sum"), ia.view(-1, 64).cumsum(dim=1).view(-1))
