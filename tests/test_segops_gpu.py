"""Parity of the CUDA segmented reduce/scan (through the C ABI) with the oracle.
Integers, max/min, fp32/fp64 sums and all scans: bit-exact.  16-bit sums: within
1e-6 * sum|x| of the float64 value (the kernel's fp32 association differs from the
reference's shuffle order)."""
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
            got = b200p.segreduce(xd, "sum").cpu().numpy().astype(np.float64)
            bound = 1e-6 * np.abs(xr).sum(axis=1)
            assert (np.abs(got - xr.sum(axis=1)) <= bound).all()
            # the oracle's shuffle-order fp32 value obeys the same bound, so the two agree to 2 bounds
            ref_f, ref_n = orc.shfl_reduce_narrow(orc.SUM, bits, bf, threads=8)
            assert (np.abs(got - ref_f) <= 2 * bound).all()
            # rounded to the input type: equal, or one unit in the last place apart where fp32 order tipped the rounding
            gn = narrow_bits(torch, b200p.segreduce(xd, "sum", narrow=True))
            differ = gn != ref_n
            assert differ.mean() < 0.01
            gv = orc.bf16_bits_to_f32(gn) if bf else orc.f16_bits_to_f32(gn)
            rv = orc.bf16_bits_to_f32(ref_n) if bf else orc.f16_bits_to_f32(ref_n)
            ulp = np.maximum(np.abs(rv), 1e-3) * (2.0 ** -7 if bf else 2.0 ** -10)
            assert (np.abs(gv - rv) <= ulp).all()
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
