"""The device-level facade a caller of the reference compiles against -- <cdna3/cdna3.hpp>,
cdna3::ex::row_softmax_lane / online_softmax_step (cdna3-prims/examples/fused_softmax.hpp:26-48)
and the per-thread asynchronous copy API dme::copy_tile_1d_stream / AsyncTile2D
(research/dme-abstraction/include/dme/dme_copy.hpp:133-160, tensor_prefetch.hpp:151-196) -- run
on the GPU by kernels that only include those headers (csrc/api_probe.cu), through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def softmax64(x):
    x = x.astype(np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


@pytest.mark.parametrize("width,which", [(64, 0), (32, 1)])
def test_row_softmax_lane(b200p, torch_cuda, width, which):
    torch = torch_cuda
    rows = 1237
    x = (np.random.default_rng(width).standard_normal((rows, width)) * 3).astype(np.float32)
    got = b200p.api_probe(which, torch.from_numpy(x).cuda(), rows).cpu().numpy().reshape(rows, width)
    assert np.abs(got - softmax64(x)).max() < 1e-6
    assert np.abs(got.sum(axis=1) - 1).max() < 1e-5


def test_online_softmax_step_streams_to_the_same_result(b200p, torch_cuda):
    torch = torch_cuda
    rows, tiles = 515, 7
    x = (np.random.default_rng(1).standard_normal((rows, tiles * 64)) * 4).astype(np.float32)
    got = b200p.api_probe(2, torch.from_numpy(x).cuda(), rows, tiles, out_elems=rows * 3).cpu().numpy().reshape(rows, 3)
    m = x.max(axis=1).astype(np.float64)
    l = np.exp(x.astype(np.float64) - m[:, None]).sum(axis=1)
    assert np.array_equal(got[:, 0], x.max(axis=1))
    assert np.abs(got[:, 1] / l - 1).max() < 1e-5               # the running denominator
    assert np.abs(got[:, 2] / l - 1).max() < 1e-5               # an accumulator rescaled by the returned factors


def test_async_tile_ping_pong_and_tile_1d(b200p, torch_cuda):
    torch = torch_cuda
    tiles = 9
    h = torch.randn(tiles, 16 * 64, device="cuda").half()
    got = b200p.api_probe(3, h, 1, tiles).view(tiles, -1)
    assert torch.equal(got, 2 * h.float())
    f = torch.randn(11, 256, device="cuda")
    got = b200p.api_probe(4, f, 1, 11).view(11, 256)
    assert torch.equal(got, f + 1)


@pytest.mark.parametrize("backend", ["primitives", "portable"])
@pytest.mark.parametrize("dt", ["float32", "float64", "int32", "int64"])
def test_register_resident_reduce_loop(b200p, torch_cuda, dt, backend):
    """The reference's microbenchmark loop (bench_reduce_dpp_types.hip:29-45) computes what a host loop computes:
    integer-valued data keeps every type exact."""
    torch = torch_cuda
    dtype = getattr(torch, dt)
    waves, reps = 64, 5
    x = (torch.arange(64 * waves, device="cuda") % 7).to(dtype)
    lane = torch.arange(64, device="cuda").to(dtype) + 1
    for op, fn in (("sum", lambda t: t.sum(dim=1)), ("max", lambda t: t.max(dim=1).values), ("min", lambda t: t.min(dim=1).values)):
        got = b200p.wave_reduce_loop(x, op, reps, backend)
        v, acc = x.view(waves, 64).clone(), torch.zeros(waves, device="cuda", dtype=dtype)
        for _ in range(reps):
            s = fn(v).to(dtype)                                 # the kernel's arithmetic wraps in the element type
            acc = acc + s
            v = (s[:, None] + lane[None, :]).to(dtype)
        assert torch.equal(got, acc), (dt, op)


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_register_resident_reduce_loop_16bit_fp32_accumulation(b200p, torch_cuda, dt):
    """16-bit inputs, fp32 accumulation, one rounding (wave::reduce_sum on a 16-bit pair) against the same in torch;
    the small integer values keep both exact."""
    torch = torch_cuda
    dtype = getattr(torch, dt)
    waves, reps = 64, 5
    x = (torch.arange(64 * waves, device="cuda") % 7).to(dtype)
    got = b200p.wave_reduce_loop(x, "sum", reps, "primitives")
    v, acc = x.view(waves, 64).clone(), torch.zeros(waves, device="cuda", dtype=torch.float32)
    idx = torch.arange(64, device="cuda")
    for _ in range(reps):
        s = v.float().sum(dim=1).to(dtype)
        acc = acc + s.float()
        dep = (s.float() > 100.0).to(dtype)
        v = ((idx % 5).to(dtype)[None, :] + dep[:, None]).to(dtype)
    assert torch.equal(got, acc.to(dtype)), dt
    native = b200p.wave_reduce_loop(x, "sum", reps, "portable")               # 16-bit accumulation: same here, the sums are small integers
    assert torch.equal(native, got), dt


@pytest.mark.parametrize("backend", ["primitives", "portable"])
@pytest.mark.parametrize("dt", ["float32", "float64", "int32", "int64"])
def test_register_resident_scan_loop(b200p, torch_cuda, dt, backend):
    """The scan loop computes what a host loop computes (small integer-valued data: exact in every type)."""
    torch = torch_cuda
    dtype = getattr(torch, dt)
    waves, reps = 64, 4
    x = (torch.arange(64 * waves, device="cuda") % 3).to(dtype) - 1          # -1, 0, 1: totals of either sign
    got = b200p.wave_scan_loop(x, reps, backend).view(waves, 64)
    v = x.view(waves, 64).clone()
    acc = torch.zeros(waves, 32, device="cuda", dtype=dtype)                 # per lane: sum of its second element over the rounds
    idx = torch.arange(64, device="cuda")
    for _ in range(reps):
        sc = torch.cumsum(v, dim=1).to(dtype)
        acc = acc + sc[:, 1::2]
        dep = (sc[:, 63:64] > 0).to(dtype)
        v = ((idx % 5).to(dtype)[None, :] + dep).to(dtype)
    assert torch.equal(got[:, 1::2], v[:, 1::2]), dt
    assert torch.equal(got[:, 0::2], v[:, 0::2] + acc), dt


@pytest.mark.parametrize("backend", ["primitives", "portable"])
@pytest.mark.parametrize("cols", [64, 512])
def test_layernorm_and_softmax_rows(b200p, torch_cuda, cols, backend):
    torch = torch_cuda
    g = torch.Generator(device="cuda"); g.manual_seed(cols)
    x = torch.randn(4099, cols, device="cuda", generator=g) * 3
    gamma, beta = torch.randn(cols, device="cuda", generator=g), torch.randn(cols, device="cuda", generator=g)
    ln = b200p.row_op("layernorm", x, gamma, beta, backend)
    ref = torch.nn.functional.layer_norm(x.double(), (cols,), gamma.double(), beta.double(), 1e-5)
    assert (ln.double() - ref).abs().max().item() < 2e-5
    sm = b200p.row_op("softmax", x, backend=backend)
    assert (sm.double() - torch.softmax(x.double(), dim=1)).abs().max().item() < 1e-6
