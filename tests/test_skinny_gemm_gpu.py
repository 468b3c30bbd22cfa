"""The decode step's projection kernel (few rows of activations against a weight matrix,
with RMSNorm / SiLU / residual fused in) against a float64 statement of the same contract:
16-bit operands, fp32 accumulation, one rounding of the output."""
import numpy as np
import pytest

import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[1, 2], ids=["weights-in-registers", "weights-through-shared-memory"], autouse=True)
def skinny_kernel(b200p, request):
    """Every test runs on both kernels: W held in registers between load and MMA, and W staged
    through a shared-memory ring by a producer thread."""
    b200p.set_tuning("runtime_skinny", request.param)
    yield request.param
    b200p.set_tuning("runtime_skinny", -1)


def w16(torch, rng, shape, kind, scale=1.0):
    a = orc.round_to((rng.standard_normal(shape) * scale).astype(np.float32), kind)
    t = torch.from_numpy(a).cuda()
    return a.astype(np.float64), (t.bfloat16() if kind == "bf16" else t.half())


def rmsnorm16(x, w, kind, eps=1e-6):
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return orc.round_to((x * inv * w).astype(np.float32), kind).astype(np.float64)


# 9 .. 16 rows take the two-fragment kernels; (16, 2048, 5632) does not fit the staged kernel's shared memory
# beside X and goes to the register kernel whatever the knob says
SHAPES = [(1, 96, 64), (2, 2560, 2048), (3, 130, 528), (4, 2048, 5632), (8, 77, 1040), (5, 33, 16),
          (9, 130, 528), (12, 2560, 2048), (16, 2048, 5632), (16, 77, 1040), (13, 33, 16)]


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_norm_prologue_store_epilogues(b200p, torch_cuda, kind, M, N, K):
    torch = torch_cuda
    rng = np.random.default_rng(M * 1000 + N)
    Wf, W = w16(torch, rng, (N, K), kind, 0.05)
    nwf, nw = w16(torch, rng, (K,), kind)
    x = rng.standard_normal((M, K)).astype(np.float32)
    X = rmsnorm16(x.astype(np.float64), nwf, kind)
    ref = X @ Wf.T
    x32 = torch.from_numpy(x).cuda()
    dt = torch.bfloat16 if kind == "bf16" else torch.float16
    out32 = torch.full((M, N), 7.0, dtype=torch.float32, device="cuda")
    b200p.skinny_gemm(W, out32, x32=x32, norm_w=nw, epilogue="store32")
    scale = np.abs(ref).max()
    # a 1-ulp flip of a normalised 16-bit activation moves the sum a little: allow 2e-3 of the scale
    assert np.abs(out32.cpu().numpy() - ref).max() < 2e-3 * scale
    out16 = torch.zeros((M, N), dtype=dt, device="cuda")
    b200p.skinny_gemm(W, out16, x32=x32, norm_w=nw, epilogue="store16")
    ulp = 2.0 ** -8 if kind == "bf16" else 2.0 ** -11
    assert np.abs(out16.float().cpu().numpy() - ref).max() < (ulp + 2e-3) * scale


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_plain_prologue_residual_epilogue(b200p, torch_cuda, kind, M, N, K):
    torch = torch_cuda
    rng = np.random.default_rng(M * 77 + K)
    Wf, W = w16(torch, rng, (N, K), kind, 0.05)
    Xf, X = w16(torch, rng, (M, K), kind)
    res = rng.standard_normal((M, N)).astype(np.float32)
    out = torch.from_numpy(res.copy()).cuda()
    b200p.skinny_gemm(W, out, x16=X, epilogue="acc32")
    ref = res.astype(np.float64) + Xf @ Wf.T
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    # a strided activation matrix (rows of a wider buffer)
    wide = torch.zeros((M, K + 24), dtype=X.dtype, device="cuda")
    wide[:, :K] = X
    out2 = torch.from_numpy(res.copy()).cuda()
    b200p.skinny_gemm(W, out2, x16=wide[:, :K], epilogue="acc32")
    assert torch.equal(out, out2)


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("M,F,K", [(2, 5632, 2048), (1, 40, 64), (8, 300, 512), (11, 300, 512), (16, 5632, 2048)])
def test_silu_epilogue(b200p, torch_cuda, kind, M, F, K):
    torch = torch_cuda
    rng = np.random.default_rng(F)
    Wf, W = w16(torch, rng, (2 * F, K), kind, 0.05)
    nwf, nw = w16(torch, rng, (K,), kind)
    x = rng.standard_normal((M, K)).astype(np.float32)
    X = rmsnorm16(x.astype(np.float64), nwf, kind)
    g, u = X @ Wf[:F].T, X @ Wf[F:].T
    ref = g / (1.0 + np.exp(-g)) * u
    dt = torch.bfloat16 if kind == "bf16" else torch.float16
    out = torch.zeros((M, F), dtype=dt, device="cuda")
    b200p.skinny_gemm(W, out, x32=torch.from_numpy(x).cuda(), norm_w=nw, epilogue="silu16")
    ulp = 2.0 ** -8 if kind == "bf16" else 2.0 ** -11
    assert np.abs(out.float().cpu().numpy() - ref).max() < (ulp + 3e-3) * max(1e-3, np.abs(ref).max())


def test_shapes_outside_the_domain_are_refused(b200p, torch_cuda):
    torch = torch_cuda
    W = torch.zeros((64, 24), dtype=torch.bfloat16, device="cuda")          # K not a multiple of 16
    X = torch.zeros((2, 24), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((2, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(b200p.B200PError):
        b200p.skinny_gemm(W, out, x16=X, epilogue="acc32")
    W = torch.zeros((64, 32), dtype=torch.bfloat16, device="cuda")
    X = torch.zeros((17, 32), dtype=torch.bfloat16, device="cuda")          # more than 16 rows
    out = torch.zeros((17, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(b200p.B200PError):
        b200p.skinny_gemm(W, out, x16=X, epilogue="acc32")
    with pytest.raises(b200p.B200PError):
        b200p.skinny_gemm(W, out[:2], x16=X[:2], epilogue="store16")         # combination that does not exist
