"""The tensor-core GEMM of the runtime's prefill projections (b200p_gemm_16, tcgen05 with the accumulator in
tensor memory) against an fp64 product of the same 16-bit operands: every epilogue, both tile widths, and
shapes whose M, N and K do not fill their last tile.  Bound: fp32 accumulation over K terms plus one rounding
of the output (16-bit outputs: half an ulp of the result)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def ops(torch, M, N, K, kind, seed, wrows=None):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    dt = torch.bfloat16 if kind == "bf16" else torch.float16
    A = (torch.randn(M, K, device="cuda", generator=g)).to(dt)
    W = (torch.randn(wrows or N, K, device="cuda", generator=g) * 0.05).to(dt)
    return A, W, dt


SHAPES = [(1024, 2560, 2048), (1024, 2048, 5632), (128, 128, 64), (200, 328, 136), (1, 40, 8), (513, 1000, 72), (96, 4096, 512)]


@pytest.mark.parametrize("tile_n", [0, 128, 256])
@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_store_and_accumulate(b200p, torch_cuda, M, N, K, kind, tile_n):
    torch = torch_cuda
    A, W, dt = ops(torch, M, N, K, kind, M + N + K)
    ref = A.double() @ W.double().T
    scale = max(1.0, ref.abs().max().item())
    ldc16, ldc32 = -(-N // 8) * 8 + 8, -(-N // 4) * 4 + 4               # rows of C on 16 bytes, a little wider than N
    b200p.set_tuning("gemm_tile_n", tile_n)
    try:
        c16 = torch.zeros(M, ldc16, dtype=dt, device="cuda")
        b200p.gemm_16(A, W, c16[:, :N], "store16")
        c32 = torch.full((M, ldc32), 7.0, device="cuda")
        b200p.gemm_16(A, W, c32[:, :N], "store32")
        res = torch.randn(M, ldc32, device="cuda")
        acc = res.clone()
        b200p.gemm_16(A, W, acc[:, :N], "acc32")
    finally:
        b200p.set_tuning("gemm_tile_n", -1)
    assert b200p.device_status() == 0
    ulp = 2.0 ** -8 if kind == "bf16" else 2.0 ** -11
    assert (c32[:, :N].double() - ref).abs().max().item() < 1e-5 * scale * max(1, K // 64)
    assert (c16[:, :N].double() - ref).abs().max().item() < (ulp + 1e-4) * scale
    assert (acc[:, :N].double() - (res[:, :N].double() + ref)).abs().max().item() < 1e-5 * scale * max(1, K // 64)
    # nothing outside [M, N] is touched
    assert (c32[:, N:] == 7.0).all() and torch.equal(acc[:, N:], res[:, N:]) and not c16[:, N:].any()


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("M,F,K", [(1024, 5632, 2048), (130, 200, 96), (7, 128, 64)])
def test_silu_gate_up_epilogue(b200p, torch_cuda, M, F, K, kind):
    torch = torch_cuda
    A, W, dt = ops(torch, M, F, K, kind, F, wrows=2 * F)
    g, u = A.double() @ W[:F].double().T, A.double() @ W[F:].double().T
    ref = g / (1.0 + torch.exp(-g)) * u
    ldc = -(-F // 8) * 8 + 8
    out = torch.zeros(M, ldc, dtype=dt, device="cuda")
    b200p.gemm_16(A, W, out[:, :F], "silu16")
    assert b200p.device_status() == 0
    ulp = 2.0 ** -8 if kind == "bf16" else 2.0 ** -11
    assert (out[:, :F].double() - ref).abs().max().item() < (ulp + 2e-3) * max(1e-3, ref.abs().max().item())
    assert not out[:, F:].any()


def test_domain_errors(b200p, torch_cuda):
    torch = torch_cuda
    A = torch.zeros(64, 36, dtype=torch.bfloat16, device="cuda")      # K not a multiple of 8
    W = torch.zeros(64, 36, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    n0 = b200p.launch_count()
    with pytest.raises(b200p.B200PError) as e:
        b200p.gemm_16(A, W, out)
    assert e.value.status == -10 and b200p.launch_count() == n0
    A = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(b200p.B200PError) as e:
        b200p.gemm_16(A, A, torch.zeros(64, 68, dtype=torch.bfloat16, device="cuda")[:, :64])   # rows of C not on 16 bytes
    assert e.value.status == -5


def test_session_prefill_uses_no_library_gemm(b200p, torch_cuda):
    """With default settings every projection of a prefill and of the decode steps runs on this library's own
    kernels; the same tokens come out with the projections sent to the GEMM library instead."""
    from oracle import runtime_ref as rr
    torch = torch_cuda
    cfg = dict(n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1024, vocab_size=1000, rope_theta=10000.0)
    w = rr.make_weights(cfg, seed=3, kind="bf16", std=0.05)
    conv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().bfloat16()
    dw = {"embed_tokens": conv(w["embed_tokens"]), "lm_head": conv(w["lm_head"]), "final_norm": conv(w["final_norm"]),
          "layers": [{k: conv(v) for k, v in L.items()} for L in w["layers"]]}
    sess = b200p.Session(cfg, dw, 160, 2)
    ids = np.random.default_rng(2).integers(0, 1000, (2, 128)).astype(np.int32)
    lg = sess.prefill_logits(ids)
    toks, _ = sess.generate(ids, 6)
    assert sess.gemm_calls > 0 and sess.blas_calls == 0
    b200p.set_tuning("runtime_gemm", 0)
    try:
        lg_lib = sess.prefill_logits(ids)
        assert sess.blas_calls > 0
    finally:
        b200p.set_tuning("runtime_gemm", -1)
    assert np.abs(lg - lg_lib).max() < 0.02 * lg_lib.std()
    sess.close()
