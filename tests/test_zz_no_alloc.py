"""The scratch-free decode entry point (for hosts that cannot lend device memory)
gives the same result as the entry point that takes a caller-provided workspace.
Collected last on purpose.  Called through the C ABI, twice in a row, on shapes
that fit the built-in scratch; a shape that does not fit is refused."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_decode_matches_workspace_decode(b200p, torch_cuda):
    torch = torch_cuda
    L = b200p.lib()
    g = torch.Generator(device="cuda"); g.manual_seed(77)
    stream = torch.cuda.current_stream().cuda_stream
    for (batch, nqh, nkvh, N, D, dt) in ((4, 32, 8, 3000, 128, torch.bfloat16), (2, 8, 8, 777, 64, torch.float16)):
        q = torch.randn(batch, nqh, D, device="cuda", generator=g).to(dt)
        K = torch.randn(batch, nkvh, N, D, device="cuda", generator=g).to(dt)
        V = torch.randn(batch, nkvh, N, D, device="cuda", generator=g).to(dt)
        args = b200p.DecodeArgs(D, N, nqh, nkvh, N, batch, b200p._dtype_code(q), 0, 0, 0, 0)
        need = L.b200p_attn_decode_workspace_bytes(C.byref(args))
        assert 0 < need <= L.b200p_attn_decode_noalloc_max_bytes()
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        ref = torch.empty_like(q)
        assert L.b200p_attn_decode(q.data_ptr(), K.data_ptr(), V.data_ptr(), ref.data_ptr(), C.byref(args),
                                   ws.data_ptr(), need, stream) == 0
        outs = []
        for _ in range(2):                                   # two calls in a row share the built-in scratch
            o = torch.full_like(q, float("nan"))
            assert L.b200p_attn_decode_noalloc(q.data_ptr(), K.data_ptr(), V.data_ptr(), o.data_ptr(), C.byref(args), stream) == 0
            outs.append(o)
        torch.cuda.synchronize()
        for o in outs:
            assert torch.isfinite(o.float()).all()
            # same kernels, same split plan: the tolerance of the decode tests (2e-2) is met with room to spare
            assert (o.float() - ref.float()).abs().max().item() <= 2e-2
            assert torch.equal(o, ref)
    # a shape whose partials do not fit the 8 MiB array is refused before any launch
    big = b200p.DecodeArgs(128, 8192, 32, 8, 8192, 1024, b200p.BF16, 0, 0, 0, 0)
    assert L.b200p_attn_decode_workspace_bytes(C.byref(big)) > L.b200p_attn_decode_noalloc_max_bytes()
    n0 = b200p.launch_count()
    q = torch.zeros(1, device="cuda")
    assert L.b200p_attn_decode_noalloc(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), C.byref(big), stream) == -10
    assert b200p.launch_count() == n0
