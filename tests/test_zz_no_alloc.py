"""The scratch-free decode entry point (for hosts that cannot lend device memory)
gives the same result as the entry point that takes a caller-provided workspace, and
both agree with the CPU oracle.  Collected last on purpose.  Called through the C ABI,
twice in a row, on shapes that fit the built-in scratch; a shape that does not fit is
refused.  A second test drives it from compiled C++ through the reference's own launcher
signatures (no workspace argument)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import oracle as orc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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
        assert L.b200p_attn_workspace_status(None, stream) == 0     # NULL = the built-in scratch; synchronises
        cpu = orc.cpu_decode(q.float().cpu().numpy(), K.float().cpu().numpy(), V.float().cpu().numpy(), D, N, nqh, nkvh,
                             batch=batch, threads=8)
        for o in outs:
            assert torch.isfinite(o.float()).all()
            # same kernels, same split plan: the tolerance of the decode tests (2e-2) is met with room to spare
            assert (o.float() - ref.float()).abs().max().item() <= 2e-2
            assert torch.equal(o, ref)
            assert np.abs(o.float().cpu().numpy() - cpu).max() < 2e-2          # and against the oracle itself
    # a shape whose partials do not fit the 8 MiB array is refused before any launch
    big = b200p.DecodeArgs(128, 8192, 32, 8, 8192, 1024, b200p.BF16, 0, 0, 0, 0)
    assert L.b200p_attn_decode_workspace_bytes(C.byref(big)) > L.b200p_attn_decode_noalloc_max_bytes()
    n0 = b200p.launch_count()
    q = torch.zeros(1, device="cuda")
    assert L.b200p_attn_decode_noalloc(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), C.byref(big), stream) == -10
    assert b200p.launch_count() == n0


@pytest.mark.parametrize("D,N,nqh,nkvh,stride", [(128, 1000, 8, 2, 1000), (64, 333, 14, 2, 512)])
def test_reference_signatures_from_compiled_cpp(b200p, torch_cuda, tmp_path, D, N, nqh, nkvh, stride):
    """cdna3::attn::decode(q, K, V, o, cfg, stream) and decode_dme(...) exactly as a caller of the
    reference writes them, from a g++-built program on the GPU, against cpu_decode (fp16: < 2e-3)."""
    exe = tmp_path / "decode_ref_signature_gpu"
    lib_dir = os.path.dirname(b200p.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-I" + os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                    os.path.join(ROOT, "tests", "cpp", "decode_ref_signature_gpu.cpp"), "-L" + lib_dir, "-lb200p",
                    "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + lib_dir + ":/usr/local/cuda/lib64", "-o", str(exe)], check=True)
    rng = np.random.default_rng(D + N)
    q = orc.round_to(rng.standard_normal((nqh, D)).astype(np.float32), "f16")
    K = orc.round_to(rng.standard_normal((nkvh, stride, D)).astype(np.float32), "f16")
    V = orc.round_to(rng.standard_normal((nkvh, stride, D)).astype(np.float32), "f16")
    fin, fout = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(fin, "wb") as f:
        for a in (q, K, V):
            f.write(a.astype(np.float16).tobytes())
    r = subprocess.run([str(exe), str(fin), str(fout), str(D), str(N), str(nqh), str(nkvh), str(stride)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    out = np.fromfile(fout, dtype=np.float16).astype(np.float32).reshape(2, nqh, D)
    ref = orc.cpu_decode(q[None], K[None], V[None], D, N, nqh, nkvh, stride_kv=stride, batch=1, threads=4)[0]
    if stride == N:
        assert np.abs(out[0] - ref).max() < 2e-3
    assert np.abs(out[1] - ref).max() < 2e-3
