"""Pin of the oracle's attention restatements: bit-for-bit equality with the
reference's OWN CPU reference functions, compiled from the reference tree into
oracle/_ref/libref_cpu.so by oracle/build_ref.py.  Skipped only when that file
was never built (it is built wherever the reference tree is present).  No GPU."""
import numpy as np
import pytest

import oracle as orc

pytestmark = pytest.mark.skipif(orc.ref_lib() is None, reason="oracle/_ref/libref_cpu.so not built")


# the reference's own configs: cdna3-prims/tests/validate_attention_api.hip:154-172 (small ones)
PREFILL = [(128, 64, 64, 2, 2, 1, 0), (128, 64, 64, 4, 2, 1, 1), (64, 128, 128, 2, 2, 1, 0),
           (64, 96, 96, 4, 1, 2, 1), (128, 64, 128, 4, 2, 1, 1)]


@pytest.mark.parametrize("D,sq,sk,nqh,nkvh,batch,causal", PREFILL)
def test_cpu_prefill_and_attn_ref(D, sq, sk, nqh, nkvh, batch, causal):
    q, k, v = orc.gen_qkv_mt19937(42, 0.5, batch * nqh * sq * D, batch * nkvh * sk * D)
    mine = orc.cpu_prefill(q, k, v, D, sq, sk, nqh, nkvh, batch, causal).ravel()
    a = orc.ref_call("ref_cpu_prefill", q, k, v, q.size, D, sq, sk, nqh, nkvh, batch, causal)
    b = orc.ref_call("ref_attn_ref", q, k, v, q.size, D, sq, sk, nqh, nkvh, batch, causal)
    assert np.array_equal(mine.view(np.uint32), a.view(np.uint32))
    assert np.array_equal(mine.view(np.uint32), b.view(np.uint32))


def test_attn_cpu_ref_step_config_head0():
    """research/flash-attention-mi300x/fa_naive.hip:258-263, :303-305: seed 42, N(0,0.5),
    B1 H8 S512 D64; the reference checks head 0."""
    D, S, H = 64, 512, 8
    q, k, v = orc.gen_qkv_mt19937(42, 0.5, H * S * D, H * S * D)
    ref = orc.ref_call("ref_attn_cpu_ref", q[:S * D], k[:S * D], v[:S * D], S * D, S, S, D)
    mine = orc.cpu_prefill(q, k, v, D, S, S, H, H, 1, 0, threads=8)[0, 0].ravel()
    assert np.array_equal(mine.view(np.uint32), ref.view(np.uint32))


def test_cpu_attention_ref_fp32_variant():
    """research/flash-attention-mi300x/kernels/fa_naive.hip:337-346: N(0,0.3), seed 42."""
    D, S = 64, 128
    a = orc.gen_normal_mt19937(42, 0.0, 0.3, 3 * S * D)
    q, k, v = a[:S * D], a[S * D:2 * S * D], a[2 * S * D:]
    ref = orc.ref_call("ref_cpu_attention_ref", q, k, v, S * D, S, D, scale=1.0 / np.sqrt(D))
    mine = orc.cpu_attention_ref_heads(q, k, v, 1, S, D, 1.0 / np.sqrt(D)).ravel()
    assert np.array_equal(mine.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("D,N,nqh,nkvh", [(128, 128, 8, 8), (64, 128, 8, 8), (128, 512, 32, 8), (64, 256, 14, 2)])
def test_cpu_decode_and_decode_ref(D, N, nqh, nkvh):
    a = orc.gen_normal_mt19937(7, 0.0, 0.5, nqh * D + 2 * nkvh * N * D)
    q, k, v = a[:nqh * D], a[nqh * D:nqh * D + nkvh * N * D], a[nqh * D + nkvh * N * D:]
    mine = orc.cpu_decode(q, k, v, D, N, nqh, nkvh).ravel()
    r1 = orc.ref_call("ref_cpu_decode", q, k, v, q.size, D, N, nqh, nkvh)
    r2 = orc.ref_call("ref_decode_ref", q, k, v, q.size, D, N, nqh, nkvh)
    assert np.array_equal(mine.view(np.uint32), r1.view(np.uint32))
    assert np.array_equal(mine.view(np.uint32), r2.view(np.uint32))


def test_strided_decode_equals_packed():
    """pack_host + decode, cdna3-prims/tests/validate_decode_dme.hip:32-41: a cache with
    stride max_seq gives the packed layout's result."""
    D, N, nqh, nkvh, max_seq = 64, 96, 14, 2, 160
    qb, ck, cv, _ = orc.gen_decode_dme_case(123, 0, D, N, nqh, nkvh, max_seq)
    q = orc.f16_bits_to_f32(qb)
    K = orc.f16_bits_to_f32(ck).reshape(nkvh, max_seq, D)
    V = orc.f16_bits_to_f32(cv).reshape(nkvh, max_seq, D)
    strided = orc.cpu_decode(q, K, V, D, N, nqh, nkvh, stride_kv=max_seq)
    packed = orc.cpu_decode(q, K[:, :N].copy(), V[:, :N].copy(), D, N, nqh, nkvh)
    assert np.array_equal(strided, packed)
    ref = orc.ref_call("ref_cpu_decode", q, K[:, :N].copy(), V[:, :N].copy(), q.size, D, N, nqh, nkvh)
    assert np.array_equal(packed.ravel().view(np.uint32), ref.view(np.uint32))
    assert not K[:, N:].any()
