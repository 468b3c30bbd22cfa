"""Generates tests/golden/reference_cpu_vectors.npz: inputs and outputs of the REFERENCE's own CPU
reference functions (attn_cpu_ref, cpu_attention_ref, cpu_prefill / attn_ref, cpu_decode / decode_ref),
compiled from the reference tree by oracle/build_ref.py into oracle/_ref/libref_cpu.so.

Run it where the reference tree is present (python tests/golden/make_golden.py); the fixture it writes
is committed, so the oracle stays pinned to the reference's outputs where the tree is absent.
Inputs follow the reference's recipes: mt19937 + normal_distribution, seeds 42 / 7, sigma 0.5 / 0.3
(research/flash-attention-mi300x/fa_naive.hip:258-268, kernels/fa_naive.hip:337-346,
cdna3-prims/tests/validate_attention_api.hip:154-172), at sizes small enough to commit."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle as orc  # noqa: E402


def main() -> int:
    if orc.ref_lib() is None:
        print("oracle/_ref/libref_cpu.so is not built: run oracle/build_ref.py where the reference tree is present")
        return 1
    out = {}
    # GQA prefill, non-causal and causal: cpu_prefill == attn_ref
    for name, (D, sq, sk, nqh, nkvh, batch, causal) in {"prefill_nc": (64, 40, 56, 4, 2, 1, 0), "prefill_c": (64, 48, 48, 4, 2, 2, 1),
                                                         "prefill_d128_c": (128, 32, 32, 2, 1, 1, 1)}.items():
        q, k, v = orc.gen_qkv_mt19937(42, 0.5, batch * nqh * sq * D, batch * nkvh * sk * D)
        o = orc.ref_call("ref_cpu_prefill", q, k, v, q.size, D, sq, sk, nqh, nkvh, batch, causal)
        o2 = orc.ref_call("ref_attn_ref", q, k, v, q.size, D, sq, sk, nqh, nkvh, batch, causal)
        assert np.array_equal(o.view(np.uint32), o2.view(np.uint32))
        out[name + "_cfg"] = np.array([D, sq, sk, nqh, nkvh, batch, causal], np.int32)
        out[name + "_q"], out[name + "_k"], out[name + "_v"], out[name + "_o"] = q, k, v, o
    # single-head step reference (fa_naive.hip:217-243)
    D, S = 64, 48
    q, k, v = orc.gen_qkv_mt19937(42, 0.5, S * D, S * D)
    out["step_cfg"] = np.array([S, D], np.int32)
    out["step_q"], out["step_k"], out["step_v"] = q, k, v
    out["step_o"] = orc.ref_call("ref_attn_cpu_ref", q, k, v, S * D, S, S, D)
    # fp32-I/O variant (kernels/fa_naive.hip:284-313)
    a = orc.gen_normal_mt19937(42, 0.0, 0.3, 3 * S * D)
    q, k, v = a[:S * D].copy(), a[S * D:2 * S * D].copy(), a[2 * S * D:].copy()
    out["fp32_cfg"] = np.array([S, D], np.int32)
    out["fp32_q"], out["fp32_k"], out["fp32_v"] = q, k, v
    out["fp32_o"] = orc.ref_call("ref_cpu_attention_ref", q, k, v, S * D, S, D, scale=1.0 / np.sqrt(D))
    # decode: cpu_decode == decode_ref
    for name, (D, N, nqh, nkvh) in {"decode_gqa": (64, 72, 8, 2), "decode_d128": (128, 40, 4, 4)}.items():
        a = orc.gen_normal_mt19937(7, 0.0, 0.5, nqh * D + 2 * nkvh * N * D)
        q, k, v = a[:nqh * D].copy(), a[nqh * D:nqh * D + nkvh * N * D].copy(), a[nqh * D + nkvh * N * D:].copy()
        o = orc.ref_call("ref_cpu_decode", q, k, v, q.size, D, N, nqh, nkvh)
        o2 = orc.ref_call("ref_decode_ref", q, k, v, q.size, D, N, nqh, nkvh)
        assert np.array_equal(o.view(np.uint32), o2.view(np.uint32))
        out[name + "_cfg"] = np.array([D, N, nqh, nkvh], np.int32)
        out[name + "_q"], out[name + "_k"], out[name + "_v"], out[name + "_o"] = q, k, v, o
    path = os.path.join(HERE, "reference_cpu_vectors.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
