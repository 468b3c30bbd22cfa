"""The committed golden vectors (tests/golden/reference_cpu_vectors.npz: inputs and outputs of
the reference's own CPU reference functions, written by tests/golden/make_golden.py where the
reference tree is present) against the oracle's restatements: bit for bit.  No GPU, and no
reference tree needed."""
import os

import numpy as np
import pytest

import oracle as orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cpu_vectors.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def bits(a):
    return np.ascontiguousarray(a, np.float32).ravel().view(np.uint32)


@pytest.mark.parametrize("name", ["prefill_nc", "prefill_c", "prefill_d128_c"])
def test_cpu_prefill(gold, name):
    D, sq, sk, nqh, nkvh, batch, causal = (int(x) for x in gold[name + "_cfg"])
    mine = orc.cpu_prefill(gold[name + "_q"], gold[name + "_k"], gold[name + "_v"], D, sq, sk, nqh, nkvh, batch, causal)
    assert np.array_equal(bits(mine), bits(gold[name + "_o"]))


def test_step_reference_single_head(gold):
    S, D = (int(x) for x in gold["step_cfg"])
    mine = orc.cpu_prefill(gold["step_q"], gold["step_k"], gold["step_v"], D, S, S, 1, 1, 1, 0)
    assert np.array_equal(bits(mine), bits(gold["step_o"]))


def test_fp32_io_reference(gold):
    S, D = (int(x) for x in gold["fp32_cfg"])
    mine = orc.cpu_attention_ref_heads(gold["fp32_q"], gold["fp32_k"], gold["fp32_v"], 1, S, D, 1.0 / np.sqrt(D))
    assert np.array_equal(bits(mine), bits(gold["fp32_o"]))


@pytest.mark.parametrize("name", ["decode_gqa", "decode_d128"])
def test_cpu_decode(gold, name):
    D, N, nqh, nkvh = (int(x) for x in gold[name + "_cfg"])
    mine = orc.cpu_decode(gold[name + "_q"], gold[name + "_k"], gold[name + "_v"], D, N, nqh, nkvh)
    assert np.array_equal(bits(mine), bits(gold[name + "_o"]))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["prefill_nc", "prefill_c", "prefill_d128_c"])
def test_cuda_prefill_against_the_reference_outputs(b200p, torch_cuda, gold, name):
    """The CUDA kernel on the golden inputs (rounded to fp16, as the reference's tests feed its GPU
    kernels) against the reference's CPU outputs: max|delta| < 2e-2."""
    torch = torch_cuda
    D, sq, sk, nqh, nkvh, batch, causal = (int(x) for x in gold[name + "_cfg"])
    dev = lambda a, shape: torch.from_numpy(np.ascontiguousarray(a)).cuda().half().view(*shape)
    got = b200p.prefill(dev(gold[name + "_q"], (batch, nqh, sq, D)), dev(gold[name + "_k"], (batch, nkvh, sk, D)),
                        dev(gold[name + "_v"], (batch, nkvh, sk, D)), causal=bool(causal))
    assert np.abs(got.float().cpu().numpy().ravel() - gold[name + "_o"]).max() < 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["decode_gqa", "decode_d128"])
def test_cuda_decode_against_the_reference_outputs(b200p, torch_cuda, gold, name):
    torch = torch_cuda
    D, N, nqh, nkvh = (int(x) for x in gold[name + "_cfg"])
    dev = lambda a, shape: torch.from_numpy(np.ascontiguousarray(a)).cuda().half().view(*shape)
    got = b200p.decode(dev(gold[name + "_q"], (1, nqh, D)), dev(gold[name + "_k"], (1, nkvh, N, D)), dev(gold[name + "_v"], (1, nkvh, N, D)))
    assert np.abs(got.float().cpu().numpy().ravel() - gold[name + "_o"]).max() < 2e-2
