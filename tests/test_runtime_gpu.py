"""The small LLM runtime (CUDA session through the C ABI) against the numpy restatement
of the reference's Session (oracle/runtime_ref.py, pinned to HuggingFace outputs by
tests/test_runtime_golden.py).  Random-init weights stand in for the HF checkpoint.  Both sides round to 16 bits at the same places, so logits differ only by
fp32 accumulation order and exp implementations, plus the occasional 1-ulp flip of a
16-bit intermediate.  Gates: max|delta logits| < 5% of the logits' standard deviation and
cosine > 0.9999 on the first decode step and on teacher-forced steps; teacher-forced argmax
agrees wherever the oracle's top-2 margin exceeds the logit tolerance (free-running token
equality is not a valid gate with random weights: near-ties, the same caveat the reference
documents in cdna3-prims/runtime/design.md:138-151)."""
import numpy as np
import pytest

import oracle as orc
from oracle import runtime_ref as rr

pytestmark = pytest.mark.gpu

SMALL = dict(n_layers=2, hidden=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1024, vocab_size=1000, rope_theta=10000.0)
WIDE = dict(n_layers=2, hidden=512, n_heads=4, n_kv_heads=4, head_dim=128, ffn_dim=768, vocab_size=777, rope_theta=10000.0)


def to_device(torch, w, kind):
    dt = torch.bfloat16 if kind == "bf16" else torch.float16
    conv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt)
    return {"embed_tokens": conv(w["embed_tokens"]), "lm_head": conv(w["lm_head"]), "final_norm": conv(w["final_norm"]),
            "layers": [{k: conv(v) for k, v in L.items()} for L in w["layers"]]}


def check_logits(got, ref):
    std = ref.std()
    assert np.abs(got - ref).max() < 0.05 * std, (np.abs(got - ref).max(), std)
    cos = (got * ref).sum() / np.sqrt((got * got).sum() * (ref * ref).sum())
    assert cos > 0.9999, cos
    return 0.05 * std


@pytest.fixture(params=[1, 0], ids=["persistent-decode-kernel", "kernel-per-phase"])
def decode_path(b200p, request):
    """The decode steps as one persistent cooperative kernel (opt-in) and as one kernel per phase (the default)."""
    b200p.set_tuning("runtime_mega", request.param)
    yield request.param
    b200p.set_tuning("runtime_mega", -1)


@pytest.mark.parametrize("cfg,kind,bias,T", [(SMALL, "bf16", False, 48), (SMALL, "f16", True, 33), (WIDE, "bf16", False, 130)])
def test_prefill_and_teacher_forced_decode(b200p, torch_cuda, decode_path, cfg, kind, bias, T):
    torch = torch_cuda
    batch, max_seq, steps = 2, 192, 6
    w = rr.make_weights(cfg, seed=11, kind=kind, std=0.05, bias=bias)
    ref = rr.RefSession(cfg, w, max_seq, batch, kind)
    sess = b200p.Session(cfg, to_device(torch, w, kind), max_seq, batch)
    rng = np.random.default_rng(5)
    ids = rng.integers(0, cfg["vocab_size"], (batch, T)).astype(np.int32)
    g, r = sess.prefill_logits(ids), ref.prefill_logits(ids)
    tol = check_logits(g, r)
    assert sess.kv_len == T
    for _ in range(steps):
        nxt = ref.argmax(r)                                   # teacher forcing with the oracle's token
        srt = np.sort(orc.round_to(r, kind), axis=-1)
        clear = (srt[:, -1] - srt[:, -2]) > 2 * tol
        gnext = np.argmax(orc.round_to(g, kind), axis=-1)
        assert (gnext[clear] == nxt[clear]).all()
        g, r = sess.step_logits(nxt), ref.step_logits(nxt)
        check_logits(g, r)
    assert b200p.device_status() == 0
    assert (sess.mega_launches == steps) if decode_path else (sess.mega_launches == 0)
    sess.close()


@pytest.mark.parametrize("batch", [3, 12])
def test_generate_equals_stepwise_greedy(b200p, torch_cuda, decode_path, batch):
    """generate() keeps the next-token ids on the device; it must produce exactly the tokens
    of the host-driven loop over prefill_logits / step_logits on the same session.  Twelve
    sequences put the decode step on the projection kernels' two-fragment (9 .. 16 row) forms."""
    torch = torch_cuda
    cfg, kind, max_seq, T, new = SMALL, "bf16", 128, 40, 12
    w = rr.make_weights(cfg, seed=3, kind=kind, std=0.05)
    dw = to_device(torch, w, kind)
    sess = b200p.Session(cfg, dw, max_seq, batch)
    ids = np.random.default_rng(9).integers(0, cfg["vocab_size"], (batch, T)).astype(np.int32)
    toks, (ttft, dec) = sess.generate(ids, new)
    assert toks.shape == (batch, new) and ttft > 0 and dec > 0
    assert sess.kv_len == T + new - 1
    # all decode steps of the call in one launch, for up to 8 sequences
    assert sess.mega_launches == (1 if decode_path and batch <= 8 else 0)
    lg = sess.prefill_logits(ids)
    manual = np.zeros_like(toks)
    for s in range(new):
        nxt = np.argmax(orc.round_to(lg, kind), axis=-1).astype(np.int32)
        manual[:, s] = nxt
        if s + 1 < new:
            lg = sess.step_logits(nxt)
    assert np.array_equal(toks, manual)
    again, _ = sess.generate(ids, new)                         # run-to-run identical, cache reset
    assert np.array_equal(toks, again)
    # first generated token against the oracle (top-1 of the first step is the reference's criterion)
    ref = rr.RefSession(cfg, w, max_seq, batch, kind)
    r = ref.prefill_logits(ids)
    srt = np.sort(orc.round_to(r, kind), axis=-1)
    clear = (srt[:, -1] - srt[:, -2]) > 0.1 * r.std()
    assert (toks[clear, 0] == ref.argmax(r)[clear]).all()
    # and every decode step's logits against the oracle, teacher-forced on this library's tokens
    lg = sess.prefill_logits(ids)
    for s in range(3):
        g, r = sess.step_logits(toks[:, s].copy()), ref.step_logits(toks[:, s].copy())
        check_logits(g, r)
    sess.close()


def test_generate_graph_replay_equals_launched_steps(b200p, torch_cuda):
    """From its second decode step on, generate() replays one captured CUDA graph whose kernels
    read position and output column on the device.  Same tokens as with the graph switched off,
    as the host-driven loop, across calls with a different prompt length and token budget."""
    torch = torch_cuda
    cfg, kind, batch, max_seq = SMALL, "bf16", 2, 1024
    w = rr.make_weights(cfg, seed=4, kind=kind, std=0.05)
    sess = b200p.Session(cfg, to_device(torch, w, kind), max_seq, batch)
    rng = np.random.default_rng(10)
    for T, new in ((300, 10), (37, 16), (300, 10)):
        ids = rng.integers(0, cfg["vocab_size"], (batch, T)).astype(np.int32)
        before = sess.graph_replays
        toks, _ = sess.generate(ids, new)
        assert sess.graph_replays - before == new - 2
        assert sess.kv_len == T + new - 1
        b200p.set_tuning("runtime_graph", 0)
        try:
            before = sess.graph_replays
            plain, _ = sess.generate(ids, new)
            assert sess.graph_replays == before
        finally:
            b200p.set_tuning("runtime_graph", -1)
        assert np.array_equal(toks, plain)
        lg = sess.prefill_logits(ids)
        for s_ in range(new):
            nxt = np.argmax(orc.round_to(lg, kind), axis=-1).astype(np.int32)
            assert np.array_equal(toks[:, s_], nxt), s_
            if s_ + 1 < new:
                lg = sess.step_logits(nxt)
    assert b200p.device_status() == 0
    sess.close()


@pytest.mark.parametrize("cfg,kind,T", [(SMALL, "bf16", 700), (WIDE, "f16", 1100)])
def test_persistent_decode_kernel_over_a_long_cache(b200p, torch_cuda, cfg, kind, T):
    """With more than 256 keys the persistent kernel's attention splits a (sequence, kv head) over several
    CTAs that merge through global scratch.  Its logits against the kernel-per-phase path's on the same cache,
    its tokens against its own host-driven loop, and a second call against the first (scratch and counters
    are left clean)."""
    torch = torch_cuda
    batch, max_seq, new = 2, 2048, 24
    w = rr.make_weights(cfg, seed=21, kind=kind, std=0.05)
    sess = b200p.Session(cfg, to_device(torch, w, kind), max_seq, batch)
    ids = np.random.default_rng(T).integers(0, cfg["vocab_size"], (batch, T)).astype(np.int32)
    lg = sess.prefill_logits(ids)
    nxt = np.argmax(orc.round_to(lg, kind), axis=-1).astype(np.int32)
    b = sess.step_logits(nxt)                                  # kernel per phase
    assert sess.mega_launches == 0
    b200p.set_tuning("runtime_mega", 1)
    try:
        sess.prefill_logits(ids)
        a = sess.step_logits(nxt)
        assert sess.mega_launches == 1
        check_logits(a, b)
        toks, _ = sess.generate(ids, new)
        lg = sess.prefill_logits(ids)
        for s_ in range(new):
            nx = np.argmax(orc.round_to(lg, kind), axis=-1).astype(np.int32)
            assert np.array_equal(toks[:, s_], nx), s_
            if s_ + 1 < new:
                lg = sess.step_logits(nx)
        again, _ = sess.generate(ids, new)
        assert np.array_equal(toks, again)
    finally:
        b200p.set_tuning("runtime_mega", -1)
    assert b200p.device_status() == 0
    sess.close()


# BASELINE config 5's dimensions (the Llama-style decoder of the reference's runtime benchmark)
C5 = dict(hidden=2048, n_heads=32, n_kv_heads=4, head_dim=64, ffn_dim=5632, vocab_size=32000, rope_theta=10000.0)


def test_config5_dimensions_against_the_oracle(b200p, torch_cuda):
    """Two layers at the full config-5 widths, batch 2, a 512-token prompt and 8 teacher-forced steps against
    the numpy restatement of the reference Session (itself pinned to HuggingFace on the exported tiny model)."""
    torch = torch_cuda
    cfg = dict(C5, n_layers=2)
    batch, T, steps = 2, 512, 8
    w = rr.make_weights(cfg, seed=5, kind="bf16", std=0.02)
    ref = rr.RefSession(cfg, w, T + steps, batch, "bf16")
    sess = b200p.Session(cfg, to_device(torch, w, "bf16"), T + steps, batch)
    ids = np.random.default_rng(0xB205).integers(0, cfg["vocab_size"], (batch, T)).astype(np.int32)
    g, r = sess.prefill_logits(ids), ref.prefill_logits(ids)
    tol = check_logits(g, r)
    for _ in range(steps):
        nxt = ref.argmax(r)
        srt = np.sort(orc.round_to(r, "bf16"), axis=-1)
        clear = (srt[:, -1] - srt[:, -2]) > 2 * tol
        assert (np.argmax(orc.round_to(g, "bf16"), axis=-1)[clear] == nxt[clear]).all()
        g, r = sess.step_logits(nxt), ref.step_logits(nxt)
        check_logits(g, r)
    assert b200p.device_status() == 0
    sess.close()


def test_config5_full_depth_generate_equals_stepwise(b200p, torch_cuda, decode_path):
    """All 22 layers at config 5 (2.2 GB of weights): generate() -- device-side greedy loop, as one persistent
    kernel or as a captured step graph -- gives exactly the tokens of the host-driven prefill_logits / step_logits loop
    (cdna3-prims/include/cdna3/runtime/session.hpp:263-296)."""
    torch = torch_cuda
    cfg = dict(C5, n_layers=22)
    batch, T, new = 2, 512, 10
    g = torch.Generator(device="cuda"); g.manual_seed(0xB205)
    H, F, D = cfg["hidden"], cfg["ffn_dim"], cfg["head_dim"]
    qd, kvd = cfg["n_heads"] * D, cfg["n_kv_heads"] * D
    wt = lambda *shape: (torch.randn(shape, device="cuda", generator=g) * 0.02).bfloat16()
    ones = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    layers = [{"Wq": wt(qd, H), "Wk": wt(kvd, H), "Wv": wt(kvd, H), "Wo": wt(H, qd), "Wgate": wt(F, H), "Wup": wt(F, H),
               "Wdown": wt(H, F), "norm_attn": ones, "norm_mlp": ones} for _ in range(cfg["n_layers"])]
    weights = {"embed_tokens": wt(cfg["vocab_size"], H), "lm_head": wt(cfg["vocab_size"], H), "final_norm": ones, "layers": layers}
    sess = b200p.Session(cfg, weights, T + new, batch)
    ids = np.random.default_rng(7).integers(0, cfg["vocab_size"], (batch, T)).astype(np.int32)
    toks, _ = sess.generate(ids, new)
    assert (sess.mega_launches == 1 and sess.graph_replays == 0) if decode_path else (sess.graph_replays == new - 2)
    lg = sess.prefill_logits(ids)
    for s_ in range(new):
        nxt = np.argmax(orc.round_to(lg, "bf16"), axis=-1).astype(np.int32)
        assert np.array_equal(toks[:, s_], nxt), s_
        if s_ + 1 < new:
            lg = sess.step_logits(nxt)
    assert b200p.device_status() == 0
    sess.close()


def test_session_argument_errors(b200p, torch_cuda):
    torch = torch_cuda
    cfg = dict(SMALL, head_dim=96)
    w = rr.make_weights(cfg, seed=1)
    with pytest.raises(b200p.B200PError) as e:
        b200p.Session(cfg, to_device(torch, w, "bf16"), 64, 1)
    assert e.value.status == -6
    w = rr.make_weights(SMALL, seed=1)
    sess = b200p.Session(SMALL, to_device(torch, w, "bf16"), 64, 1)
    with pytest.raises(b200p.B200PError) as e:
        sess.generate(np.zeros((1, 60), np.int32), 10)          # 60 + 9 > max_seq
    assert e.value.status == -4
    sess.close()


def test_strided_prefill_matches_dense(b200p, torch_cuda):
    """b200p_attn_prefill_strided on token-major Q/O and a KV-cache slice equals the dense call."""
    torch = torch_cuda
    B, T, nq, nkv, D, max_seq = 2, 200, 8, 2, 64, 320
    g = torch.Generator(device="cuda"); g.manual_seed(8)
    qkv = (torch.randn(B, T, (nq + 2 * nkv) * D, device="cuda", generator=g) * 0.5).bfloat16()
    cacheK = (torch.randn(B, nkv, max_seq, D, device="cuda", generator=g) * 0.5).bfloat16()
    cacheV = (torch.randn(B, nkv, max_seq, D, device="cuda", generator=g) * 0.5).bfloat16()
    Qv = qkv[:, :, :nq * D].view(B, T, nq, D).permute(0, 2, 1, 3)          # [B, nq, T, D] view, token-major memory
    Kv, Vv = cacheK[:, :, :T], cacheV[:, :, :T]
    out_tok = torch.empty(B, T, nq * D, device="cuda", dtype=torch.bfloat16)
    Ov = out_tok.view(B, T, nq, D).permute(0, 2, 1, 3)
    b200p.prefill_strided(Qv, Kv, Vv, Ov, causal=True)
    dense = b200p.prefill(Qv.contiguous(), Kv.contiguous(), Vv.contiguous(), causal=True)
    assert torch.equal(Ov.contiguous(), dense)
