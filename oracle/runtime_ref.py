"""CPU restatement (numpy) of the reference's small LLM runtime, for parity checks of the
session around the attention kernels.  TEST INFRASTRUCTURE ONLY.

Follows cdna3-prims/include/cdna3/runtime/session.hpp:141-237 (run_layers), :120-135
(fill_rope), :263-331 (generate / greedy_from_last) and the kernels of
cdna3-prims/include/cdna3/runtime/forward.hpp (RMSNorm :34-56, RoPE :135-148, SiLU*up
:154-160, embedding :174-183, argmax :244-262), with the GEMM contract of
rocblas_gemm.hpp:112-209: activations are cast to the 16-bit type, products accumulate in
fp32, Q/K/V come out 16-bit, O-proj / gate / up / down come out fp32.

Pinned the way the reference pins its own runtime (cdna3-prims/tests/validate_runtime.hip:
67-86, diag_logits.hip:23-66): against HuggingFace outputs on an exported model.  The
checkpoints the reference used are not available offline, so tests/golden/tiny_llama holds a
tiny random-init Llama exported by the reference's own export_model.py together with
HuggingFace's first-step logits and greedy tokens for it (tests/golden/make_runtime_golden.py);
tests/test_runtime_golden.py checks this file against them.  The attention inside it is the
pinned oracle (cpu_prefill / cpu_decode).

Two deliberate differences from the reference, shared with the CUDA session so that the
two stay comparable: the final norm's output is cast to 16-bit before lm_head (the
reference feeds fp32 activations to its naive lm_head kernel), and argmax ties go to the
lowest index (the reference's tree leaves ties unspecified).
"""
from __future__ import annotations

import numpy as np

from . import cpu_decode, cpu_prefill, round_to


def make_weights(cfg: dict, seed: int, kind: str = "bf16", std: float = 0.02, bias: bool = False) -> dict:
    """Random-init weights ~ N(0, std) rounded to the 16-bit type; norm weights = 1
    (stand-in for the HF checkpoint the reference loads)."""
    rng = np.random.default_rng(seed)
    H, F, D = cfg["hidden"], cfg["ffn_dim"], cfg["head_dim"]
    qd, kvd, V = cfg["n_heads"] * D, cfg["n_kv_heads"] * D, cfg["vocab_size"]

    def w(*shape):
        return round_to((rng.standard_normal(shape, dtype=np.float32) * np.float32(std)), kind)

    layers = []
    for _ in range(cfg["n_layers"]):
        L = {"Wq": w(qd, H), "Wk": w(kvd, H), "Wv": w(kvd, H), "Wo": w(H, qd), "Wgate": w(F, H), "Wup": w(F, H),
             "Wdown": w(H, F), "norm_attn": np.ones(H, np.float32), "norm_mlp": np.ones(H, np.float32)}
        if bias:
            L.update({"bq": w(qd), "bk": w(kvd), "bv": w(kvd)})
        layers.append(L)
    return {"embed_tokens": w(V, H), "lm_head": w(V, H), "final_norm": np.ones(H, np.float32), "layers": layers}


def load_export(model_dir: str):
    """A model directory in the reference's export format (cdna3-prims/runtime/export_model.py:
    meta.json + one raw fp16 .bin per tensor) -> (cfg, weights) as make_weights returns them."""
    import json
    import os
    meta = json.load(open(os.path.join(model_dir, "meta.json")))
    cfg = {k: meta[k] for k in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn_dim", "vocab_size")}
    cfg["rope_theta"] = float(meta.get("rope_theta", 10000.0))
    H, F, D = cfg["hidden"], cfg["ffn_dim"], cfg["head_dim"]
    qd, kvd, V = cfg["n_heads"] * D, cfg["n_kv_heads"] * D, cfg["vocab_size"]

    def t(name, *shape):
        return np.fromfile(os.path.join(model_dir, name + ".bin"), dtype=np.float16).astype(np.float32).reshape(shape)

    layers = []
    for i in range(cfg["n_layers"]):
        p = f"layer_{i}_"
        L = {"Wq": t(p + "q_proj", qd, H), "Wk": t(p + "k_proj", kvd, H), "Wv": t(p + "v_proj", kvd, H), "Wo": t(p + "o_proj", H, qd),
             "Wgate": t(p + "gate_proj", F, H), "Wup": t(p + "up_proj", F, H), "Wdown": t(p + "down_proj", H, F),
             "norm_attn": t(p + "norm_attn", H), "norm_mlp": t(p + "norm_mlp", H)}
        if meta.get("qkv_bias"):
            L.update({"bq": t(p + "q_bias", qd), "bk": t(p + "k_bias", kvd), "bv": t(p + "v_bias", kvd)})
        layers.append(L)
    return cfg, {"embed_tokens": t("embed_tokens", V, H), "lm_head": t("lm_head", V, H), "final_norm": t("final_norm", H), "layers": layers}


def rope_table(cfg: dict, max_seq: int):
    """session.hpp:120-135 in float32: freq = 1 / theta^(2d/D); angle = pos * freq."""
    D = cfg["head_dim"]
    theta = np.float32(cfg.get("rope_theta", 10000.0))
    d = np.arange(D // 2, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(theta, (np.float32(2.0) * d) / np.float32(D), dtype=np.float32)).astype(np.float32)
    ang = (np.arange(max_seq, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


class RefSession:
    def __init__(self, cfg: dict, weights: dict, max_seq: int, batch: int, kind: str = "bf16"):
        self.cfg, self.w, self.max_seq, self.batch, self.kind = cfg, weights, max_seq, batch, kind
        c = cfg
        self.cos, self.sin = rope_table(cfg, max_seq)
        self.K = np.zeros((c["n_layers"], batch, c["n_kv_heads"], max_seq, c["head_dim"]), np.float32)
        self.V = np.zeros_like(self.K)
        self.kv_len = 0

    def r(self, x):
        return round_to(x, self.kind)

    @staticmethod
    def rmsnorm(x, w, eps=1e-6):
        inv = 1.0 / np.sqrt((x.astype(np.float32) ** 2).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))
        return (x * inv.astype(np.float32) * w).astype(np.float32)

    def run_layers(self, hidden, T, pos0):
        """hidden [B, T, H] fp32 -> final hidden [B, T, H] fp32."""
        c = self.cfg
        B, D, nq, nkv = self.batch, c["head_dim"], c["n_heads"], c["n_kv_heads"]
        half = D // 2
        cos, sin = self.cos[pos0:pos0 + T], self.sin[pos0:pos0 + T]
        for li, L in enumerate(self.w["layers"]):
            x = self.r(self.rmsnorm(hidden, L["norm_attn"]))
            q = self.r(x @ L["Wq"].T); k = self.r(x @ L["Wk"].T); v = self.r(x @ L["Wv"].T)
            if "bq" in L:
                q = self.r(q + L["bq"]); k = self.r(k + L["bk"]); v = self.r(v + L["bv"])
            q = q.reshape(B, T, nq, D); k = k.reshape(B, T, nkv, D); v = v.reshape(B, T, nkv, D)

            def rope(t):
                a, b = t[..., :half], t[..., half:]
                cc, ss = cos[None, :, None, :], sin[None, :, None, :]
                return self.r(np.concatenate([a * cc - b * ss, b * cc + a * ss], axis=-1).astype(np.float32))

            q, k = rope(q), rope(k)
            self.K[li, :, :, pos0:pos0 + T] = k.transpose(0, 2, 1, 3)
            self.V[li, :, :, pos0:pos0 + T] = v.transpose(0, 2, 1, 3)
            if T > 1:
                assert pos0 == 0
                o = cpu_prefill(np.ascontiguousarray(q.transpose(0, 2, 1, 3)), np.ascontiguousarray(self.K[li, :, :, :T]),
                                np.ascontiguousarray(self.V[li, :, :, :T]), D, T, T, nq, nkv, B, 1, threads=8)
                attn = self.r(o).transpose(0, 2, 1, 3).reshape(B, T, nq * D)
            else:
                N = pos0 + 1
                o = cpu_decode(np.ascontiguousarray(q.reshape(B, nq, D)), self.K[li], self.V[li], D, N, nq, nkv,
                               stride_kv=self.max_seq, batch=B, threads=8)
                attn = self.r(o).reshape(B, 1, nq * D)
            hidden = hidden + (attn @ L["Wo"].T).astype(np.float32)
            x = self.r(self.rmsnorm(hidden, L["norm_mlp"]))
            g = (x @ L["Wgate"].T).astype(np.float32); u = (x @ L["Wup"].T).astype(np.float32)
            act = self.r((g / (1.0 + np.exp(-g, dtype=np.float32))) * u)
            hidden = hidden + (act @ L["Wdown"].T).astype(np.float32)
        return hidden

    def logits_last(self, hidden):
        x = self.r(self.rmsnorm(hidden[:, -1], self.w["final_norm"]))
        return (x @ self.w["lm_head"].T).astype(np.float32)

    def embed(self, ids):
        return self.w["embed_tokens"][np.asarray(ids)].astype(np.float32)

    def prefill_logits(self, ids):
        ids = np.asarray(ids).reshape(self.batch, -1)
        T = ids.shape[1]
        self.kv_len = 0
        h = self.run_layers(self.embed(ids), T, 0)
        self.kv_len = T
        return self.logits_last(h)

    def step_logits(self, token_ids):
        ids = np.asarray(token_ids).reshape(self.batch, 1)
        h = self.run_layers(self.embed(ids), 1, self.kv_len)
        self.kv_len += 1
        return self.logits_last(h)

    def argmax(self, logits):
        return np.argmax(self.r(logits), axis=-1).astype(np.int32)      # first maximum, 16-bit logits

    def generate(self, ids, max_new):
        out = np.zeros((self.batch, max_new), np.int32)
        nxt = self.argmax(self.prefill_logits(ids))
        out[:, 0] = nxt
        for s in range(1, max_new):
            nxt = self.argmax(self.step_logits(nxt))
            out[:, s] = nxt
        return out
