"""PyTorch custom operators over the C ABI: torch.ops.b200p.flash_attn and
torch.ops.b200p.flash_attn_decode, with the signatures and layout contracts of the
reference's torch.ops.amdinstinct.flash_attn / flash_attn_decode
(research/flash-attention-mi300x/llm_integration/torch_op/fa_torch_op.hip:36-67,
fa_decode_op.hip:26-57):

    flash_attn(q [nQH, seq, D], k [nKVH, seq, D], v [nKVH, seq, D]) -> o [nQH, seq, D]
        head-major, GQA (nQH % nKVH == 0), CAUSAL, D in {64, 128}
    flash_attn_decode(q [nQH, D], k_cache [nKVH, N, D], v_cache [nKVH, N, D]) -> o [nQH, D]

fp16 like the reference, or bf16.  Batched forms (a leading batch dimension) are accepted too.
The operators are registered with torch.library when register() is called (importing this
module does not touch torch); the implementations call libb200p through ctypes on the
current CUDA stream.  No autograd formula: forward only, as in the reference.
"""
from __future__ import annotations

_registered = False


def register():
    """Define torch.ops.b200p.{flash_attn, flash_attn_decode}.  Idempotent."""
    global _registered
    if _registered:
        return
    import torch
    from . import prefill, decode_noalloc, decode, decode_workspace, B200PError

    def _check(t, name, dims):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError(f"{name} must be fp16 or bf16")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
        if t.dim() not in dims:
            raise RuntimeError(f"{name}: wrong rank")

    lib = torch.library.Library("b200p", "DEF")
    lib.define("flash_attn(Tensor q, Tensor k, Tensor v) -> Tensor")
    lib.define("flash_attn_decode(Tensor q, Tensor k_cache, Tensor v_cache) -> Tensor")

    def flash_attn(q, k, v):
        for t, n in ((q, "q"), (k, "k"), (v, "v")):
            _check(t, n, (3, 4))
        squeeze = q.dim() == 3
        q4, k4, v4 = (t.unsqueeze(0) if squeeze else t for t in (q, k, v))
        if k4.shape[2] != q4.shape[2] or v4.shape != k4.shape:
            raise RuntimeError("k/v seq must match q and each other")
        if k4.shape[3] != q4.shape[3]:
            raise RuntimeError("k/v head_dim must match q")
        if q4.shape[1] % k4.shape[1] != 0:
            raise RuntimeError("nQH must be a multiple of nKVH (GQA)")
        if q4.shape[3] not in (64, 128):
            raise RuntimeError("D must be 64 or 128")
        o = prefill(q4, k4, v4, causal=True)
        return o.squeeze(0) if squeeze else o

    def flash_attn_decode(q, k_cache, v_cache):
        _check(q, "q", (2, 3)); _check(k_cache, "k_cache", (3, 4)); _check(v_cache, "v_cache", (3, 4))
        if k_cache.shape != v_cache.shape or k_cache.shape[-1] != q.shape[-1]:
            raise RuntimeError("k/v cache shape mismatch")
        if q.shape[-2] % k_cache.shape[-3] != 0:
            raise RuntimeError("nQH must be a multiple of nKVH (GQA)")
        out = torch.empty_like(q)
        try:
            return decode_noalloc(q, k_cache, v_cache, out=out)      # scratch inside the library when it fits
        except B200PError as e:
            if e.status != -10:
                raise
        return decode(q, k_cache, v_cache, out=out, workspace=decode_workspace(q, k_cache))

    lib.impl("flash_attn", flash_attn, "CUDA")
    lib.impl("flash_attn_decode", flash_attn_decode, "CUDA")

    # shape propagation for tracing / meta tensors
    lib.impl("flash_attn", lambda q, k, v: torch.empty_like(q), "Meta")
    lib.impl("flash_attn_decode", lambda q, k, v: torch.empty_like(q), "Meta")
    register._lib = lib                         # keep the library object alive
    _registered = True
