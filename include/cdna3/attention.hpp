// ---------------------------------------------------------------------------
// cdna3/attention.hpp -- the reference's unified attention API on B200.
//
// Source-compatible stand-in for cdna3-prims/include/cdna3/attention.hpp:
// the same namespace, config structs (field for field, :63-78 and
// detail/fa_decode_dme_kernel.hpp:45-48) and launcher names (prefill :86-109,
// decode :117-137, decode_dme :152-173).  The launchers forward to the C ABI of
// libb200p.so instead of instantiating kernels in the caller, so host code
// needs no CUDA compiler: only cuda_runtime / cuda_fp16 types.
//
// Differences from the reference, all additive:
//  * cudaStream_t / int status instead of hipStream_t / hipError_t (0 = success,
//    > 0 a cudaError_t, < 0 a B200P_E_* code; unsupported D is reported before
//    any launch like the reference's hipErrorInvalidValue);
//  * decode needs scratch for its split-KV partials.  The reference's launchers
//    allocate nothing and neither do these: pass a workspace sized by
//    decode_workspace_bytes(), or use the *_noalloc forms that use the
//    library's built-in 8 MiB scratch;
//  * __nv_bfloat16 overloads, and batched decode (decode_batched).
// ---------------------------------------------------------------------------
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../b200p.h"

namespace cdna3 {
namespace attn {

struct PrefillCfg {
    int D;          // head dimension (64 or 128)
    int seqQ;       // query sequence length
    int seqK;       // key/value sequence length
    int nQHeads;    // number of query heads
    int nKVHeads;   // number of KV heads (nQH for MHA; nQH/G for GQA)
    int batch;      // batch size
    int causal;     // 1 = causal mask, 0 = full attention
};
static_assert(sizeof(PrefillCfg) == sizeof(b200p_prefill_cfg), "PrefillCfg must match the C ABI struct");

struct DecodeCfg {
    int D;          // head dimension (64 or 128)
    int N;          // KV-cache length (number of cached keys)
    int nQHeads;
    int nKVHeads;
};

struct DecodeDmeCfg {
    int D, N, nQHeads, nKVHeads;
    int stride_kv;  // keys between KV heads in the cache: [nKVHeads, max_seq, D]
};

namespace detail {
inline int dtype_of(const __half*)        { return B200P_F16; }
inline int dtype_of(const __nv_bfloat16*) { return B200P_BF16; }
inline b200p_decode_args args(int D, int N, int nQH, int nKVH, int stride_kv, int batch, int dtype) {
    b200p_decode_args a{};
    a.D = D; a.N = N; a.nQHeads = nQH; a.nKVHeads = nKVH; a.stride_kv = stride_kv; a.batch = batch; a.dtype = dtype;
    a.kv_batch_stride = 0; a.key_offset = 0; a.q_batch_stride = 0; a.o_batch_stride = 0;
    return a;
}
} // namespace detail

// Q[batch x nQH x seqQ x D], K/V[batch x nKVH x seqK x D], O same as Q.
template <typename T>
inline int prefill(const T* Q, const T* K, const T* V, T* O, const PrefillCfg& cfg, cudaStream_t stream = nullptr) {
    return b200p_attn_prefill(Q, K, V, O, reinterpret_cast<const b200p_prefill_cfg*>(&cfg), detail::dtype_of(Q), stream);
}

// Scratch the decode launchers need for this shape (batch = 1 in the reference).
inline size_t decode_workspace_bytes(const DecodeCfg& c, int batch = 1) {
    const b200p_decode_args a = detail::args(c.D, c.N, c.nQHeads, c.nKVHeads, c.N, batch, B200P_F16);
    return b200p_attn_decode_workspace_bytes(&a);
}

// q[nQH x D], K[nKVH x N x D], V[nKVH x N x D], o[nQH x D]
template <typename T>
inline int decode(const T* q, const T* K, const T* V, T* o, const DecodeCfg& c,
                  void* workspace, size_t workspace_bytes, cudaStream_t stream = nullptr) {
    const b200p_decode_args a = detail::args(c.D, c.N, c.nQHeads, c.nKVHeads, c.N, 1, detail::dtype_of(q));
    return b200p_attn_decode(q, K, V, o, &a, workspace, workspace_bytes, stream);
}
// K/V: the strided cache [nKVHeads, max_seq, D]; the caller passes the layer base.
template <typename T>
inline int decode_dme(const T* q, const T* K, const T* V, T* o, const DecodeDmeCfg& c,
                      void* workspace, size_t workspace_bytes, cudaStream_t stream = nullptr) {
    const b200p_decode_args a = detail::args(c.D, c.N, c.nQHeads, c.nKVHeads, c.stride_kv, 1, detail::dtype_of(q));
    return b200p_attn_decode(q, K, V, o, &a, workspace, workspace_bytes, stream);
}
// The reference's exact signatures (no workspace argument): scratch comes from the
// library's built-in array; shapes that need more than it holds return B200P_E_RANGE.
template <typename T>
inline int decode(const T* q, const T* K, const T* V, T* o, const DecodeCfg& c, cudaStream_t stream = nullptr) {
    const b200p_decode_args a = detail::args(c.D, c.N, c.nQHeads, c.nKVHeads, c.N, 1, detail::dtype_of(q));
    return b200p_attn_decode_noalloc(q, K, V, o, &a, stream);
}
template <typename T>
inline int decode_dme(const T* q, const T* K, const T* V, T* o, const DecodeDmeCfg& c, cudaStream_t stream = nullptr) {
    const b200p_decode_args a = detail::args(c.D, c.N, c.nQHeads, c.nKVHeads, c.stride_kv, 1, detail::dtype_of(q));
    return b200p_attn_decode_noalloc(q, K, V, o, &a, stream);
}
// `batch` sequences in one launch: q,o [batch, nQH, D]; K,V [batch, nKVH, stride_kv, D].
template <typename T>
inline int decode_batched(const T* q, const T* K, const T* V, T* o, const DecodeDmeCfg& c, int batch,
                          void* workspace, size_t workspace_bytes, cudaStream_t stream = nullptr) {
    const b200p_decode_args a = detail::args(c.D, c.N, c.nQHeads, c.nKVHeads, c.stride_kv, batch, detail::dtype_of(q));
    return b200p_attn_decode(q, K, V, o, &a, workspace, workspace_bytes, stream);
}

} // namespace attn
} // namespace cdna3
