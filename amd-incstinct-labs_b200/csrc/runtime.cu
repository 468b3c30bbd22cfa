// ---------------------------------------------------------------------------
// runtime.cu -- the small LLM runtime around the attention kernels.
//
// Stands in for cdna3::runtime::Session (cdna3-prims/include/cdna3/runtime/
// session.hpp:52-331), KVCache (kv_cache.hpp:19-52), the forward kernels of
// forward.hpp:34-262 and the rocBLAS wrappers of rocblas_gemm.hpp:112-209, for
// a batch of equal-length sequences.  Same arithmetic contract as the
// reference: hidden state fp32, weights and GEMM operands 16-bit with fp32
// accumulation, attention I/O 16-bit, RMSNorm eps 1e-6, rotate-half RoPE with a
// host-computed table, greedy argmax over 16-bit logits.
//
// What is organised differently for a B200:
//  * attention reads the token-major projections and the KV cache in place
//    through strided TMA tensor maps, so the four repack_kernel launches per
//    layer and pack_kv are gone (session.hpp:193-207);
//  * RoPE, the optional QKV bias and the scatter into the cache are one kernel;
//    RMSNorm writes the GEMM's 16-bit operand directly; SiLU*up writes the down
//    projection's operand; residual adds are the GEMMs' beta = 1 accumulation;
//  * Q/K/V and gate/up projections are one GEMM each over concatenated weights;
//  * GEMMs are library calls (cuBLAS), as they are rocBLAS calls in the reference;
//  * the greedy loop keeps the next-token ids on the device: no per-token
//    device-to-host copy (session.hpp:329), one copy at the end;
//  * the RoPE table is built once per session, not per step (session.hpp:120-135).
// RMSNorm and argmax reduce with the warp primitives of wave64.cuh.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "attn_common.cuh"
#include "wave_primitives/wave64.cuh"
#include "skinny_gemm.cuh"
#include "decode_mega.cuh"
#include "status_rc.hpp"
#include "gemm_tc.cuh"
#include "b200p_runtime.h"
#include <cublas_v2.h>
#include <cmath>
#include <vector>

namespace b200p {
int decode_prepared(const void* q, const void* K, const void* V, void* o, const b200p_decode_args* a,
                    const int* n_dev, int n_add, void* ws, size_t ws_bytes, cudaStream_t st);
int prefill_dispatch_strided(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                             const b200p_attn_strides* strides, float* debug_s, cudaStream_t st);
namespace {

// ---- kernels ------------------------------------------------------------------------------
// forward.hpp:174-183: out[t, :] = float(embed[ids[t], :])
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ embed, const int* __restrict__ ids, float* __restrict__ out, int M, int H) {
    griddep_launch_dependents();
    const int t = blockIdx.x;
    if (t >= M) return;
    const T* src = embed + size_t(ids[t]) * H;
    float* dst = out + size_t(t) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_float(src[i]);
}

// forward.hpp:34-56 RMSNorm (y = x * rsqrt(mean(x^2) + eps) * w), writing the 16-bit GEMM operand.
// Output row r is the norm of source row r * src_row_stride + src_row_offset (stride > 1: the last token of each
// sequence).  One warp per row: float4 loads, up to 8 of them per lane kept in registers between the sum of squares
// and the scaling (rows up to 1024 floats per pass of 32 lanes x 8 x 4; longer rows are read twice, the second
// time from cache), 8-byte stores.  H must be a multiple of 4.
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_cast_kernel(const float* __restrict__ X, const T* __restrict__ W, T* __restrict__ Y,
                    int rows, int H, float eps, int src_row_stride, int src_row_offset) {
    const int r = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (r >= rows) return;
    const float4* x = reinterpret_cast<const float4*>(X + (size_t(r) * src_row_stride + src_row_offset) * H);
    uint2* y = reinterpret_cast<uint2*>(Y + size_t(r) * H);
    const uint2* w = reinterpret_cast<const uint2*>(W);
    const int quads = H / 4;
    constexpr int CACHE = 16;                                 // quads per lane held in registers: rows up to 2048 floats
    float4 c[CACHE];
    float ss = 0.f;
    #pragma unroll
    for (int i = 0; i < CACHE; ++i) {
        const int q = lane + 32 * i;
        if (q < quads) { c[i] = x[q]; ss += c[i].x * c[i].x + c[i].y * c[i].y + c[i].z * c[i].z + c[i].w * c[i].w; }
    }
    for (int q = lane + 32 * CACHE; q < quads; q += 32) { const float4 v = x[q]; ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
    const float inv = rsqrtf(wave::dpp::reduce_sum(ss) / H + eps);
    const bool w_vec = (reinterpret_cast<uintptr_t>(W) & 7) == 0;        // caller-owned weights may be any 2-byte aligned view
    auto put = [&](int q, const float4& v) {
        uint2 wv;
        if (w_vec) wv = w[q];
        else { const unsigned short* ws = reinterpret_cast<const unsigned short*>(W) + 4 * q;
               wv.x = ws[0] | (unsigned(ws[1]) << 16); wv.y = ws[2] | (unsigned(ws[3]) << 16); }
        const T* w4 = reinterpret_cast<const T*>(&wv);
        uint2 o;
        o.x = pack2<T>(v.x * inv * to_float(w4[0]), v.y * inv * to_float(w4[1]));
        o.y = pack2<T>(v.z * inv * to_float(w4[2]), v.w * inv * to_float(w4[3]));
        y[q] = o;
    };
    #pragma unroll
    for (int i = 0; i < CACHE; ++i) { const int q = lane + 32 * i; if (q < quads) put(q, c[i]); }
    for (int q = lane + 32 * CACHE; q < quads; q += 32) put(q, x[q]);
}

// forward.hpp:135-148 RoPE (rotate-half) on Q and K in place, rocblas_gemm.hpp:56-63 bias add, and
// forward.hpp:211-224 scatter of K, V into the cache, for token-major qkv [B*T, qd + 2*kvd].
// One thread per (token, head slot, 8 columns d0 .. d0 + 7 < D/2): it owns those and their partners d + D/2, as two
// 16-byte vectors each way.
template <typename T>
__global__ void rope_scatter_kernel(T* __restrict__ qkv, const T* __restrict__ bias, const float* __restrict__ cos_t,
                                    const float* __restrict__ sin_t, T* __restrict__ kcache, T* __restrict__ vcache,
                                    int B, int Tn, int nQH, int nKVH, int D, int pos0, int max_seq,
                                    const int* __restrict__ pos_dev) {
    griddep_launch_dependents();
    if (pos_dev) pos0 = min(*pos_dev, max_seq - Tn);         // device-side position (graph replay), kept inside the cache
    const int half = D / 2, chunks = half / 8;
    const int slots = nQH + 2 * nKVH;                       // q heads, k heads, v heads
    const size_t total = size_t(B) * Tn * slots * chunks;
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int d0 = int(idx % chunks) * 8;
    const int slot = int((idx / chunks) % slots);
    const size_t tok = idx / (size_t(chunks) * slots);       // b * Tn + s
    const int s = int(tok % Tn), b = int(tok / Tn);
    const int W = slots * D;
    T* row = qkv + tok * W + size_t(slot) * D;
    uint4 va = *reinterpret_cast<const uint4*>(row + d0), vb = *reinterpret_cast<const uint4*>(row + d0 + half);
    T* a = reinterpret_cast<T*>(&va);
    T* h = reinterpret_cast<T*>(&vb);
    const bool rotate = slot < nQH + nKVH;
    if (bias) {                                              // fp16 GEMM output + fp16 bias, rounded (bias_add_f16_kernel)
        const uint4 ba = *reinterpret_cast<const uint4*>(bias + slot * D + d0), bb = *reinterpret_cast<const uint4*>(bias + slot * D + d0 + half);
        const T* pa = reinterpret_cast<const T*>(&ba);
        const T* pb = reinterpret_cast<const T*>(&bb);
        #pragma unroll
        for (int i = 0; i < 8; ++i) { a[i] = from_float<T>(to_float(a[i]) + to_float(pa[i])); h[i] = from_float<T>(to_float(h[i]) + to_float(pb[i])); }
    }
    if (rotate) {
        const int pos = pos0 + s;
        const float4* cp = reinterpret_cast<const float4*>(cos_t + size_t(pos) * half + d0);
        const float4* sp = reinterpret_cast<const float4*>(sin_t + size_t(pos) * half + d0);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x0 = to_float(a[i]), x1 = to_float(h[i]);
            a[i] = from_float<T>(x0 * cs[i] - x1 * sn[i]);   // d < D/2:  t*c + (-t[d+D/2])*s
            h[i] = from_float<T>(x1 * cs[i] + x0 * sn[i]);   // d >= D/2: t*c + ( t[d-D/2])*s
        }
    }
    if (rotate || bias) {
        *reinterpret_cast<uint4*>(row + d0) = va; *reinterpret_cast<uint4*>(row + d0 + half) = vb;
    }
    if (slot >= nQH) {                                       // k or v: into cache[b][kvh][pos][:]
        const bool is_k = slot < nQH + nKVH;
        const int kvh = is_k ? slot - nQH : slot - nQH - nKVH;
        T* dst = (is_k ? kcache : vcache) + ((size_t(b) * nKVH + kvh) * max_seq + pos0 + s) * D;
        *reinterpret_cast<uint4*>(dst + d0) = va; *reinterpret_cast<uint4*>(dst + d0 + half) = vb;
    }
}

// forward.hpp:154-160: silu(gate) * up in fp32, written as the down projection's 16-bit operand.
// gu is [M, 2F]: gate in the first F columns, up in the last F.
template <typename T>
__global__ void silu_mul_cast_kernel(const float* __restrict__ gu, T* __restrict__ act, size_t M, int F) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= M * F) return;
    const size_t m = i / F; const int f = int(i % F);
    const float g = gu[m * 2 * F + f], u = gu[m * 2 * F + F + f];
    act[i] = from_float<T>((g / (1.f + expf(-g))) * u);
}

// forward.hpp:244-262 argmax over a [V] row of 16-bit logits; ties go to the lowest index.
// The row is spread over gridDim.y blocks: each folds its slice into a 64-bit key
// (order-preserving value bits, then the complemented index) and merges it into keys[row] with
// atomicMax; the last block of a row to arrive (ticket counter) writes the id for the next
// step and the output token, and clears key and counter for the next launch.
template <typename T>
__global__ void argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ next_ids,
                              int* __restrict__ tokens, int tokens_stride, int step, const int* __restrict__ step_dev,
                              unsigned long long* __restrict__ keys, unsigned int* __restrict__ tickets) {
    griddep_launch_dependents();
    if (step_dev) step = min(*step_dev, tokens_stride - 1);
    __shared__ unsigned long long red[32];
    const int rowi = blockIdx.x;
    const float* row = logits + size_t(rowi) * V;
    const int per = (V + gridDim.y - 1) / gridDim.y;
    const int i0 = blockIdx.y * per, i1 = min(i0 + per, V);
    unsigned long long best = 0;
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float v = to_float(from_float<T>(row[i]));                 // the reference's logits are 16-bit
        unsigned u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);                  // order-preserving key
        const unsigned long long key = (unsigned long long)u << 32 | (0xffffffffu - unsigned(i));
        best = key > best ? key : best;
    }
    best = wave::dpp::reduce_max(best);                                  // 64-bit butterfly over the warp
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nw = blockDim.x / 32;
    if (lane == 0) red[warp] = best;
    __syncthreads();
    if (warp == 0) {
        unsigned long long t = lane < nw ? red[lane] : 0ull;
        t = wave::dpp::reduce_max(t);
        if (lane == 0) {
            atomicMax(&keys[rowi], t);
            __threadfence();
            if (atomicAdd(&tickets[rowi], 1u) == gridDim.y - 1) {        // every slice of the row is in
                __threadfence();
                const unsigned long long k = atomicExch(&keys[rowi], 0ull);
                tickets[rowi] = 0u;
                const int id = int(0xffffffffu - unsigned(k & 0xffffffffu));
                next_ids[rowi] = id;
                if (tokens) tokens[size_t(rowi) * tokens_stride + step] = id;
            }
        }
    }
}

template <typename T>
__global__ void concat_rows_kernel(T* __restrict__ dst, const T* __restrict__ a, size_t na, const T* __restrict__ b, size_t nb,
                                   const T* __restrict__ c, size_t nc) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < na) dst[i] = a[i];
    else if (i < na + nb) dst[i] = b[i - na];
    else if (i < na + nb + nc) dst[i] = c[i - na - nb];
}

// Device-side step state of the greedy loop: state[0] = position of the token being
// decoded (= keys already in the cache), state[1] = column of the output it produces.
__global__ void set_state_kernel(int* state, int pos, int step) { state[0] = pos; state[1] = step; }
__global__ void advance_state_kernel(int* state) { state[0] += 1; state[1] += 1; }

// argmax: rows x slices of ~2048 logits
inline dim3 argmax_grid(int rows, int V) { return dim3(unsigned(rows), unsigned((V + 2047) / 2048), 1); }

inline unsigned blocks(size_t n, int tpb = 256) { return unsigned((n + tpb - 1) / tpb); }

} // namespace
} // namespace b200p

using namespace b200p;

struct b200p_session {
    b200p_model_config c{};
    int dtype = B200P_BF16, max_seq = 0, batch = 0, kv_len = 0, cap_tokens = 0, cap_new = 0;
    int qd = 0, kvd = 0, W = 0;
    const void *embed = nullptr, *lm_head = nullptr, *final_norm = nullptr;
    std::vector<b200p_layer_weights> layers;
    std::vector<void*> Wqkv, Wgu, bqkv;                 // session-owned concatenations
    cublasHandle_t blas = nullptr;
    float *hidden = nullptr, *gu = nullptr, *logits = nullptr, *cos_t = nullptr, *sin_t = nullptr;
    void *norm = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr, *last_norm = nullptr;
    void *kcache = nullptr, *vcache = nullptr, *decode_ws = nullptr;
    size_t decode_ws_bytes = 0;
    int *d_ids = nullptr, *d_next = nullptr, *d_tokens = nullptr, *d_state = nullptr;
    int* d_abort = nullptr;                              // abort word of the session's streaming GEMMs (cleared per call, read after it)
    bool skinny_aligned = true;                          // every weight the skinny kernels read is 16-byte aligned
    unsigned long long* d_keys = nullptr;                // argmax merge keys [batch], zero between launches
    unsigned int* d_tickets = nullptr;                   // argmax arrival counters [batch]
    void* blas_ws = nullptr;
    static constexpr size_t kBlasWsBytes = size_t(64) << 20;
    // one decode step (embed -> layers -> logits -> argmax -> advance) as an executable graph
    cudaStream_t capture_stream = nullptr;
    cudaGraphExec_t step_graph = nullptr;
    const void* graph_hidden = nullptr; const int* graph_tokens = nullptr; int graph_max_new = 0; unsigned graph_epoch = 0;
    unsigned long long graph_replays = 0, graph_kernels = 0;   // kernels of this library inside one replay
    unsigned long long gemm_calls = 0, blas_calls = 0;      // all projections / those that went to the GEMM library
    // the decode loop as one persistent kernel (decode_mega.cuh): per-layer pointer table, split scratch, counters
    MegaLayer* mega_layers = nullptr;
    float* mega_part = nullptr;
    unsigned* mega_words = nullptr;                      // [0] grid barrier, [1] key readers
    unsigned long long mega_launches = 0;
    std::vector<void*> owned;

    template <typename P> cudaError_t alloc(P** p, size_t bytes) {
        cudaError_t e = cudaMalloc(reinterpret_cast<void**>(p), bytes ? bytes : 16);
        if (e == cudaSuccess) owned.push_back(*p);
        return e;
    }
    void release(void* p) {
        for (auto& q : owned) if (q == p && p) { cudaFree(p); q = nullptr; }
    }
    size_t esz() const { return 2; }
    size_t layer_cache_elems() const { return size_t(batch) * c.n_kv_heads * max_seq * c.head_dim; }
};

namespace {

cudaDataType cuda_type(int dtype) { return dtype == B200P_F16 ? CUDA_R_16F : CUDA_R_16BF; }

// C[M,N] (row-major) = A[M,K] . W[N,K]^T (+ C if accumulate); A, W 16-bit, fp32 accumulation
// (rocblas_gemm.hpp:112-209: transpose/none with the operands swapped).
int gemm(b200p_session* s, const void* A, const void* Wt, void* Cm, int M, int N, int K, bool c_is_f32, bool accumulate,
         cudaStream_t st) {
    if (tuning(KNOB_RUNTIME_GEMM, 1) != 0 && !(accumulate && !c_is_f32)) {
        // this library's tensor-core GEMM; shapes or pointers outside its domain take the library call below
        const int epi = !c_is_f32 ? GEMM_EPI_STORE16 : accumulate ? GEMM_EPI_ACC32 : GEMM_EPI_STORE32;
        const int rc = gemm_tc(s->dtype, epi, A, Wt, Cm, M, N, K, K, K, N, st);
        if (rc == B200P_OK) { ++s->gemm_calls; return rc; }
        if (rc != B200P_E_RANGE && rc != B200P_E_ALIGN) return rc;
    }
    ++s->blas_calls;
    const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
    cublasSetStream(s->blas, st);
    cublasSetWorkspace(s->blas, s->blas_ws, b200p_session::kBlasWsBytes);   // SetStream resets it; a fixed one is capturable
    const cudaDataType t = cuda_type(s->dtype);
    const cublasStatus_t r = cublasGemmEx(s->blas, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, Wt, t, K, A, t, K, &beta,
                                          Cm, c_is_f32 ? CUDA_R_32F : t, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    ++s->gemm_calls;
    return r == CUBLAS_STATUS_SUCCESS ? B200P_OK : int(cudaErrorUnknown);
}

void drop_step_graph(b200p_session* s);

template <typename T>
int ensure_scratch(b200p_session* s, int Tn, int max_new) {
    const int M = s->batch * Tn;
    if (M > s->cap_tokens) {
        const auto& c = s->c;
        cudaError_t e = cudaSuccess;
        // scratch is grown, never shrunk; the superseded buffers are released once the device is idle
        if (s->cap_tokens > 0) {
            if ((e = cudaDeviceSynchronize())) return int(e);
            void* old[] = {s->hidden, s->norm, s->qkv, s->attn, s->gu, s->act, s->d_ids};
            for (void* q : old) s->release(q);
            drop_step_graph(s);                                 // the captured step names the old buffers
        }
        if ((e = s->alloc(&s->hidden, size_t(M) * c.hidden * 4))) return int(e);
        if ((e = s->alloc(&s->norm, size_t(M) * c.hidden * 2))) return int(e);
        if ((e = s->alloc(&s->qkv, size_t(M) * s->W * 2))) return int(e);
        if ((e = s->alloc(&s->attn, size_t(M) * s->qd * 2))) return int(e);
        if ((e = s->alloc(&s->gu, size_t(M) * 2 * c.ffn_dim * 4))) return int(e);
        if ((e = s->alloc(&s->act, size_t(M) * c.ffn_dim * 2))) return int(e);
        if ((e = s->alloc(&s->d_ids, size_t(M) * sizeof(int)))) return int(e);
        s->cap_tokens = M;
    }
    if (max_new > s->cap_new) {
        if (cudaError_t e = s->alloc(&s->d_tokens, size_t(s->batch) * max_new * sizeof(int))) return int(e);
        s->cap_new = max_new;
    }
    return B200P_OK;
}

// session.hpp:141-237 run_layers: hidden [B*Tn, H] in, final hidden out.
// Whether the decode step's projections run as skinny_gemm_kernel (few rows: a stream over
// the weights with the norm / SiLU / residual work fused in) instead of library GEMMs.
bool skinny_ok(const b200p_session* s, int M) {
    const auto& c = s->c;
    return tuning(KNOB_RUNTIME_SKINNY, 2) != 0 && s->skinny_aligned && M <= kSkinnyMaxM && c.hidden % 16 == 0 && c.ffn_dim % 16 == 0 &&
           s->qd % 16 == 0 && size_t(M <= 8 ? 8 : 16) * size_t((c.ffn_dim > c.hidden ? c.ffn_dim : c.hidden) + kSkinnyXPad) * 2 <= 190 * 1024;
}

// One decoder layer of the decode step (one new token per sequence) on the skinny kernels:
// norm+QKV, RoPE/scatter, attention, O (+= residual), norm+gate/up+SiLU, down (+= residual).
template <typename T>
int decode_layer_skinny(b200p_session* s, int li, int pos0, cudaStream_t st, const int* pos_dev) {
    const auto& c = s->c;
    const int H = c.hidden, F = c.ffn_dim, D = c.head_dim, B = s->batch;
    const int qd = s->qd, W = s->W;
    const b200p_layer_weights& L = s->layers[li];
    T* kc = static_cast<T*>(s->kcache) + size_t(li) * s->layer_cache_elems();
    T* vc = static_cast<T*>(s->vcache) + size_t(li) * s->layer_cache_elems();
    SkinnyArgs a{};
    a.M = B; a.eps = 1e-6f; a.abort_word = s->d_abort;
    a.W = s->Wqkv[li]; a.X32 = s->hidden; a.norm_w = L.norm_attn; a.out = s->qkv; a.N = W; a.K = H; a.ldo = W;
    if (tuning(KNOB_RUNTIME_ROPE_FUSED, 1) != 0) {
        // 1.-4. attention RMSNorm, Q/K/V projection, bias, RoPE and the K/V scatter into the cache: one kernel
        a.rope.bias = s->bqkv[li]; a.rope.cos_t = s->cos_t; a.rope.sin_t = s->sin_t; a.rope.kcache = kc; a.rope.vcache = vc;
        a.rope.pos_dev = pos_dev; a.rope.pos0 = pos0; a.rope.nQH = c.n_heads; a.rope.nKVH = c.n_kv_heads; a.rope.D = D; a.rope.max_seq = s->max_seq;
        if (int e = launch_skinny<T, PRO_RMSNORM, EPI_ROPE>(a, st)) return e;
    } else {
        // 1.+2. attention RMSNorm fused into the Q/K/V projection; 3.+4. bias, RoPE, K/V into the cache
        if (int e = launch_skinny<T, PRO_RMSNORM, EPI_STORE16>(a, st)) return e;
        const size_t n = size_t(B) * (c.n_heads + 2 * c.n_kv_heads) * (D / 16);
        rope_scatter_kernel<T><<<blocks(n), 256, 0, st>>>(static_cast<T*>(s->qkv), static_cast<const T*>(s->bqkv[li]),
                                                          s->cos_t, s->sin_t, kc, vc, B, 1, c.n_heads, c.n_kv_heads, D, pos0, s->max_seq, pos_dev);
        launched();
    }
    // 5. attention over the cache
    {
        b200p_decode_args d{};
        d.D = D; d.N = pos_dev ? s->max_seq : pos0 + 1; d.nQHeads = c.n_heads; d.nKVHeads = c.n_kv_heads; d.stride_kv = s->max_seq;
        d.batch = B; d.dtype = s->dtype; d.kv_batch_stride = (long long)c.n_kv_heads * s->max_seq * D;
        d.key_offset = 0; d.q_batch_stride = W; d.o_batch_stride = qd;
        // the session's workspace stays prepared (zeroed at creation): no clearing memset per layer
        if (int e = decode_prepared(s->qkv, kc, vc, s->attn, &d, pos_dev, 1, s->decode_ws, s->decode_ws_bytes, st)) return e;
    }
    // 6. O projection accumulated into the residual stream
    a = SkinnyArgs{}; a.M = B; a.eps = 1e-6f; a.abort_word = s->d_abort;
    a.W = L.Wo; a.X16 = s->attn; a.ldx = qd; a.out = s->hidden; a.N = H; a.K = qd; a.ldo = H;
    if (int e = launch_skinny<T, PRO_PLAIN, EPI_ACC32>(a, st)) return e;
    // 7.+8. MLP RMSNorm fused into gate/up, SiLU(gate) * up as the epilogue
    a = SkinnyArgs{}; a.M = B; a.eps = 1e-6f; a.abort_word = s->d_abort;
    a.W = s->Wgu[li]; a.X32 = s->hidden; a.norm_w = L.norm_mlp; a.out = s->act; a.N = F; a.K = H; a.ldo = F;
    if (int e = launch_skinny<T, PRO_RMSNORM, EPI_SILU16>(a, st)) return e;
    //    down projection accumulated into the residual stream
    a = SkinnyArgs{}; a.M = B; a.eps = 1e-6f; a.abort_word = s->d_abort;
    a.W = L.Wdown; a.X16 = s->act; a.ldx = F; a.out = s->hidden; a.N = H; a.K = F; a.ldo = H;
    if (int e = launch_skinny<T, PRO_PLAIN, EPI_ACC32>(a, st)) return e;
    s->gemm_calls += 4;
    return B200P_OK;
}

template <typename T>
int run_layers(b200p_session* s, int Tn, int pos0, cudaStream_t st, const int* pos_dev = nullptr) {
    const auto& c = s->c;
    const int H = c.hidden, F = c.ffn_dim, D = c.head_dim, B = s->batch, M = B * Tn;
    const int qd = s->qd, W = s->W;
    if (Tn == 1 && skinny_ok(s, M)) {
        for (int li = 0; li < c.n_layers; ++li)
            if (int e = decode_layer_skinny<T>(s, li, pos0, st, pos_dev)) return e;
        return B200P_OK;
    }
    for (int li = 0; li < c.n_layers; ++li) {
        const b200p_layer_weights& L = s->layers[li];
        T* kc = static_cast<T*>(s->kcache) + size_t(li) * s->layer_cache_elems();
        T* vc = static_cast<T*>(s->vcache) + size_t(li) * s->layer_cache_elems();
        // 1. attention RMSNorm -> 16-bit operand
        rmsnorm_cast_kernel<T><<<blocks(size_t(M) * 32), 256, 0, st>>>(s->hidden, static_cast<const T*>(L.norm_attn), static_cast<T*>(s->norm), M, H, 1e-6f, 1, 0);
        launched();
        // 2. Q, K, V projections in one GEMM -> qkv [M, qd + 2 kvd] 16-bit
        if (int e = gemm(s, s->norm, s->Wqkv[li], s->qkv, M, W, H, false, false, st)) return e;
        // 3.+4. bias, RoPE on Q and K, K/V into the cache at [pos0, pos0 + Tn)
        {
            const size_t n = size_t(M) * (c.n_heads + 2 * c.n_kv_heads) * (D / 16);
            rope_scatter_kernel<T><<<blocks(n), 256, 0, st>>>(static_cast<T*>(s->qkv), static_cast<const T*>(s->bqkv[li]),
                                                              s->cos_t, s->sin_t, kc, vc, B, Tn, c.n_heads, c.n_kv_heads, D, pos0, s->max_seq, pos_dev);
            launched();
        }
        // 5. attention over the cache, in place
        if (Tn > 1) {
            if (pos0 != 0) return B200P_E_OP;                 // like the reference, prefill starts from an empty cache
            b200p_prefill_cfg pc{D, Tn, Tn, c.n_heads, c.n_kv_heads, B, 1};
            b200p_attn_strides a{};
            a.q_seq = W; a.q_head = D; a.q_batch = (long long)Tn * W;
            a.k_seq = D; a.k_head = (long long)s->max_seq * D; a.k_batch = (long long)c.n_kv_heads * s->max_seq * D;
            a.v_seq = a.k_seq; a.v_head = a.k_head; a.v_batch = a.k_batch;
            a.o_seq = qd; a.o_head = D; a.o_batch = (long long)Tn * qd;
            if (int e = prefill_dispatch_strided(s->qkv, kc, vc, s->attn, &pc, s->dtype, &a, nullptr, st)) return e;
        } else {
            b200p_decode_args a{};
            a.D = D; a.N = pos0 + 1; a.nQHeads = c.n_heads; a.nKVHeads = c.n_kv_heads; a.stride_kv = s->max_seq;
            a.batch = B; a.dtype = s->dtype; a.kv_batch_stride = (long long)c.n_kv_heads * s->max_seq * D;
            a.key_offset = 0; a.q_batch_stride = W; a.o_batch_stride = qd;
            if (pos_dev) {                                      // key count = *pos_dev + 1, bound = the cache length
                a.N = s->max_seq;
                if (int e = b200p_attn_decode_dyn(s->qkv, kc, vc, s->attn, &a, pos_dev, 1, s->decode_ws, s->decode_ws_bytes, st)) return e;
            } else if (int e = b200p_attn_decode(s->qkv, kc, vc, s->attn, &a, s->decode_ws, s->decode_ws_bytes, st)) return e;
        }
        // 6. O projection, accumulated into the residual stream
        if (int e = gemm(s, s->attn, L.Wo, s->hidden, M, H, qd, true, true, st)) return e;
        // 7. MLP RMSNorm
        rmsnorm_cast_kernel<T><<<blocks(size_t(M) * 32), 256, 0, st>>>(s->hidden, static_cast<const T*>(L.norm_mlp), static_cast<T*>(s->norm), M, H, 1e-6f, 1, 0);
        launched();
        // 8. gate and up in one GEMM with SiLU(gate) * up as its epilogue (or, through the GEMM library: fp32 out and a
        //    separate kernel), down accumulated into the residual stream
        int fused = B200P_E_RANGE;
        if (tuning(KNOB_RUNTIME_GEMM, 1) != 0) {
            fused = gemm_tc(s->dtype, GEMM_EPI_SILU16, s->norm, s->Wgu[li], s->act, M, F, H, H, H, F, st);
            if (fused == B200P_OK) ++s->gemm_calls;
            else if (fused != B200P_E_RANGE && fused != B200P_E_ALIGN) return fused;
        }
        if (fused != B200P_OK) {
            if (int e = gemm(s, s->norm, s->Wgu[li], s->gu, M, 2 * F, H, true, false, st)) return e;
            silu_mul_cast_kernel<T><<<blocks(size_t(M) * F), 256, 0, st>>>(s->gu, static_cast<T*>(s->act), size_t(M), F);
            launched();
        }
        if (int e = gemm(s, s->act, L.Wdown, s->hidden, M, H, F, true, true, st)) return e;
    }
    return B200P_OK;
}

// final norm of the LAST token of every sequence + lm_head -> fp32 logits [B, V]
template <typename T>
int last_logits(b200p_session* s, int Tn, cudaStream_t st) {
    const auto& c = s->c;
    rmsnorm_cast_kernel<T><<<blocks(size_t(s->batch) * 32), 256, 0, st>>>(s->hidden, static_cast<const T*>(s->final_norm), static_cast<T*>(s->last_norm),
                                                                          s->batch, c.hidden, 1e-6f, Tn, Tn - 1);
    launched();
    return gemm(s, s->last_norm, s->lm_head, s->logits, s->batch, c.vocab_size, c.hidden, true, false, st);
}

// The same for the decode step (one token per sequence): final norm fused into lm_head.
template <typename T>
int last_logits_skinny(b200p_session* s, cudaStream_t st) {
    const auto& c = s->c;
    SkinnyArgs a{};
    a.M = s->batch; a.eps = 1e-6f; a.abort_word = s->d_abort;
    a.W = s->lm_head; a.X32 = s->hidden; a.norm_w = s->final_norm; a.out = s->logits; a.N = c.vocab_size; a.K = c.hidden; a.ldo = c.vocab_size;
    ++s->gemm_calls;
    return launch_skinny<T, PRO_RMSNORM, EPI_STORE32>(a, st);
}

// After a prefill: the last token's rows are gathered by the norm kernel, then the few-row lm_head product is the
// streaming kernel's case (M = batch), not a tensor-core tile's.
template <typename T>
int last_logits_prefill(b200p_session* s, int Tn, cudaStream_t st) {
    const auto& c = s->c;
    if (!skinny_ok(s, s->batch) || tuning(KNOB_RUNTIME_GEMM, 1) == 0) return last_logits<T>(s, Tn, st);
    rmsnorm_cast_kernel<T><<<blocks(size_t(s->batch) * 32), 256, 0, st>>>(s->hidden, static_cast<const T*>(s->final_norm), static_cast<T*>(s->last_norm),
                                                                          s->batch, c.hidden, 1e-6f, Tn, Tn - 1);
    launched();
    SkinnyArgs a{};
    a.M = s->batch; a.eps = 1e-6f; a.abort_word = s->d_abort;
    a.W = s->lm_head; a.X16 = s->last_norm; a.ldx = c.hidden; a.out = s->logits; a.N = c.vocab_size; a.K = c.hidden; a.ldo = c.vocab_size;
    ++s->gemm_calls;
    return launch_skinny<T, PRO_PLAIN, EPI_STORE32>(a, st);
}

template <typename T>
int embed(b200p_session* s, int M, cudaStream_t st) {
    embed_gather_kernel<T><<<M, 256, 0, st>>>(static_cast<const T*>(s->embed), s->d_ids, s->hidden, M, s->c.hidden);
    return launched();
}

// ---- the decode loop as one persistent kernel (decode_mega.cuh) ---------------------------------------
struct MegaPlan { const void* kernel = nullptr; int nstages = 0, x_bytes = 0, tab_bytes = 0, stage_bytes = 0; size_t dyn = 0; };

template <typename T>
const void* mega_kernel(int D) {
    return D == 64 ? reinterpret_cast<const void*>(decode_mega_kernel<T, 2>) : D == 128 ? reinterpret_cast<const void*>(decode_mega_kernel<T, 4>) : nullptr;
}

// Whether (and how) this session's decode steps run as the persistent kernel: the projection kernels' domain,
// at most 8 sequences, heads of 64 or 128 columns, a device that launches
// cooperatively, and room for at least two weight stages beside X.
template <typename T>
bool mega_plan(const b200p_session* s, MegaPlan* out) {
    const auto& c = s->c;
    if (tuning(KNOB_RUNTIME_MEGA, 0) == 0 || tuning(KNOB_RUNTIME_SKINNY, 2) != 2 || !s->mega_layers) return false;
    if (!skinny_ok(s, s->batch) || s->batch > kMegaMaxRows || c.n_kv_heads < 1 || c.n_heads % c.n_kv_heads != 0) return false;
    const int D = c.head_dim;
    MegaPlan pl;
    pl.kernel = mega_kernel<T>(D);
    if (!pl.kernel || device_status_ptr() == nullptr) return false;
    const int B = s->batch, Mp = B <= 1 ? 1 : B <= 2 ? 2 : B <= 4 ? 4 : 8;
    const int maxK = std::max(std::max(c.hidden, c.ffn_dim), s->qd);
    const int slab = std::min(kSkinnySlab, maxK);
    const size_t x_need = size_t(Mp) * (maxK + kSkinnyXPad) * 2;
    const size_t att_need = size_t(kSkinnyWarps) * (2 * D + 2) * sizeof(float);
    pl.x_bytes = int((std::max(x_need, att_need) + 127) / 128 * 128);
    pl.stage_bytes = 16 * (slab * 2 + 16);
    const int budget = 232448 - 8704;                          // shared memory per CTA minus the kernel's static part
    pl.tab_bytes = int((size_t(c.n_layers) * sizeof(MegaLayer) + 127) / 128 * 128);
    pl.nstages = std::min(kSkinnyMaxStages, (budget - pl.x_bytes - pl.tab_bytes) / pl.stage_bytes);
    if (pl.nstages < 2) return false;
    pl.dyn = size_t(pl.x_bytes) + pl.tab_bytes + size_t(pl.nstages) * pl.stage_bytes;
    int dev = 0, coop = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop) {
        cudaGetLastError();
        return false;
    }
    if (cudaFuncSetAttribute(pl.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(pl.dyn)) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pl.kernel, kSkinnyStreamThreads, pl.dyn) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        return false;
    }
    *out = pl;
    return true;
}

// n_steps decode steps from the device-side state (position, output column) and the ids in ids_in.
template <typename T>
int mega_launch(b200p_session* s, const MegaPlan& pl, const int* ids_in, int n_steps, bool want_argmax, int* tokens, int tokens_stride,
                cudaStream_t st) {
    const auto& c = s->c;
    if (cudaError_t e = cudaMemsetAsync(s->mega_words, 0, sizeof(unsigned), st)) return int(e);      // the grid barrier's counter
    MegaParams p{};
    p.layers = s->mega_layers; p.n_layers = c.n_layers; p.B = s->batch; p.H = c.hidden; p.F = c.ffn_dim; p.D = c.head_dim;
    p.nQH = c.n_heads; p.nKVH = c.n_kv_heads; p.V = c.vocab_size; p.max_seq = s->max_seq;
    p.embed = s->embed; p.lm_head = s->lm_head; p.final_norm = s->final_norm;
    p.hidden = s->hidden; p.qkv = s->qkv; p.act = s->act; p.logits = s->logits;
    p.kcache = s->kcache; p.vcache = s->vcache; p.layer_cache_elems = s->layer_cache_elems();
    p.cos_t = s->cos_t; p.sin_t = s->sin_t;
    p.part = s->mega_part;
    p.ids_in = ids_in; p.next_ids = s->d_next; p.tokens = tokens; p.tokens_stride = tokens_stride; p.state = s->d_state;
    p.keys = s->d_keys; p.key_ticket = s->mega_words + 1; p.bar = s->mega_words;
    p.status = s->d_abort; p.sticky = device_status_ptr();
    p.n_steps = n_steps; p.want_argmax = want_argmax ? 1 : 0;
    p.nstages = pl.nstages; p.slab_cols = kSkinnySlab; p.x_bytes = pl.x_bytes; p.tab_bytes = pl.tab_bytes; p.stage_bytes = pl.stage_bytes;
    p.ahead = tuning(KNOB_RUNTIME_MEGA_AHEAD, 0);              // measured: 1.03 ms per token without, 1.07 / 1.08 / 1.17 at 2 / 4 / 8 stages
    p.eps = 1e-6f; p.scale_log2 = (1.f / sqrtf(float(c.head_dim))) * 1.4426950408889634f;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(sm_count())); cfg.blockDim = dim3(kSkinnyStreamThreads); cfg.dynamicSmemBytes = pl.dyn; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    void* args[] = {&p};
    const cudaError_t le = cudaLaunchKernelExC(&cfg, pl.kernel, args);
    if (le != cudaSuccess) { cudaGetLastError(); return int(le); }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    ++s->mega_launches;
    s->gemm_calls += (unsigned long long)(n_steps) * (4ull * c.n_layers + 1);
    return B200P_OK;
}

// One greedy decode step with every per-step quantity read on the device: embed the ids the
// previous argmax left in d_next, run the layers at position state[0], argmax into column
// state[1] of the token table, advance the state.  Launch parameters never change, so the
// step can be captured once and replayed.
template <typename T>
int decode_step_device_state(b200p_session* s, int max_new, cudaStream_t st) {
    const int B = s->batch, V = s->c.vocab_size;
    embed_gather_kernel<T><<<B, 256, 0, st>>>(static_cast<const T*>(s->embed), s->d_next, s->hidden, B, s->c.hidden);
    launched();
    if (int e = run_layers<T>(s, 1, 0, st, s->d_state)) return e;
    if (int e = skinny_ok(s, B) ? last_logits_skinny<T>(s, st) : last_logits<T>(s, 1, st)) return e;
    argmax_kernel<T><<<argmax_grid(B, V), 256, 0, st>>>(s->logits, V, s->d_next, s->d_tokens, max_new, 0, s->d_state + 1, s->d_keys, s->d_tickets);
    advance_state_kernel<<<1, 1, 0, st>>>(s->d_state);
    return launched(2);
}

void drop_step_graph(b200p_session* s) {
    if (s->step_graph) cudaGraphExecDestroy(s->step_graph);
    s->step_graph = nullptr;
}

// Capture the decode step on the session's own stream (the caller's may be the legacy default
// stream, which cannot be captured) and instantiate it.  The graph bakes in the scratch
// pointers and the token table's row length, so it is rebuilt when those change.  Called only
// after the same step has run once eagerly (modules loaded, attributes set).
template <typename T>
int build_step_graph(b200p_session* s, int max_new) {
    drop_step_graph(s);
    if (!s->capture_stream && cudaStreamCreateWithFlags(&s->capture_stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        return B200P_E_NO_DEVICE;
    }
    if (cudaError_t e = cudaStreamBeginCapture(s->capture_stream, cudaStreamCaptureModeThreadLocal)) { cudaGetLastError(); return int(e); }
    const unsigned long long gemms = s->gemm_calls, launches = g_launches.load();
    const int rc = decode_step_device_state<T>(s, max_new, s->capture_stream);
    s->gemm_calls = gemms;                                   // recording is not running: take the counts back
    s->graph_kernels = g_launches.load() - launches;
    g_launches.fetch_sub(s->graph_kernels);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(s->capture_stream, &graph);
    if (rc || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc ? rc : int(ce ? ce : cudaErrorUnknown);
    }
    const cudaError_t ie = cudaGraphInstantiate(&s->step_graph, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) { s->step_graph = nullptr; cudaGetLastError(); return int(ie); }
    s->graph_hidden = s->hidden; s->graph_tokens = s->d_tokens; s->graph_max_new = max_new; s->graph_epoch = tuning_epoch();
    return B200P_OK;
}

// Status words of a call: the session's abort word (streaming GEMMs) and the status word at the head of
// its decode workspace.  Cleared on the stream when a call starts; read back behind the call's work.
int clear_status(b200p_session* s, cudaStream_t st) {
    if (cudaError_t e = cudaMemsetAsync(s->d_abort, 0, sizeof(int), st)) return int(e);
    return int(cudaMemsetAsync(s->decode_ws, 0, sizeof(int), st));
}
// Enqueues the read-back into words[2] (host); valid after the stream has been synchronised.
int fetch_status(b200p_session* s, int* words, cudaStream_t st) {
    if (cudaError_t e = cudaMemcpyAsync(&words[0], s->d_abort, sizeof(int), cudaMemcpyDeviceToHost, st)) return int(e);
    return int(cudaMemcpyAsync(&words[1], s->decode_ws, sizeof(int), cudaMemcpyDeviceToHost, st));
}

template <typename T>
int generate(b200p_session* s, const int* ids, int Tn, int max_new, int* out, float* timings, cudaStream_t st) {
    if (int e = ensure_scratch<T>(s, Tn, max_new)) return e;
    const int B = s->batch, V = s->c.vocab_size;
    const bool use_graph = tuning(KNOB_RUNTIME_GRAPH, 1) != 0;
    const int gemms_per_step = 4 * s->c.n_layers + 1;
    cudaEvent_t e0, e1, e2;
    cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
    int rc = B200P_OK;
    do {
        if ((rc = clear_status(s, st))) break;
        cudaEventRecord(e0, st);
        if (cudaError_t e = cudaMemcpyAsync(s->d_ids, ids, size_t(B) * Tn * sizeof(int), cudaMemcpyHostToDevice, st)) { rc = int(e); break; }
        if ((rc = embed<T>(s, B * Tn, st))) break;
        s->kv_len = 0;
        if ((rc = run_layers<T>(s, Tn, 0, st))) break;
        s->kv_len = Tn;
        if ((rc = last_logits_prefill<T>(s, Tn, st))) break;
        argmax_kernel<T><<<argmax_grid(B, V), 256, 0, st>>>(s->logits, V, s->d_next, s->d_tokens, max_new, 0, nullptr, s->d_keys, s->d_tickets);
        set_state_kernel<<<1, 1, 0, st>>>(s->d_state, Tn, 1);
        launched(2);
        cudaEventRecord(e1, st);
        MegaPlan mega;
        const bool use_mega = max_new > 1 && mega_plan<T>(s, &mega);
        if (use_mega) {
            // all remaining steps in one launch: the ids, the position and the output column stay on the device
            if (Tn + max_new - 2 >= s->max_seq) { rc = B200P_E_RANGE; break; }
            if ((rc = mega_launch<T>(s, mega, s->d_next, max_new - 1, true, s->d_tokens, max_new, st))) break;
            s->kv_len += max_new - 1;
        }
        for (int step = 1; step < max_new && !use_mega; ++step) {
            if (s->kv_len >= s->max_seq) { rc = B200P_E_RANGE; break; }
            if (use_graph && step >= 2) {
                // the first decode step ran eagerly below; from the second on, replay the captured step
                if (!s->step_graph || s->graph_hidden != s->hidden || s->graph_tokens != s->d_tokens || s->graph_max_new != max_new ||
                    s->graph_epoch != tuning_epoch()) {
                    if (build_step_graph<T>(s, max_new) != B200P_OK) drop_step_graph(s);
                }
                if (s->step_graph) {
                    if (cudaError_t e = cudaGraphLaunch(s->step_graph, st)) { rc = int(e); break; }
                    s->kv_len += 1;
                    s->gemm_calls += gemms_per_step;
                    g_launches.fetch_add(s->graph_kernels, std::memory_order_relaxed);
                    ++s->graph_replays;
                    continue;
                }
            }
            if ((rc = decode_step_device_state<T>(s, max_new, st))) break;
            s->kv_len += 1;
        }
        if (rc) break;
        cudaEventRecord(e2, st);
        if (cudaError_t e = cudaMemcpyAsync(out, s->d_tokens, size_t(B) * max_new * sizeof(int), cudaMemcpyDeviceToHost, st)) { rc = int(e); break; }
        int words[2] = {0, 0};
        if ((rc = fetch_status(s, words, st))) break;
        if (cudaError_t e = cudaStreamSynchronize(st)) { rc = int(e); break; }
        if ((rc = status_words_rc(words, 2))) break;            // a bounded wait gave up: the tokens are not to be trusted
        if (timings) { cudaEventElapsedTime(&timings[0], e0, e1); cudaEventElapsedTime(&timings[1], e1, e2); }
    } while (false);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    return rc;
}

template <typename T>
int prefill_logits(b200p_session* s, const int* ids, int Tn, float* logits, cudaStream_t st) {
    if (int e = ensure_scratch<T>(s, Tn, 1)) return e;
    const int B = s->batch;
    if (int e = clear_status(s, st)) return e;
    if (cudaError_t e = cudaMemcpyAsync(s->d_ids, ids, size_t(B) * Tn * sizeof(int), cudaMemcpyHostToDevice, st)) return int(e);
    if (int e = embed<T>(s, B * Tn, st)) return e;
    s->kv_len = 0;
    if (int e = run_layers<T>(s, Tn, 0, st)) return e;
    s->kv_len = Tn;
    if (int e = last_logits_prefill<T>(s, Tn, st)) return e;
    if (cudaError_t e = cudaMemcpyAsync(logits, s->logits, size_t(B) * s->c.vocab_size * 4, cudaMemcpyDeviceToHost, st)) return int(e);
    int words[2] = {0, 0};
    if (int e = fetch_status(s, words, st)) return e;
    if (cudaError_t e = cudaStreamSynchronize(st)) return int(e);
    return status_words_rc(words, 2);
}

template <typename T>
int step_logits(b200p_session* s, const int* ids, float* logits, cudaStream_t st) {
    if (int e = ensure_scratch<T>(s, 1, 1)) return e;
    if (s->kv_len >= s->max_seq) return B200P_E_RANGE;
    const int B = s->batch;
    if (int e = clear_status(s, st)) return e;
    if (cudaError_t e = cudaMemcpyAsync(s->d_ids, ids, size_t(B) * sizeof(int), cudaMemcpyHostToDevice, st)) return int(e);
    // same device-side position and split plan as the greedy loop, so that both give the same bits
    set_state_kernel<<<1, 1, 0, st>>>(s->d_state, s->kv_len, 0);
    launched();
    MegaPlan mega;
    if (mega_plan<T>(s, &mega)) {
        // the greedy loop's kernel for one step, logits only: same arithmetic, so both give the same bits
        if (int e = mega_launch<T>(s, mega, s->d_ids, 1, false, nullptr, 0, st)) return e;
        s->kv_len += 1;
    } else {
        if (int e = embed<T>(s, B, st)) return e;
        if (int e = run_layers<T>(s, 1, 0, st, s->d_state)) return e;
        s->kv_len += 1;
        if (int e = skinny_ok(s, B) ? last_logits_skinny<T>(s, st) : last_logits<T>(s, 1, st)) return e;
    }
    if (cudaError_t e = cudaMemcpyAsync(logits, s->logits, size_t(B) * s->c.vocab_size * 4, cudaMemcpyDeviceToHost, st)) return int(e);
    int words[2] = {0, 0};
    if (int e = fetch_status(s, words, st)) return e;
    if (cudaError_t e = cudaStreamSynchronize(st)) return int(e);
    return status_words_rc(words, 2);
}

template <typename T>
int build(b200p_session* s, const b200p_model_weights* w) {
    const auto& c = s->c;
    const int H = c.hidden, F = c.ffn_dim, D = c.head_dim;
    cudaError_t e;
    for (int li = 0; li < c.n_layers; ++li) {
        const b200p_layer_weights& L = s->layers[li];
        T *wqkv = nullptr, *wgu = nullptr, *b = nullptr;
        const size_t nq = size_t(s->qd) * H, nk = size_t(s->kvd) * H, nf = size_t(F) * H;
        if ((e = s->alloc(&wqkv, (nq + 2 * nk) * 2))) return int(e);
        if ((e = s->alloc(&wgu, 2 * nf * 2))) return int(e);
        concat_rows_kernel<T><<<blocks(nq + 2 * nk), 256>>>(wqkv, (const T*)L.Wq, nq, (const T*)L.Wk, nk, (const T*)L.Wv, nk);
        concat_rows_kernel<T><<<blocks(2 * nf), 256>>>(wgu, (const T*)L.Wgate, nf, (const T*)L.Wup, nf, (const T*)nullptr, 0);
        launched(2);
        if (L.bq && L.bk && L.bv) {
            if ((e = s->alloc(&b, size_t(s->W) * 2))) return int(e);
            concat_rows_kernel<T><<<blocks(s->W), 256>>>(b, (const T*)L.bq, s->qd, (const T*)L.bk, s->kvd, (const T*)L.bv, s->kvd);
            launched();
        }
        s->Wqkv.push_back(wqkv); s->Wgu.push_back(wgu); s->bqkv.push_back(b);
    }
    // RoPE table, session.hpp:120-135: freq = 1 / theta^(2d/D), angle = pos * freq
    std::vector<float> cosv(size_t(s->max_seq) * D / 2), sinv(cosv.size());
    for (int pos = 0; pos < s->max_seq; ++pos)
        for (int d = 0; d < D / 2; ++d) {
            const float freq = 1.f / powf(c.rope_theta, (2.f * d) / D);
            const float ang = pos * freq;
            cosv[size_t(pos) * (D / 2) + d] = cosf(ang);
            sinv[size_t(pos) * (D / 2) + d] = sinf(ang);
        }
    if ((e = s->alloc(&s->cos_t, cosv.size() * 4))) return int(e);
    if ((e = s->alloc(&s->sin_t, sinv.size() * 4))) return int(e);
    if ((e = cudaMemcpy(s->cos_t, cosv.data(), cosv.size() * 4, cudaMemcpyHostToDevice))) return int(e);
    if ((e = cudaMemcpy(s->sin_t, sinv.data(), sinv.size() * 4, cudaMemcpyHostToDevice))) return int(e);
    // KV cache [L][B][kvh][max_seq][D], zero-filled like kv_cache.hpp:34-37
    const size_t cache_bytes = size_t(c.n_layers) * s->layer_cache_elems() * 2;
    if ((e = s->alloc(&s->kcache, cache_bytes))) return int(e);
    if ((e = s->alloc(&s->vcache, cache_bytes))) return int(e);
    if ((e = cudaMemset(s->kcache, 0, cache_bytes))) return int(e);
    if ((e = cudaMemset(s->vcache, 0, cache_bytes))) return int(e);
    if ((e = s->alloc(&s->logits, size_t(s->batch) * c.vocab_size * 4))) return int(e);
    if ((e = s->alloc(&s->last_norm, size_t(s->batch) * H * 2))) return int(e);
    if ((e = s->alloc(&s->d_next, size_t(s->batch) * sizeof(int)))) return int(e);
    if ((e = s->alloc(&s->d_state, 2 * sizeof(int)))) return int(e);
    if ((e = s->alloc(&s->d_abort, sizeof(int)))) return int(e);
    if ((e = cudaMemset(s->d_abort, 0, sizeof(int)))) return int(e);
    // caller-owned weights the skinny kernels stream: misaligned views take the library GEMMs instead
    s->skinny_aligned = aligned(s->lm_head, 16) && aligned(s->final_norm, 8);
    for (const auto& L : s->layers)
        s->skinny_aligned = s->skinny_aligned && aligned(L.Wo, 16) && aligned(L.Wdown, 16) && aligned(L.norm_attn, 8) && aligned(L.norm_mlp, 8);
    if ((e = s->alloc(&s->d_keys, size_t(s->batch) * sizeof(unsigned long long)))) return int(e);
    if ((e = s->alloc(&s->d_tickets, size_t(s->batch) * sizeof(unsigned int)))) return int(e);
    if ((e = cudaMemset(s->d_keys, 0, size_t(s->batch) * sizeof(unsigned long long)))) return int(e);
    if ((e = cudaMemset(s->d_tickets, 0, size_t(s->batch) * sizeof(unsigned int)))) return int(e);
    if ((e = s->alloc(&s->blas_ws, b200p_session::kBlasWsBytes))) return int(e);
    // the persistent decode kernel's tables and scratch (decode_mega.cuh), when the shape is in its domain
    if (s->batch <= kMegaMaxRows && c.n_heads / c.n_kv_heads <= kMegaMaxGroup) {
        std::vector<MegaLayer> ml(c.n_layers);
        for (int li = 0; li < c.n_layers; ++li) {
            const b200p_layer_weights& L = s->layers[li];
            ml[li] = MegaLayer{s->Wqkv[li], s->bqkv[li], L.Wo, s->Wgu[li], L.Wdown, L.norm_attn, L.norm_mlp};
        }
        const size_t units = size_t(s->batch) * c.n_heads;
        if ((e = s->alloc(&s->mega_layers, ml.size() * sizeof(MegaLayer)))) return int(e);
        if ((e = cudaMemcpy(s->mega_layers, ml.data(), ml.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice))) return int(e);
        if ((e = s->alloc(&s->mega_part, units * kMegaMaxSplits * kMegaPartPad(D) * sizeof(float)))) return int(e);
        if ((e = s->alloc(&s->mega_words, 2 * sizeof(unsigned)))) return int(e);
        if ((e = cudaMemset(s->mega_words, 0, 2 * sizeof(unsigned)))) return int(e);
    }
    // decode scratch for the longest cache
    b200p_decode_args a{};
    a.D = D; a.N = s->max_seq; a.nQHeads = c.n_heads; a.nKVHeads = c.n_kv_heads; a.stride_kv = s->max_seq; a.batch = s->batch; a.dtype = s->dtype;
    size_t need = 0;
    for (int n = 1; n <= s->max_seq; n = n < 128 ? 128 : n * 2) {       // the split plan depends on N: take the largest need
        a.N = n < s->max_seq ? n : s->max_seq;
        const size_t b = b200p_attn_decode_workspace_bytes(&a);
        need = b > need ? b : need;
        if (a.N == s->max_seq) break;
    }
    s->decode_ws_bytes = need * 2;
    if ((e = s->alloc(&s->decode_ws, s->decode_ws_bytes))) return int(e);
    if ((e = cudaMemset(s->decode_ws, 0, s->decode_ws_bytes))) return int(e);
    if (cublasCreate(&s->blas) != CUBLAS_STATUS_SUCCESS) return int(cudaErrorUnknown);
    return int(cudaDeviceSynchronize());
}

} // namespace

extern "C" b200p_session* b200p_session_create(const b200p_model_weights* w, int max_seq, int batch, int* status) {
    int dummy; if (!status) status = &dummy;
    *status = B200P_OK;
    if (!w || !w->layers || !w->embed_tokens || !w->lm_head || !w->final_norm) { *status = B200P_E_NULL; return nullptr; }
    if (w->dtype != B200P_F16 && w->dtype != B200P_BF16) { *status = B200P_E_DTYPE; return nullptr; }
    const auto& c = w->cfg;
    if ((c.head_dim != 64 && c.head_dim != 128) || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.n_heads % c.n_kv_heads != 0 ||
        c.hidden % 8 != 0 || c.ffn_dim % 8 != 0) { *status = B200P_E_DIM; return nullptr; }
    if (max_seq <= 0 || batch <= 0 || c.n_layers <= 0 || c.vocab_size <= 0) { *status = B200P_E_LENGTH; return nullptr; }
    if (sm_count() <= 0) { *status = B200P_E_NO_DEVICE; return nullptr; }
    b200p_session* s = new b200p_session();
    s->c = c; s->dtype = w->dtype; s->max_seq = max_seq; s->batch = batch;
    s->qd = c.n_heads * c.head_dim; s->kvd = c.n_kv_heads * c.head_dim; s->W = s->qd + 2 * s->kvd;
    s->embed = w->embed_tokens; s->lm_head = w->lm_head; s->final_norm = w->final_norm;
    s->layers.assign(w->layers, w->layers + c.n_layers);
    for (const auto& L : s->layers)
        if (!L.Wq || !L.Wk || !L.Wv || !L.Wo || !L.Wgate || !L.Wup || !L.Wdown || !L.norm_attn || !L.norm_mlp) {
            *status = B200P_E_NULL; delete s; return nullptr;
        }
    const int rc = w->dtype == B200P_F16 ? build<__half>(s, w) : build<__nv_bfloat16>(s, w);
    if (rc) { *status = rc; b200p_session_destroy(s); return nullptr; }
    return s;
}

extern "C" void b200p_session_destroy(b200p_session* s) {
    if (!s) return;
    cudaDeviceSynchronize();
    if (s->step_graph) cudaGraphExecDestroy(s->step_graph);
    if (s->capture_stream) cudaStreamDestroy(s->capture_stream);
    if (s->blas) cublasDestroy(s->blas);
    for (void* p : s->owned) cudaFree(p);
    delete s;
}

extern "C" int b200p_session_generate(b200p_session* s, const int* ids, int T, int max_new, int* out, float* timings,
                                      b200p_stream_t stream) {
    if (!s || !ids || !out) return B200P_E_NULL;
    if (T <= 0 || max_new <= 0 || T + max_new - 1 > s->max_seq) return B200P_E_LENGTH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return s->dtype == B200P_F16 ? generate<__half>(s, ids, T, max_new, out, timings, st)
                                 : generate<__nv_bfloat16>(s, ids, T, max_new, out, timings, st);
}

extern "C" int b200p_session_prefill_logits(b200p_session* s, const int* ids, int T, float* logits, b200p_stream_t stream) {
    if (!s || !ids || !logits) return B200P_E_NULL;
    if (T <= 0 || T > s->max_seq) return B200P_E_LENGTH;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return s->dtype == B200P_F16 ? prefill_logits<__half>(s, ids, T, logits, st) : prefill_logits<__nv_bfloat16>(s, ids, T, logits, st);
}

extern "C" int b200p_session_step_logits(b200p_session* s, const int* ids, float* logits, b200p_stream_t stream) {
    if (!s || !ids || !logits) return B200P_E_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return s->dtype == B200P_F16 ? step_logits<__half>(s, ids, logits, st) : step_logits<__nv_bfloat16>(s, ids, logits, st);
}

extern "C" int b200p_skinny_gemm(int dtype, int prologue, int epilogue, const void* W, const void* x16, const float* x32,
                                 const void* norm_w, void* out, int M, int N, int K, int ldx, int ldo, float eps,
                                 b200p_stream_t stream) {
    if (!W || !out) return B200P_E_NULL;
    if (dtype != B200P_F16 && dtype != B200P_BF16) return B200P_E_DTYPE;
    if (prologue == PRO_PLAIN ? !x16 : (!x32 || !norm_w)) return B200P_E_NULL;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    SkinnyArgs a{};
    a.W = W; a.X16 = x16; a.X32 = x32; a.norm_w = norm_w; a.out = out; a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldo = ldo; a.eps = eps;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto run = [&](auto tag) -> int {
        using T = decltype(tag);
        if (prologue == PRO_RMSNORM) {
            switch (epilogue) {
                case EPI_STORE16: return launch_skinny<T, PRO_RMSNORM, EPI_STORE16>(a, st);
                case EPI_STORE32: return launch_skinny<T, PRO_RMSNORM, EPI_STORE32>(a, st);
                case EPI_SILU16:  return launch_skinny<T, PRO_RMSNORM, EPI_SILU16>(a, st);
            }
        } else if (prologue == PRO_PLAIN) {
            if (epilogue == EPI_ACC32) return launch_skinny<T, PRO_PLAIN, EPI_ACC32>(a, st);
        }
        return B200P_E_OP;                                   // only the combinations the decode step uses exist
    };
    return dtype == B200P_F16 ? run(__half{}) : run(__nv_bfloat16{});
}

extern "C" int b200p_session_kv_len(const b200p_session* s) { return s ? s->kv_len : -1; }
extern "C" unsigned long long b200p_session_gemm_calls(const b200p_session* s) { return s ? s->gemm_calls : 0; }
extern "C" unsigned long long b200p_session_blas_calls(const b200p_session* s) { return s ? s->blas_calls : 0; }
extern "C" unsigned long long b200p_session_graph_replays(const b200p_session* s) { return s ? s->graph_replays : 0; }
extern "C" unsigned long long b200p_session_mega_launches(const b200p_session* s) { return s ? s->mega_launches : 0; }
