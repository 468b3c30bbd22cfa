// ---------------------------------------------------------------------------
// decode.cu -- split-KV decode attention (one new query token per sequence).
//
// Stands in for fa_decode_kernel<D,W> and fa_decode_dme_kernel<D,W,kBc>
// (cdna3-prims/include/cdna3/detail/fa_decode_kernel.hpp:21-94,
//  cdna3-prims/include/cdna3/detail/fa_decode_dme_kernel.hpp:64-208) behind
// cdna3::attn::decode / decode_dme (cdna3-prims/include/cdna3/attention.hpp:
// 117-137, 152-173), with a batch dimension added.
//
// The reference launches one block per QUERY head (every KV head is streamed
// `group` times) and performs one 64-lane reduction per key.  Here:
//  * a CTA owns (sequence, KV head, KV split) and serves ALL query heads of the
//    group, so each K/V byte leaves HBM once;
//  * a producer warp streams contiguous [TK, D] K and V tiles into a ring of
//    shared-memory stages with bulk async copies completing on mbarriers
//    (dme/dme_tma.cuh), the multi-stage successor of the reference's DME
//    ping-pong;
//  * 8 consumer warps read the tile with 16-byte shared loads.  A key row is
//    covered by 8 lanes (D/8 dims each), so a warp handles 4 keys per step and
//    the q.k dot product needs a 3-step xor butterfly instead of a 64-lane
//    reduction per key;
//  * the online softmax runs per warp and per tile: one running max per head
//    shared by the warp (wave::dpp::reduce_max style butterfly over the lane
//    groups), O rescaled at most once per tile and only when a max moved;
//  * warps are merged through shared memory, splits through a workspace and a
//    small combine kernel, both with the reference's merge
//    m = max m_w; l = sum e^{m_w-m} l_w; O = sum e^{m_w-m} O_w / l
//    (fa_decode_kernel.hpp:75-92).
// HBM-bound: algorithmic bytes = K and V once + q + o.
//
// Scores are kept in the log2 domain (s * log2e/sqrt(D)) so that exp is one
// ex2.approx; the reference uses __expf, the oracle expf.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "attn_common.cuh"
#include "dme/dme_tma.cuh"
#include "mma_sync.cuh"
#include "tensor_map.cuh"
#include "wave_primitives/wave64.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200p {
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr float kNegBig = -1e30f;

// Tiles and stages per head dim: [TK keys][D] of K and of V per stage.
template <int D> struct DecodeShape {
    static constexpr int TK = 128;
    static constexpr int STAGES = (D == 128) ? 3 : 4;
    static constexpr int TILE_BYTES = TK * D * 2;            // one of K / V
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
};

struct DecodeParams {
    const void* q; const void* K; const void* V;
    float* part_o;        // [batch][nQH][splits][D]  unnormalised partial outputs
    float* part_ml;       // [batch][nQH][splits][2]  running max (log2 domain), sum
    int*   status;        // != 0 after a bounded wait gave up
    int N, nQH, nKVH, group, batch, splits, keys_per_split;
    long long kv_head_stride;     // elements between KV heads   (stride_kv * D)
    long long kv_batch_stride;    // elements between sequences
    long long key_offset;         // first key of this launch inside each head (KV shards)
    long long q_batch_stride;     // elements between sequences in q
    float scale_log2;             // log2(e) / sqrt(D)
    const int* n_dev;             // non-null: keys = min(*n_dev + n_add, N), read by the kernels (N is then the bound)
    int n_add;
    // Fused combine (tensor-core kernel, 16-bit output): the last CTA of a (sequence, KV head)
    // to finish merges that unit's splits and writes o; tickets[batch * nKVH] count arrivals
    // and reset themselves.  Null: the partials are left for a separate combine launch.
    void* fused_o; unsigned int* tickets; long long o_batch_stride;
    int pdl;                      // host only: launch the tensor-core kernel as a programmatic dependent
    int o_pairs;                  // fused output: rows start on 4 bytes, so two 16-bit results go out as one word
};

// Key count and keys per split of this launch.  With a device-side count the split
// length is derived here exactly as plan_decode() derives it on the host (whole
// 128-key tiles), over a grid sized for the bound; splits past the end are empty.
__device__ __forceinline__ void decode_extent(const DecodeParams& p, int& N, int& per) {
    N = p.N; per = p.keys_per_split;
    if (p.n_dev) {
        N = min(max(*p.n_dev + p.n_add, 0), p.N);
        per = ((N + p.splits - 1) / p.splits + 127) / 128 * 128;
    }
}

template <typename T> __device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]);
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& w, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& w, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}
template <typename T> __device__ __forceinline__ float load_scalar(const T* p);
template <> __device__ __forceinline__ float load_scalar<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float load_scalar<__half>(const __half* p) { return __half2float(*p); }

// ---------------------------------------------------------------------------
// T: 16-bit storage type; D: head dim; GH: query heads a warp serves (1, 2, 4).
// Warp w serves head set (w % head_sets) and the 4-key groups (w / head_sets),
// (w / head_sets) + slices, ... of every tile.
// ---------------------------------------------------------------------------
template <typename T, int D, int GH>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_splitkv_kernel(const DecodeParams p) {
    using Sh = DecodeShape<D>;
    constexpr int TK = Sh::TK, STAGES = Sh::STAGES;
    constexpr int DPL = D / 8;            // dims per lane
    constexpr int CH = DPL / 8;           // 16-byte chunks per lane per row

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = smem_raw;
    uint64_t* full_bar  = reinterpret_cast<uint64_t*>(smem_raw + STAGES * Sh::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    __shared__ int s_failed;

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    griddep_launch_dependents();                  // a programmatic dependent may begin its own prefetch
    int N, per;
    decode_extent(p, N, per);
    const int k0 = min(split * per, N);
    const int k1 = min(k0 + per, N);
    const int ntiles = (k1 - k0 + TK - 1) / TK;

    const T* Kh = static_cast<const T*>(p.K) + size_t(b) * p.kv_batch_stride + size_t(kvh) * p.kv_head_stride + size_t(p.key_offset) * D;
    const T* Vh = static_cast<const T*>(p.V) + size_t(b) * p.kv_batch_stride + size_t(kvh) * p.kv_head_stride + size_t(p.key_offset) * D;

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; ++s) { dme::mbar_init(&full_bar[s], 1); dme::mbar_init(&empty_bar[s], kConsumerWarps); }
        dme::mbar_init_fence();
    }
    __syncthreads();

    // head sets: ceil(group / GH) rounded up to a power of two that divides the warp count
    int head_sets = (p.group + GH - 1) / GH;
    { int hs = 1; while (hs < head_sets) hs <<= 1; head_sets = hs; }
    const int slices = kConsumerWarps / head_sets;      // warps sharing a head set split the keys

    if (warp == kConsumerWarps) {
        // ------------------------------- producer ---------------------------------------
        if (lane == 0) {
            const uint64_t pol = dme::policy_evict_first();
            dme::Ring<STAGES> ring;
            for (int t = 0; t < ntiles; ++t) {
                if (t >= STAGES && !dme::wait(&empty_bar[ring.stage], ring.phase ^ 1u, p.status)) { atomicExch(&s_failed, 1); break; }
                const int key = k0 + t * TK;
                const uint32_t bytes = uint32_t(min(TK, k1 - key)) * D * 2;
                unsigned char* dst = tiles + ring.stage * Sh::STAGE_BYTES;
                dme::mbar_arrive_expect_tx(&full_bar[ring.stage], 2 * bytes);
                dme::copy_tile_1d_stream(dst, Kh + size_t(key) * D, bytes, &full_bar[ring.stage], pol);
                dme::copy_tile_1d_stream(dst + Sh::TILE_BYTES, Vh + size_t(key) * D, bytes, &full_bar[ring.stage], pol);
                ring.advance();
            }
        }
    } else {
        // ------------------------------- consumers --------------------------------------
        const int hset = warp % head_sets, slice = warp / head_sets;
        const int g = lane / 8, j8 = lane % 8;           // key group, position in the row
        const int h0 = hset * GH;                        // first head (inside the group) of this warp

        // q for this warp's heads, the lane's dims: chunk c covers dims 64c + 8*j8 .. +7
        float q[GH][DPL];
        #pragma unroll
        for (int h = 0; h < GH; ++h) {
            const bool live = h0 + h < p.group;
            const T* qp = static_cast<const T*>(p.q) + size_t(b) * p.q_batch_stride + (size_t(kvh) * p.group + (live ? h0 + h : 0)) * D;
            #pragma unroll
            for (int c = 0; c < CH; ++c) {
                #pragma unroll
                for (int i = 0; i < 8; ++i) q[h][c * 8 + i] = live ? load_scalar(qp + c * 64 + j8 * 8 + i) * p.scale_log2 : 0.f;
            }
        }
        float m[GH], l[GH], acc[GH][DPL];
        #pragma unroll
        for (int h = 0; h < GH; ++h) {
            m[h] = kNegBig; l[h] = 0.f;
            #pragma unroll
            for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
        }

        const int groups_per_tile = TK / 4;              // 4-key groups in a tile
        dme::Ring<STAGES> ring;
        bool ok = true;
        for (int t = 0; t < ntiles && ok; ++t) {
            if (!dme::wait(&full_bar[ring.stage], ring.phase, p.status)) { atomicExch(&s_failed, 1); ok = false; break; }
            const unsigned char* kt = tiles + ring.stage * Sh::STAGE_BYTES;
            const unsigned char* vt = kt + Sh::TILE_BYTES;
            const int valid = min(TK, k1 - (k0 + t * TK));      // keys present in this tile

            constexpr int STEPS_MAX = TK / 4 / 1;
            (void)STEPS_MAX;
            // this warp's key groups: slice, slice + slices, ...
            // scores for up to TK/(4*slices) steps; slices >= 1 so at most TK/4 -- but
            // registers only for the common case, larger counts loop in chunks of 4 steps.
            for (int gbase = slice; gbase < groups_per_tile; gbase += slices * 4) {
                float s[4][GH];
                bool live[4];
                #pragma unroll
                for (int st = 0; st < 4; ++st) {
                    const int kg = gbase + st * slices;
                    const int key = kg * 4 + g;
                    live[st] = kg < groups_per_tile && key < valid;
                    float part[GH];
                    #pragma unroll
                    for (int h = 0; h < GH; ++h) part[h] = 0.f;
                    if (live[st]) {
                        #pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            const uint4 w = *reinterpret_cast<const uint4*>(kt + size_t(key) * (D * 2) + c * 128 + j8 * 16);
                            float kf[8];
                            unpack8<T>(w, kf);
                            #pragma unroll
                            for (int h = 0; h < GH; ++h) {
                                #pragma unroll
                                for (int i = 0; i < 8; ++i) part[h] = fmaf(q[h][c * 8 + i], kf[i], part[h]);
                            }
                        }
                    }
                    #pragma unroll
                    for (int h = 0; h < GH; ++h) {
                        float v = part[h];
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                        v += __shfl_xor_sync(0xffffffffu, v, 4);
                        s[st][h] = live[st] ? v : kNegBig;
                    }
                }
                // running max per head, shared by the whole warp
                float alpha[GH];
                bool moved = false;
                #pragma unroll
                for (int h = 0; h < GH; ++h) {
                    float mx = fmaxf(fmaxf(s[0][h], s[1][h]), fmaxf(s[2][h], s[3][h]));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float mn = fmaxf(m[h], mx);
                    alpha[h] = exp2f(m[h] - mn);
                    moved |= (mn != m[h]);
                    m[h] = mn;
                }
                if (moved) {                       // warp-uniform: m is warp-wide
                    #pragma unroll
                    for (int h = 0; h < GH; ++h) {
                        l[h] *= alpha[h];
                        #pragma unroll
                        for (int d = 0; d < DPL; ++d) acc[h][d] *= alpha[h];
                    }
                }
                #pragma unroll
                for (int st = 0; st < 4; ++st) {
                    float pr[GH];
                    #pragma unroll
                    for (int h = 0; h < GH; ++h) { pr[h] = live[st] ? exp2f(s[st][h] - m[h]) : 0.f; l[h] += pr[h]; }
                    if (live[st]) {
                        const int key = (gbase + st * slices) * 4 + g;
                        #pragma unroll
                        for (int c = 0; c < CH; ++c) {
                            const uint4 w = *reinterpret_cast<const uint4*>(vt + size_t(key) * (D * 2) + c * 128 + j8 * 16);
                            float vf[8];
                            unpack8<T>(w, vf);
                            #pragma unroll
                            for (int h = 0; h < GH; ++h) {
                                #pragma unroll
                                for (int i = 0; i < 8; ++i) acc[h][c * 8 + i] = fmaf(pr[h], vf[i], acc[h][c * 8 + i]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) dme::mbar_arrive(&empty_bar[ring.stage]);
            ring.advance();
        }

        // l was summed 8x per key (all 8 lanes of a row hold the same p): keep one copy
        // per key group by summing over the 4 groups only.  acc: sum over the 4 groups.
        #pragma unroll
        for (int h = 0; h < GH; ++h) {
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 8);
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 16);
            #pragma unroll
            for (int d = 0; d < DPL; ++d) {
                float v = acc[h][d];
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                acc[h][d] = v;
            }
        }

        // ---- merge the warps of a head set through shared memory (tiles are dead now:
        // every warp passes the barrier below only after its last tile) ----
        asm volatile("bar.sync 1, %0;" :: "r"(kConsumerWarps * 32) : "memory");
        float* sm_o  = reinterpret_cast<float*>(tiles);                       // [warp][GH][D]
        float* sm_ml = sm_o + kConsumerWarps * GH * D;                        // [warp][GH][2]
        if (g == 0) {
            #pragma unroll
            for (int h = 0; h < GH; ++h) {
                #pragma unroll
                for (int c = 0; c < CH; ++c) {
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) sm_o[(warp * GH + h) * D + c * 64 + j8 * 8 + i] = acc[h][c * 8 + i];
                }
                if (j8 == 0) { sm_ml[(warp * GH + h) * 2] = m[h]; sm_ml[(warp * GH + h) * 2 + 1] = l[h]; }
            }
        }
        asm volatile("bar.sync 1, %0;" :: "r"(kConsumerWarps * 32) : "memory");
        // thread x merges output element (head hh of the group, dim d) over the slices
        for (int e = threadIdx.x; e < head_sets * GH * D; e += kConsumerWarps * 32) {
            const int hh = e / D, d = e % D;                 // hh = hset * GH + h
            if (hh >= p.group) continue;
            const int hs = hh / GH, h = hh % GH;
            float M = kNegBig;
            for (int sl = 0; sl < slices; ++sl) M = fmaxf(M, sm_ml[((sl * head_sets + hs) * GH + h) * 2]);
            float L = 0.f, O = 0.f;
            for (int sl = 0; sl < slices; ++sl) {
                const int w = sl * head_sets + hs;
                const float f = exp2f(sm_ml[(w * GH + h) * 2] - M);
                L += f * sm_ml[(w * GH + h) * 2 + 1];
                O += f * sm_o[(w * GH + h) * D + d];
            }
            const size_t row = (size_t(b) * p.nQH + size_t(kvh) * p.group + hh) * p.splits + split;
            p.part_o[row * D + d] = O;
            if (d == 0) { p.part_ml[row * 2] = M; p.part_ml[row * 2 + 1] = L; }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_failed) atomicExch(p.status, 1);
}


// ---------------------------------------------------------------------------
// Tensor-core variant (the default).  Same CTA ownership, ring and merges as
// above, but:
//  * tiles arrive through 4-D TMA tensor maps (dims D, keys, KV heads,
//    sequences) in 64-element boxes with the 128-byte swizzle, so ldmatrix reads
//    them without bank conflicts and keys past the end of the cache read as 0;
//  * the query heads of the group are the M = 16 rows of mma.sync m16n8k16
//    (rows past the group are zero): S = Q.K^T and O += P.V cost two MMAs per key
//    instead of ~50 scalar instructions, which takes the kernel from
//    issue-bound to HBM-bound;
//  * a score row lives on the 4 lanes of a quad: row max / row sum are
//    wave::lane_group_reduce<4> butterflies.
// Each of the 8 consumer warps takes 16 of the tile's 128 keys.
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_mma_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV) {
    using Sh = DecodeShape<D>;
    constexpr int TK = Sh::TK, STAGES = Sh::STAGES;
    constexpr int SUB = D / 64;                 // 64-element boxes per row
    constexpr int SUB_BYTES = TK * 128;
    constexpr int KS = D / 16;                  // k-steps of Q.K^T
    static_assert(TK == kConsumerWarps * 16, "one 16-key chunk per warp per tile");

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = smem_raw;
    uint64_t* full_bar  = reinterpret_cast<uint64_t*>(smem_raw + STAGES * Sh::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    __shared__ int s_failed;

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    griddep_launch_dependents();                  // a programmatic dependent may begin its own prefetch

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; ++s) { dme::mbar_init(&full_bar[s], 1); dme::mbar_init(&empty_bar[s], kConsumerWarps); }
        dme::mbar_init_fence();
    }
    __syncthreads();
    // Launched as a programmatic dependent (the runtime's decode step, p.pdl) the CTA is resident and set up by
    // now, possibly while its predecessor -- the projection that writes this step's q and the cache row of the
    // newest key -- is still running.  The key count and every cache row but the newest were written by launches
    // that completed before the predecessor could start, so the producer reads the count and fetches the tiles
    // that end before the newest key first, and waits for the predecessor only before the tile that holds it;
    // the consumers wait before they touch q.
    if (!p.pdl) griddep_wait();
    int N, per;
    decode_extent(p, N, per);
    const int k0 = min(split * per, N);
    const int k1 = min(k0 + per, N);
    const int ntiles = (k1 - k0 + TK - 1) / TK;

    if (warp == kConsumerWarps) {
        if (lane == 0) {
            dme::prefetch_tensor_map(&mapK);
            dme::prefetch_tensor_map(&mapV);
            const uint64_t pol = dme::policy_evict_first();
            dme::Ring<STAGES> ring;
            bool waited = !p.pdl;
            for (int t = 0; t < ntiles; ++t) {
                if (!waited && k0 + (t + 1) * TK >= N) { griddep_wait(); waited = true; }      // this tile reaches the newest key
                if (t >= STAGES && !dme::wait(&empty_bar[ring.stage], ring.phase ^ 1u, p.status)) { atomicExch(&s_failed, 1); break; }
                const int key = int(p.key_offset) + k0 + t * TK;
                unsigned char* dst = tiles + ring.stage * Sh::STAGE_BYTES;
                dme::mbar_arrive_expect_tx(&full_bar[ring.stage], Sh::STAGE_BYTES);
                #pragma unroll
                for (int sb = 0; sb < SUB; ++sb) {
                    dme::copy_tile_4d_stream(dst + sb * SUB_BYTES, &mapK, sb * 64, key, kvh, b, &full_bar[ring.stage], pol);
                    dme::copy_tile_4d_stream(dst + Sh::TILE_BYTES + sb * SUB_BYTES, &mapV, sb * 64, key, kvh, b, &full_bar[ring.stage], pol);
                }
                ring.advance();
            }
        }
    } else {
        const int g = lane / 4, t4 = lane % 4;
        if (p.pdl) griddep_wait();                    // q comes from the predecessor
        // Q fragments: rows g and g+8 are heads of the group (zero past it)
        uint32_t qa[KS][4];
        {
            const T* qbase = static_cast<const T*>(p.q) + size_t(b) * p.q_batch_stride + size_t(kvh) * p.group * D;
            const bool v0 = g < p.group, v1 = g + 8 < p.group;
            const uint32_t* r0 = reinterpret_cast<const uint32_t*>(qbase + size_t(v0 ? g : 0) * D);
            const uint32_t* r1 = reinterpret_cast<const uint32_t*>(qbase + size_t(v1 ? g + 8 : 0) * D);
            #pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                qa[ks][0] = v0 ? r0[ks * 8 + t4] : 0u;
                qa[ks][1] = v1 ? r1[ks * 8 + t4] : 0u;
                qa[ks][2] = v0 ? r0[ks * 8 + 4 + t4] : 0u;
                qa[ks][3] = v1 ? r1[ks * 8 + 4 + t4] : 0u;
            }
        }
        float o[D / 8][4];
        #pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; }
        float m0 = kNegBig, m1 = kNegBig, l0 = 0.f, l1 = 0.f;

        const int mi = lane / 8, r8 = lane % 8;
        const int row0 = warp * 16;
        const int krow = row0 + (mi >> 1) * 8 + r8, kchunk = mi & 1;      // K: matrices (n-tile, chunk)
        const int vrow = row0 + (mi & 1) * 8 + r8,  vchunk = mi >> 1;     // V: matrices (key half, chunk)

        dme::Ring<STAGES> ring;
        for (int t = 0; t < ntiles; ++t) {
            if (!dme::wait(&full_bar[ring.stage], ring.phase, p.status)) { atomicExch(&s_failed, 1); break; }
            const uint32_t kt = dme::smem_addr(tiles + ring.stage * Sh::STAGE_BYTES);
            const uint32_t vt = kt + Sh::TILE_BYTES;

            // even and odd k-steps accumulate apart (four independent chains of KS / 2 instead of two of KS) and meet in one
            // add.  (Issuing the next tile's scores before this tile's softmax as well measured slower.)
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float s_odd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            #pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int cc = 2 * ks + kchunk;
                uint32_t bk[4];
                ldmatrix_x4(bk, kt + (cc >> 3) * SUB_BYTES + swz128(krow, cc & 7));
                mma_16816<T>((ks & 1) ? s_odd[0] : s[0], qa[ks], bk[0], bk[1]);
                mma_16816<T>((ks & 1) ? s_odd[1] : s[1], qa[ks], bk[2], bk[3]);
            }
            #pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                #pragma unroll
                for (int j = 0; j < 4; ++j) s[nt][j] += s_odd[nt][j];
            }
            // scale to the log2 domain, mask keys past the end of this split
            const int key_base = k0 + t * TK + row0 + 2 * t4;
            #pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool live = key_base + nt * 8 + (j & 1) < k1;
                    s[nt][j] = live ? s[nt][j] * p.scale_log2 : kNegBig;
                }
            }
            float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            mx0 = wave::lane_group_reduce<4>(mx0, wave::MaxOp{});
            mx1 = wave::lane_group_reduce<4>(mx1, wave::MaxOp{});
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
            if (__any_sync(0xffffffffu, n0 != m0 || n1 != m1)) {
                const float a0 = fast_exp2(m0 - n0), a1 = fast_exp2(m1 - n1);
                l0 *= a0; l1 *= a1;
                #pragma unroll
                for (int nt = 0; nt < D / 8; ++nt) { o[nt][0] *= a0; o[nt][1] *= a0; o[nt][2] *= a1; o[nt][3] *= a1; }
                m0 = n0; m1 = n1;
            }
            float pr[2][4];
            #pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                #pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool live = key_base + nt * 8 + (j & 1) < k1;
                    pr[nt][j] = live ? fast_exp2(s[nt][j] - (j < 2 ? m0 : m1)) : 0.f;
                }
                l0 += pr[nt][0] + pr[nt][1];
                l1 += pr[nt][2] + pr[nt][3];
            }
            uint32_t pa[4];
            pa[0] = pack2<T>(pr[0][0], pr[0][1]);
            pa[1] = pack2<T>(pr[0][2], pr[0][3]);
            pa[2] = pack2<T>(pr[1][0], pr[1][1]);
            pa[3] = pack2<T>(pr[1][2], pr[1][3]);
            #pragma unroll
            for (int n2 = 0; n2 < D / 16; ++n2) {
                const int cc = 2 * n2 + vchunk;
                uint32_t bv[4];
                ldmatrix_x4_trans(bv, vt + (cc >> 3) * SUB_BYTES + swz128(vrow, cc & 7));
                mma_16816<T>(o[2 * n2], pa, bv[0], bv[1]);
                mma_16816<T>(o[2 * n2 + 1], pa, bv[2], bv[3]);
            }
            __syncwarp();
            if (lane == 0) dme::mbar_arrive(&empty_bar[ring.stage]);
            ring.advance();
        }
        l0 = wave::lane_group_reduce<4>(l0, wave::SumOp{});
        l1 = wave::lane_group_reduce<4>(l1, wave::SumOp{});

        // ---- merge the 8 warps through shared memory (tiles are dead past this barrier) ----
        asm volatile("bar.sync 1, %0;" :: "r"(kConsumerWarps * 32) : "memory");
        // rows of D + 8 floats: the eight row groups of a half-warp's 8-byte stores fall on different banks
        constexpr int DP = D + 8;
        float* sm_o  = reinterpret_cast<float*>(tiles);                 // [warp][16][DP]
        float* sm_ml = sm_o + kConsumerWarps * 16 * DP;                 // [warp][16][2]
        #pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g) * DP + nt * 8 + 2 * t4])     = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g + 8) * DP + nt * 8 + 2 * t4]) = make_float2(o[nt][2], o[nt][3]);
        }
        if (t4 == 0) {
            sm_ml[(warp * 16 + g) * 2] = m0;     sm_ml[(warp * 16 + g) * 2 + 1] = l0;
            sm_ml[(warp * 16 + g + 8) * 2] = m1; sm_ml[(warp * 16 + g + 8) * 2 + 1] = l1;
        }
        asm volatile("bar.sync 1, %0;" :: "r"(kConsumerWarps * 32) : "memory");
        // a thread merges pairs of columns of one head: the eight warps' factors are computed once per pair
        for (int e = 2 * threadIdx.x; e < p.group * D; e += 2 * kConsumerWarps * 32) {
            const int hh = e / D, d = e % D;
            float M = kNegBig;
            #pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) M = fmaxf(M, sm_ml[(w * 16 + hh) * 2]);
            float L = 0.f, O0 = 0.f, O1 = 0.f;
            #pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                const float2 ml = *reinterpret_cast<const float2*>(&sm_ml[(w * 16 + hh) * 2]);
                const float f = fast_exp2(ml.x - M);
                const float2 ov = *reinterpret_cast<const float2*>(&sm_o[(w * 16 + hh) * DP + d]);
                L += f * ml.y;
                O0 += f * ov.x; O1 += f * ov.y;
            }
            if (p.fused_o && p.splits == 1) {
                // the only split of its unit: this is the result, no partials and no merge
                T* dst = static_cast<T*>(p.fused_o) + size_t(b) * p.o_batch_stride + (size_t(kvh) * p.group + hh) * D + d;
                const float r0 = L > 0.f ? O0 / L : O0, r1 = L > 0.f ? O1 / L : O1;
                if (p.o_pairs) *reinterpret_cast<uint32_t*>(dst) = pack2<T>(r0, r1);
                else { dst[0] = from_float<T>(r0); dst[1] = from_float<T>(r1); }
                continue;
            }
            const size_t row = (size_t(b) * p.nQH + size_t(kvh) * p.group + hh) * p.splits + split;
            *reinterpret_cast<float2*>(&p.part_o[row * D + d]) = make_float2(O0, O1);
            if (d == 0) { p.part_ml[row * 2] = M; p.part_ml[row * 2 + 1] = L; }
        }
    }
    if (p.fused_o && p.splits > 1) {
        // ---- the last CTA of this (sequence, KV head) merges the unit's splits: the reference's
        // merge (fa_decode_kernel.hpp:75-92) without a second launch -------------------------------
        __shared__ int s_last;
        __threadfence();                                   // this CTA's partials are visible device-wide ...
        __syncthreads();
        if (threadIdx.x == 0) {                            // ... before its ticket is
            unsigned int* tk = p.tickets + size_t(b) * p.nKVH + kvh;
            const unsigned int t = atomicAdd(tk, 1u);
            s_last = (t == unsigned(p.splits) - 1u);
            if (s_last) *tk = 0u;                          // ready for the next launch on this stream
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            constexpr int PER = D / 32;
            for (int hh = warp; hh < p.group; hh += kDecodeThreads / 32) {
                const size_t row = size_t(b) * p.nQH + size_t(kvh) * p.group + hh;
                const float* ml = p.part_ml + row * p.splits * 2;
                const float* po = p.part_o + row * p.splits * D;
                float M = kNegBig;
                for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(ml + 2 * s));
                float L = 0.f, acc[PER];
                #pragma unroll
                for (int i = 0; i < PER; ++i) acc[i] = 0.f;
                for (int s = 0; s < p.splits; ++s) {
                    const float f = exp2f(__ldcg(ml + 2 * s) - M);
                    L += f * __ldcg(ml + 2 * s + 1);
                    #pragma unroll
                    for (int i = 0; i < PER; ++i) acc[i] += f * __ldcg(po + size_t(s) * D + lane + 32 * i);
                }
                const float inv = L > 0.f ? 1.f / L : 1.f;
                T* orow = static_cast<T*>(p.fused_o) + size_t(b) * p.o_batch_stride + (size_t(kvh) * p.group + hh) * D;
                #pragma unroll
                for (int i = 0; i < PER; ++i) orow[lane + 32 * i] = from_float<T>(acc[i] * inv);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_failed) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------
// Combine the splits of every (sequence, query head): the reference's merge
// (fa_decode_kernel.hpp:75-92) in the log2 domain.  One warp per row.
// MODE 0: o = O / l in the 16-bit output type.
// MODE 1: normalised O in fp32 plus lse (natural log), the form exchanged
//         between GPUs when the KV sequence is sharded.
// ---------------------------------------------------------------------------
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(128)
decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits, int rows,
                      int rows_per_seq, long long o_batch_stride,
                      T* __restrict__ o, float* __restrict__ o_f32, float* __restrict__ lse) {
    griddep_launch_dependents();
    const int row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= rows) return;
    constexpr int PER = D / 32;
    float M = kNegBig;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(size_t(row) * splits + s) * 2]);
    float L = 0.f, acc[PER];
    #pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float f = exp2f(part_ml[(size_t(row) * splits + s) * 2] - M);
        L += f * part_ml[(size_t(row) * splits + s) * 2 + 1];
        #pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += f * part_o[(size_t(row) * splits + s) * D + lane + 32 * i];
    }
    const float inv = L > 0.f ? 1.f / L : 1.f;
    #pragma unroll
    for (int i = 0; i < PER; ++i) {
        const float v = acc[i] * inv;
        if (MODE == 0) o[size_t(row / rows_per_seq) * o_batch_stride + size_t(row % rows_per_seq) * D + lane + 32 * i] = from_float<T>(v);
        else           o_f32[size_t(row) * D + lane + 32 * i] = v;
    }
    if (MODE == 1 && lane == 0) lse[row] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
}

// Merge G normalised partials by their lse (KV sequence sharded over G ranks):
// O = sum_g e^{lse_g - M} O_g / sum_g e^{lse_g - M}.  Part g starts at o_parts + g*o_stride
// ([rows][D]) and lse_parts + g*l_stride ([rows]).
template <typename T, int D>
__global__ void __launch_bounds__(128)
merge_lse_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts, int G, int rows,
                 long long o_stride, long long l_stride, T* __restrict__ o) {
    const int row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= rows) return;
    constexpr int PER = D / 32;
    float M = -INFINITY;
    for (int g = 0; g < G; ++g) M = fmaxf(M, lse_parts[size_t(g) * l_stride + row]);
    float den = 0.f, acc[PER];
    #pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int g = 0; g < G; ++g) {
        const float w = (M == -INFINITY) ? 0.f : __expf(lse_parts[size_t(g) * l_stride + row] - M);
        den += w;
        #pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += w * o_parts[size_t(g) * o_stride + size_t(row) * D + lane + 32 * i];
    }
    const float inv = den > 0.f ? 1.f / den : 1.f;
    #pragma unroll
    for (int i = 0; i < PER; ++i) o[size_t(row) * D + lane + 32 * i] = from_float<T>(acc[i] * inv);
}

// ---------------------------------------------------------------------------
// Exchange of the (O, lse) partials over peer memory (KV sequence sharded over the
// GPUs of one node).  Instead of writing its partial locally and handing it to a
// collective, the combine kernel stores each normalised row straight into slot
// [parity][rank] of EVERY rank's receive buffer (plain peer stores over NVLink, no
// multicast), and the last CTA to finish publishes the step number in word [rank]
// of every rank's flag array.  The merge kernel on each GPU then waits, bounded,
// until all flag words have reached the step number and merges from its own memory.
// Receive buffers are double-buffered by step parity: a rank can be at most one
// step ahead of the slowest one, because its next merge needs that rank's flag.
// ---------------------------------------------------------------------------
struct PeerTable {
    float* slots[B200P_MAX_PEERS];
    int*   flags[B200P_MAX_PEERS];
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

template <int D>
__global__ void __launch_bounds__(128)
decode_combine_push_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits, int rows,
                           PeerTable peers, int rank, int world, int seq, int* __restrict__ counter) {
    const int row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
    constexpr int PER = D / 32;
    if (row < rows) {
        float M = kNegBig;
        for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[(size_t(row) * splits + s) * 2]);
        float L = 0.f, acc[PER];
        #pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float f = exp2f(part_ml[(size_t(row) * splits + s) * 2] - M);
            L += f * part_ml[(size_t(row) * splits + s) * 2 + 1];
            #pragma unroll
            for (int i = 0; i < PER; ++i) acc[i] += f * part_o[(size_t(row) * splits + s) * D + lane + 32 * i];
        }
        const float inv = L > 0.f ? 1.f / L : 1.f;
        const float lse = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        const size_t n = size_t(rows) * (D + 1);
        const size_t slot = (size_t(seq & 1) * world + rank) * n;
        for (int g = 0; g < world; ++g) {
            float* dst = peers.slots[(rank + g) % world] + slot;         // start with the own GPU, then round the ring
            #pragma unroll
            for (int i = 0; i < PER; ++i) dst[size_t(row) * D + lane + 32 * i] = acc[i] * inv;
            if (lane == 0) dst[size_t(rows) * D + row] = lse;
        }
    }
    // publish: every CTA fences its stores, the last one to count in raises the flags
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int old = atomicAdd(counter, 1);
        if (old == int(gridDim.x) - 1) {
            *counter = 0;                                                // ready for the next launch on this stream
            __threadfence_system();
            for (int g = 0; g < world; ++g) st_release_sys(peers.flags[(rank + g) % world] + rank, seq);
        }
    }
}

// Merge after the peer exchange: waits (bounded by wait_ns of wall time) until every
// rank's flag word has reached `seq`, then merges the `world` packed partials of this
// step's parity.  A wait that runs out sets *status to 1 and the launch finishes
// without hanging (its output is then meaningless).
template <typename T, int D>
__global__ void __launch_bounds__(128)
merge_lse_wait_kernel(const float* slots, const int* flags, int world, int seq, int rows,
                      T* __restrict__ o, int* status, unsigned long long wait_ns) {
    if (threadIdx.x < world) {
        const int* f = flags + threadIdx.x;
        if (ld_acquire_sys(f) < seq) {
            const uint64_t t0 = dme::global_timer_ns();
            for (;;) {
                bool ok = false;
                #pragma unroll 1
                for (int i = 0; i < 64 && !ok; ++i) ok = ld_acquire_sys(f) >= seq;
                if (ok) break;
                if (*reinterpret_cast<volatile int*>(status) != 0) break;
                if (dme::global_timer_ns() - t0 > wait_ns) { atomicExch(status, 1); break; }
            }
        }
    }
    __syncthreads();
    const int row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= rows) return;
    constexpr int PER = D / 32;
    const size_t n = size_t(rows) * (D + 1);
    const float* base = slots + size_t(seq & 1) * world * n;
    float M = -INFINITY;
    for (int g = 0; g < world; ++g) M = fmaxf(M, __ldcg(base + g * n + size_t(rows) * D + row));
    float den = 0.f, acc[PER];
    #pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int g = 0; g < world; ++g) {
        const float w = (M == -INFINITY) ? 0.f : __expf(__ldcg(base + g * n + size_t(rows) * D + row) - M);
        den += w;
        #pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += w * __ldcg(base + g * n + size_t(row) * D + lane + 32 * i);
    }
    const float inv = den > 0.f ? 1.f / den : 1.f;
    #pragma unroll
    for (int i = 0; i < PER; ++i) o[size_t(row) * D + lane + 32 * i] = from_float<T>(acc[i] * inv);
}

// ---- host side ------------------------------------------------------------------------
struct DecodePlan { int splits, keys_per_split; size_t ws_bytes, off_tickets, off_ml, off_o; };

DecodePlan plan_decode(int D, int N, int nQH, int nKVH, int batch) {
    DecodePlan pl{};
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long long units = (long long)batch * nKVH;
    int splits = tuning(KNOB_DECODE_SPLITS, 0);
    if (splits <= 0) {
        // enough CTAs for ~8 rounds over the SMs, at least 256 keys per split
        const long long want = (8LL * sms + units - 1) / units;
        const long long cap = (N + 255) / 256;
        splits = int(want < 1 ? 1 : (want > cap ? cap : want));
        // a short sequence fits the ring in one or two fills: splitting it buys no bandwidth and costs the merge
        if (N <= 1024) splits = 1;
    }
    if (splits < 1) splits = 1;
    if (splits > 65535) splits = 65535;
    int per = (N + splits - 1) / splits;
    per = (per + 127) / 128 * 128;                      // whole tiles per split
    splits = (N + per - 1) / per;
    if (splits < 1) splits = 1;
    pl.splits = splits; pl.keys_per_split = per;
    const size_t rows = size_t(batch) * nQH;
    pl.off_tickets = 256;                               // [0,256): status word; then one arrival counter per (sequence, KV head)
    pl.off_ml = pl.off_tickets + ((size_t(batch) * nKVH * sizeof(unsigned int) + 255) / 256) * 256;
    pl.off_o = pl.off_ml + ((rows * splits * 2 * sizeof(float) + 255) / 256) * 256;
    pl.ws_bytes = pl.off_o + rows * splits * D * sizeof(float);
    return pl;
}

int validate(const b200p_decode_args* a) {
    if (!a) return B200P_E_NULL;
    if (a->dtype != B200P_F16 && a->dtype != B200P_BF16) return B200P_E_DTYPE;
    if (a->D != 64 && a->D != 128) return B200P_E_DIM;                       // attention.hpp:134-136
    if (a->nQHeads <= 0 || a->nKVHeads <= 0 || a->nQHeads % a->nKVHeads != 0) return B200P_E_DIM;
    if (a->nQHeads / a->nKVHeads > 32) return B200P_E_DIM;
    if (a->N <= 0 || a->batch <= 0) return B200P_E_LENGTH;
    if (a->batch > 65535 || a->nKVHeads > 65535) return B200P_E_RANGE;
    if (a->key_offset < 0 || a->stride_kv < a->N + a->key_offset) return B200P_E_LENGTH;
    return B200P_OK;
}

template <typename T, int D, int GH>
int launch_decode_gh(const DecodeParams& p, cudaStream_t st) {
    using Sh = DecodeShape<D>;
    auto kern = decode_splitkv_kernel<T, D, GH>;
    static bool attr_set[64] = {};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Sh::SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        attr_set[dev] = true;
    }
    dim3 grid(p.splits, p.nKVH, p.batch);
    kern<<<grid, kDecodeThreads, Sh::SMEM_BYTES, st>>>(p);
    return launched();
}
template <typename T, int D>
int launch_decode(const DecodeParams& p, cudaStream_t st) {
    if (p.group == 1) return launch_decode_gh<T, D, 1>(p, st);
    if (p.group == 2) return launch_decode_gh<T, D, 2>(p, st);
    return launch_decode_gh<T, D, 4>(p, st);
}
template <typename T>
int launch_decode_d(const DecodeParams& p, int D, cudaStream_t st) {
    return D == 128 ? launch_decode<T, 128>(p, st) : launch_decode<T, 64>(p, st);
}

template <typename T, int D>
int launch_decode_mma(const DecodeParams& p, const b200p_decode_args* a, cudaStream_t st) {
    using Sh = DecodeShape<D>;
    // K/V as 4-D tensors (D, keys, KV heads, sequences); keys past key_offset + N read as zero.
    // With a device-side key count N is only the bound: rows between the live count and the end
    // of the last 128-key tile are fetched as stored and masked in the softmax (their P is 0).
    CUtensorMap mk, mv;
    const uint64_t dims[4] = {uint64_t(D), uint64_t(a->key_offset + a->N), uint64_t(a->nKVHeads), uint64_t(a->batch)};
    const uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(p.kv_head_stride) * 2, uint64_t(p.kv_batch_stride) * 2};
    const uint32_t box[4] = {64, uint32_t(Sh::TK), 1, 1};
    const CUtensorMapDataType dt = a->dtype == B200P_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    cudaError_t e = make_tensor_map(&mk, dt, 4, p.K, dims, strides, box, Swizzle::B128);
    if (e == cudaSuccess) e = make_tensor_map(&mv, dt, 4, p.V, dims, strides, box, Swizzle::B128);
    if (e != cudaSuccess) return int(e);
    auto kern = decode_mma_kernel<T, D>;
    static bool attr_set[64] = {};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Sh::SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        attr_set[dev] = true;
    }
    dim3 grid(p.splits, p.nKVH, p.batch);
    if (p.pdl) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid; cfg.blockDim = dim3(kDecodeThreads); cfg.dynamicSmemBytes = Sh::SMEM_BYTES; cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, p, mk, mv);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return le == cudaSuccess ? B200P_OK : int(le);
    }
    kern<<<grid, kDecodeThreads, Sh::SMEM_BYTES, st>>>(p, mk, mv);
    return launched();
}
template <typename T>
int launch_decode_mma_d(const DecodeParams& p, const b200p_decode_args* a, cudaStream_t st) {
    return a->D == 128 ? launch_decode_mma<T, 128>(p, a, st) : launch_decode_mma<T, 64>(p, a, st);
}

template <typename T, int D>
int launch_combine(const float* po, const float* pml, int splits, int rows, int rows_per_seq, long long o_bs,
                   void* o, float* o32, float* lse, cudaStream_t st) {
    const int grid = (rows + 3) / 4;
    if (o) decode_combine_kernel<T, D, 0><<<grid, 128, 0, st>>>(po, pml, splits, rows, rows_per_seq, o_bs, static_cast<T*>(o), nullptr, nullptr);
    else   decode_combine_kernel<T, D, 1><<<grid, 128, 0, st>>>(po, pml, splits, rows, rows_per_seq, o_bs, nullptr, o32, lse);
    return launched();
}

int validate_peers(const b200p_peer_exchange* px) {
    if (!px || !px->counter) return B200P_E_NULL;
    if (px->world < 1 || px->world > B200P_MAX_PEERS || px->rank < 0 || px->rank >= px->world) return B200P_E_RANGE;
    for (int g = 0; g < px->world; ++g) {
        if (!px->slots[g] || !px->flags[g]) return B200P_E_NULL;
        if (!aligned(px->slots[g], 4) || !aligned(px->flags[g], 4)) return B200P_E_ALIGN;
    }
    return B200P_OK;
}

int run_decode(const b200p_decode_args* a, const void* q, const void* K, const void* V,
               void* o, float* o_f32, float* lse, void* ws, size_t ws_bytes, cudaStream_t st,
               const b200p_peer_exchange* px = nullptr, int seq = 0, const int* n_dev = nullptr, int n_add = 0,
               bool prepared = false) {
    if (int e = validate(a)) return e;
    if (!q || !K || !V || (!px && !o && !(o_f32 && lse))) return B200P_E_NULL;
    if (px) {
        if (int e = validate_peers(px)) return e;
        if (seq < 1) return B200P_E_RANGE;
    }
    if (!aligned(K, 16) || !aligned(V, 16) || !aligned(q, 2)) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    const DecodePlan pl = plan_decode(a->D, a->N, a->nQHeads, a->nKVHeads, a->batch);
    if (!ws || ws_bytes < pl.ws_bytes || !aligned(ws, 256)) return B200P_E_WORKSPACE;

    DecodeParams p{};
    p.q = q; p.K = K; p.V = V;
    p.status = static_cast<int*>(ws);
    p.part_ml = reinterpret_cast<float*>(static_cast<char*>(ws) + pl.off_ml);
    p.part_o  = reinterpret_cast<float*>(static_cast<char*>(ws) + pl.off_o);
    p.N = a->N; p.nQH = a->nQHeads; p.nKVH = a->nKVHeads; p.group = a->nQHeads / a->nKVHeads; p.batch = a->batch;
    p.splits = pl.splits; p.keys_per_split = pl.keys_per_split;
    p.kv_head_stride = (long long)a->stride_kv * a->D;
    p.kv_batch_stride = a->kv_batch_stride > 0 ? a->kv_batch_stride : (long long)a->nKVHeads * a->stride_kv * a->D;
    p.key_offset = a->key_offset;
    p.q_batch_stride = a->q_batch_stride > 0 ? a->q_batch_stride : (long long)a->nQHeads * a->D;
    if (p.q_batch_stride % 2) return B200P_E_ALIGN;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(a->D));
    p.n_dev = n_dev; p.n_add = n_add;
    // K/V rows must start on 16 bytes for the bulk copies
    if ((p.kv_head_stride * 2) % 16 || (p.kv_batch_stride * 2) % 16) return B200P_E_ALIGN;

    // variant 1 (default): TMA tensor maps + mma.sync; variant 0: bulk copies + vector FMAs.
    // The tensor-core kernel holds the whole group in one M = 16 tile.
    const bool use_mma = tuning(KNOB_DECODE_VARIANT, 1) == 1 && p.group <= 16 && aligned(q, 4);
    const long long obs = a->o_batch_stride > 0 ? a->o_batch_stride : (long long)a->nQHeads * a->D;
    // 16-bit output from the tensor-core kernel: the combine is fused into it (last CTA of a unit merges)
    const bool fused = use_mma && o && !px && tuning(KNOB_DECODE_FUSED_COMBINE, 1) != 0;
    p.pdl = prepared && fused && tuning(KNOB_RUNTIME_PDL, 1) != 0;     // the runtime's decode step only
    if (fused) {
        p.fused_o = o; p.o_batch_stride = obs;
        p.o_pairs = aligned(o, 4) && obs % 2 == 0;
        p.tickets = reinterpret_cast<unsigned int*>(static_cast<char*>(ws) + pl.off_tickets);
    }
    // Clear the status word and the arrival counters, unless the caller keeps the workspace
    // prepared (both zero before the first launch; the counters reset themselves, and the
    // status word only ever changes when a bounded wait gives up).
    if (!prepared) {
        const cudaError_t ce = cudaMemsetAsync(ws, 0, pl.off_ml, st);
        if (ce != cudaSuccess) return int(ce);
    }
    int e;
    if (use_mma) e = a->dtype == B200P_F16 ? launch_decode_mma_d<__half>(p, a, st) : launch_decode_mma_d<__nv_bfloat16>(p, a, st);
    else         e = a->dtype == B200P_F16 ? launch_decode_d<__half>(p, a->D, st) : launch_decode_d<__nv_bfloat16>(p, a->D, st);
    if (e) return e;
    if (fused) return B200P_OK;
    const int rows = a->batch * a->nQHeads, rps = a->nQHeads;
    if (px) {
        PeerTable pt{};
        for (int g = 0; g < px->world; ++g) { pt.slots[g] = px->slots[g]; pt.flags[g] = px->flags[g]; }
        const int grid = (rows + 3) / 4;
        if (a->D == 128) decode_combine_push_kernel<128><<<grid, 128, 0, st>>>(p.part_o, p.part_ml, pl.splits, rows, pt, px->rank, px->world, seq, px->counter);
        else             decode_combine_push_kernel<64><<<grid, 128, 0, st>>>(p.part_o, p.part_ml, pl.splits, rows, pt, px->rank, px->world, seq, px->counter);
        return launched();
    }
    if (a->dtype == B200P_F16)
        return a->D == 128 ? launch_combine<__half, 128>(p.part_o, p.part_ml, pl.splits, rows, rps, obs, o, o_f32, lse, st)
                           : launch_combine<__half, 64>(p.part_o, p.part_ml, pl.splits, rows, rps, obs, o, o_f32, lse, st);
    return a->D == 128 ? launch_combine<__nv_bfloat16, 128>(p.part_o, p.part_ml, pl.splits, rows, rps, obs, o, o_f32, lse, st)
                       : launch_combine<__nv_bfloat16, 64>(p.part_o, p.part_ml, pl.splits, rows, rps, obs, o, o_f32, lse, st);
}

} // namespace

// For callers inside the library that keep their workspace prepared (status word and arrival
// counters zero before the first use): decode without the clearing memset, key count by value
// (n_dev null) or read on the device.
int decode_prepared(const void* q, const void* K, const void* V, void* o, const b200p_decode_args* a,
                    const int* n_dev, int n_add, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (!o) return B200P_E_NULL;
    return run_decode(a, q, K, V, o, nullptr, nullptr, ws, ws_bytes, st, nullptr, 0, n_dev, n_add, true);
}
} // namespace b200p

using namespace b200p;

extern "C" size_t b200p_attn_decode_workspace_bytes(const b200p_decode_args* a) {
    if (validate(a) != B200P_OK) return 0;
    return plan_decode(a->D, a->N, a->nQHeads, a->nKVHeads, a->batch).ws_bytes;
}

extern "C" int b200p_attn_decode(const void* q, const void* K, const void* V, void* o,
                                 const b200p_decode_args* a, void* workspace, size_t workspace_bytes,
                                 b200p_stream_t stream) {
    if (!o) return B200P_E_NULL;
    return run_decode(a, q, K, V, o, nullptr, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int b200p_attn_decode_dyn(const void* q, const void* K, const void* V, void* o,
                                     const b200p_decode_args* a, const int* n_dev, int n_add,
                                     void* workspace, size_t workspace_bytes, b200p_stream_t stream) {
    if (!o || !n_dev) return B200P_E_NULL;
    return run_decode(a, q, K, V, o, nullptr, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream),
                      nullptr, 0, n_dev, n_add);
}

extern "C" int b200p_attn_decode_partial(const void* q, const void* K, const void* V, float* o_f32, float* lse,
                                         const b200p_decode_args* a, void* workspace, size_t workspace_bytes,
                                         b200p_stream_t stream) {
    if (!o_f32 || !lse) return B200P_E_NULL;
    return run_decode(a, q, K, V, nullptr, o_f32, lse, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int b200p_attn_merge_lse(const float* o_parts, const float* lse_parts, int parts, int rows, int D,
                                    long long o_part_stride, long long lse_part_stride,
                                    int dtype, void* o, b200p_stream_t stream) {
    const long long os = o_part_stride > 0 ? o_part_stride : (long long)rows * D;
    const long long ls = lse_part_stride > 0 ? lse_part_stride : (long long)rows;
    if (!o_parts || !lse_parts || !o) return B200P_E_NULL;
    if (dtype != B200P_F16 && dtype != B200P_BF16) return B200P_E_DTYPE;
    if (D != 64 && D != 128) return B200P_E_DIM;
    if (parts <= 0 || rows <= 0) return B200P_E_LENGTH;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (rows + 3) / 4;
    if (dtype == B200P_F16) {
        if (D == 128) merge_lse_kernel<__half, 128><<<grid, 128, 0, st>>>(o_parts, lse_parts, parts, rows, os, ls, static_cast<__half*>(o));
        else          merge_lse_kernel<__half, 64><<<grid, 128, 0, st>>>(o_parts, lse_parts, parts, rows, os, ls, static_cast<__half*>(o));
    } else {
        if (D == 128) merge_lse_kernel<__nv_bfloat16, 128><<<grid, 128, 0, st>>>(o_parts, lse_parts, parts, rows, os, ls, static_cast<__nv_bfloat16*>(o));
        else          merge_lse_kernel<__nv_bfloat16, 64><<<grid, 128, 0, st>>>(o_parts, lse_parts, parts, rows, os, ls, static_cast<__nv_bfloat16*>(o));
    }
    return launched();
}

extern "C" int b200p_attn_decode_push(const void* q, const void* K, const void* V,
                                      const b200p_decode_args* a, void* workspace, size_t workspace_bytes,
                                      const b200p_peer_exchange* px, int seq, b200p_stream_t stream) {
    if (!px) return B200P_E_NULL;
    return run_decode(a, q, K, V, nullptr, nullptr, nullptr, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream), px, seq);
}

extern "C" int b200p_attn_merge_lse_wait(const b200p_peer_exchange* px, int seq, int rows, int D, int dtype,
                                         void* o, int* status, unsigned long long wait_ns, b200p_stream_t stream) {
    if (!o || !status) return B200P_E_NULL;
    if (int e = validate_peers(px)) return e;
    if (dtype != B200P_F16 && dtype != B200P_BF16) return B200P_E_DTYPE;
    if (D != 64 && D != 128) return B200P_E_DIM;
    if (rows <= 0) return B200P_E_LENGTH;
    if (seq < 1) return B200P_E_RANGE;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    if (wait_ns == 0) wait_ns = dme::kWaitLimitNs;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (rows + 3) / 4;
    const float* slots = px->slots[px->rank];
    const int* flags = px->flags[px->rank];
    const int w = px->world;
    if (dtype == B200P_F16) {
        if (D == 128) merge_lse_wait_kernel<__half, 128><<<grid, 128, 0, st>>>(slots, flags, w, seq, rows, static_cast<__half*>(o), status, wait_ns);
        else          merge_lse_wait_kernel<__half, 64><<<grid, 128, 0, st>>>(slots, flags, w, seq, rows, static_cast<__half*>(o), status, wait_ns);
    } else {
        if (D == 128) merge_lse_wait_kernel<__nv_bfloat16, 128><<<grid, 128, 0, st>>>(slots, flags, w, seq, rows, static_cast<__nv_bfloat16*>(o), status, wait_ns);
        else          merge_lse_wait_kernel<__nv_bfloat16, 64><<<grid, 128, 0, st>>>(slots, flags, w, seq, rows, static_cast<__nv_bfloat16*>(o), status, wait_ns);
    }
    return launched();
}

// ---------------------------------------------------------------------------
// Decode without caller-provided scratch.
//
// Some hosts of this library cannot hand it device memory: a serving loop whose
// memory plan was frozen at start-up, or an embedding runtime that only passes
// the tensors it owns and has no allocator to lend.  For them the split-KV
// partials live in this fixed array, which is part of the library image: every
// GPU that loads the library carries these bytes until the process exits.
// The array's name is only a host-side handle; the device address is looked up
// once per device (with that device current) and handed to the kernels.
// ---------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;        // 8 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
// Per device, filled at first use.  Two host threads that make their first call on a device at the same
// time both look the address up and store the same value: a benign race.
static void* g_noalloc_ptr[64] = {};

extern "C" size_t b200p_attn_decode_noalloc_max_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int b200p_attn_decode_noalloc(const void* q, const void* K, const void* V, void* o,
                                         const b200p_decode_args* a, b200p_stream_t stream) {
    if (!o) return B200P_E_NULL;
    if (int e = validate(a)) return e;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    const DecodePlan pl = plan_decode(a->D, a->N, a->nQHeads, a->nKVHeads, a->batch);
    if (pl.ws_bytes > kNoAllocScratchBytes) return B200P_E_RANGE;      // shapes too large for the built-in scratch
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200P_E_NO_DEVICE;
    if (!g_noalloc_ptr[dev]) {
        // set-up, once per device: resolve the array's device address
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return int(e);
        g_noalloc_ptr[dev] = ptr;
    }
    // run_decode clears the status word at the front of the scratch; the partials
    // behind it are overwritten before they are read.
    return run_decode(a, q, K, V, o, nullptr, nullptr, g_noalloc_ptr[dev], kNoAllocScratchBytes,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int b200p_attn_workspace_status(const void* workspace, b200p_stream_t stream) {
    if (!workspace) {
        // NULL names the library's built-in scratch (b200p_attn_decode_noalloc) on the current device
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200P_E_NO_DEVICE;
        workspace = g_noalloc_ptr[dev];
        if (!workspace) return B200P_OK;                        // never used on this device: nothing can have failed
    }
    int h = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&h, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return int(e);
    return h == 0 ? B200P_OK : B200P_E_TIMEOUT;
}
