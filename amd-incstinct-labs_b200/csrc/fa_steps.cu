// ---------------------------------------------------------------------------
// fa_steps.cu -- the reference's FA2 build-order steps on warp primitives.
//
//   step 0  fa_naive  research/flash-attention-mi300x/fa_naive.hip:72-212
//           one wave per query row, portable shfl_down softmax reductions
//   step 1  fa_dpp    research/flash-attention-mi300x/fa_dpp.hip:52-167
//           the same with wave::dpp::reduce_max_bcast / reduce_sum_bcast
//   step 2  fa_dme    research/flash-attention-mi300x/fa_dme.hip:74-221
//           step 1 + K/V tiles double-buffered by asynchronous copies
//   (step 3, fa_mfma2, is the tcgen05 kernel in prefill.cu)
// and, with fp32 I/O, the reference's fp32 kernels
//   research/flash-attention-mi300x/kernels/fa_naive.hip:118-278
//   research/flash-attention-mi300x/kernels/fa_dpp.hip:167-313
// whose launch takes (seq_len, n_heads, scale).
//
// Tiling is the reference's: Br = 16 query rows per CTA (one warp per row),
// Bc = 64 keys per tile.  A 64-key score row is held by ONE 32-lane warp as an
// adjacent pair per lane (keys 2l, 2l+1), which is exactly the shape the pair
// overloads of wave64.cuh reduce; O stays in registers (D/32 dims per lane)
// instead of the reference's LDS accumulator.
// These kernels exist for parity with the reference's steps and to exercise the
// primitives and the TMA ring in a simple setting; at the reference's config
// (0.54 GFLOP, 4 MiB) they are launch-bound on a B200.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "attn_common.cuh"
#include "dme/dme_tma.cuh"
#include "wave_primitives/wave64.cuh"

namespace b200p {
int prefill_dispatch(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                     float* debug_s, cudaStream_t st);
namespace {

constexpr int kBr = 16, kBc = 64;

// The reference's portable reduction: v op= shfl_down(v, o), then broadcast lane 0
// (fa_naive.hip:48-58), on a pair per lane.
template <typename Op>
__device__ __forceinline__ float portable_reduce_bcast(float a, float b, Op op) {
    float v = op(a, b);
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_down_sync(0xffffffffu, v, o));
    return __shfl_sync(0xffffffffu, v, 0);
}

template <typename T> __device__ __forceinline__ float exp_for(float x);
template <> __device__ __forceinline__ float exp_for<float>(float x)         { return expf(x); }
template <> __device__ __forceinline__ float exp_for<__half>(float x)        { return __expf(x); }
template <> __device__ __forceinline__ float exp_for<__nv_bfloat16>(float x) { return __expf(x); }

template <typename T, int D, int STEP>
__global__ void __launch_bounds__(kBr * 32)
fa_step_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V, T* __restrict__ O,
               int seq_q, int seq_k, int heads, float scale, int* abort_word, int* sticky) {
    constexpr int DPL = D / 32;                           // output dims per lane
    constexpr uint32_t kTileBytes = kBc * D * sizeof(T);
    extern __shared__ __align__(128) unsigned char smem[];
    T* Kt = reinterpret_cast<T*>(smem);                                    // [2][Bc*D] (one buffer used for STEP < 2)
    T* Vt = reinterpret_cast<T*>(smem + 2 * kTileBytes);
    float* prow = reinterpret_cast<float*>(smem + 4 * kTileBytes);         // [Br][Bc]
    float* qs = prow + kBr * kBc;                                          // [Br][D]
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + 4 * kTileBytes + (kBr * kBc + kBr * D) * sizeof(float));
    __shared__ int s_failed;

    // blockIdx.x = batch * heads * (seq_q/Br) + head * (seq_q/Br) + qblk   (fa_naive.hip:70-71)
    const int qblocks = seq_q / kBr;
    const int qblk = blockIdx.x % qblocks;
    const int bh = blockIdx.x / qblocks;                                   // batch * heads + head
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const T* Qrow = Q + (size_t(bh) * seq_q + qblk * kBr + warp) * D;
    const T* Kb = K + size_t(bh) * seq_k * D;
    const T* Vb = V + size_t(bh) * seq_k * D;
    T* Orow = O + (size_t(bh) * seq_q + qblk * kBr + warp) * D;
    const int ntiles = seq_k / kBc;

    if (STEP == 2 && threadIdx.x == 0) {
        s_failed = 0;
        dme::mbar_init(&full[0], 1); dme::mbar_init(&full[1], 1);
        dme::mbar_init_fence();
    }
    // This warp's query row as fp32.  With 16-bit keys a lane reads 8 floats of q per 16-byte key chunk, so the eight
    // lanes of a shared-memory phase read pieces 32 bytes apart, 256 bytes in all: pieces 0 and 4 would share their
    // banks.  The row is therefore stored with its float4 index f at f ^ ((f >> 3) & 1).
    constexpr bool kSwizzleQ = sizeof(T) == 2;
    auto qpos = [](int f4) -> int { return kSwizzleQ ? (f4 ^ ((f4 >> 3) & 1)) : f4; };
    float* q = qs + warp * D;
    for (int d = lane; d < D; d += 32) q[qpos(d / 4) * 4 + d % 4] = to_float(Qrow[d]);
    __syncthreads();
    if (STEP == 2 && threadIdx.x == 0) {                  // prologue: tile 0 -> buffer 0
        dme::mbar_arrive_expect_tx(&full[0], 2 * kTileBytes);
        dme::copy_tile_1d(Kt, Kb, kTileBytes, &full[0]);
        dme::copy_tile_1d(Vt, Vb, kTileBytes, &full[0]);
    }

    float m = -1e38f, l = 0.f;                            // the reference's initial running max
    float o[DPL];
    #pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.f;
    bool ok = true;

    for (int j = 0; j < ntiles; ++j) {
        const int buf = (STEP == 2) ? (j & 1) : 0;
        const T* Kc = Kt + buf * kBc * D;
        const T* Vc = Vt + buf * kBc * D;
        if (STEP == 2) {
            if (threadIdx.x == 0 && j + 1 < ntiles) {     // prefetch tile j+1 into the other buffer
                const int nb = (j + 1) & 1;
                dme::mbar_arrive_expect_tx(&full[nb], 2 * kTileBytes);
                dme::copy_tile_1d(Kt + nb * kBc * D, Kb + size_t(j + 1) * kBc * D, kTileBytes, &full[nb]);
                dme::copy_tile_1d(Vt + nb * kBc * D, Vb + size_t(j + 1) * kBc * D, kTileBytes, &full[nb]);
            }
            if (!dme::wait(&full[buf], uint32_t(j >> 1) & 1u, abort_word)) { ok = false; }
        } else {
            // cooperative synchronous tile load, 16 bytes per thread per step
            const uint4* ks = reinterpret_cast<const uint4*>(Kb + size_t(j) * kBc * D);
            const uint4* vs = reinterpret_cast<const uint4*>(Vb + size_t(j) * kBc * D);
            uint4* kd = reinterpret_cast<uint4*>(Kt);
            uint4* vd = reinterpret_cast<uint4*>(Vt);
            for (int i = threadIdx.x; i < int(kTileBytes / 16); i += kBr * 32) { kd[i] = ks[i]; vd[i] = vs[i]; }
            __syncthreads();
        }
        // S[row][2l], S[row][2l+1].  Every lane reads its own two key rows, which lie a multiple of 128 bytes apart:
        // read in the same order they would all hit the same banks.  Lane l starts at 16-byte chunk l of its rows and
        // wraps, so the eight lanes of a shared-memory phase read eight different chunks (and eight different pieces of q).
        float s0 = 0.f, s1 = 0.f;
        {
            constexpr int EPC = 16 / int(sizeof(T)), NCH = D / EPC;           // elements per chunk, chunks per row
            const uint4* kr0 = reinterpret_cast<const uint4*>(Kc + (2 * lane) * D);
            const uint4* kr1 = kr0 + NCH;
            #pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int cc = (c + lane) & (NCH - 1);
                const uint4 ka = kr0[cc], kb = kr1[cc];
                const T* ea = reinterpret_cast<const T*>(&ka);
                const T* eb = reinterpret_cast<const T*>(&kb);
                float qv[EPC];
                #pragma unroll
                for (int e = 0; e < EPC; e += 4) *reinterpret_cast<float4*>(&qv[e]) = *reinterpret_cast<const float4*>(q + qpos((cc * EPC + e) / 4) * 4);
                #pragma unroll
                for (int e = 0; e < EPC; ++e) { s0 = fmaf(qv[e], to_float(ea[e]), s0); s1 = fmaf(qv[e], to_float(eb[e]), s1); }
            }
        }
        s0 *= scale; s1 *= scale;
        // online softmax (cdna3-prims/examples/fused_softmax.hpp:38-48)
        float rmax, rsum;
        if (STEP == 0) rmax = portable_reduce_bcast(s0, s1, wave::MaxOp{});
        else           rmax = wave::dpp::reduce_max_bcast(s0, s1);
        const float m_new = fmaxf(m, rmax);
        const float p0 = exp_for<T>(s0 - m_new), p1 = exp_for<T>(s1 - m_new);
        if (STEP == 0) rsum = portable_reduce_bcast(p0, p1, wave::SumOp{});
        else           rsum = wave::dpp::reduce_sum_bcast(p0, p1);
        const float resc = exp_for<T>(m - m_new);
        l = resc * l + rsum;
        m = m_new;
        #pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] *= resc;
        // O[row][d] += sum_k P[row][k] * V[k][d]
        prow[warp * kBc + 2 * lane] = p0;
        prow[warp * kBc + 2 * lane + 1] = p1;
        __syncwarp();
        #pragma unroll 4
        for (int k = 0; k < kBc; k += 4) {
            const float4 p4 = *reinterpret_cast<const float4*>(&prow[warp * kBc + k]);      // broadcast read
            const float pk[4] = {p4.x, p4.y, p4.z, p4.w};
            #pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                #pragma unroll
                for (int i = 0; i < DPL; ++i) o[i] = fmaf(pk[kk], to_float(Vc[(k + kk) * D + lane * DPL + i]), o[i]);
            }
        }
        __syncthreads();                                  // tile buffers and prow are reused next iteration
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;            // kernels/fa_naive.hip: l_inv = l > 0 ? 1/l : 0
    #pragma unroll
    for (int i = 0; i < DPL; ++i) Orow[lane * DPL + i] = from_float<T>(o[i] * inv);
    if (STEP == 2) {
        if (!ok) atomicExch(&s_failed, 1);
        __syncthreads();
        if (threadIdx.x == 0 && s_failed) atomicExch(sticky, 1);
    }
}

// ---------------------------------------------------------------------------
// The reference's fp32-I/O kernels, one query row per block (Br = 1):
//   research/flash-attention-mi300x/kernels/fa_naive.hip:118-278   (DPP = false)
//   research/flash-attention-mi300x/kernels/fa_dpp.hip:96-155,167-313 (DPP = true)
// Bc keys per tile are spread over Bc/64 "waves"; here a wave is one 32-lane warp
// holding the 64 scores as an adjacent pair per lane.  Row max and row sum are the
// reference's two-phase reduction (block_reduce_max_sum): inside the wave with the
// pair primitives (shfl_down order for the naive kernel), across the waves through
// 2 * waves floats of shared memory.  Keys past seq_len are padded with the lowest
// float and contribute p = 0 (kernels/fa_naive.hip:158-169,233); any seq_len works.
// O[row] = sum_k p_k V[k] / l with l_inv = l > 0 ? 1/l : 0.
// ---------------------------------------------------------------------------
template <int BC, int D, bool DPP>
__global__ void __launch_bounds__(BC / 2)
fa_rows_f32_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                   float* __restrict__ O, int seq_len, int n_heads, float scale) {
    constexpr int WAVES = BC / 64, THREADS = BC / 2;
    constexpr float kLowest = -3.402823466e+38f;
    __shared__ __align__(16) float q_s[D];
    __shared__ float p_s[BC];
    __shared__ float red[2 * WAVES];
    const int tid = threadIdx.x, wave_i = tid / 32, lane = tid % 32;
    const int row = blockIdx.x, bh = blockIdx.y;               // bh = batch * n_heads + head
    const size_t base = size_t(bh) * seq_len * D;
    for (int d = tid; d < D; d += THREADS) q_s[d] = Q[base + size_t(row) * D + d];
    __syncthreads();

    float m = kLowest, l = 0.f;
    constexpr int DPT = (D + THREADS - 1) / THREADS;           // output dims per thread: d = tid + i * THREADS
    float o[DPT];
    #pragma unroll
    for (int i = 0; i < DPT; ++i) o[i] = 0.f;

    const int tiles = (seq_len + BC - 1) / BC;
    for (int j = 0; j < tiles; ++j) {
        const int kv0 = j * BC;
        const int k0 = kv0 + wave_i * 64 + 2 * lane, k1 = k0 + 1;
        float s0 = kLowest, s1 = kLowest;
        if (k0 < seq_len) {
            const float4* kr = reinterpret_cast<const float4*>(K + base + size_t(k0) * D);
            float a = 0.f;
            #pragma unroll 4
            for (int d4 = 0; d4 < D / 4; ++d4) {
                const float4 kv = kr[d4]; const float4 qv = *reinterpret_cast<const float4*>(&q_s[4 * d4]);
                a = fmaf(qv.x, kv.x, a); a = fmaf(qv.y, kv.y, a); a = fmaf(qv.z, kv.z, a); a = fmaf(qv.w, kv.w, a);
            }
            s0 = a * scale;
        }
        if (k1 < seq_len) {
            const float4* kr = reinterpret_cast<const float4*>(K + base + size_t(k1) * D);
            float a = 0.f;
            #pragma unroll 4
            for (int d4 = 0; d4 < D / 4; ++d4) {
                const float4 kv = kr[d4]; const float4 qv = *reinterpret_cast<const float4*>(&q_s[4 * d4]);
                a = fmaf(qv.x, kv.x, a); a = fmaf(qv.y, kv.y, a); a = fmaf(qv.z, kv.z, a); a = fmaf(qv.w, kv.w, a);
            }
            s1 = a * scale;
        }
        // phase 1: inside the wave; phase 2: across the waves of the block
        float tmax = DPP ? wave::dpp::reduce_max_bcast(s0, s1) : portable_reduce_bcast(s0, s1, wave::MaxOp{});
        if (WAVES > 1) {
            if (lane == 0) red[wave_i] = tmax;
            __syncthreads();
            tmax = red[0];
            #pragma unroll
            for (int w = 1; w < WAVES; ++w) tmax = tmax > red[w] ? tmax : red[w];
        }
        const float m_new = fmaxf(m, tmax);                    // running max (fused_softmax.hpp:38-48)
        const float p0 = k0 < seq_len ? expf(s0 - m_new) : 0.f;
        const float p1 = k1 < seq_len ? expf(s1 - m_new) : 0.f;
        float tsum = DPP ? wave::dpp::reduce_sum_bcast(p0, p1) : portable_reduce_bcast(p0, p1, wave::SumOp{});
        if (WAVES > 1) {
            if (lane == 0) red[WAVES + wave_i] = tsum;
            __syncthreads();
            tsum = red[WAVES];
            #pragma unroll
            for (int w = 1; w < WAVES; ++w) tsum += red[WAVES + w];
        }
        const float alpha = expf(m - m_new);
        m = m_new;
        l = alpha * l + tsum;
        p_s[wave_i * 64 + 2 * lane] = p0;
        p_s[wave_i * 64 + 2 * lane + 1] = p1;
        __syncthreads();
        const int live = min(BC, seq_len - kv0);
        #pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = tid + i * THREADS;
            if (d < D) {
                float acc = o[i] * alpha;
                const float* vcol = V + base + size_t(kv0) * D + d;
                #pragma unroll 4
                for (int k = 0; k < live; ++k) acc = fmaf(p_s[k], vcol[size_t(k) * D], acc);
                o[i] = acc;
            }
        }
        __syncthreads();                                       // p_s and red are rewritten by the next tile
    }
    const float l_inv = l > 0.f ? 1.f / l : 0.f;
    #pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = tid + i * THREADS;
        if (d < D) O[base + size_t(row) * D + d] = o[i] * l_inv;
    }
}

template <int BC, int D>
int launch_rows(bool dpp, const float* Q, const float* K, const float* V, float* O, int batch, int heads, int seq_len,
                float scale, cudaStream_t st) {
    const dim3 grid(unsigned(seq_len), unsigned(batch) * unsigned(heads));
    if (dpp) fa_rows_f32_kernel<BC, D, true><<<grid, BC / 2, 0, st>>>(Q, K, V, O, seq_len, heads, scale);
    else     fa_rows_f32_kernel<BC, D, false><<<grid, BC / 2, 0, st>>>(Q, K, V, O, seq_len, heads, scale);
    return launched();
}
template <int D>
int launch_rows_bc(int bc, bool dpp, const float* Q, const float* K, const float* V, float* O, int batch, int heads,
                   int seq_len, float scale, cudaStream_t st) {
    switch (bc) {
        case 64:  return launch_rows<64, D>(dpp, Q, K, V, O, batch, heads, seq_len, scale, st);
        case 128: return launch_rows<128, D>(dpp, Q, K, V, O, batch, heads, seq_len, scale, st);
        case 256: return launch_rows<256, D>(dpp, Q, K, V, O, batch, heads, seq_len, scale, st);
    }
    return B200P_E_OP;
}

template <typename T, int D, int STEP>
int launch_step(const void* Q, const void* K, const void* V, void* O, int batch, int heads, int seq_q, int seq_k,
                float scale, cudaStream_t st) {
    const size_t smem = 4 * size_t(kBc) * D * sizeof(T) + (kBr * kBc + kBr * D) * sizeof(float) + 64;
    int* sticky = device_status_ptr();
    if (!sticky) return B200P_E_NO_DEVICE;
    LaunchSlot slot{};                                         // the launch's own abort word (only the async step waits)
    if (STEP == 2) { if (int se = take_launch_slot(st, &slot)) return se; }
    auto kern = fa_step_kernel<T, D, STEP>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
    }
    const unsigned grid = unsigned(batch) * heads * (seq_q / kBr);
    kern<<<grid, kBr * 32, smem, st>>>(static_cast<const T*>(Q), static_cast<const T*>(K), static_cast<const T*>(V),
                                       static_cast<T*>(O), seq_q, seq_k, heads, scale, slot.abort, sticky);
    return launched();
}
template <typename T, int D>
int launch_step_s(int step, const void* Q, const void* K, const void* V, void* O, int batch, int heads, int seq_q,
                  int seq_k, float scale, cudaStream_t st) {
    switch (step) {
        case 0: return launch_step<T, D, 0>(Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
        case 1: return launch_step<T, D, 1>(Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
        case 2: return launch_step<T, D, 2>(Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
    }
    return B200P_E_OP;
}
template <typename T>
int launch_step_d(int step, int D, const void* Q, const void* K, const void* V, void* O, int batch, int heads,
                  int seq_q, int seq_k, float scale, cudaStream_t st) {
    return D == 64 ? launch_step_s<T, 64>(step, Q, K, V, O, batch, heads, seq_q, seq_k, scale, st)
                   : launch_step_s<T, 128>(step, Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
}

} // namespace
} // namespace b200p

using namespace b200p;

extern "C" int b200p_fa_rows_f32(int variant, int bc, const float* Q, const float* K, const float* V, float* O,
                                 int batch, int heads, int seq_len, int D, float scale, b200p_stream_t stream) {
    if (variant != 0 && variant != 1) return B200P_E_OP;
    if (bc != 64 && bc != 128 && bc != 256) return B200P_E_OP;
    if (D != 64 && D != 128) return B200P_E_DIM;
    if (batch <= 0 || heads <= 0 || seq_len <= 0) return B200P_E_LENGTH;
    if ((long long)batch * heads > 65535) return B200P_E_RANGE;
    if (!Q || !K || !V || !O) return B200P_E_NULL;
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16)) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    if (scale == 0.f) scale = 1.f / sqrtf(float(D));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return D == 64 ? launch_rows_bc<64>(bc, variant == 1, Q, K, V, O, batch, heads, seq_len, scale, st)
                   : launch_rows_bc<128>(bc, variant == 1, Q, K, V, O, batch, heads, seq_len, scale, st);
}

extern "C" int b200p_fa_step(int step, int dtype, const void* Q, const void* K, const void* V, void* O,
                             int batch, int heads, int seq_q, int seq_k, int D, float scale, b200p_stream_t stream) {
    if (step < 0 || step > 3) return B200P_E_OP;
    if (dtype != B200P_F16 && dtype != B200P_BF16 && dtype != B200P_F32) return B200P_E_DTYPE;
    if (D != 64 && D != 128) return B200P_E_DIM;
    if (batch <= 0 || heads <= 0 || seq_q <= 0 || seq_k <= 0) return B200P_E_LENGTH;
    if (!Q || !K || !V || !O) return B200P_E_NULL;
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16)) return B200P_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (step == 3) {
        // the tensor-core step: 16-bit operands, fixed scale 1/sqrt(D) like fa_mfma2.hip
        if (dtype == B200P_F32) return B200P_E_DTYPE;
        if (scale != 0.f && fabsf(scale * sqrtf(float(D)) - 1.f) > 1e-6f) return B200P_E_OP;
        b200p_prefill_cfg c{D, seq_q, seq_k, heads, heads, batch, 0};
        return prefill_dispatch(Q, K, V, O, &c, dtype, nullptr, st);
    }
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    if (scale == 0.f) scale = 1.f / sqrtf(float(D));
    if (seq_q % kBr != 0 || seq_k % kBc != 0) {
        // Lengths off the Br = 16 / Bc = 64 tiling: the fp32-I/O kernels take any seq_len by padding the
        // keys past the end (kernels/fa_naive.hip:158-169); the 16-bit step kernels keep the reference's tiling.
        if (dtype != B200P_F32 || seq_q != seq_k) return B200P_E_LENGTH;
        return b200p_fa_rows_f32(step == 0 ? 0 : 1, 64, static_cast<const float*>(Q), static_cast<const float*>(K),
                                 static_cast<const float*>(V), static_cast<float*>(O), batch, heads, seq_q, D, scale, stream);
    }
    switch (dtype) {
        case B200P_F16:  return launch_step_d<__half>(step, D, Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
        case B200P_BF16: return launch_step_d<__nv_bfloat16>(step, D, Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
        default:         return launch_step_d<float>(step, D, Q, K, V, O, batch, heads, seq_q, seq_k, scale, st);
    }
}
