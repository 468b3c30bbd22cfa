// ---------------------------------------------------------------------------
// gemm_tc.cu -- C[M,N] = A[M,K] . W[N,K]^T on the 5th-generation tensor cores,
// for the runtime's prefill projections.
//
// Stands in for the reference's rocBLAS wrappers RocblasHandle::gemm_*
// (cdna3-prims/include/cdna3/runtime/rocblas_gemm.hpp:112-209) at their call sites in
// Session::run_layers (cdna3-prims/include/cdna3/runtime/session.hpp:147-160,171-173,
// 220,227-230): 16-bit A (activations, row-major) and W (nn.Linear layout [out, in]),
// fp32 accumulation, and the element-wise kernels that follow those GEMMs in the
// reference folded into the epilogue:
//   EPI_STORE16  C 16-bit                              (Q/K/V projection)
//   EPI_STORE32  C fp32                                (logits)
//   EPI_ACC32    C fp32 += A.W^T                       (O and down projections + add_f32_kernel)
//   EPI_SILU16   W = [gate; up] (2N rows); C 16-bit = SiLU(A.gate^T) * (A.up^T)
//                                                      (gate/up GEMMs + silu_mul_f32_kernel)
//
// Both operands are K-major, so a tile is the Q.K^T case of the attention kernel:
// TMA loads [rows][64 x 16-bit] boxes with the 128-byte swizzle into a ring of
// shared-memory stages, ONE thread issues tcgen05.mma (M = 128, N = BN, K = 16) with the
// fp32 accumulator in tensor memory, and a warpgroup reads the finished accumulator
// back (one row per thread), applies the epilogue and hands the result to the TMA
// engine 128 bytes of columns at a time: rows go to a swizzled shared-memory staging
// tile (two buffers), and one thread issues a tensor-map store -- or, for the residual
// form, a tensor-map fp32 add-reduction into C, so the read-modify-write happens in L2
// without a register round trip.  Rows past M and columns past N are clipped by the
// tensor map, so there is no tail code.  CTAs are persistent (one per SM) and
// walk the tiles m-fastest, so the CTAs in flight at any time share a few W tiles in
// L2; two accumulator buffers (2 x 256 columns = all of tensor memory) let the
// epilogue of tile i run under the MMAs of tile i+1.
//   warp 0  TMA producer      warp 1  MMA issuer      warps 2-5  epilogue
// Rows of A past M and rows of W past N are read as zeros by TMA (tensor-map bounds)
// and masked in the epilogue; a K tail inside the last 64-column block is zero-filled too.
// Every mbarrier wait is bounded; a wait that gives up raises the launch's abort word.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "attn_common.cuh"
#include "dme/dme_tma.cuh"
#include "mma_sync.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"
#include "gemm_tc.cuh"

namespace b200p {
namespace {

constexpr int kTM = 128;                  // rows of C per tile
constexpr int kTK = 64;                   // K per stage: one 128-byte swizzle row of 16-bit elements
constexpr int kGemmThreads = 6 * 32;

template <int BN> struct GemmShape {
    static constexpr int A_BYTES = kTM * kTK * 2;            // 16 KB
    static constexpr int B_BYTES = BN * kTK * 2;             // 16 / 32 KB
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN == 256 ? 4 : 6;
    static constexpr int OFF_OUT = STAGES * STAGE_BYTES;     // two staging tiles [128 rows][128 B] for the epilogue
    static constexpr int OUT_BYTES = kTM * 128;
    static constexpr int OFF_BAR = OFF_OUT + 2 * OUT_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 256;
};

struct GemmParams {
    void* C;
    long long ldc;
    int M, N, K;
    int tiles_m, tiles_n;
    int* abort_word; int* sticky;
};

template <typename T> struct GFmt;
template <> struct GFmt<__half>        { static constexpr int id = 0; };
template <> struct GFmt<__nv_bfloat16> { static constexpr int id = 1; };

// BN: accumulator columns per tile (for EPI_SILU16: BN/2 gate columns and the BN/2 matching up columns).
template <typename T, int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW,
               const __grid_constant__ CUtensorMap mapC) {
    using Sh = GemmShape<BN>;
    constexpr int ST = Sh::STAGES;
    constexpr int OUT_N = EPI == GEMM_EPI_SILU16 ? BN / 2 : BN;     // output columns per tile
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Sh::OFF_BAR);
    uint64_t* full = bars;                  // [ST]
    uint64_t* empty = bars + ST;            // [ST]
    uint64_t* acc_full = empty + ST;        // [2]
    uint64_t* acc_empty = acc_full + 2;     // [2]
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_failed;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int ntiles = p.tiles_m * p.tiles_n;
    const int kblocks = (p.K + kTK - 1) / kTK;

    if (threadIdx.x == 0) {
        s_failed = 0;
        for (int s = 0; s < ST; ++s) { dme::mbar_init(&full[s], 1); dme::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { dme::mbar_init(&acc_full[b], 1); dme::mbar_init(&acc_empty[b], 128); }
        dme::mbar_init_fence();
    }
    if (warp == 1) { tc::tmem_alloc(&s_tmem_base, 512); tc::tmem_relinquish(); }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem_base;
    bool ok = true;

    if (warp == 0) {
        // ---------------------------------- TMA producer ----------------------------------
        if (lane == 0) {
            dme::prefetch_tensor_map(&mapA); dme::prefetch_tensor_map(&mapW);
            dme::Ring<ST> r; int loads = 0;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (loads >= ST && !dme::wait(&empty[r.stage], r.phase ^ 1u, p.abort_word)) { ok = false; break; }
                    unsigned char* sa = smem + r.stage * Sh::STAGE_BYTES;
                    dme::mbar_arrive_expect_tx(&full[r.stage], Sh::STAGE_BYTES);
                    dme::copy_tile_2d(sa, &mapA, kb * kTK, tm * kTM, &full[r.stage]);
                    if (EPI == GEMM_EPI_SILU16) {           // gate rows, then the matching up rows N further down
                        dme::copy_tile_2d(sa + Sh::A_BYTES, &mapW, kb * kTK, tn * OUT_N, &full[r.stage]);
                        dme::copy_tile_2d(sa + Sh::A_BYTES + Sh::B_BYTES / 2, &mapW, kb * kTK, p.N + tn * OUT_N, &full[r.stage]);
                    } else if (BN == 256) {                 // a box holds at most 256 rows; two boxes of 128 keep one map for both tile widths
                        dme::copy_tile_2d(sa + Sh::A_BYTES, &mapW, kb * kTK, tn * BN, &full[r.stage]);
                        dme::copy_tile_2d(sa + Sh::A_BYTES + Sh::B_BYTES / 2, &mapW, kb * kTK, tn * BN + 128, &full[r.stage]);
                    } else {
                        dme::copy_tile_2d(sa + Sh::A_BYTES, &mapW, kb * kTK, tn * BN, &full[r.stage]);
                    }
                    r.advance(); ++loads;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------- MMA issuer ------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = tc::instr_desc_f16(kTM, BN, GFmt<T>::id, 0, 0);
            dme::Ring<ST> r;
            int it = 0;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
                const int b = it & 1;
                // the epilogue of the tile that used this accumulator buffer two tiles ago must have read it
                if (it >= 2 && !dme::wait(&acc_empty[b], uint32_t(((it >> 1) - 1) & 1), p.abort_word)) { ok = false; break; }
                tc::fence_after_sync();
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!dme::wait(&full[r.stage], r.phase, p.abort_word)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t sa = dme::smem_addr(smem + r.stage * Sh::STAGE_BYTES);
                    const uint64_t ad = tc::smem_desc_sw128(sa, 16, 1024);
                    const uint64_t bd = tc::smem_desc_sw128(sa + Sh::A_BYTES, 16, 1024);
                    #pragma unroll
                    for (int ks = 0; ks < kTK / 16; ++ks)
                        tc::mma_ss(tmem + b * 256, ad + uint64_t(ks * 2), bd + uint64_t(ks * 2), idesc, (kb | ks) != 0);
                    tc::commit(&empty[r.stage]);
                    r.advance();
                }
                if (!ok) break;
                tc::commit(&acc_full[b]);
            }
        }
    } else {
        // ---------------------------------- epilogue warps --------------------------------
        constexpr bool OUT16 = EPI == GEMM_EPI_STORE16 || EPI == GEMM_EPI_SILU16;
        constexpr int GCOLS = OUT16 ? 64 : 32;                // output columns per 128-byte group
        const int q = warp & 3;                               // TMEM lane quarter this warp may touch
        const int r = q * 32 + lane;                          // row inside the tile
        const uint32_t lane_base = uint32_t(32 * q) << 16;
        const bool issuer = threadIdx.x == 64;                // first epilogue thread: issues and tracks the stores
        if (issuer) dme::prefetch_tensor_map(&mapC);
        int it = 0, grp = 0;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
            const int b = it & 1;
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            // The 128 epilogue threads meet at named barriers below, so they must leave this loop TOGETHER: the outcome
            // of the wait is and-reduced over all of them (a barrier every one of them reaches) before anyone acts on it.
            const bool got = dme::wait(&acc_full[b], uint32_t((it >> 1) & 1), p.abort_word);
            uint32_t all_got;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, 3, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(all_got) : "r"(uint32_t(got)) : "memory");
            if (!all_got) { ok = false; break; }
            tc::fence_after_sync();
            const uint32_t tacc = tmem + lane_base + uint32_t(b * 256);
            #pragma unroll 1
            for (int c = 0; c < OUT_N / GCOLS; ++c, ++grp) {
                uint32_t v[GCOLS], w[32];                      // accumulator columns of this group; 128 bytes of output
                #pragma unroll
                for (int h = 0; h < GCOLS / 32; ++h) tc::ld_32x32b_x32(tacc + c * GCOLS + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[h * 32]));
                if (EPI == GEMM_EPI_SILU16) {
                    uint32_t u[GCOLS];
                    #pragma unroll
                    for (int h = 0; h < GCOLS / 32; ++h) tc::ld_32x32b_x32(tacc + OUT_N + c * GCOLS + h * 32, *reinterpret_cast<uint32_t(*)[32]>(&u[h * 32]));
                    tc::wait_ld();
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {              // SiLU on the SFU: one ex2 and one approximate divide per element
                        const float g0 = __uint_as_float(v[2 * i]), g1 = __uint_as_float(v[2 * i + 1]);
                        w[i] = pack2<T>(__fdividef(g0, 1.f + __expf(-g0)) * __uint_as_float(u[2 * i]),
                                        __fdividef(g1, 1.f + __expf(-g1)) * __uint_as_float(u[2 * i + 1]));
                    }
                } else {
                    tc::wait_ld();
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = OUT16 ? pack2<T>(__uint_as_float(v[(2 * i) % GCOLS]), __uint_as_float(v[(2 * i + 1) % GCOLS])) : v[i % GCOLS];
                }
                // staging buffer grp & 1: the store issued from it two groups ago must have read it out
                unsigned char* stage = smem + Sh::OFF_OUT + (grp & 1) * Sh::OUT_BYTES;
                if (issuer) dme::store_wait_read<1>();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                #pragma unroll
                for (int ch = 0; ch < 8; ++ch)                  // row r, 16-byte chunk ch, 128-byte swizzle
                    *reinterpret_cast<uint4*>(stage + swz128(r, ch)) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
                dme::fence_proxy_async_smem();
                asm volatile("bar.sync 2, 128;" ::: "memory");
                if (issuer) {
                    if (EPI == GEMM_EPI_ACC32) dme::reduce_add_tile_2d(&mapC, tn * OUT_N + c * GCOLS, tm * kTM, stage);
                    else                       dme::store_tile_2d(&mapC, tn * OUT_N + c * GCOLS, tm * kTM, stage);
                    dme::store_commit();
                }
            }
            tc::fence_before_sync();
            dme::mbar_arrive(&acc_empty[b]);
        }
        if (issuer) dme::store_wait_all();
    }
    if (!ok) atomicExch(&s_failed, 1);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    if (warp == 1) tc::tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && s_failed) atomicExch(p.sticky, 1);
}

template <typename T, int BN, int EPI>
int launch_gemm(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw, long long ldc,
                int dtype, cudaStream_t st) {
    using Sh = GemmShape<BN>;
    constexpr int OUT_N = EPI == GEMM_EPI_SILU16 ? BN / 2 : BN;
    const CUtensorMapDataType dt = dtype == B200P_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap ma, mw;
    const uint64_t ad[2] = {uint64_t(K), uint64_t(M)}, as[1] = {uint64_t(lda) * 2};
    const uint64_t wrows = EPI == GEMM_EPI_SILU16 ? uint64_t(2) * N : uint64_t(N);
    const uint64_t wd[2] = {uint64_t(K), wrows}, ws[1] = {uint64_t(ldw) * 2};
    const uint32_t boxa[2] = {kTK, kTM}, boxw[2] = {kTK, 128};
    cudaError_t e = make_tensor_map(&ma, dt, 2, A, ad, as, boxa, Swizzle::B128);
    if (e == cudaSuccess) e = make_tensor_map(&mw, dt, 2, W, wd, ws, boxw, Swizzle::B128);
    // C: boxes of 128 rows x 128 bytes, written (or add-reduced) from the epilogue's staging tiles
    constexpr bool OUT16 = EPI == GEMM_EPI_STORE16 || EPI == GEMM_EPI_SILU16;
    CUtensorMap mc;
    const uint64_t cd[2] = {uint64_t(N), uint64_t(M)}, cs[1] = {uint64_t(ldc) * (OUT16 ? 2 : 4)};
    const uint32_t boxc[2] = {OUT16 ? 64u : 32u, kTM};
    if (e == cudaSuccess) e = make_tensor_map(&mc, OUT16 ? dt : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, C, cd, cs, boxc, Swizzle::B128);
    if (e != cudaSuccess) return int(e);
    auto kern = gemm_tc_kernel<T, BN, EPI>;
    static bool attr_set[64] = {};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Sh::SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        attr_set[dev] = true;
    }
    GemmParams p{};
    p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K;
    p.tiles_m = (M + kTM - 1) / kTM; p.tiles_n = (N + OUT_N - 1) / OUT_N;
    p.sticky = device_status_ptr();
    if (!p.sticky) return B200P_E_NO_DEVICE;
    LaunchSlot slot{};
    if (int se = take_launch_slot(st, &slot)) return se;
    p.abort_word = slot.abort;
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const int sms = sm_count();
    kern<<<unsigned(tiles < sms ? tiles : sms), kGemmThreads, Sh::SMEM_BYTES, st>>>(p, ma, mw, mc);
    return launched();
}

template <typename T, int EPI>
int launch_gemm_bn(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw, long long ldc,
                   int dtype, cudaStream_t st) {
    if (EPI == GEMM_EPI_SILU16) return launch_gemm<T, 256, EPI>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
    // A 128 x 256 tile moves 1.5 bytes of shared memory per flop-unit against 2 for a 128 x 128 tile (both the TMA
    // writes and the MMA reads share the 128 bytes per clock of an SM), so per column it costs 3/4 of the narrow
    // tile's time; but the launch takes whole waves of tiles over the SMs.  Pick the width with the smaller
    // waves x time-per-tile (narrow tile = 2 units, wide = 3).
    const long long tm = (M + kTM - 1) / kTM, sms = sm_count();
    const long long waves128 = (tm * ((N + 127) / 128) + sms - 1) / sms, waves256 = (tm * ((N + 255) / 256) + sms - 1) / sms;
    const int forced = tuning(KNOB_GEMM_TILE_N, 0);
    const bool use_wide = forced == 256 || (forced != 128 && 3 * waves256 <= 2 * waves128);
    return use_wide ? launch_gemm<T, 256, EPI>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st)
                    : launch_gemm<T, 128, EPI>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
}

template <typename T>
int launch_gemm_epi(int epi, const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                    long long ldc, int dtype, cudaStream_t st) {
    switch (epi) {
        case GEMM_EPI_STORE16: return launch_gemm_bn<T, GEMM_EPI_STORE16>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
        case GEMM_EPI_ACC32:   return launch_gemm_bn<T, GEMM_EPI_ACC32>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
        case GEMM_EPI_STORE32: return launch_gemm_bn<T, GEMM_EPI_STORE32>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
        case GEMM_EPI_SILU16:  return launch_gemm_bn<T, GEMM_EPI_SILU16>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
    }
    return B200P_E_OP;
}

} // namespace

int gemm_tc(int dtype, int epi, const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
            long long ldc, cudaStream_t st) {
    if (!A || !W || !C) return B200P_E_NULL;
    if (dtype != B200P_F16 && dtype != B200P_BF16) return B200P_E_DTYPE;
    if (M <= 0 || N <= 0 || K <= 0) return B200P_E_LENGTH;
    // TMA: 16-byte aligned bases and row strides for A, W and C
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K || ldc < N) return B200P_E_RANGE;
    if (!aligned(A, 16) || !aligned(W, 16) || !aligned(C, 16)) return B200P_E_ALIGN;
    const bool c16 = epi == GEMM_EPI_STORE16 || epi == GEMM_EPI_SILU16;
    if ((ldc * (c16 ? 2 : 4)) % 16 != 0) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    return dtype == B200P_F16 ? launch_gemm_epi<__half>(epi, A, W, C, M, N, K, lda, ldw, ldc, dtype, st)
                              : launch_gemm_epi<__nv_bfloat16>(epi, A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
}

} // namespace b200p

extern "C" int b200p_gemm_16(int dtype, int epilogue, const void* A, const void* W, void* C, int M, int N, int K,
                             long long lda, long long ldw, long long ldc, b200p_stream_t stream) {
    return b200p::gemm_tc(dtype, epilogue, A, W, C, M, N, K, lda, ldw, ldc, static_cast<cudaStream_t>(stream));
}
