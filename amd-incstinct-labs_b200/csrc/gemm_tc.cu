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
// back (one row per thread) for the epilogue.  CTAs are persistent (one per SM) and
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
    static constexpr int OFF_BAR = STAGES * STAGE_BYTES;
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

__device__ __forceinline__ void st_v8(void* p, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                 :: "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "l"(p) : "memory");
}
__device__ __forceinline__ void ld_v8(const void* p, uint32_t (&w)[8]) {
    asm volatile("ld.global.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(p) : "memory");
}

// BN: accumulator columns per tile (for EPI_SILU16: BN/2 gate columns and the BN/2 matching up columns).
template <typename T, int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW) {
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
        const int q = warp & 3;                               // TMEM lane quarter this warp may touch
        const int r = q * 32 + lane;                          // row inside the tile
        const uint32_t lane_base = uint32_t(32 * q) << 16;
        int it = 0;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++it) {
            const int b = it & 1;
            const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            if (!dme::wait(&acc_full[b], uint32_t((it >> 1) & 1), p.abort_word)) { ok = false; break; }
            tc::fence_after_sync();
            const int row = tm * kTM + r;
            const int col0 = tn * OUT_N;
            const uint32_t tacc = tmem + lane_base + uint32_t(b * 256);
            #pragma unroll 1
            for (int c = 0; c < OUT_N / 32; ++c) {
                uint32_t v[32];
                tc::ld_32x32b_x32(tacc + c * 32, v);
                uint32_t u[32];
                if (EPI == GEMM_EPI_SILU16) tc::ld_32x32b_x32(tacc + OUT_N + c * 32, u);
                tc::wait_ld();
                const int col = col0 + c * 32;
                if (row < p.M && col < p.N) {
                    const bool whole = col + 32 <= p.N;
                    if (EPI == GEMM_EPI_STORE16 || EPI == GEMM_EPI_SILU16) {
                        T* dst = static_cast<T*>(p.C) + size_t(row) * p.ldc + col;
                        uint32_t w[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float x0 = __uint_as_float(v[2 * i]), x1 = __uint_as_float(v[2 * i + 1]);
                            if (EPI == GEMM_EPI_SILU16) {
                                x0 = (x0 / (1.f + __expf(-x0))) * __uint_as_float(u[2 * i]);
                                x1 = (x1 / (1.f + __expf(-x1))) * __uint_as_float(u[2 * i + 1]);
                            }
                            w[i] = pack2<T>(x0, x1);
                        }
                        if (whole) {
                            st_v8(dst, *reinterpret_cast<uint32_t(*)[8]>(&w[0]));
                            st_v8(dst + 16, *reinterpret_cast<uint32_t(*)[8]>(&w[8]));
                        } else {
                            const T* h = reinterpret_cast<const T*>(w);
                            for (int i = 0; col + i < p.N; ++i) dst[i] = h[i];
                        }
                    } else {
                        float* dst = static_cast<float*>(p.C) + size_t(row) * p.ldc + col;
                        if (whole) {
                            #pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                uint32_t w[8];
                                if (EPI == GEMM_EPI_ACC32) {
                                    ld_v8(dst + g * 8, w);
                                    #pragma unroll
                                    for (int i = 0; i < 8; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) + __uint_as_float(v[g * 8 + i]));
                                } else {
                                    #pragma unroll
                                    for (int i = 0; i < 8; ++i) w[i] = v[g * 8 + i];
                                }
                                st_v8(dst + g * 8, w);
                            }
                        } else {
                            for (int i = 0; col + i < p.N; ++i)
                                dst[i] = EPI == GEMM_EPI_ACC32 ? dst[i] + __uint_as_float(v[i]) : __uint_as_float(v[i]);
                        }
                    }
                }
            }
            tc::fence_before_sync();
            dme::mbar_arrive(&acc_empty[b]);
        }
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
    kern<<<unsigned(tiles < sms ? tiles : sms), kGemmThreads, Sh::SMEM_BYTES, st>>>(p, ma, mw);
    return launched();
}

template <typename T, int EPI>
int launch_gemm_bn(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw, long long ldc,
                   int dtype, cudaStream_t st) {
    if (EPI == GEMM_EPI_SILU16) return launch_gemm<T, 256, EPI>(A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
    // wide tiles read less shared memory per flop; narrow tiles when the wide ones would leave SMs without work
    const long long wide = (long long)((M + kTM - 1) / kTM) * ((N + 255) / 256);
    const int forced = tuning(KNOB_GEMM_TILE_N, 0);
    const bool use_wide = forced == 256 || (forced != 128 && wide >= sm_count());
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
    // TMA: 16-byte aligned bases and row strides; the epilogue's 32-byte stores need rows of C on 32 bytes
    if (K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K || ldc < N) return B200P_E_RANGE;
    if (!aligned(A, 16) || !aligned(W, 16) || !aligned(C, 32)) return B200P_E_ALIGN;
    const bool c16 = epi == GEMM_EPI_STORE16 || epi == GEMM_EPI_SILU16;
    if ((ldc * (c16 ? 2 : 4)) % 32 != 0) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    return dtype == B200P_F16 ? launch_gemm_epi<__half>(epi, A, W, C, M, N, K, lda, ldw, ldc, dtype, st)
                              : launch_gemm_epi<__nv_bfloat16>(epi, A, W, C, M, N, K, lda, ldw, ldc, dtype, st);
}

} // namespace b200p

extern "C" int b200p_gemm_16(int dtype, int epilogue, const void* A, const void* W, void* C, int M, int N, int K,
                             long long lda, long long ldw, long long ldc, b200p_stream_t stream) {
    return b200p::gemm_tc(dtype, epilogue, A, W, C, M, N, K, lda, ldw, ldc, static_cast<cudaStream_t>(stream));
}
