// ---------------------------------------------------------------------------
// wave_bench.cu -- kernels that measure the DEVICE-level wave API in the
// reference's own terms, and two small "real kernels" built on it.
//
// 1. Register-resident reduce loop (research/wave-primitives/benchmarks/
//    bench_reduce_dpp_types.hip:29-45): every wave reduces its 64 values kReps
//    times, feeding the result back into the inputs so that nothing can be
//    hoisted; no memory traffic inside the loop.  A wave is one warp holding a
//    pair per lane.  Backends: 0 = wave::dpp::reduce_* (xor butterfly, redux.sync
//    where the type has it), 1 = the portable shfl_down loop + broadcast the
//    reference benchmarks against (wave_reduce.hpp:40-46).
// 2. LayerNorm and softmax over rows of 64 * E elements, one warp per row, E pairs
//    per lane (research/wave-primitives/benchmarks/bench_layernorm.hip:47-96,
//    bench_softmax.hip): two row reductions each, with the same two backends.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "wave_primitives/wave64.cuh"

namespace b200p {
namespace {

template <typename T, typename Op>
__device__ __forceinline__ T portable_pair_reduce_bcast(T a, T b, Op op) {
    T v = op(a, b);
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_down_sync(0xffffffffu, v, o));
    return __shfl_sync(0xffffffffu, v, 0);
}

template <typename T, int OP, int BACKEND>
__global__ void __launch_bounds__(256)
wave_reduce_loop_kernel(const T* __restrict__ in, T* __restrict__ out, int reps) {
    const size_t wave_i = size_t(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    const unsigned l = threadIdx.x % 32;
    T a = in[wave_i * 64 + 2 * l], b = in[wave_i * 64 + 2 * l + 1];
    T acc = T(0);
    #pragma unroll 1
    for (int r = 0; r < reps; ++r) {
        T s;
        if (BACKEND == 0) {
            if (OP == 0)      s = wave::dpp::reduce_sum(a, b);
            else if (OP == 1) s = wave::dpp::reduce_max(a, b);
            else              s = wave::dpp::reduce_min(a, b);
        } else {
            if (OP == 0)      s = portable_pair_reduce_bcast(a, b, wave::SumOp{});
            else if (OP == 1) s = portable_pair_reduce_bcast(a, b, wave::MaxOp{});
            else              s = portable_pair_reduce_bcast(a, b, wave::MinOp{});
        }
        acc = acc + s;
        // per-lane perturbation: the inputs of the next repetition depend on this one's result
        a = s + T(2 * l) + T(1);
        b = s + T(2 * l + 1) + T(1);
    }
    if (l == 31) out[wave_i] = acc;
}

// 16-bit inputs: the sum is accumulated in fp32 and rounded once (wave::reduce_sum(__half / bf16 pair),
// research/wave-primitives/benchmarks/bench_h3_h4_multitype.hip's fp32-acc form); backend 1 accumulates in the 16-bit
// type itself with the portable shuffle-down loop (the "native" form the reference compares against).
template <typename T, int BACKEND>
__global__ void __launch_bounds__(256)
wave_reduce_loop16_kernel(const T* __restrict__ in, T* __restrict__ out, int reps) {
    const size_t wave_i = size_t(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    const unsigned l = threadIdx.x % 32;
    T a = in[wave_i * 64 + 2 * l], b = in[wave_i * 64 + 2 * l + 1];
    float acc = 0.f;
    #pragma unroll 1
    for (int r = 0; r < reps; ++r) {
        T s;
        if (BACKEND == 0) s = wave::reduce_sum(a, b);
        else {
            T v = a + b;
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = v + __shfl_down_sync(0xffffffffu, v, o);
            s = __shfl_sync(0xffffffffu, v, 0);
        }
        acc += float(s);
        // next repetition: small values that depend on this one's result
        const T dep = float(s) > 100.f ? T(1.f) : T(0.f);
        a = T(float((2 * l) % 5)) + dep;
        b = T(float((2 * l + 1) % 5)) + dep;
    }
    if (l == 31) out[wave_i] = T(acc);
}

template <typename T, int BACKEND>
int launch_loop(int op, const void* in, void* out, int waves, int reps, cudaStream_t st) {
    const int grid = waves / 8;
    const T* i = static_cast<const T*>(in); T* o = static_cast<T*>(out);
    switch (op) {
        case B200P_SUM: wave_reduce_loop_kernel<T, 0, BACKEND><<<grid, 256, 0, st>>>(i, o, reps); break;
        case B200P_MAX: wave_reduce_loop_kernel<T, 1, BACKEND><<<grid, 256, 0, st>>>(i, o, reps); break;
        default:        wave_reduce_loop_kernel<T, 2, BACKEND><<<grid, 256, 0, st>>>(i, o, reps); break;
    }
    return launched();
}

// The scan loop (research/wave-primitives/benchmarks/bench_scan_dpp.hip): every wave takes the inclusive prefix
// sum of its 64 values `reps` times, the last element fed back into the inputs of the next repetition.  Backend 0:
// wave::dpp::scan_inclusive_sum on the pair; backend 1: the portable form (pair prefix, shuffle-up ladder over the
// lanes' totals, add the exclusive lane prefix).
template <typename T>
__device__ __forceinline__ void portable_pair_scan(T& a, T& b) {
    b = a + b;
    T t = b;
    const unsigned l = threadIdx.x % 32;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const T u = __shfl_up_sync(0xffffffffu, t, o); if (l >= unsigned(o)) t = t + u; }
    const T excl = t - b;
    a = a + excl; b = b + excl;
}
template <typename T, int BACKEND>
__global__ void __launch_bounds__(256)
wave_scan_loop_kernel(const T* __restrict__ in, T* __restrict__ out, int reps) {
    const size_t wave_i = size_t(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    const unsigned l = threadIdx.x % 32;
    T a = in[wave_i * 64 + 2 * l], b = in[wave_i * 64 + 2 * l + 1];
    T acc = T(0);
    #pragma unroll 1
    for (int r = 0; r < reps; ++r) {
        if (BACKEND == 0) wave::dpp::scan_inclusive_sum(a, b);
        else              portable_pair_scan(a, b);
        acc = acc + b;                                           // lane 31 holds the wave's total in b
        const T last = __shfl_sync(0xffffffffu, b, 31);
        // next repetition: small values that depend on this one's result (the total's parity for integers, its sign for floats)
        const T dep = last > T(0) ? T(1) : T(0);
        a = T((2 * l) % 5) + dep;
        b = T((2 * l + 1) % 5) + dep;
    }
    out[wave_i * 64 + 2 * l] = a + acc;                          // every lane's state is observable
    out[wave_i * 64 + 2 * l + 1] = b;
}

template <int BACKEND> __device__ __forceinline__ float row_sum(float a, float b) {
    return BACKEND == 0 ? wave::dpp::reduce_sum_bcast(a, b) : portable_pair_reduce_bcast(a, b, wave::SumOp{});
}
template <int BACKEND> __device__ __forceinline__ float row_max(float a, float b) {
    return BACKEND == 0 ? wave::dpp::reduce_max_bcast(a, b) : portable_pair_reduce_bcast(a, b, wave::MaxOp{});
}

// which 0: y = (x - mean) / sqrt(var + eps) * gamma + beta;  which 1: y = softmax(x).  Row = 64 * E floats; lane l holds
// the float2 at columns 64 e + 2 l (e = 0 .. E-1), so a warp reads whole 256-byte runs.  A warp takes R consecutive
// rows at a time, all their loads issued before the first reduction: with 64-column rows one row per warp leaves
// 16 KB in flight per SM, a quarter of what the memory system needs to stay busy.
template <int E, int R, int BACKEND>
__global__ void __launch_bounds__(256)
row_op_kernel(int which, const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              float* __restrict__ out, int rows, float eps) {
    const int row0 = (blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32) * R;
    if (row0 >= rows) return;
    const unsigned l = threadIdx.x % 32;
    constexpr int COLS = 64 * E;
    float2 v[R][E];
    #pragma unroll
    for (int r = 0; r < R; ++r) {
        const float2* xr = reinterpret_cast<const float2*>(x + size_t(min(row0 + r, rows - 1)) * COLS);
        #pragma unroll
        for (int e = 0; e < E; ++e) v[r][e] = xr[e * 32 + l];
    }
    if (which == 0) {
        float2 g[E], bt[E];
        #pragma unroll
        for (int e = 0; e < E; ++e) { g[e] = reinterpret_cast<const float2*>(gamma)[e * 32 + l]; bt[e] = reinterpret_cast<const float2*>(beta)[e * 32 + l]; }
        float mean[R], inv[R];
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            float sa = 0.f, sb = 0.f;
            #pragma unroll
            for (int e = 0; e < E; ++e) { sa += v[r][e].x; sb += v[r][e].y; }
            mean[r] = row_sum<BACKEND>(sa, sb) * (1.f / COLS);
        }
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            float qa = 0.f, qb = 0.f;
            #pragma unroll
            for (int e = 0; e < E; ++e) { const float dx = v[r][e].x - mean[r], dy = v[r][e].y - mean[r]; qa += dx * dx; qb += dy * dy; }
            inv[r] = rsqrtf(row_sum<BACKEND>(qa, qb) * (1.f / COLS) + eps);
        }
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row0 + r < rows) {
                float2* orow = reinterpret_cast<float2*>(out + size_t(row0 + r) * COLS);
                #pragma unroll
                for (int e = 0; e < E; ++e)
                    orow[e * 32 + l] = make_float2((v[r][e].x - mean[r]) * inv[r] * g[e].x + bt[e].x, (v[r][e].y - mean[r]) * inv[r] * g[e].y + bt[e].y);
            }
        }
    } else {
        float m[R], inv[R];
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            float ma = v[r][0].x, mb = v[r][0].y;
            #pragma unroll
            for (int e = 1; e < E; ++e) { ma = fmaxf(ma, v[r][e].x); mb = fmaxf(mb, v[r][e].y); }
            m[r] = row_max<BACKEND>(ma, mb);
        }
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            float sa = 0.f, sb = 0.f;
            #pragma unroll
            for (int e = 0; e < E; ++e) { v[r][e].x = __expf(v[r][e].x - m[r]); v[r][e].y = __expf(v[r][e].y - m[r]); sa += v[r][e].x; sb += v[r][e].y; }
            inv[r] = 1.f / row_sum<BACKEND>(sa, sb);
        }
        #pragma unroll
        for (int r = 0; r < R; ++r) {
            if (row0 + r < rows) {
                float2* orow = reinterpret_cast<float2*>(out + size_t(row0 + r) * COLS);
                #pragma unroll
                for (int e = 0; e < E; ++e) orow[e * 32 + l] = make_float2(v[r][e].x * inv[r], v[r][e].y * inv[r]);
            }
        }
    }
}

template <int E, int R>
int launch_row(int which, int backend, const float* x, const float* g, const float* b, float* out, int rows, float eps, cudaStream_t st) {
    const int grid = (rows + 8 * R - 1) / (8 * R);
    if (backend == 0) row_op_kernel<E, R, 0><<<grid, 256, 0, st>>>(which, x, g, b, out, rows, eps);
    else              row_op_kernel<E, R, 1><<<grid, 256, 0, st>>>(which, x, g, b, out, rows, eps);
    return launched();
}

} // namespace
} // namespace b200p

using namespace b200p;

extern "C" int b200p_wave_reduce_loop(int op, int dtype, int backend, const void* in, void* out, int n_waves, int reps,
                                      b200p_stream_t stream) {
    if (op < B200P_SUM || op > B200P_MIN || (backend != 0 && backend != 1)) return B200P_E_OP;
    const bool narrow = dtype == B200P_F16 || dtype == B200P_BF16;
    if (!narrow && (dtype < B200P_F32 || dtype > B200P_I64)) return B200P_E_DTYPE;
    if (narrow && op != B200P_SUM) return B200P_E_OP;
    if (n_waves <= 0 || n_waves % 8 != 0 || reps <= 0) return B200P_E_LENGTH;
    if (!in || !out) return B200P_E_NULL;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (narrow) {
        const int grid = n_waves / 8;
        if (dtype == B200P_F16) {
            if (backend == 0) wave_reduce_loop16_kernel<__half, 0><<<grid, 256, 0, st>>>(static_cast<const __half*>(in), static_cast<__half*>(out), reps);
            else              wave_reduce_loop16_kernel<__half, 1><<<grid, 256, 0, st>>>(static_cast<const __half*>(in), static_cast<__half*>(out), reps);
        } else {
            if (backend == 0) wave_reduce_loop16_kernel<__nv_bfloat16, 0><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), reps);
            else              wave_reduce_loop16_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), reps);
        }
        return launched();
    }
    switch (dtype) {
        case B200P_F32: return backend == 0 ? launch_loop<float, 0>(op, in, out, n_waves, reps, st) : launch_loop<float, 1>(op, in, out, n_waves, reps, st);
        case B200P_F64: return backend == 0 ? launch_loop<double, 0>(op, in, out, n_waves, reps, st) : launch_loop<double, 1>(op, in, out, n_waves, reps, st);
        case B200P_I32: return backend == 0 ? launch_loop<int, 0>(op, in, out, n_waves, reps, st) : launch_loop<int, 1>(op, in, out, n_waves, reps, st);
        default:        return backend == 0 ? launch_loop<long long, 0>(op, in, out, n_waves, reps, st) : launch_loop<long long, 1>(op, in, out, n_waves, reps, st);
    }
}

extern "C" int b200p_wave_scan_loop(int dtype, int backend, const void* in, void* out, int n_waves, int reps, b200p_stream_t stream) {
    if (backend != 0 && backend != 1) return B200P_E_OP;
    if (dtype < B200P_F32 || dtype > B200P_I64) return B200P_E_DTYPE;
    if (n_waves <= 0 || n_waves % 8 != 0 || reps <= 0) return B200P_E_LENGTH;
    if (!in || !out) return B200P_E_NULL;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = n_waves / 8;
    #define B200P_SCAN_LOOP(T) \
        if (backend == 0) wave_scan_loop_kernel<T, 0><<<grid, 256, 0, st>>>(static_cast<const T*>(in), static_cast<T*>(out), reps); \
        else              wave_scan_loop_kernel<T, 1><<<grid, 256, 0, st>>>(static_cast<const T*>(in), static_cast<T*>(out), reps);
    switch (dtype) {
        case B200P_F32: B200P_SCAN_LOOP(float) break;
        case B200P_F64: B200P_SCAN_LOOP(double) break;
        case B200P_I32: B200P_SCAN_LOOP(int) break;
        default:        B200P_SCAN_LOOP(long long) break;
    }
    #undef B200P_SCAN_LOOP
    return launched();
}

extern "C" int b200p_row_op(int which, int backend, int cols, const float* x, const float* gamma, const float* beta, float* out,
                            int rows, float eps, b200p_stream_t stream) {
    if ((which != 0 && which != 1) || (backend != 0 && backend != 1)) return B200P_E_OP;
    if (cols != 64 && cols != 512) return B200P_E_LENGTH;
    if (rows <= 0) return B200P_E_LENGTH;
    if (!x || !out || (which == 0 && (!gamma || !beta))) return B200P_E_NULL;
    if (!aligned(x, 8) || !aligned(out, 8) || (which == 0 && (!aligned(gamma, 8) || !aligned(beta, 8)))) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return cols == 64 ? launch_row<1, 8>(which, backend, x, gamma, beta, out, rows, eps, st)
                      : launch_row<8, 1>(which, backend, x, gamma, beta, out, rows, eps, st);
}
