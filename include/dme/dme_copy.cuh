// ---------------------------------------------------------------------------
// dme/dme_copy.cuh -- the per-thread asynchronous copy API of the reference's
// dme-abstraction headers, under its own names and signatures:
//   research/dme-abstraction/include/dme/dme_copy.hpp:62-94,133-160
//     copy_element / copy_element_stream / wait / wait_lds /
//     copy_tile_1d<T,N> / copy_tile_1d_stream<T,N>
//   research/dme-abstraction/include/dme/tensor_prefetch.hpp:64-79,100-125,151-196
//     prefetch_tile2d_fp16 / prefetch_tile2d_strided_fp16 / AsyncTile2D
//
// The reference issues one 4-byte global_load_lds per lane and waits with
// s_waitcnt.  The sm_100a counterpart with the same shape -- every thread names
// its own source and destination, completion is awaited per thread -- is
// cp.async: the copy bypasses registers, and wait() retires all copies the
// calling thread has issued.  As in the reference, a __syncthreads() after wait()
// publishes the tile to the other threads.  The "stream" forms bypass L1
// (cp.async.cg needs 16-byte transfers; 4- and 8-byte elements use .ca, which
// still leaves no register round trip).
//
// These wrappers keep reference call sites compiling unchanged.  The kernels of
// this library move whole tiles with ONE elected thread and an mbarrier instead
// (dme_tma.cuh): fewer instructions and any number of stages in flight.
// ---------------------------------------------------------------------------
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace dme {

namespace detail {
__device__ __forceinline__ uint32_t shared_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
template <int BYTES> __device__ __forceinline__ void cp_async(void* dst_shared, const void* src_global);
template <> __device__ __forceinline__ void cp_async<4>(void* d, const void* s) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(shared_addr(d)), "l"(s) : "memory");
}
template <> __device__ __forceinline__ void cp_async<8>(void* d, const void* s) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(shared_addr(d)), "l"(s) : "memory");
}
template <> __device__ __forceinline__ void cp_async<16>(void* d, const void* s) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(shared_addr(d)), "l"(s) : "memory");
}
__device__ __forceinline__ unsigned lane() { unsigned l; asm("mov.u32 %0, %%laneid;" : "=r"(l)); return l; }
} // namespace detail

// One element per calling thread, global -> shared, asynchronously (dme_copy.hpp:62-74).
template <typename T>
__device__ __forceinline__ void copy_element(const T* __restrict__ src_global, T* __restrict__ dst_shared) {
    static_assert(sizeof(T) == 4 || sizeof(T) == 8 || sizeof(T) == 16, "copy_element: 4-, 8- or 16-byte elements");
    detail::cp_async<int(sizeof(T))>(dst_shared, src_global);
}
// The streaming form (dme_copy.hpp:77-86).
template <typename T>
__device__ __forceinline__ void copy_element_stream(const T* __restrict__ src_global, T* __restrict__ dst_shared) {
    copy_element<T>(src_global, dst_shared);
}

// Wait for every asynchronous copy this thread has issued (dme_copy.hpp:92-94).  Follow with
// __syncthreads() before other threads read the destination.
__device__ __forceinline__ void wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void wait_lds() { wait(); }

// Cooperative copy of kElems elements by ONE WARP: lane l copies elements l, l + 32, ...
// (dme_copy.hpp:133-146; the reference's wave has 64 lanes, hence kElems % 64 there).
template <typename T, int kElems>
__device__ __forceinline__ void copy_tile_1d(const T* __restrict__ src, T* __restrict__ dst_shared) {
    static_assert(kElems % 32 == 0, "copy_tile_1d: kElems must be a multiple of the warp width");
    const unsigned l = detail::lane();
    #pragma unroll
    for (int i = 0; i < kElems / 32; ++i) copy_element<T>(src + l + i * 32, dst_shared + l + i * 32);
}
template <typename T, int kElems>
__device__ __forceinline__ void copy_tile_1d_stream(const T* __restrict__ src, T* __restrict__ dst_shared) {
    copy_tile_1d<T, kElems>(src, dst_shared);
}

// A packed [kRows][kCols] fp16 tile, spread over `nthreads` threads in 16-byte pieces
// (tensor_prefetch.hpp:64-79 moves it in 4-byte pieces).  base and dst 16-byte aligned.
template <int kRows, int kCols>
__device__ __forceinline__ void prefetch_tile2d_fp16(const __half* __restrict__ base_global, __half* __restrict__ dst_shared,
                                                     int tid, int nthreads) {
    static_assert(kRows * kCols % 128 == 0, "prefetch_tile2d_fp16: kRows*kCols must be a multiple of 128");
    constexpr int kVecs = kRows * kCols / 8;
    const uint4* src = reinterpret_cast<const uint4*>(base_global);
    uint4* dst = reinterpret_cast<uint4*>(dst_shared);
    for (int i = tid; i < kVecs; i += nthreads) detail::cp_async<16>(dst + i, src + i);
}
// The same with `stride_row` elements between consecutive rows in global memory, e.g. a KV
// cache [heads, max_seq, D] (tensor_prefetch.hpp:100-125).  stride_row % 8 == 0.
template <int kRows, int kCols>
__device__ __forceinline__ void prefetch_tile2d_strided_fp16(const __half* __restrict__ base_global, __half* __restrict__ dst_shared,
                                                             int stride_row, int tid, int nthreads) {
    static_assert(kCols % 8 == 0, "prefetch_tile2d_strided_fp16: kCols must be a multiple of 8");
    constexpr int kVecsPerRow = kCols / 8, kVecs = kRows * kVecsPerRow;
    for (int i = tid; i < kVecs; i += nthreads) {
        const int row = i / kVecsPerRow, v = i % kVecsPerRow;
        detail::cp_async<16>(dst_shared + size_t(i) * 8, base_global + size_t(row) * stride_row + size_t(v) * 8);
    }
}

// Ping/pong state of a double-buffered K or V tile stream (tensor_prefetch.hpp:151-196), same
// methods and call order: prologue; then per iteration prefetch_next, compute on cur(), wait_next,
// advance.
template <int kRows, int kCols>
struct AsyncTile2D {
    int cur_ = 0;
    __device__ __forceinline__ int cur()  const { return cur_; }
    __device__ __forceinline__ int next() const { return cur_ ^ 1; }
    __device__ __forceinline__ void advance() { cur_ ^= 1; }

    __device__ __forceinline__ void prologue(const __half* __restrict__ base_global, __half dst_shared[][kRows * kCols],
                                             int tid, int nthreads) {
        prefetch_tile2d_fp16<kRows, kCols>(base_global, dst_shared[0], tid, nthreads);
        wait();
        __syncthreads();
        cur_ = 0;
    }
    __device__ __forceinline__ void prefetch_next(const __half* __restrict__ base_global, __half dst_shared[][kRows * kCols],
                                                  int next_tile_idx, int n_tiles, int tid, int nthreads) {
        if (next_tile_idx < n_tiles)
            prefetch_tile2d_fp16<kRows, kCols>(base_global + size_t(next_tile_idx) * kRows * kCols, dst_shared[next()], tid, nthreads);
    }
    __device__ __forceinline__ void wait_next(int next_tile_idx, int n_tiles) {
        if (next_tile_idx < n_tiles) wait();
        __syncthreads();
    }
};

} // namespace dme
