// ---------------------------------------------------------------------------
// dme/dme_tma.cuh -- asynchronous global -> shared tile copies for sm_100a.
//
// Plays the role of the reference's dme-abstraction headers
//   research/dme-abstraction/include/dme/dme_copy.hpp:77-94,133-146
//     (copy_element_stream / copy_tile_1d_stream / wait)
//   research/dme-abstraction/include/dme/tensor_prefetch.hpp:64-79,151-196
//     (prefetch_tile2d_fp16 / AsyncTile2D ping-pong)
// The reference issues one 4-byte global_load_lds per lane and waits with
// s_waitcnt; here ONE elected thread hands a whole contiguous tile to the TMA
// engine (cp.async.bulk) and completion is signalled through an mbarrier that
// the consumers poll, so any number of stages can be in flight.
//
// Every wait is BOUNDED: wait() returns false after kWaitLimitNs instead of
// spinning for ever, so a lost copy turns into an error status, not a hang.
//
// Alignment: source, destination and byte count of a bulk copy must be
// multiples of 16 bytes.  No multicast form is used anywhere.
// ---------------------------------------------------------------------------
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace dme {

constexpr uint64_t kWaitLimitNs = 2000000000ull;   // a wait gives up after ~2 s of wall time

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier --------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
// Make freshly initialised barriers visible to the async proxy (call once, by
// the initialising thread, before the CTA-wide barrier that publishes them).
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_addr(bar)) : "memory");
}
// Arrive and announce `bytes` of asynchronous copies that will complete on this barrier.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait for the phase with the given parity.  false = gave up (after
// kWaitLimitNs; the clock is read once per 256 polls).
// `abort_flag` (optional, global memory): a word that is non-zero once ANY wait of the launch has
// given up; every other wait then gives up at its next check instead of running out its own limit, so
// a launch whose pipeline is broken ends within about one limit, not one limit per CTA.
__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, int* abort_flag = nullptr) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (abort_flag && *reinterpret_cast<volatile int*>(abort_flag) != 0) return false;
        if (global_timer_ns() - t0 > kWaitLimitNs) {
            if (abort_flag) atomicExch(abort_flag, 1);
            return false;
        }
    }
}

// ---- L2 policy for data that is read exactly once -------------------------------------
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// ---- copies (issued by ONE thread) -----------------------------------------------------
// Contiguous `bytes` from global to shared; completion adds `bytes` to `bar`'s
// transaction count.  The streaming form marks the lines evict-first in L2
// (the reference's sc0 "streaming" hint, dme_copy.hpp:77-86).
__device__ __forceinline__ void copy_tile_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void copy_tile_1d_stream(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar,
                                                    uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 :: "r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy) : "memory");
}

// Hint: bring `bytes` (a multiple of 16, from a 16-byte aligned address) of global memory into L2; nothing to wait for.
__device__ __forceinline__ void prefetch_l2(const void* gmem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(gmem_src), "r"(bytes) : "memory");
}

// Tiled tensor-map copies: box at element coordinates (x, y[, z, w]); x * element size
// must be a multiple of 16 bytes.
__device__ __forceinline__ void copy_tile_2d(void* smem_dst, const void* tensor_map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_addr(smem_dst)), "l"(tensor_map), "r"(smem_addr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void copy_tile_4d(void* smem_dst, const void* tensor_map, int x, int y, int z, int w, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 :: "r"(smem_addr(smem_dst)), "l"(tensor_map), "r"(smem_addr(bar)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// Streaming form: lines are marked evict-first in L2 (data read exactly once).
__device__ __forceinline__ void copy_tile_4d_stream(void* smem_dst, const void* tensor_map, int x, int y, int z, int w,
                                                    uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
                 :: "r"(smem_addr(smem_dst)), "l"(tensor_map), "r"(smem_addr(bar)), "r"(x), "r"(y), "r"(z), "r"(w), "l"(policy) : "memory");
}
// ---- shared -> global tile stores (issued by ONE thread, completion tracked in bulk groups) -----------
// The box at element coordinates (x, y) of the tensor map is written from a dense (swizzled as the map says)
// shared-memory tile; rows and columns outside the tensor are clipped by the hardware.  x * element size must
// be a multiple of 16 bytes and no coordinate may be negative.  Make the generic-proxy writes of the tile
// visible first (fence_proxy_async_smem + a barrier over the writing threads).
__device__ __forceinline__ void store_tile_2d(const void* tensor_map, int x, int y, const void* smem_src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(tensor_map), "r"(smem_addr(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void store_tile_4d(const void* tensor_map, int x, int y, int z, int w, const void* smem_src) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :: "l"(tensor_map), "r"(smem_addr(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// The same with an fp32 add into global memory instead of a plain write (every element of the box is
// read-modified-written once, in L2).
__device__ __forceinline__ void reduce_add_tile_2d(const void* tensor_map, int x, int y, const void* smem_src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(tensor_map), "r"(smem_addr(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's committed store groups still READ their shared-memory source
// (the source of the older ones may be overwritten) ...
template <int N> __device__ __forceinline__ void store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
// ... and until all of them have completed.
__device__ __forceinline__ void store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void prefetch_tensor_map(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" :: "l"(tensor_map) : "memory");
}

// Order generic-proxy shared-memory writes before later async-proxy accesses
// (needed before a TMA store or an MMA that reads what threads just wrote).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- ring of stages ---------------------------------------------------------------------
// Producer / consumer bookkeeping for an N-stage ring: stage index and the
// parity of the phase to wait for (the reference's AsyncTile2D ping/pong,
// tensor_prefetch.hpp:151-196, generalised to N stages).
template <int STAGES>
struct Ring {
    int stage = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void advance() {
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
    }
};

} // namespace dme
