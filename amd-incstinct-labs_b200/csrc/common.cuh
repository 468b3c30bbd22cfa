// Shared host-side plumbing of libb200p: status codes, the launch counter,
// tuning knobs and device properties.
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <cstdint>
#include "b200p.h"

namespace b200p {

extern std::atomic<unsigned long long> g_launches;

// Number of SMs of the current device (cached per device), 0 if there is none.
int sm_count();
// Value of a tuning knob (see b200p_set_tuning), or `dflt` when unset (< 0).
int tuning(int knob, int dflt);
// Counts b200p_set_tuning calls: anything that bakes knob values in (a captured graph) compares it.
unsigned tuning_epoch();

enum Knob {
    KNOB_SEG_VEC_BYTES = 0,     // 16 or 32: bytes one lane loads per instruction
    KNOB_SEG_CTAS_PER_SM,       // resident CTAs per SM for the streaming kernels
    KNOB_SCAN_FP_EXACT,         // 1: reference association for fp scans, 0: fast
    KNOB_DECODE_SPLITS,         // split-KV count override
    KNOB_DECODE_FUSED_COMBINE,  // 1: the tensor-core decode kernel merges its splits itself, 0: separate combine launch
    KNOB_DECODE_VARIANT,        // 1: tensor-map + mma.sync kernel, 0: bulk-copy + vector kernel
    KNOB_PREFILL_VARIANT,
    KNOB_RUNTIME_GRAPH,         // 1: the runtime replays its decode step as a CUDA graph, 0: launches it every step
    KNOB_RUNTIME_PDL,           // 1: skinny kernels launch as programmatic dependents (weights prefetched before the wait)
    KNOB_RUNTIME_ROPE_FUSED,    // 1: RoPE + KV scatter in the Q/K/V projection's epilogue, 0: separate kernel
    KNOB_RUNTIME_SKINNY,        // decode-step projections: 0 library GEMMs, 1 skinny_gemm_kernel (W in registers),
                                // 2 skinny_stream_kernel (W through shared memory; default)
    KNOB_SCAN16_LANE,           // 1: 16-bit scans hold a whole segment per lane, 0: four lanes per segment
    KNOB_RUNTIME_GEMM,          // prefill projections: 1 the tcgen05 GEMM of this library (default), 0 library GEMMs
    KNOB_GEMM_TILE_N,           // 128 or 256: force the tensor-core GEMM's tile width (0: chosen from the shape)
    KNOB_RUNTIME_MEGA,          // 1: the greedy loop's decode steps run as one persistent cooperative kernel, 0: kernel per phase (default)
    KNOB_RUNTIME_MEGA_AHEAD,    // persistent decode kernel: stages of L2 prefetch in front of the shared-memory ring's loads
    KNOB_COUNT
};

// Device address of the library's sticky status word on the current device: raised at
// kernel exit by any kernel one of whose bounded waits gave up, reported and cleared by
// b200p_device_status.  nullptr without a device.
int* device_status_ptr();

// Per-launch scratch words.  Every launch of a kernel with bounded waits or a device-side
// work counter takes the next slot of a ring of kLaunchSlots slots on the current device
// and clears it on its own stream before the kernel:
//   work  : zero at launch; persistent CTAs draw their later work items from it;
//   abort : zero at launch; set by the first wait of THIS launch that gives up and polled
//           by its other waits, so one lost copy ends the launch within about one wait
//           limit -- and never touches a launch that is in flight on another stream.
// The ring wraps: at most kLaunchSlots such launches may be enqueued and unfinished on a
// device at a time.
constexpr unsigned kLaunchSlots = 1024;
struct LaunchSlot { int* work; int* abort; };
// B200P_OK, B200P_E_NO_DEVICE or the cudaError_t of the clearing memset.
int take_launch_slot(cudaStream_t st, LaunchSlot* out);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Record a launch and translate the launch status.
inline int launched(unsigned n = 1) {
    g_launches.fetch_add(n, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? B200P_OK : int(e);
}

// Programmatic dependent launch (PTX griddepcontrol).  launch_dependents: the next kernel in
// the stream, if it was launched as a programmatic dependent, may start once every CTA of this
// grid has passed this point or exited.  wait: blocks until all predecessor grids have
// completed and their writes are visible; returns at once in a normally launched kernel.
#ifdef __CUDACC__
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

} // namespace b200p
