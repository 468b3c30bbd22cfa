// core.cu -- process-wide state of libb200p: launch counter, tuning knobs,
// device properties, status strings.
#include "common.cuh"
#include <climits>
#include <cstring>
#include <mutex>

namespace b200p {

std::atomic<unsigned long long> g_launches{0};

namespace {
std::atomic<int> g_knobs[KNOB_COUNT];
std::atomic<unsigned> g_tuning_epoch{0};
struct KnobInit { KnobInit() { for (auto& k : g_knobs) k.store(-1); } } g_knob_init;
const char* const kKnobNames[KNOB_COUNT] = {
    "seg_vec_bytes", "seg_ctas_per_sm", "scan_fp_exact", "decode_splits", "decode_fused_combine", "decode_variant", "prefill_variant",
    "runtime_graph", "runtime_pdl", "runtime_rope_fused", "runtime_skinny", "scan16_lane", "runtime_gemm", "gemm_tile_n",
    "runtime_mega", "runtime_mega_ahead",
};
constexpr int kMaxDevices = 64;
std::atomic<int> g_sms[kMaxDevices];
} // namespace

int sm_count() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return 0; }
    int v = g_sms[dev].load(std::memory_order_relaxed);
    if (v > 0) return v;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); return 0; }
    g_sms[dev].store(sms, std::memory_order_relaxed);
    return sms;
}

// Sticky status word and the per-launch slot ring (see common.cuh).  Kernels receive
// addresses inside these arrays as parameters; only this file names the symbols.
__device__ int g_device_status = 0;
__device__ int g_launch_slots[kLaunchSlots][2];

namespace {
struct DevicePtrs { int* status; int* slots; };
DevicePtrs* device_ptrs() {
    static DevicePtrs ptrs[kMaxDevices] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev].status) {
        void *a = nullptr, *b = nullptr;
        if (cudaGetSymbolAddress(&a, g_device_status) != cudaSuccess || cudaGetSymbolAddress(&b, g_launch_slots) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        ptrs[dev].status = static_cast<int*>(a); ptrs[dev].slots = static_cast<int*>(b);
    }
    return &ptrs[dev];
}
std::atomic<unsigned> g_next_slot{0};
} // namespace

int* device_status_ptr() {
    DevicePtrs* d = device_ptrs();
    return d ? d->status : nullptr;
}

int take_launch_slot(cudaStream_t st, LaunchSlot* out) {
    DevicePtrs* d = device_ptrs();
    if (!d) return B200P_E_NO_DEVICE;
    int* base = d->slots + 2 * (g_next_slot.fetch_add(1, std::memory_order_relaxed) % kLaunchSlots);
    if (cudaError_t e = cudaMemsetAsync(base, 0, 2 * sizeof(int), st)) return int(e);
    out->work = base; out->abort = base + 1;
    return B200P_OK;
}

unsigned tuning_epoch() { return g_tuning_epoch.load(std::memory_order_relaxed); }

int tuning(int knob, int dflt) {
    const int v = g_knobs[knob].load(std::memory_order_relaxed);
    return v < 0 ? dflt : v;
}

} // namespace b200p

using namespace b200p;

extern "C" const char* b200p_version(void) { return "b200p 0.1 (sm_100a)"; }

extern "C" const char* b200p_strerror(int s) {
    switch (s) {
        case B200P_OK:          return "success";
        case B200P_E_NULL:      return "null pointer";
        case B200P_E_DTYPE:     return "unsupported dtype";
        case B200P_E_OP:        return "unknown op, step or variant";
        case B200P_E_LENGTH:    return "length not a multiple of the segment or tile size";
        case B200P_E_ALIGN:     return "pointer not sufficiently aligned";
        case B200P_E_DIM:       return "unsupported head dimension or head counts";
        case B200P_E_WORKSPACE: return "workspace missing or too small";
        case B200P_E_NO_DEVICE: return "no usable CUDA device";
        case B200P_E_TIMEOUT:   return "a bounded device-side wait gave up";
        case B200P_E_RANGE:     return "size beyond a documented maximum";
        case B200P_E_IO:        return "model file missing, short or malformed";
    }
    if (s > 0) return cudaGetErrorString(static_cast<cudaError_t>(s));
    return "unknown status";
}

extern "C" unsigned long long b200p_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int b200p_device_status(int clear) {
    int h = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&h, g_device_status, sizeof(int));
    if (e == cudaSuccess && clear && h != 0) { const int z = 0; e = cudaMemcpyToSymbol(g_device_status, &z, sizeof(z)); }
    if (e != cudaSuccess) return int(e);
    return h == 0 ? B200P_OK : B200P_E_TIMEOUT;
}

extern "C" int b200p_set_tuning(const char* key, int value) {
    if (!key) return INT_MIN;
    for (int i = 0; i < KNOB_COUNT; ++i) {
        if (std::strcmp(key, kKnobNames[i]) == 0) { g_tuning_epoch.fetch_add(1); return g_knobs[i].exchange(value); }
    }
    return INT_MIN;
}
