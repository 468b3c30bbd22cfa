// Host stand-in for one 32-lane warp, used to check the cross-lane logic of
// wave_primitives/wave64.cuh without a GPU.  32 host threads run the same
// device function in lockstep; every *_sync intrinsic is "publish my value,
// barrier, read the source lane's value, barrier", which is exactly the
// semantics of the hardware instruction when all 32 lanes take part.
#pragma once
#include <barrier>
#include <cstdint>
#include <cstring>

#define __device__
#define __host__
#define __forceinline__ inline

namespace warp_shim {
inline std::barrier<>& bar() { static std::barrier<> b(32); return b; }
inline unsigned long long* slots() { static unsigned long long s[32]; return s; }
inline thread_local unsigned t_lane = 0;

template <typename T> inline T exchange(T v, int src) {
    static_assert(sizeof(T) <= 8, "slot size");
    unsigned long long raw = 0;
    std::memcpy(&raw, &v, sizeof(T));
    slots()[t_lane] = raw;
    bar().arrive_and_wait();
    T r;
    std::memcpy(&r, &slots()[src & 31], sizeof(T));
    bar().arrive_and_wait();
    return r;
}
template <typename T, typename F> inline T group_reduce(unsigned mask, T v, F f) {
    unsigned long long raw = 0;
    std::memcpy(&raw, &v, sizeof(T));
    slots()[t_lane] = raw;
    bar().arrive_and_wait();
    bool first = true; T acc{};
    for (int l = 0; l < 32; ++l) if (mask >> l & 1u) {
        T x; std::memcpy(&x, &slots()[l], sizeof(T));
        acc = first ? x : f(acc, x); first = false;
    }
    bar().arrive_and_wait();
    return acc;
}
} // namespace warp_shim

template <typename T> inline T __shfl_xor_sync(unsigned, T v, int m)       { return warp_shim::exchange(v, int(warp_shim::t_lane) ^ m); }
template <typename T> inline T __shfl_sync(unsigned, T v, int src)         { return warp_shim::exchange(v, src); }
template <typename T> inline T __shfl_up_sync(unsigned, T v, unsigned d) {
    const int src = int(warp_shim::t_lane) - int(d);
    return warp_shim::exchange(v, src < 0 ? int(warp_shim::t_lane) : src);   // out of range: own value
}
inline int __reduce_add_sync(unsigned m, int v) { return warp_shim::group_reduce(m, v, [](int a, int b) { return int(unsigned(a) + unsigned(b)); }); }
inline int __reduce_max_sync(unsigned m, int v) { return warp_shim::group_reduce(m, v, [](int a, int b) { return a > b ? a : b; }); }
inline int __reduce_min_sync(unsigned m, int v) { return warp_shim::group_reduce(m, v, [](int a, int b) { return a < b ? a : b; }); }

namespace wave {
inline unsigned lane_id() { return warp_shim::t_lane; }
inline unsigned lane_id_here() { return warp_shim::t_lane; }
namespace detail {
inline float redux_max_f32(unsigned m, float v) { return warp_shim::group_reduce(m, v, [](float a, float b) { return a > b ? a : b; }); }
inline float redux_min_f32(unsigned m, float v) { return warp_shim::group_reduce(m, v, [](float a, float b) { return a < b ? a : b; }); }
} // namespace detail
} // namespace wave
