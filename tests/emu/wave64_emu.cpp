// Runs the device functions of wave_primitives/wave64.cuh on the host warp
// shim.  One call = one warp: the input holds 32*VEC elements (32*VEC/64
// segments); lane l owns elements [l*VEC, (l+1)*VEC).
// Build: g++ -O1 -std=c++20 -pthread -shared -fPIC -I include
//        -DWAVE64_HOST_EMULATION='"../../tests/emu/warp_shim.hpp"' (path relative
//        to the header) tests/emu/wave64_emu.cpp
#include "wave_primitives/wave64.cuh"
#include <thread>
#include <vector>

namespace {
enum { FN_REDUCE = 0, FN_SCAN_DPP = 1, FN_SCAN_FAST = 2, FN_SCAN_KS64 = 3, FN_SCAN_EXCL_DPP = 4, FN_PAIR_API = 5 };

template <typename F> void run_warp(F f) {
    std::vector<std::thread> th;
    for (unsigned l = 0; l < 32; ++l) th.emplace_back([=]() { warp_shim::t_lane = l; f(l); });
    for (auto& t : th) t.join();
}

template <typename T, typename Op, int VEC>
void run(int fn, const T* in, T* out) {
    run_warp([=](unsigned l) {
        T v[VEC];
        for (int i = 0; i < VEC; ++i) v[i] = in[l * VEC + i];
        const Op op{};
        const T id = Op::template identity<T>();
        if (fn == FN_REDUCE) {
            T r = wave::segment_reduce<VEC>(v, op);
            for (int i = 0; i < VEC; ++i) out[l * VEC + i] = r;
            return;
        }
        if (fn == FN_SCAN_DPP)           wave::segment_scan_dpp_order<VEC>(v, op, id);
        else if (fn == FN_SCAN_FAST)     wave::segment_scan_fast<VEC>(v, op, id);
        else if (fn == FN_SCAN_KS64)     wave::row_scan_kogge_stone<VEC, 64>(v, op, id);
        else if (fn == FN_SCAN_EXCL_DPP) { wave::segment_scan_dpp_order<VEC>(v, op, id); wave::segment_shift_right<VEC>(v, T(0)); }
        for (int i = 0; i < VEC; ++i) out[l * VEC + i] = v[i];
    });
}

// the public pair-per-lane API (VEC = 2): fn2 0 reduce, 1 inclusive, 2 exclusive sum
template <typename T> void run_pair(int fn2, int op, const T* in, T* out) {
    run_warp([=](unsigned l) {
        T a = in[2 * l], b = in[2 * l + 1];
        if (fn2 == 0) {
            T r = op == 0 ? wave::dpp::reduce_sum_bcast(a, b) : op == 1 ? wave::dpp::reduce_max_bcast(a, b) : wave::dpp::reduce_min_bcast(a, b);
            out[2 * l] = r; out[2 * l + 1] = r;
        } else {
            if (fn2 == 2) wave::dpp::scan_exclusive_sum(a, b);
            else if (op == 0) wave::dpp::scan_inclusive_sum(a, b);
            else if (op == 1) wave::dpp::scan_inclusive_max(a, b);
            else wave::dpp::scan_inclusive_min(a, b);
            out[2 * l] = a; out[2 * l + 1] = b;
        }
    });
}

template <typename T, int VEC> int by_op(int fn, int op, const T* in, T* out) {
    if (op == 0) run<T, wave::SumOp, VEC>(fn, in, out);
    else if (op == 1) run<T, wave::MaxOp, VEC>(fn, in, out);
    else run<T, wave::MinOp, VEC>(fn, in, out);
    return 0;
}
template <typename T> int by_vec(int fn, int op, int vec, const void* in, void* out) {
    const T* i = static_cast<const T*>(in); T* o = static_cast<T*>(out);
    switch (vec) {
        case 2: return by_op<T, 2>(fn, op, i, o);
        case 4: return by_op<T, 4>(fn, op, i, o);
        case 8: return by_op<T, 8>(fn, op, i, o);
        case 16: return by_op<T, 16>(fn, op, i, o);
    }
    return -1;
}
} // namespace

// lane_scan_kogge_stone<64>: every lane scans a whole 64-element segment of its own (32 segments per call).
template <typename Op> void run_lane_scan(const float* in, float* out) {
    run_warp([=](unsigned l) {
        float v[64];
        for (int i = 0; i < 64; ++i) v[i] = in[l * 64 + i];
        wave::lane_scan_kogge_stone<64>(v, Op{});
        for (int i = 0; i < 64; ++i) out[l * 64 + i] = v[i];
    });
}
extern "C" int emu_lane_scan(int op, const float* in, float* out) {
    if (op == 0) run_lane_scan<wave::SumOp>(in, out);
    else if (op == 1) run_lane_scan<wave::MaxOp>(in, out);
    else run_lane_scan<wave::MinOp>(in, out);
    return 0;
}

// dtype: 0 f32, 1 f64, 2 i32, 3 i64
extern "C" int emu_run(int fn, int op, int dtype, int vec, const void* in, void* out) {
    if (fn == FN_PAIR_API) return -1;
    switch (dtype) {
        case 0: return by_vec<float>(fn, op, vec, in, out);
        case 1: return by_vec<double>(fn, op, vec, in, out);
        case 2: return by_vec<int>(fn, op, vec, in, out);
        case 3: return by_vec<long long>(fn, op, vec, in, out);
    }
    return -1;
}
extern "C" int emu_pair(int fn2, int op, int dtype, const void* in, void* out) {
    switch (dtype) {
        case 0: run_pair<float>(fn2, op, (const float*)in, (float*)out); return 0;
        case 1: run_pair<double>(fn2, op, (const double*)in, (double*)out); return 0;
        case 2: run_pair<int>(fn2, op, (const int*)in, (int*)out); return 0;
        case 3: run_pair<long long>(fn2, op, (const long long*)in, (long long*)out); return 0;
    }
    return -1;
}
