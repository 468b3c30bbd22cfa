// 16- and 32-byte streaming loads/stores (sm_100a has 256-bit global accesses).
// Loads bypass L1 allocation; 32-byte loads also mark the line evict-first in
// L2, since every byte of these kernels' inputs is read exactly once.
#pragma once
#include <cstdint>

namespace b200p {

template <int BYTES> struct VecIO;

template <> struct VecIO<16> {
    static constexpr int WORDS = 4;
    static __device__ __forceinline__ void load(const void* p, uint32_t (&w)[4]) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "l"(p));
    }
    static __device__ __forceinline__ void store(void* p, const uint32_t (&w)[4]) {
        asm volatile("st.global.L1::no_allocate.v4.u32 [%4], {%0,%1,%2,%3};"
                     :: "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "l"(p) : "memory");
    }
};

template <> struct VecIO<32> {
    static constexpr int WORDS = 8;
    static __device__ __forceinline__ void load(const void* p, uint32_t (&w)[8]) {
        asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]),
                       "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "l"(p));
    }
    static __device__ __forceinline__ void store(void* p, const uint32_t (&w)[8]) {
        asm volatile("st.global.L1::no_allocate.v8.b32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};"
                     :: "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                        "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]), "l"(p) : "memory");
    }
};

} // namespace b200p
