// ---------------------------------------------------------------------------
// cdna3/cdna3.hpp -- one include for the device-level primitives, as the
// reference's umbrella header gives its users
// (cdna3-prims/include/cdna3/cdna3.hpp:31-45):
//
//   #include <cdna3/cdna3.hpp>
//   wave::dpp::reduce_sum(a, b)              cross-lane reduction, no shared memory
//   dme::copy_tile_1d_stream<T, N>(src, dst) asynchronous global -> shared copies
//   dme::copy_tile_4d(...), dme::Ring<N>     TMA tile copies with mbarrier stages
//
// The attention launchers (cdna3::attn::prefill / decode / decode_dme) are a
// separate include, <cdna3/attention.hpp>, as in the reference.  The reference's
// typed MFMA accessors (cdna3::mfma) describe the 16x16x16 lane mapping of its
// matrix cores and have no counterpart here: the tensor-core tiles of this
// library are issued by one thread per CTA from shared and tensor memory.
// ---------------------------------------------------------------------------
#pragma once

#include "../wave_primitives/wave64.cuh"
#include "../dme/dme_copy.cuh"
#include "../dme/dme_tma.cuh"

namespace cdna3 {

// Tracks the reference facade's API level (cdna3.hpp:39-43).
static constexpr int VERSION_MAJOR = 0;
static constexpr int VERSION_MINOR = 2;

} // namespace cdna3
