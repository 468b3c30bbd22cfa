// Host-side construction of TMA tensor maps (CUtensorMap) without linking
// libcuda: cuTensorMapEncodeTiled is fetched through the runtime's driver
// entry-point query.  Maps are built per call from the caller's pointers and
// passed to kernels as __grid_constant__ parameters; nothing is cached.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace b200p {

enum class Swizzle { None, B32, B64, B128 };

// Up to 5 dimensions of a 16-bit (or other) element tensor.
// dims[0] is the innermost (contiguous) extent in elements; strides_bytes[i]
// is the byte stride of dimension i+1 (dimension 0 is dense); box[i] the tile
// extent.  Requirements checked by the driver: base 16-byte aligned, strides
// multiples of 16 bytes, box[0]*elem_bytes a multiple of 16 and, with a
// swizzle, no larger than the swizzle span.
// Returns cudaSuccess or an error; on success *out is ready for use.
cudaError_t make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                            const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                            Swizzle swizzle, bool l2_promote_256 = true);

} // namespace b200p
