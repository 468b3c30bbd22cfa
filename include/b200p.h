/* ---------------------------------------------------------------------------
 * b200p.h -- C ABI of libb200p.so: the B200 (sm_100a) implementation of the
 * wave reduce/scan primitives and FA2 attention kernels.
 *
 * The reference project has no FFI layer: its operator API is header-only HIP
 * C++ compiled into the caller.  Every entry point below therefore names the
 * reference C++ interface it stands in for; the C++ wrappers with the
 * reference's own names and struct layouts live in include/cdna3/attention.hpp
 * and include/wave_primitives/wave64.cuh and forward to this ABI.
 *
 * Conventions (same as the reference launchers, cdna3-prims/include/cdna3/
 * attention.hpp:86-109): the caller owns every device pointer; nothing here
 * allocates, frees or synchronises; work is enqueued on `stream` (the default
 * stream if NULL); arguments are checked BEFORE any launch.  Return value:
 * 0 = success, > 0 = a cudaError_t from the launch, < 0 = B200P_E_*.
 * There is no CPU fallback: without a CUDA device every compute entry point
 * returns an error.
 * ------------------------------------------------------------------------- */
#ifndef B200P_H_
#define B200P_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* b200p_stream_t;            /* a cudaStream_t */

/* ---- status codes ------------------------------------------------------- */
enum {
    B200P_OK              =  0,
    B200P_E_NULL          = -1,   /* a required pointer is NULL                 */
    B200P_E_DTYPE         = -2,   /* dtype not supported by this entry point    */
    B200P_E_OP            = -3,   /* unknown op / step / variant                */
    B200P_E_LENGTH        = -4,   /* n_elems not a multiple of 64, seq not a multiple of the tile */
    B200P_E_ALIGN         = -5,   /* pointer not 16-byte aligned                */
    B200P_E_DIM           = -6,   /* unsupported head dim / heads not divisible */
    B200P_E_WORKSPACE     = -7,   /* workspace missing or too small             */
    B200P_E_NO_DEVICE     = -8,   /* no usable CUDA device                      */
    B200P_E_TIMEOUT       = -9,   /* a bounded device-side wait gave up         */
    B200P_E_RANGE         = -10   /* size beyond a documented maximum           */
};

/* ---- element types and ops ---------------------------------------------- */
enum { B200P_F32 = 0, B200P_F64 = 1, B200P_I32 = 2, B200P_I64 = 3, B200P_F16 = 4, B200P_BF16 = 5 };
enum { B200P_SUM = 0, B200P_MAX = 1, B200P_MIN = 2 };

const char* b200p_version(void);
const char* b200p_strerror(int status);
/* Number of kernels this library has launched in this process (all streams). */
unsigned long long b200p_launch_count(void);
/* Internal tuning knobs (vector width, CTAs per SM, split counts, ...).
 * Returns the previous value, or INT32_MIN for an unknown key. */
int b200p_set_tuning(const char* key, int value);

/* =========================================================================
 * Segmented wave reduce / scan over an array.
 * Every run of 64 consecutive elements is one "wave64" and is reduced or
 * scanned on its own, exactly as a wave of the reference would with one
 * element per lane.
 * ========================================================================= */

/* Stands in for wave::dpp::reduce_sum / reduce_max / reduce_min (+ *_bcast),
 * research/wave-primitives/include/wave_primitives/wave_reduce_dpp.hpp:106-113,
 * and for the fp32-accumulating 16-bit overloads wave::reduce_* in
 * research/wave-primitives/include/wave_primitives/wave_reduce.hpp:48-119.
 * in : n_elems values (n_elems % 64 == 0).  out : n_elems/64 values, of the
 * input type for f32/f64/i32/i64 and fp32 for f16/bf16. */
int b200p_segreduce(int op, int dtype, const void* in, void* out,
                    size_t n_elems, b200p_stream_t stream);
/* f16/bf16 only: the result rounded to the input type, which is what the
 * reference overloads return (wave_reduce.hpp:53, :62). */
int b200p_segreduce_narrow(int op, int dtype, const void* in, void* out,
                           size_t n_elems, b200p_stream_t stream);

/* Stands in for wave::dpp::scan_inclusive_sum / _max / _min
 * (wave_scan_dpp.hpp:70-72) and wave::scan_inclusive_sum(__half|bf16)
 * (wave_scan.hpp:52-74).  out has n_elems values of the input type. */
int b200p_segscan_inclusive(int op, int dtype, const void* in, void* out,
                            size_t n_elems, b200p_stream_t stream);
/* Stands in for wave::dpp::scan_exclusive_sum (wave_scan_dpp.hpp:74-87);
 * f32/f64/i32/i64. */
int b200p_segscan_exclusive_sum(int dtype, const void* in, void* out,
                                size_t n_elems, b200p_stream_t stream);

/* One wave64 through the DEVICE-level API of wave_primitives/wave64.cuh (the
 * pair-per-lane overloads), the way the reference's probe kernels call it
 * (research/wave-primitives/tests/probe_scan_dpp.hip:13-17).
 * fn: 0 reduce (result replicated to all 64 outputs), 1 inclusive scan,
 *     2 exclusive sum scan.  in/out: 64 values of `dtype` (16-bit reduce
 *     returns the input type). */
int b200p_wave_probe(int fn, int op, int dtype, const void* in64, void* out64,
                     b200p_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200P_H_ */
