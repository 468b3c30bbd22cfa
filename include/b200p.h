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
    B200P_E_RANGE         = -10,  /* size beyond a documented maximum           */
    B200P_E_IO            = -11   /* a model file is missing, short or malformed */
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

/* b200p_wave_probe over n_waves independent waves (in/out: 64 * n_waves values),
 * one warp per wave: the device-level API on arbitrary data. */
int b200p_wave_probe_n(int fn, int op, int dtype, const void* in, void* out, int n_waves,
                       b200p_stream_t stream);

/* One wave through the vote and bitwise wrappers of wave64.cuh (the reference's
 * research/wave-primitives/include/wave_primitives/wave_ballot.hpp:23-75 and
 * wave_reduce.hpp reduce_and / reduce_or), pair per lane with predicate "value > 0":
 * out8[0] ballot (64 bits, bit i = element i), [1] any, [2] all, [3] popcount,
 * [4] reduce_and, [5] reduce_or of the 64 ints, [6] the 32-lane ballot of the lanes'
 * first elements, [7] lane_mask_lt() of lane 5. */
int b200p_wave_vote_probe(const int* in64, unsigned long long* out8, b200p_stream_t stream);

/* The register-resident reduce loop with which the reference measures its device-level primitives
 * (research/wave-primitives/benchmarks/bench_reduce_dpp_types.hip:29-45): each of n_waves waves (a multiple of 8;
 * in: 64 * n_waves values, out: n_waves values) reduces its 64 values `reps` times with the result fed back into
 * the inputs, no memory traffic inside the loop.  backend 0: wave::dpp::reduce_* of wave64.cuh (pair per lane);
 * backend 1: the portable shuffle-down loop + broadcast the reference compares against.  f32 / f64 / i32 / i64;
 * f16 / bf16 for the sum only (bench_h3_h4_multitype.hip): backend 0 accumulates in fp32 and rounds once
 * (wave::reduce_sum on a 16-bit pair), backend 1 accumulates in the 16-bit type (the "native" form).
 * The caller times the launch; throughput = 64 * n_waves * reps elements per launch. */
int b200p_wave_reduce_loop(int op, int dtype, int backend, const void* in, void* out, int n_waves, int reps,
                           b200p_stream_t stream);

/* The same for the inclusive prefix sum (research/wave-primitives/benchmarks/bench_scan_dpp.hip): each wave scans its
 * 64 values `reps` times, the total fed back into the inputs of the next repetition.  in and out: 64 * n_waves values (out
 * receives the waves' final state).  backend 0: wave::dpp::scan_inclusive_sum (pair per lane); backend 1: the
 * portable shuffle-up ladder.  f32 / f64 / i32 / i64.  Throughput = 64 * n_waves * reps elements per launch. */
int b200p_wave_scan_loop(int dtype, int backend, const void* in, void* out, int n_waves, int reps, b200p_stream_t stream);

/* The reference's two "real kernel" benchmarks of the primitives, one wave per row
 * (research/wave-primitives/benchmarks/bench_layernorm.hip:47-96, bench_softmax.hip):
 * which 0: out = LayerNorm(x) * gamma + beta (two row sums);  which 1: out = softmax(x) (row max + row sum).
 * x, out [rows, cols] fp32 with cols 64 or 512; gamma, beta [cols] (LayerNorm only); backend as above. */
int b200p_row_op(int which, int backend, int cols, const float* x, const float* gamma, const float* beta, float* out,
                 int rows, float eps, b200p_stream_t stream);

/* Kernels that use the facade headers the way a caller of the reference would
 * (cdna3-prims/tests/compile_smoke.hip:24-50; include <cdna3/cdna3.hpp> and
 * <cdna3/examples/fused_softmax.hpp>):
 *   which 0: cdna3::ex::row_softmax_lane over `rows` rows of 64 fp32 scores (pair per lane);
 *   which 1: the same, rows of 32 scores, one per lane;
 *   which 2: cdna3::ex::online_softmax_step over `tiles` 64-score tiles per row; out[row] =
 *            (running max, denominator, sum of exp(s - max) accumulated like an O column);
 *   which 3: dme::AsyncTile2D<16,64> ping/pong over `tiles` packed fp16 tiles (`in` is fp16),
 *            out = 2 * in as fp32;
 *   which 4: dme::copy_tile_1d_stream<float,256> per warp over `tiles` tiles, out = in + 1. */
int b200p_api_probe(int which, const void* in, float* out, int rows, int tiles, b200p_stream_t stream);

/* =========================================================================
 * FA2 attention.
 * Layouts are the reference's (cdna3-prims/include/cdna3/attention.hpp:83-85,
 * 112-116, 146-148): Q,O [batch, nQH, seqQ, D]; K,V [batch, nKVH, seqK, D];
 * decode q,o [nQH, D] and K,V [nKVH, N, D] or the strided cache
 * [nKVH, max_seq, D]; nQH % nKVH == 0; scale fixed at 1/sqrt(D); 16-bit I/O,
 * fp32 softmax and accumulation.  dtype is B200P_F16 (the reference's type) or
 * B200P_BF16.
 * ========================================================================= */

/* Decode arguments.  The first four fields are cdna3::attn::DecodeCfg
 * (attention.hpp:73-78), stride_kv is DecodeDmeCfg::stride_kv
 * (cdna3-prims/include/cdna3/detail/fa_decode_dme_kernel.hpp:45-48); the rest
 * extends the reference's single sequence to a batch and to a shard of the
 * KV sequence. */
typedef struct b200p_decode_args {
    int D;                     /* head dimension: 64 or 128                               */
    int N;                     /* number of cached keys attended to                       */
    int nQHeads;
    int nKVHeads;
    int stride_kv;             /* keys between consecutive KV heads: N if packed, max_seq
                                  for the cache layout                                    */
    int batch;                 /* sequences; q,o are [batch, nQH, D] (reference: 1)       */
    int dtype;                 /* B200P_F16 or B200P_BF16                                 */
    long long kv_batch_stride; /* elements between sequences in K and V;
                                  0 = nKVHeads * stride_kv * D                            */
    long long key_offset;      /* first key of each head to attend to (a KV shard starts
                                  here); N keys are read from it                          */
    long long q_batch_stride;  /* elements between sequences in q; 0 = nQHeads * D        */
    long long o_batch_stride;  /* elements between sequences in o; 0 = nQHeads * D        */
} b200p_decode_args;

/* Bytes of caller-owned scratch the decode entry points need for these
 * arguments (split-KV partials + a status word); 0 for invalid arguments.
 * The launchers allocate nothing, like the reference's (attention.hpp:117-137). */
size_t b200p_attn_decode_workspace_bytes(const b200p_decode_args* args);

/* Stands in for cdna3::attn::decode (attention.hpp:117-137, packed K/V:
 * stride_kv = N) and cdna3::attn::decode_dme (attention.hpp:152-173, strided
 * cache: stride_kv = max_seq).  workspace: 256-byte aligned device memory of at
 * least b200p_attn_decode_workspace_bytes(args). */
int b200p_attn_decode(const void* q, const void* K, const void* V, void* o,
                      const b200p_decode_args* args, void* workspace, size_t workspace_bytes,
                      b200p_stream_t stream);

/* b200p_attn_decode with the key count read on the device: the kernels attend to
 * min(*n_dev + n_add, args->N) keys, where args->N is now only an upper bound that
 * sizes the grid, the split plan and the workspace.  The launch parameters then do
 * not change from step to step, so a decode step can be captured once in a CUDA
 * graph and replayed while a device-side counter advances (the reference passes N
 * by value, attention.hpp:117-137, and re-launches every step).  K and V rows
 * between the live count and the next multiple of 128 (inside args->N) are fetched
 * and multiplied by a zero probability: they must hold finite values. */
int b200p_attn_decode_dyn(const void* q, const void* K, const void* V, void* o,
                          const b200p_decode_args* args, const int* n_dev, int n_add,
                          void* workspace, size_t workspace_bytes, b200p_stream_t stream);

/* The same attention over a shard of the KV sequence, returning what the
 * cross-shard combine needs: o_f32 [batch, nQH, D] normalised over the shard and
 * lse [batch, nQH] (natural log of the shard's softmax denominator, including
 * the running max).  No counterpart in the reference, which is single-GPU; the
 * merge it feeds is the reference's split-KV merge
 * (cdna3-prims/include/cdna3/detail/fa_decode_kernel.hpp:75-92). */
int b200p_attn_decode_partial(const void* q, const void* K, const void* V, float* o_f32, float* lse,
                              const b200p_decode_args* args, void* workspace, size_t workspace_bytes,
                              b200p_stream_t stream);

/* Merge `parts` shard results -> o [rows, D] in `dtype`.  Part g is
 * o_parts + g*o_part_stride ([rows, D] fp32) and lse_parts + g*lse_part_stride
 * ([rows]); a stride of 0 means densely packed parts.  With both strides equal
 * to rows*(D+1) the parts can be the rows of ONE all-gathered buffer that holds
 * each rank's O followed by its lse.
 * O = sum_g e^{lse_g-M} O_g / sum_g e^{lse_g-M} (fa_decode_kernel.hpp:75-92). */
int b200p_attn_merge_lse(const float* o_parts, const float* lse_parts, int parts, int rows, int D,
                         long long o_part_stride, long long lse_part_stride,
                         int dtype, void* o, b200p_stream_t stream);

/* The (O, lse) exchange fused into the kernels, over peer memory of one NVLink
 * domain, in place of decode_partial -> all-gather -> merge_lse.  No counterpart
 * in the reference (single GPU).
 *
 * Every rank owns a receive buffer of 2 * world * rows*(D+1) floats (two step
 * parities x one packed partial per source rank: O [rows, D], then lse [rows]),
 * an array of `world` int flag words and one local int counter, all zero before
 * the first step.  slots[g] / flags[g] are rank g's buffer and flag array as
 * addressable FROM THIS GPU (peer-mapped device pointers; entry [rank] is the
 * local one).  The caller obtains them however it shares memory between its
 * processes (CUDA IPC, symmetric memory); the library only stores through them.
 *
 * b200p_attn_decode_push: decode over this rank's KV shard, then store the
 *   shard's normalised O and lse into slot [seq & 1][rank] of every rank's
 *   buffer and, when all of it is written, store `seq` into flag word [rank] of
 *   every rank.  `seq` starts at 1 and grows by one per step on all ranks alike.
 * b200p_attn_merge_lse_wait: wait until all `world` local flag words are >= seq
 *   (at most wait_ns nanoseconds of wall time, 0 = 2 s), then merge the world
 *   partials of parity seq & 1 from the LOCAL buffer into o [rows, D].  A wait
 *   that runs out sets *status (device int, caller-cleared) to 1 and the launch
 *   ends; it never hangs.  Plain loads and stores only: no multicast.
 * Each rank must run on its own GPU: a rank's merge waits for the other ranks'
 * kernels, which is only safe when those run concurrently elsewhere. */
#define B200P_MAX_PEERS 16
typedef struct b200p_peer_exchange {
    int    rank, world;
    float* slots[B200P_MAX_PEERS];
    int*   flags[B200P_MAX_PEERS];
    int*   counter;
} b200p_peer_exchange;

int b200p_attn_decode_push(const void* q, const void* K, const void* V,
                           const b200p_decode_args* args, void* workspace, size_t workspace_bytes,
                           const b200p_peer_exchange* px, int seq, b200p_stream_t stream);

int b200p_attn_merge_lse_wait(const b200p_peer_exchange* px, int seq, int rows, int D, int dtype,
                              void* o, int* status, unsigned long long wait_ns, b200p_stream_t stream);

/* Decode for callers that cannot supply scratch memory -- a serving loop whose
 * memory plan is fixed at start-up, or a host runtime that passes only its own
 * tensors and has no allocator to lend.  This entry point has no counterpart in
 * the reference.  It is b200p_attn_decode with the split-KV scratch held in a
 * fixed array inside the library (b200p_attn_decode_noalloc_max_bytes() bytes,
 * 8 MiB, resident on every GPU that loads the library until the process ends)
 * and it allocates nothing itself.  Arguments whose scratch need exceeds that
 * size (compare b200p_attn_decode_workspace_bytes) are rejected with
 * B200P_E_RANGE.  The first call on each device looks up the array's device
 * address; make that first call outside any stream capture.  All calls share
 * the one array: two calls whose kernels can overlap on the GPU (different
 * streams, no dependency) race on it -- serialise them.  Two host threads that
 * make their first call on a device at the same moment both perform the address
 * look-up and store the same value, which is harmless.  A bounded wait that gave
 * up inside such a call is reported by b200p_attn_workspace_status(NULL, stream). */
int b200p_attn_decode_noalloc(const void* q, const void* K, const void* V, void* o,
                              const b200p_decode_args* args, b200p_stream_t stream);
size_t b200p_attn_decode_noalloc_max_bytes(void);

/* Synchronises `stream` and reports whether a kernel that used `workspace`
 * abandoned a bounded wait (B200P_E_TIMEOUT) or not (0).  workspace = NULL names
 * the built-in scratch of b200p_attn_decode_noalloc on the current device. */
int b200p_attn_workspace_status(const void* workspace, b200p_stream_t stream);

/* cdna3::attn::PrefillCfg, field for field (attention.hpp:63-71). */
typedef struct b200p_prefill_cfg {
    int D;          /* head dimension: 64 or 128                         */
    int seqQ;       /* query length (any; the reference needs a multiple of 16*W) */
    int seqK;       /* key/value length                                  */
    int nQHeads;
    int nKVHeads;   /* nQHeads % nKVHeads == 0                           */
    int batch;
    int causal;     /* 1: key k is masked for query q iff k > q          */
} b200p_prefill_cfg;

/* Stands in for cdna3::attn::prefill (attention.hpp:86-109) and its kernel
 * fa_multiwave_kernel<D,W> (cdna3-prims/include/cdna3/detail/
 * fa_prefill_kernel.hpp:43-177).  Q,O [batch, nQH, seqQ, D]; K,V
 * [batch, nKVH, seqK, D]; dtype B200P_F16 or B200P_BF16.  Unsupported D returns
 * B200P_E_DIM before any launch, as the reference returns hipErrorInvalidValue. */
int b200p_attn_prefill(const void* Q, const void* K, const void* V, void* O,
                       const b200p_prefill_cfg* cfg, int dtype, b200p_stream_t stream);

/* Element strides of Q, K, V and O for b200p_attn_prefill_strided: for each
 * tensor the distance between consecutive tokens, heads and sequences (the
 * head dimension D is always contiguous).  Every stride must be a multiple of
 * 8 elements. */
typedef struct b200p_attn_strides {
    long long q_seq, q_head, q_batch;
    long long k_seq, k_head, k_batch;
    long long v_seq, v_head, v_batch;
    long long o_seq, o_head, o_batch;
} b200p_attn_strides;

/* b200p_attn_prefill on tensors that are not in the dense head-major layout.
 * It lets a runtime attend straight over token-major projections
 * [batch, seq, heads, D] and over its KV cache [batch, nKVH, max_seq, D], which
 * removes the four repack_kernel launches per layer and the packed K/V copies of
 * cdna3-prims/include/cdna3/runtime/session.hpp:193-207. */
int b200p_attn_prefill_strided(const void* Q, const void* K, const void* V, void* O,
                               const b200p_prefill_cfg* cfg, int dtype, const b200p_attn_strides* strides,
                               b200p_stream_t stream);

/* The same launch, additionally writing the raw (unscaled) fp32 score tile
 * S = Q.K^T of the LAST 256-row query block's first 128 rows against keys
 * 0..127 of (batch 0, head 0) to raw_scores[128][128]: the known-answer probe
 * of the tensor-core operand layouts (the role of the reference's
 * research/flash-attention-mi300x/tests/probe_mfma_mapping.hip). */
int b200p_attn_prefill_debug(const void* Q, const void* K, const void* V, void* O,
                             const b200p_prefill_cfg* cfg, int dtype, float* raw_scores,
                             b200p_stream_t stream);

/* The reference's FA2 build-order steps at their own tiling (Br = 16 query rows
 * per block, Bc = 64 keys per tile, one warp per query row), MHA, non-causal:
 *   step 0  fa_naive  research/flash-attention-mi300x/fa_naive.hip:72-212
 *   step 1  fa_dpp    research/flash-attention-mi300x/fa_dpp.hip:52-167
 *   step 2  fa_dme    research/flash-attention-mi300x/fa_dme.hip:74-221
 *   step 3  fa_mfma2  research/flash-attention-mi300x/fa_mfma2.hip:63-217
 *           (the tensor-core kernel of b200p_attn_prefill; 16-bit types only)
 * Q,K,V,O [batch, heads, seq, D]; dtype B200P_F16 (the reference's), B200P_BF16
 * or, for steps 0-2, B200P_F32 -- the fp32-I/O kernels whose launch takes
 * (seq_len, n_heads, scale): research/flash-attention-mi300x/kernels/
 * fa_naive.hip:118-278, kernels/fa_dpp.hip:167-313.  scale = 0 means 1/sqrt(D).
 * seq_q % 16 == 0 and seq_k % 64 == 0 for steps 0-2 (the reference's tiling), except
 * B200P_F32 with seq_q == seq_k, which accepts any length (see b200p_fa_rows_f32). */
int b200p_fa_step(int step, int dtype, const void* Q, const void* K, const void* V, void* O,
                  int batch, int heads, int seq_q, int seq_k, int D, float scale, b200p_stream_t stream);

/* The reference's fp32-I/O kernels with one query row per block and Bc keys per
 * tile over Bc/64 waves: research/flash-attention-mi300x/kernels/fa_naive.hip:118-278
 * (variant 0, portable shuffle reductions) and kernels/fa_dpp.hip:96-155,167-313
 * (variant 1, wave primitives + the two-phase block reduction).  Same launch
 * arguments as the reference: (seq_len, n_heads, scale); Q,K,V,O [batch, heads,
 * seq_len, D] fp32; bc 64, 128 or 256; any seq_len (keys past the end are padded
 * as in kernels/fa_naive.hip:158-169); scale = 0 means 1/sqrt(D).
 * b200p_fa_step with B200P_F32 and lengths off its tiling routes here with bc = 64. */
int b200p_fa_rows_f32(int variant, int bc, const float* Q, const float* K, const float* V, float* O,
                      int batch, int heads, int seq_len, int D, float scale, b200p_stream_t stream);

/* Synchronises the device and reports whether any kernel of this library
 * abandoned a bounded wait since the last clear (B200P_E_TIMEOUT) or not (0). */
int b200p_device_status(int clear);

#ifdef __cplusplus
}
#endif
#endif /* B200P_H_ */
