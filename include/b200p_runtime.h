/* ---------------------------------------------------------------------------
 * b200p_runtime.h -- C ABI of the small LLM runtime around the attention
 * kernels: the reference's cdna3::runtime::Session
 * (cdna3-prims/include/cdna3/runtime/session.hpp:52-331) with its KVCache
 * (kv_cache.hpp:19-52) and the forward kernels of forward.hpp, for a batch of
 * equal-length sequences on one GPU.
 *
 * Like the reference Session, a session OWNS its scratch buffers and its KV
 * cache (allocated at creation, freed at destruction); the weights are the
 * caller's device memory (the reference's ModelLoader role: model_loader.hpp:
 * 134-204).  Calls on one session must come from one host thread at a time.
 * ------------------------------------------------------------------------- */
#ifndef B200P_RUNTIME_H_
#define B200P_RUNTIME_H_

#include "b200p.h"

#ifdef __cplusplus
extern "C" {
#endif

/* cdna3::runtime::ModelConfig, field for field (model_loader.hpp:51-60). */
typedef struct b200p_model_config {
    int n_layers;
    int hidden;
    int n_heads;
    int n_kv_heads;
    int head_dim;      /* 64 or 128 */
    int ffn_dim;
    int vocab_size;
    float rope_theta;
} b200p_model_config;

/* One decoder layer's weights: 16-bit, row-major [out, in] (HF nn.Linear layout,
 * forward.hpp:58-60).  Biases and may be NULL (Llama); norm weights are [hidden].
 * cdna3::runtime::LayerWeights (model_loader.hpp:62-78). */
typedef struct b200p_layer_weights {
    const void* Wq;        /* [n_heads*head_dim, hidden]    */
    const void* Wk;        /* [n_kv_heads*head_dim, hidden] */
    const void* Wv;        /* [n_kv_heads*head_dim, hidden] */
    const void* Wo;        /* [hidden, n_heads*head_dim]    */
    const void* bq;
    const void* bk;
    const void* bv;
    const void* Wgate;     /* [ffn_dim, hidden] */
    const void* Wup;       /* [ffn_dim, hidden] */
    const void* Wdown;     /* [hidden, ffn_dim] */
    const void* norm_attn; /* [hidden] */
    const void* norm_mlp;  /* [hidden] */
} b200p_layer_weights;

typedef struct b200p_model_weights {
    b200p_model_config cfg;
    int dtype;                          /* B200P_F16 or B200P_BF16: weights and activations */
    const void* embed_tokens;           /* [vocab, hidden] */
    const void* lm_head;                /* [vocab, hidden] */
    const void* final_norm;             /* [hidden]        */
    const b200p_layer_weights* layers;  /* host array of n_layers entries (device pointers inside) */
} b200p_model_weights;

/* cdna3::runtime::ModelLoader (model_loader.hpp:134-204): a model directory in the
 * reference's export format -- meta.json plus one raw 16-bit .bin file per tensor
 * (embed_tokens, lm_head, final_norm, layer_<i>_{q,k,v,o}_proj, layer_<i>_{q,k,v}_bias
 * when meta has qkv_bias, layer_<i>_{gate,up,down}_proj, layer_<i>_norm_{attn,mlp}).
 * The files hold fp16 bits unless meta.json says "dtype": "bf16".
 * b200p_model_read_meta only parses meta.json (no device needed); b200p_model_load
 * uploads every tensor into device memory that the model object owns;
 * b200p_model_weights_of gives the table a session is created from (valid until
 * b200p_model_free).  Failures are status codes (B200P_E_IO for a missing, short or
 * malformed file), where the reference throws. */
typedef struct b200p_model b200p_model;
int b200p_model_read_meta(const char* model_dir, b200p_model_config* cfg, int* qkv_bias, int* dtype);
b200p_model* b200p_model_load(const char* model_dir, int* status);
const b200p_model_weights* b200p_model_weights_of(const b200p_model* model);
void b200p_model_free(b200p_model* model);

typedef struct b200p_session b200p_session;

/* Session(model, max_seq) (session.hpp:253-259) for `batch` sequences.
 * Returns NULL and sets *status on failure. */
b200p_session* b200p_session_create(const b200p_model_weights* weights, int max_seq, int batch, int* status);
void b200p_session_destroy(b200p_session* s);

/* Session::generate (session.hpp:263-296): greedy decoding.
 * input_ids: host, [batch, T] token ids; out_tokens: host, [batch, max_new_tokens].
 * Prefill of the T prompt tokens from an empty cache, then max_new_tokens - 1
 * single-token steps.  The next-token ids stay on the device between steps (the
 * reference copies one int to the host per token, session.hpp:329); one copy at the
 * end returns them.  timings_ms (optional, host, 2 floats): time to first token and
 * total decode time, measured with events on `stream`. */
int b200p_session_generate(b200p_session* s, const int* input_ids, int T, int max_new_tokens,
                           int* out_tokens, float* timings_ms, b200p_stream_t stream);

/* Session::prefill_logits (session.hpp:299-318): prefill only; fp32 logits of the
 * last prompt token of every sequence, host [batch, vocab]. */
int b200p_session_prefill_logits(b200p_session* s, const int* input_ids, int T, float* logits, b200p_stream_t stream);

/* One more token per sequence on top of the current cache (teacher forcing):
 * feeds token_ids [batch] (host) at position kv_len, returns logits [batch, vocab]. */
int b200p_session_step_logits(b200p_session* s, const int* token_ids, float* logits, b200p_stream_t stream);

/* The decode step's projection kernel on its own: Y[M, N] = X[M, K] . W[N, K]^T for M <= 16,
 * 16-bit operands, fp32 accumulation.  Stands in for the rocBLAS calls of the decode step
 * (rocblas_gemm.hpp:112-209) together with the kernels around them:
 *   prologue 0: X = x16 [M, ldx] (16-bit);
 *   prologue 1: X = RMSNorm(x32 [M, K] fp32) * norm_w, rounded to 16 bits (forward.hpp:34-56);
 *   epilogue 0: out 16-bit [M, ldo];  2: out fp32;  1: out fp32 += Y (residual);
 *   epilogue 3: W is [2N, K] (gate rows, then up rows), out 16-bit = SiLU(gate) * up
 *               (forward.hpp:154-160).
 * Combinations: prologue 1 with epilogues 0, 2, 3; prologue 0 with epilogue 1.
 * K must be a multiple of 16; B200P_E_RANGE for shapes outside the kernel's domain. */
int b200p_skinny_gemm(int dtype, int prologue, int epilogue, const void* W, const void* x16, const float* x32,
                      const void* norm_w, void* out, int M, int N, int K, int ldx, int ldo, float eps,
                      b200p_stream_t stream);

/* C[M, N] = A[M, K] . W[N, K]^T on the tensor cores (tcgen05, fp32 accumulation in tensor memory), the
 * prefill-side counterpart of b200p_skinny_gemm: stands in for RocblasHandle::gemm_* at their call sites in
 * Session::run_layers (rocblas_gemm.hpp:112-209; session.hpp:147-160,171-173,220,227-230) with the element-wise
 * kernel that follows each GEMM in the reference folded into the epilogue:
 *   epilogue 0: C 16-bit;  2: C fp32;  1: C fp32 += product (the residual add, forward.hpp add_f32_kernel);
 *   epilogue 3: W is [2N, K] (gate rows, then up rows), C 16-bit = SiLU(gate) * up (forward.hpp:154-160).
 * A [M, lda] and W [N, ldw] 16-bit, row-major; lda, ldw, K multiples of 8; A, W, C and the rows of C 16-byte
 * aligned.  B200P_E_RANGE / B200P_E_ALIGN for anything else (nothing is launched). */
int b200p_gemm_16(int dtype, int epilogue, const void* A, const void* W, void* C, int M, int N, int K,
                  long long lda, long long ldw, long long ldc, b200p_stream_t stream);

int b200p_session_kv_len(const b200p_session* s);
/* Projections (matrix products) issued by the session so far, and how many of them went to the GEMM
 * library (cuBLAS) rather than to this library's own kernels: 0 unless a shape or pointer is outside
 * those kernels' domain or b200p_set_tuning("runtime_gemm" / "runtime_skinny", 0). */
unsigned long long b200p_session_gemm_calls(const b200p_session* s);
unsigned long long b200p_session_blas_calls(const b200p_session* s);
/* Decode steps of b200p_session_generate that ran as replays of the captured step graph
 * (every step after the first of a call when the steps run kernel by kernel, unless
 * b200p_set_tuning("runtime_graph", 0)). */
unsigned long long b200p_session_graph_replays(const b200p_session* s);
/* Launches of the persistent decode kernel.  After b200p_set_tuning("runtime_mega", 1),
 * b200p_session_generate runs ALL the decode steps of a call as one cooperative launch (one CTA per
 * SM, weights streamed through the phase boundaries, grid barriers with bounded waits between
 * phases) and b200p_session_step_logits runs its step as one such launch, when the session has at
 * most 8 sequences and the projection kernels' shapes.  Off by default: measured slower than the
 * kernel-per-phase step replayed as a graph (session.hpp:263-331). */
unsigned long long b200p_session_mega_launches(const b200p_session* s);

#ifdef __cplusplus
}
#endif
#endif /* B200P_RUNTIME_H_ */
