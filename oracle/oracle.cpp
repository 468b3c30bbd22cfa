// ---------------------------------------------------------------------------
// oracle.cpp -- CPU restatement of the reference's algorithms for the wave
// reduce/scan primitives and the FA2 attention path.
//
// THIS IS TEST INFRASTRUCTURE.  It is the checker the CUDA path is compared
// with and the timed CPU baseline; nothing in the product library calls it.
//
// Pinning: the attention functions are checked bit-for-bit against the
// reference's own CPU reference functions compiled from the reference tree
// (oracle/build_ref.py -> oracle/_ref/libref_cpu.so), and the reduce/scan
// emulators against every known-answer vector the reference's tests hold
// (lanes 0..63 -> 2016/63/0, ones -> i+1, ...; tests/test_oracle.py).
//
// Each function names the reference file:line it follows (paths relative to
// the reference project root).
// Build: g++ -O2 -std=c++17 -ffp-contract=off -shared -fPIC -pthread
// ---------------------------------------------------------------------------
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <random>
#include <thread>
#include <vector>

namespace {

// ---- 16-bit float conversions (round to nearest even, like __float2half /
// hip_bfloat16(float)) -------------------------------------------------------
inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x0040u);   // quiet NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}
inline float bf16_to_f32(uint16_t h) { return u2f(uint32_t(h) << 16); }

inline uint16_t f32_to_f16(float f) {
    const uint32_t u = f2u(f);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t abs = u & 0x7fffffffu;
    if (abs > 0x7f800000u) return uint16_t(sign | 0x7e00u);                 // NaN
    if (abs >= 0x47800000u) {                                               // >= 65536: inf (65520..65536 handled below)
        return uint16_t(sign | 0x7c00u);
    }
    if (abs < 0x38800000u) {                                                // subnormal half or zero
        if (abs < 0x33000000u) return uint16_t(sign);                       // < 2^-25 rounds to zero
        const int e = int(abs >> 23);                                       // biased exponent, 102..112
        uint32_t m = (abs & 0x7fffffu) | 0x800000u;                         // 24-bit significand
        const int shift = 126 - e;                                          // 14..24
        const uint32_t q = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1);
        uint32_t r = q + ((rem > half || (rem == half && (q & 1u))) ? 1u : 0u);
        return uint16_t(sign | r);
    }
    uint32_t r = abs - 0x38000000u;                                         // rebias 127 -> 15
    const uint32_t rem = r & 0x1fffu;
    r >>= 13;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;                 // may carry into inf: correct
    return uint16_t(sign | r);
}
inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = uint32_t(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return u2f(sign);
        int s = 0;
        while (!(m & 0x400u)) { m <<= 1; ++s; }
        m &= 0x3ffu;
        return u2f(sign | uint32_t(127 - 15 - s + 1) << 23 | (m << 13));
    }
    if (e == 31) return u2f(sign | 0x7f800000u | (m << 13));
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

// ---- ops: the reference's functors, research/wave-primitives/include/
// wave_primitives/wave_reduce_dpp.hpp:101-103 and identities :56-58 ---------
enum { OP_SUM = 0, OP_MAX = 1, OP_MIN = 2 };
template <typename T> inline T apply(int op, T a, T b) {
    if (op == OP_SUM) return a + b;
    if (op == OP_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
template <typename T> inline T identity(int op) {
    if (op == OP_SUM) return T(0);
    if (op == OP_MAX) return std::numeric_limits<T>::lowest();
    return std::numeric_limits<T>::max();
}
// int overflow must wrap like the GPU's two's-complement add
template <> inline int apply<int>(int op, int a, int b) {
    if (op == OP_SUM) return int(uint32_t(a) + uint32_t(b));
    if (op == OP_MAX) return a > b ? a : b;
    return a < b ? a : b;
}
template <> inline long long apply<long long>(int op, long long a, long long b) {
    if (op == OP_SUM) return (long long)((unsigned long long)a + (unsigned long long)b);
    if (op == OP_MAX) return a > b ? a : b;
    return a < b ? a : b;
}

// ---- DPP lane routing on a 64-lane wave, as documented at
// wave_reduce_dpp.hpp:20-30: lanes with no source read `old`. ----------------
template <typename T> void row_shr(const T* v, T* moved, int n, T old) {
    for (int i = 0; i < 64; ++i) moved[i] = ((i & 15) >= n) ? v[i - n] : old;
}
template <typename T> void row_bcast15(const T* v, T* moved, T old) {   // 15->[16..31], 31->[32..47], 47->[48..63]
    for (int i = 0; i < 64; ++i) moved[i] = (i >= 16) ? v[(i & ~15) - 1] : old;
}
template <typename T> void row_bcast31(const T* v, T* moved, T old) {   // 31->[32..63]
    for (int i = 0; i < 64; ++i) moved[i] = (i >= 32) ? v[31] : old;
}

// dpp_reduce, wave_reduce_dpp.hpp:68-77: v = op(v, moved) six times; result on lane 63.
template <typename T> T dpp_reduce64(const T* x, int op) {
    T v[64], m[64];
    const T id = identity<T>(op);
    for (int i = 0; i < 64; ++i) v[i] = x[i];
    const int shr[4] = {1, 2, 4, 8};
    for (int s = 0; s < 4; ++s) {
        row_shr(v, m, shr[s], id);
        for (int i = 0; i < 64; ++i) v[i] = apply(op, v[i], m[i]);
    }
    row_bcast15(v, m, id);
    for (int i = 0; i < 64; ++i) v[i] = apply(op, v[i], m[i]);
    row_bcast31(v, m, id);
    for (int i = 0; i < 64; ++i) v[i] = apply(op, v[i], m[i]);
    return v[63];
}

// scan_inclusive, wave_scan_dpp.hpp:51-68.
template <typename T> void dpp_scan64(const T* x, T* out, int op) {
    T v[64], m[64], c1[64], c1b[64], c1c[64];
    const T id = identity<T>(op);
    for (int i = 0; i < 64; ++i) v[i] = x[i];
    const int shr[4] = {1, 2, 4, 8};
    for (int s = 0; s < 4; ++s) {
        row_shr(v, m, shr[s], id);
        for (int i = 0; i < 64; ++i) v[i] = apply(op, v[i], m[i]);
    }
    row_bcast15(v, c1, id);
    row_bcast15(c1, c1b, id);
    row_bcast15(c1b, c1c, id);
    for (int L = 0; L < 64; ++L) {
        T carry = id;
        if (L >= 16) carry = c1[L];
        if (L >= 32) carry = apply(op, carry, c1b[L]);
        if (L >= 48) carry = apply(op, carry, c1c[L]);
        out[L] = (L >= 16) ? apply(op, v[L], carry) : v[L];
    }
}

// scan_exclusive_sum, wave_scan_dpp.hpp:74-87.
template <typename T> void dpp_scan_excl64(const T* x, T* out) {
    T inc[64], ex[64], carry[64];
    dpp_scan64(x, inc, OP_SUM);
    row_shr(inc, ex, 1, T(0));
    row_bcast15(inc, carry, T(0));
    for (int L = 0; L < 64; ++L) out[L] = ((L & 15) == 0 && L != 0) ? carry[L] : ex[L];
}

// Portable reduce on a 64-wide wave, wave_reduce.hpp:40-63 / :69-91 / :97-119:
// f op= shfl_down(f, offset) for offset 32..1; lanes whose source is out of
// range read their own value; result on lane 0.
inline float shfl_reduce64(const float* x, int op) {
    float v[64], m[64];
    for (int i = 0; i < 64; ++i) v[i] = x[i];
    for (int o = 32; o > 0; o >>= 1) {
        for (int i = 0; i < 64; ++i) m[i] = (i + o < 64) ? v[i + o] : v[i];
        for (int i = 0; i < 64; ++i) {
            if (op == OP_SUM) v[i] = v[i] + m[i];
            else if (op == OP_MAX) v[i] = std::max(v[i], m[i]);
            else v[i] = std::min(v[i], m[i]);
        }
    }
    return v[0];
}
// Portable Hillis-Steele scan, wave_scan.hpp:40-74.
inline void shfl_scan64(const float* x, float* out, int op) {
    float v[64], m[64];
    for (int i = 0; i < 64; ++i) v[i] = x[i];
    for (int o = 1; o < 64; o <<= 1) {
        for (int i = 0; i < 64; ++i) m[i] = (i >= o) ? v[i - o] : v[i];
        for (int i = 0; i < 64; ++i) {
            if (i < o) continue;
            if (op == OP_SUM) v[i] = v[i] + m[i];
            else if (op == OP_MAX) v[i] = std::max(v[i], m[i]);
            else v[i] = std::min(v[i], m[i]);
        }
    }
    for (int i = 0; i < 64; ++i) out[i] = v[i];
}

// Run fn(unit) for unit in [0, n) on `threads` host threads (independent units).
template <typename F> void parallel_for(size_t n, int threads, F fn) {
    if (threads <= 1 || n <= 1) { for (size_t i = 0; i < n; ++i) fn(i); return; }
    std::vector<std::thread> pool;
    const size_t t = std::min<size_t>(size_t(threads), n);
    for (size_t w = 0; w < t; ++w)
        pool.emplace_back([=]() { for (size_t i = w; i < n; i += t) fn(i); });
    for (auto& th : pool) th.join();
}

template <typename T> void seg_reduce(int op, const T* in, T* out, size_t nseg, int threads) {
    const size_t chunk = 4096;
    parallel_for((nseg + chunk - 1) / chunk, threads, [=](size_t c) {
        const size_t e = std::min(nseg, (c + 1) * chunk);
        for (size_t s = c * chunk; s < e; ++s) out[s] = dpp_reduce64(in + s * 64, op);
    });
}
template <typename T> void seg_scan(int op, const T* in, T* out, size_t nseg, int excl, int threads) {
    const size_t chunk = 4096;
    parallel_for((nseg + chunk - 1) / chunk, threads, [=](size_t c) {
        const size_t e = std::min(nseg, (c + 1) * chunk);
        for (size_t s = c * chunk; s < e; ++s) {
            if (excl) dpp_scan_excl64(in + s * 64, out + s * 64);
            else      dpp_scan64(in + s * 64, out + s * 64, op);
        }
    });
}


// ---- the reference's CPU-side statement of reduce/scan: sequential loops -------------
// The reference checks its GPU results against a plain loop over the wave's
// values (research/wave-primitives/benchmarks/bench_reduce_dpp_types.hip:60-62,
// `exp_sum = exp_sum + i`) and against closed-form prefixes (research/
// wave-primitives/tests/probe_scan_dpp.hip:23-35).  These are those loops per
// 64-element segment; they are what the CPU baseline times.  Integer and
// max/min results equal the tree forms bit for bit; floating-point sums differ
// from them by rounding only.
template <typename T> void seq_reduce(int op, const T* in, T* out, size_t nseg, int threads) {
    const size_t chunk = 8192;
    parallel_for((nseg + chunk - 1) / chunk, threads, [=](size_t c) {
        const size_t e = std::min(nseg, (c + 1) * chunk);
        for (size_t s = c * chunk; s < e; ++s) {
            const T* x = in + s * 64;
            T acc = x[0];
            for (int i = 1; i < 64; ++i) acc = apply(op, acc, x[i]);
            out[s] = acc;
        }
    });
}
template <typename T> void seq_scan(int op, const T* in, T* out, size_t nseg, int threads) {
    const size_t chunk = 8192;
    parallel_for((nseg + chunk - 1) / chunk, threads, [=](size_t c) {
        const size_t e = std::min(nseg, (c + 1) * chunk);
        for (size_t s = c * chunk; s < e; ++s) {
            const T* x = in + s * 64; T* y = out + s * 64;
            T acc = x[0]; y[0] = acc;
            for (int i = 1; i < 64; ++i) { acc = apply(op, acc, x[i]); y[i] = acc; }
        }
    });
}

// ---------------------------------------------------------------------------
// Attention.
// One (batch, q-head) unit of cpu_prefill, cdna3-prims/tests/
// validate_attention_api.hip:27-51 (identical arithmetic: attn_ref,
// research/flash-attention-mi300x/fa_robust.hip:186-218, and with
// causal=0, group=1: attn_cpu_ref, research/flash-attention-mi300x/
// fa_naive.hip:217-243).  P is normalised BEFORE P.V.
// ---------------------------------------------------------------------------
void prefill_unit(const float* Q, const float* K, const float* V, float* O,
                  int D, int seqQ, int seqK, int nQH, int nKVH, int causal, int b, int h) {
    const float scale = 1.f / sqrtf((float)D);
    const int group = nQH / nKVH;
    const int kvh = h / group;
    std::vector<float> S((size_t)seqK);
    for (int q = 0; q < seqQ; ++q) {
        const int kmax = causal ? std::min(seqK, q + 1) : seqK;
        float mx = -1e38f;
        const float* qp = &Q[(((size_t)b * nQH + h) * seqQ + q) * D];
        for (int k = 0; k < kmax; ++k) {
            float dot = 0;
            const float* kp = &K[(((size_t)b * nKVH + kvh) * seqK + k) * D];
            for (int d = 0; d < D; ++d) dot += qp[d] * kp[d];
            S[k] = dot * scale;
            mx = std::max(mx, S[k]);
        }
        float se = 0;
        for (int k = 0; k < kmax; ++k) { S[k] = expf(S[k] - mx); se += S[k]; }
        for (int k = 0; k < kmax; ++k) S[k] /= se;
        float* op = &O[(((size_t)b * nQH + h) * seqQ + q) * D];
        for (int d = 0; d < D; ++d) {
            float o = 0;
            for (int k = 0; k < kmax; ++k) {
                const float* vp = &V[(((size_t)b * nKVH + kvh) * seqK + k) * D];
                o += S[k] * vp[d];
            }
            op[d] = o;
        }
    }
}

// One q-head of cpu_decode, validate_attention_api.hip:53-72 (identical:
// decode_ref, research/flash-attention-mi300x/fa_decode.hip:34-52).  K/V rows
// of a kv-head are `stride_kv` keys apart between heads (stride_kv = N for the
// packed layout; = max_seq for the cache layout read by decode_dme,
// cdna3-prims/include/cdna3/detail/fa_decode_dme_kernel.hpp:84-86).
void decode_unit(const float* q, const float* K, const float* V, float* o,
                 int D, int N, int nQH, int nKVH, long long stride_kv, int h) {
    const float scale = 1.f / sqrtf((float)D);
    const int group = nQH / nKVH;
    const int kvh = h / group;
    std::vector<float> S((size_t)N);
    float mx = -1e38f;
    const float* qp = &q[(size_t)h * D];
    for (int k = 0; k < N; ++k) {
        float dot = 0;
        const float* kp = &K[((size_t)kvh * stride_kv + k) * D];
        for (int d = 0; d < D; ++d) dot += qp[d] * kp[d];
        S[k] = dot * scale;
        mx = std::max(mx, S[k]);
    }
    float se = 0;
    for (int k = 0; k < N; ++k) { S[k] = expf(S[k] - mx); se += S[k]; }
    float* op = &o[(size_t)h * D];
    for (int d = 0; d < D; ++d) {
        float acc = 0;
        for (int k = 0; k < N; ++k) {
            const float* vp = &V[((size_t)kvh * stride_kv + k) * D];
            acc += (S[k] / se) * vp[d];
        }
        op[d] = acc;
    }
}

} // namespace

extern "C" {

// ---- conversions ------------------------------------------------------------
void orc_f32_to_f16(const float* in, uint16_t* out, size_t n)  { for (size_t i = 0; i < n; ++i) out[i] = f32_to_f16(in[i]); }
void orc_f16_to_f32(const uint16_t* in, float* out, size_t n)  { for (size_t i = 0; i < n; ++i) out[i] = f16_to_f32(in[i]); }
void orc_f32_to_bf16(const float* in, uint16_t* out, size_t n) { for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]); }
void orc_bf16_to_f32(const uint16_t* in, float* out, size_t n) { for (size_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]); }

// ---- seeded generators --------------------------------------------------------
// The reference's input recipe: std::mt19937(seed) + normal_distribution<float>
// drawn in one stream (Q, then K, then V), e.g. research/flash-attention-mi300x/
// fa_naive.hip:258-263, cdna3-prims/tests/validate_attention_api.hip:82-84.
void orc_gen_normal_mt19937(uint32_t seed, float mean, float stddev, float* out, size_t n) {
    std::mt19937 rng(seed);
    std::normal_distribution<float> dist(mean, stddev);
    for (size_t i = 0; i < n; ++i) out[i] = dist(rng);
}
// validate_decode_dme's recipe (cdna3-prims/tests/validate_decode_dme.hip:51-95):
// ONE mt19937(123) stream across all configs; per config q first, then for each
// (head, n, d) a K value followed by a V value, each rounded to fp16 on the way
// into a zero-filled cache [nKVH, max_seq, D].  `skip` draws are discarded first
// so that config i can be regenerated without the earlier ones' buffers.
void orc_gen_decode_dme_case(uint32_t seed, size_t skip, int D, int N, int nQH, int nKVH, int max_seq,
                             uint16_t* q, uint16_t* cacheK, uint16_t* cacheV) {
    std::mt19937 rng(seed);
    std::normal_distribution<float> dist(0.f, 0.5f);
    for (size_t i = 0; i < skip; ++i) (void)dist(rng);
    for (size_t i = 0; i < (size_t)nQH * D; ++i) q[i] = f32_to_f16(dist(rng));
    std::memset(cacheK, 0, (size_t)nKVH * max_seq * D * 2);
    std::memset(cacheV, 0, (size_t)nKVH * max_seq * D * 2);
    for (int h = 0; h < nKVH; ++h)
        for (int n = 0; n < N; ++n)
            for (int d = 0; d < D; ++d) {
                cacheK[(size_t)h * max_seq * D + (size_t)n * D + d] = f32_to_f16(dist(rng));
                cacheV[(size_t)h * max_seq * D + (size_t)n * D + d] = f32_to_f16(dist(rng));
            }
}

// ---- segmented reduce / scan, reference association -----------------------------
void orc_dpp_reduce_f32(int op, const float* in, float* out, size_t nseg, int threads)         { seg_reduce(op, in, out, nseg, threads); }
void orc_dpp_reduce_f64(int op, const double* in, double* out, size_t nseg, int threads)       { seg_reduce(op, in, out, nseg, threads); }
void orc_dpp_reduce_i32(int op, const int* in, int* out, size_t nseg, int threads)             { seg_reduce(op, in, out, nseg, threads); }
void orc_dpp_reduce_i64(int op, const long long* in, long long* out, size_t nseg, int threads) { seg_reduce(op, in, out, nseg, threads); }

void orc_dpp_scan_f32(int op, const float* in, float* out, size_t nseg, int excl, int threads)         { seg_scan(op, in, out, nseg, excl, threads); }
void orc_dpp_scan_f64(int op, const double* in, double* out, size_t nseg, int excl, int threads)       { seg_scan(op, in, out, nseg, excl, threads); }
void orc_dpp_scan_i32(int op, const int* in, int* out, size_t nseg, int excl, int threads)             { seg_scan(op, in, out, nseg, excl, threads); }
void orc_dpp_scan_i64(int op, const long long* in, long long* out, size_t nseg, int excl, int threads) { seg_scan(op, in, out, nseg, excl, threads); }


void orc_seq_reduce_f32(int op, const float* in, float* out, size_t nseg, int threads)         { seq_reduce(op, in, out, nseg, threads); }
void orc_seq_reduce_f64(int op, const double* in, double* out, size_t nseg, int threads)       { seq_reduce(op, in, out, nseg, threads); }
void orc_seq_reduce_i32(int op, const int* in, int* out, size_t nseg, int threads)             { seq_reduce(op, in, out, nseg, threads); }
void orc_seq_reduce_i64(int op, const long long* in, long long* out, size_t nseg, int threads) { seq_reduce(op, in, out, nseg, threads); }
void orc_seq_scan_f32(int op, const float* in, float* out, size_t nseg, int threads)           { seq_scan(op, in, out, nseg, threads); }
void orc_seq_scan_f64(int op, const double* in, double* out, size_t nseg, int threads)         { seq_scan(op, in, out, nseg, threads); }
void orc_seq_scan_i32(int op, const int* in, int* out, size_t nseg, int threads)               { seq_scan(op, in, out, nseg, threads); }
void orc_seq_scan_i64(int op, const long long* in, long long* out, size_t nseg, int threads)   { seq_scan(op, in, out, nseg, threads); }

// 16-bit inputs, fp32 accumulation, portable shfl_down order
// (wave_reduce.hpp:48-63).  out_f32: the float before rounding; out_narrow: what
// the reference returns.  Either may be NULL.
void orc_shfl_reduce_narrow(int op, int is_bf16, const uint16_t* in, float* out_f32, uint16_t* out_narrow,
                            size_t nseg, int threads) {
    const size_t chunk = 4096;
    parallel_for((nseg + chunk - 1) / chunk, threads, [=](size_t c) {
        const size_t e = std::min(nseg, (c + 1) * chunk);
        float x[64];
        for (size_t s = c * chunk; s < e; ++s) {
            for (int i = 0; i < 64; ++i) x[i] = is_bf16 ? bf16_to_f32(in[s * 64 + i]) : f16_to_f32(in[s * 64 + i]);
            const float r = shfl_reduce64(x, op);
            if (out_f32) out_f32[s] = r;
            if (out_narrow) out_narrow[s] = is_bf16 ? f32_to_bf16(r) : f32_to_f16(r);
        }
    });
}
// wave::scan_inclusive_sum(__half | bf16) (+max/min), wave_scan.hpp:52-74.
void orc_shfl_scan_narrow(int op, int is_bf16, const uint16_t* in, uint16_t* out, size_t nseg, int threads) {
    const size_t chunk = 4096;
    parallel_for((nseg + chunk - 1) / chunk, threads, [=](size_t c) {
        const size_t e = std::min(nseg, (c + 1) * chunk);
        float x[64], y[64];
        for (size_t s = c * chunk; s < e; ++s) {
            for (int i = 0; i < 64; ++i) x[i] = is_bf16 ? bf16_to_f32(in[s * 64 + i]) : f16_to_f32(in[s * 64 + i]);
            shfl_scan64(x, y, op);
            for (int i = 0; i < 64; ++i) out[s * 64 + i] = is_bf16 ? f32_to_bf16(y[i]) : f32_to_f16(y[i]);
        }
    });
}
// The portable float reduce (result on lane 0), wave_reduce.hpp:40-46 -- used
// for the fp16 accuracy known-answer (64 x 0.1 -> 6.4, bench_all_types.hip:95-127).
float orc_shfl_reduce_f32(int op, const float* in64) { return shfl_reduce64(in64, op); }

// ---- attention ----------------------------------------------------------------
// cpu_prefill over all (batch, head) units; units run on `threads` host threads,
// per-unit arithmetic untouched.
void orc_cpu_prefill(const float* Q, const float* K, const float* V, float* O,
                     int D, int seqQ, int seqK, int nQH, int nKVH, int batch, int causal, int threads) {
    parallel_for((size_t)batch * nQH, threads, [=](size_t u) {
        prefill_unit(Q, K, V, O, D, seqQ, seqK, nQH, nKVH, causal, int(u / nQH), int(u % nQH));
    });
}
// Only the listed (batch*nQH + head) units: bounded CPU-baseline samples.
void orc_cpu_prefill_units(const float* Q, const float* K, const float* V, float* O,
                           int D, int seqQ, int seqK, int nQH, int nKVH, int causal,
                           const int* units, int n_units, int threads) {
    parallel_for((size_t)n_units, threads, [=](size_t i) {
        prefill_unit(Q, K, V, O, D, seqQ, seqK, nQH, nKVH, causal, units[i] / nQH, units[i] % nQH);
    });
}

// cpu_attention_ref, research/flash-attention-mi300x/kernels/fa_naive.hip:284-313:
// single head, max starts at -inf, divides by sum_exp AFTER accumulating P.V.
void orc_cpu_attention_ref(const float* Q, const float* K, const float* V, float* O,
                           int seq_len, int d, float scale) {
    std::vector<float> scores((size_t)seq_len);
    for (int i = 0; i < seq_len; ++i) {
        float max_s = -std::numeric_limits<float>::infinity();
        for (int j = 0; j < seq_len; ++j) {
            float s = 0.0f;
            for (int dd = 0; dd < d; ++dd) s += Q[i * d + dd] * K[j * d + dd];
            scores[j] = s * scale;
            max_s = std::max(max_s, scores[j]);
        }
        float sum_exp = 0.0f;
        for (int j = 0; j < seq_len; ++j) { scores[j] = expf(scores[j] - max_s); sum_exp += scores[j]; }
        for (int dd = 0; dd < d; ++dd) {
            float acc = 0.0f;
            for (int j = 0; j < seq_len; ++j) acc += scores[j] * V[j * d + dd];
            O[i * d + dd] = acc / sum_exp;
        }
    }
}
// The same over [units] heads laid out back to back (batch*heads, seq, d).
void orc_cpu_attention_ref_heads(const float* Q, const float* K, const float* V, float* O,
                                 int n_units, int seq_len, int d, float scale, int threads) {
    const size_t hs = (size_t)seq_len * d;
    parallel_for((size_t)n_units, threads, [=](size_t u) {
        orc_cpu_attention_ref(Q + u * hs, K + u * hs, V + u * hs, O + u * hs, seq_len, d, scale);
    });
}

// cpu_decode with a batch dimension and a kv-head stride (see decode_unit).
// q,o: [batch, nQH, D]; K,V: [batch, nKVH, stride_kv, D] with kv_batch_stride
// elements between sequences.
void orc_cpu_decode(const float* q, const float* K, const float* V, float* o,
                    int D, int N, int nQH, int nKVH, long long stride_kv,
                    int batch, long long kv_batch_stride, int threads) {
    parallel_for((size_t)batch * nQH, threads, [=](size_t u) {
        const size_t b = u / nQH;
        decode_unit(q + b * (size_t)nQH * D, K + b * (size_t)kv_batch_stride, V + b * (size_t)kv_batch_stride,
                    o + b * (size_t)nQH * D, D, N, nQH, nKVH, stride_kv, int(u % nQH));
    });
}

// Split-KV merge, cdna3-prims/include/cdna3/detail/fa_decode_kernel.hpp:75-92:
//   m = max_w m_w;  l = sum_w e^{m_w-m} l_w;  O = sum_w e^{m_w-m} O_w / l (l>0 else 1)
// O_parts: [parts, rows, D] UNNORMALISED partial outputs, m/l: [parts, rows].
// expf stands in for the kernel's __expf.
void orc_merge_partials(const float* O_parts, const float* m_parts, const float* l_parts,
                        float* out, int parts, size_t rows, int D) {
    for (size_t r = 0; r < rows; ++r) {
        float m = -1e38f;
        for (int w = 0; w < parts; ++w) m = fmaxf(m, m_parts[w * rows + r]);
        float l = 0.f;
        std::vector<float> acc((size_t)D, 0.f);
        for (int w = 0; w < parts; ++w) {
            const float f = expf(m_parts[w * rows + r] - m);
            l += f * l_parts[w * rows + r];
            for (int d = 0; d < D; ++d) acc[d] += f * O_parts[((size_t)w * rows + r) * D + d];
        }
        const float inv = (l > 0.f) ? 1.f / l : 1.f;
        for (int d = 0; d < D; ++d) out[r * D + d] = acc[d] * inv;
    }
}
// The same merge stated on NORMALISED partials and their log-sum-exp, the form
// that crosses GPUs: O = sum_g e^{lse_g - M} O_g / sum_g e^{lse_g - M}.
void orc_merge_lse(const float* O_parts, const float* lse_parts, float* out, float* lse_out,
                   int parts, size_t rows, int D) {
    for (size_t r = 0; r < rows; ++r) {
        float M = -INFINITY;
        for (int g = 0; g < parts; ++g) M = fmaxf(M, lse_parts[g * rows + r]);
        float den = 0.f;
        std::vector<float> acc((size_t)D, 0.f);
        for (int g = 0; g < parts; ++g) {
            const float w = (M == -INFINITY) ? 0.f : expf(lse_parts[g * rows + r] - M);
            den += w;
            for (int d = 0; d < D; ++d) acc[d] += w * O_parts[((size_t)g * rows + r) * D + d];
        }
        const float inv = den > 0.f ? 1.f / den : 1.f;
        for (int d = 0; d < D; ++d) out[r * D + d] = acc[d] * inv;
        if (lse_out) lse_out[r] = den > 0.f ? M + logf(den) : -INFINITY;
    }
}

int orc_hardware_threads(void) { return int(std::thread::hardware_concurrency()); }

} // extern "C"
