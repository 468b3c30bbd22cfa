// ---------------------------------------------------------------------------
// decode_mega.cuh -- the greedy decode loop of the runtime as ONE persistent kernel.
//
// cdna3::runtime::Session::generate (session.hpp:263-331) launches every kernel of every decode
// step from the host: per layer a norm, three projections, RoPE, the cache scatter, attention, the
// output projection, a norm, two more projections, SiLU, the down projection, then the final norm,
// lm_head and argmax.  Run as separate kernels (however fused), each of them drains the machine
// before the next one can start to fill it, and with one new token per sequence the step is a
// stream over the weights that takes ~13 us per layer: the gaps cost more than the work.
//
// Here one cooperative launch of one CTA per SM runs n_steps whole steps.  Every CTA has
//  * one producer thread that streams ITS share of every weight matrix, in the fixed order of the
//    step, through a ring of shared-memory stages (stream_produce).  Weights do not depend on
//    activations, so the producer never waits for anything but ring space: it runs through the
//    phase boundaries, and while the consumers stand at a grid barrier the next projection's
//    weights are already arriving;
//  * eight consumer warps that walk the phases of the step -- Q/K/V projection (RMSNorm prologue;
//    bias, RoPE and the cache scatter as epilogue), attention over the cache, output projection
//    (+= residual), gate/up projection (RMSNorm prologue, SiLU * up epilogue), down projection
//    (+= residual), and after the last layer lm_head (final norm prologue, fp32 logits and the
//    running argmax key as epilogue) -- with a grid barrier after each.
// The projections are stream_consume / skinny_prologue / skinny_epilogue of skinny_gemm.cuh, the
// very code of the per-kernel path.  Attention is written here for this setting (a handful of
// query rows against a cache that is short next to the weights): a unit is one (sequence,
// kv head, key split), cut so that every CTA gets at most one; in its CTA each warp takes one
// query head and 32-key chunks, one key per lane for q.k, one output column pair per lane for
// p.v, every load of a chunk in flight before its first use, fp32 throughout; the splits of a
// (sequence, head) meet through global scratch and the last one to arrive merges them, in split
// order (no extra barrier, same bits every run).
//
// Grid barrier: one counter in global memory, zero at launch; arrival is a release add, the wait
// polls with relaxed loads and fences once the count is there.  Like every wait of this library it
// is bounded (~2 s) and polls the launch's abort word; a wait that gives up raises it, every later
// wait then returns at once, the kernel runs through its remaining control flow without hanging and
// the host reports B200P_E_TIMEOUT.  The launch is cooperative so that all CTAs are resident by
// construction.
//
// Measured (B200, 22 layers of hidden 2048 / ffn 5632, 2 sequences, 512 + 128 tokens): 0.87 to 1.14 ms
// per token, against 0.64 ms for the kernel-per-phase step replayed as a CUDA graph.  Timed per phase
// on one CTA, a layer is 38 to 48 us of which the five products take 12 to 14 (the weights' HBM time):
// each grid barrier costs 2 to 3 us, each all-to-all read of the activations after it (RMSNorm
// prologue, merge of the attention splits) 1 to 4 us -- they queue behind the weight prefetch that keeps
// the memory system full -- and attention 4 to 8 us.  Five dependent exchanges per layer at 4 to 6 us
// each leave no room under the kernel-per-phase step, whose kernel boundaries cost about the same and
// whose launches the graph and programmatic dependent launch already overlap.  An L2 prefetch running
// ahead of the ring's loads ("runtime_mega_ahead" stages, default 0) made it slower still: 1.03 ms per
// token without, 1.07 / 1.08 / 1.17 at 2 / 4 / 8 stages.  So this kernel is opt-in:
// b200p_set_tuning("runtime_mega", 1).
// ---------------------------------------------------------------------------
#pragma once
#include "skinny_gemm.cuh"

namespace b200p {

struct MegaLayer {
    const void *Wqkv, *bqkv, *Wo, *Wgu, *Wdown, *norm_attn, *norm_mlp;
};

constexpr int kMegaMaxSplits = 32;     // key splits of one (sequence, kv head)
constexpr int kMegaMaxGroup = 8;       // query heads per kv head
constexpr int kMegaMaxRows = 8;        // sequences (rows of X)
// floats between the partial states of p.part: D of o, then m, l, and padding to a 16-byte multiple
constexpr __host__ __device__ int kMegaPartPad(int D) { return D + 4; }

struct MegaParams {
    const MegaLayer* layers;
    int n_layers, B, H, F, D, nQH, nKVH, V, max_seq;
    const void *embed, *lm_head, *final_norm;
    float* hidden;                     // [B][H] fp32 residual stream
    void *qkv, *act;                   // [B][(nQH + 2 nKVH) D], [B][F] 16-bit
    float* logits;                     // [B][V]
    void *kcache, *vcache;             // [layer][B][nKVH][max_seq][D] 16-bit
    size_t layer_cache_elems;
    const float *cos_t, *sin_t;
    float* part;                       // [B nQH][kMegaMaxSplits][kMegaPartPad(D)] fp32: unnormalised o, then m, l
    const int* ids_in;                 // [B] token ids of the first step
    int* next_ids;                     // [B] the ids the last argmax chose
    int* tokens; int tokens_stride;    // [B][tokens_stride] output table or null
    int* state;                        // state[0] = position of the token being decoded, state[1] = output column
    unsigned long long* keys;          // [B] argmax merge keys, zero between uses
    unsigned* key_ticket;              // readers of keys, zero between uses
    unsigned* bar;                     // grid barrier counter, zero at launch
    int* status;                       // abort word of the launch
    int* sticky;
    int n_steps, want_argmax;
    int nstages, slab_cols, x_bytes, tab_bytes, stage_bytes;
    int ahead;                         // stages of L2 prefetch in front of the ring's loads (0: none)
    float eps, scale_log2;
};

// ---- the weight ring: skinny_stream_kernel's scheme as functions, so that one ring serves a sequence of products ----
// The ring of W stages in shared memory and one side's place in it.  A stage is stage_bytes long whatever the
// product's K (the rows inside it are slab * 2 + 16 bytes apart), so one ring serves a sequence of products.
constexpr int kSkinnyMaxStages = 8;
struct StreamRing {
    unsigned char* stages;
    int stage_bytes, nstages;
    uint64_t* full_bar;     // [nstages] 1 arrival (the producer's expect_tx) + the copies' bytes
    uint64_t* empty_bar;    // [nstages] kSkinnyWarps arrivals
};
struct RingPos { int stage = 0; uint32_t phase = 0; int uses = 0; };

__device__ __forceinline__ void stream_ring_init(const StreamRing& r) {          // one thread, before a CTA-wide barrier
    for (int s = 0; s < r.nstages; ++s) { dme::mbar_init(&r.full_bar[s], 1); dme::mbar_init(&r.empty_bar[s], kSkinnyWarps); }
    dme::mbar_init_fence();
}
__device__ __forceinline__ int stream_groups(int epi, int N) { return epi == EPI_SILU16 ? (N + 7) / 8 : (N + 15) / 16; }

// Row of W that line rr (0..15) of row group grp's stage holds: 16 consecutive rows; for EPI_SILU16 8 gate rows
// and the 8 up rows that go with them; for EPI_ROPE 8 rows d and the 8 rows d + D/2 of one head (ropeD = head size).
__device__ __forceinline__ size_t stream_row(int epi, int N, int ropeD, int grp, int rr) {
    if (epi == EPI_SILU16) return rr < 8 ? size_t(min(grp * 8 + rr, N - 1)) : size_t(N) + size_t(min(grp * 8 + rr - 8, N - 1));
    if (epi == EPI_ROPE) { const int cph = ropeD / 16; return size_t(grp / cph) * ropeD + size_t(grp % cph) * 8 + (rr & 7) + (rr >= 8 ? ropeD / 2 : 0); }
    return size_t(min(grp * 16 + rr, N - 1));
}
struct StreamNoAfter { __device__ __forceinline__ void operator()() const {} };

// Producer side of one product, called by all 32 lanes of the producer warp (they stay together; lane 0 waits
// for the stage to be free, announces the bytes and issues the 16 row copies): the row groups cta, cta + ncta,
// ... of W into the ring, slab by slab.  W is constant, so this runs as far ahead of the consumers as the ring
// allows.  false (in every lane): a wait gave up.  after(): called by all lanes once per stage issued.
// (Lanes 0..15 issuing one row copy each in the same instruction was measured slower, 0.721 vs 0.696 ms per token.)
template <typename T, int EPI, class After = StreamNoAfter>
__device__ __forceinline__ bool stream_produce(const SkinnyArgs& a, const StreamRing& r, RingPos& rp, int slab_cols,
                                               int* status, uint64_t pol, int cta, int ncta, After after = After()) {
    const int lane = threadIdx.x % 32;
    const int K = a.K;
    const int slab = K < slab_cols ? K : slab_cols;               // columns per stage
    const int nslab = (K + slab - 1) / slab;
    const int rowb = slab * 2 + 16;                               // bytes between rows of a stage
    const int ngroups = stream_groups(EPI, a.N);
    for (int grp = cta; grp < ngroups; grp += ncta) {
        for (int sl = 0; sl < nslab; ++sl) {
            if (rp.uses >= r.nstages) {
                int ok = 1;
                if (lane == 0) ok = dme::wait(&r.empty_bar[rp.stage], rp.phase ^ 1u, status) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
            }
            const int c0 = sl * slab, cols = min(slab, K - c0);
            unsigned char* dst = r.stages + size_t(rp.stage) * r.stage_bytes;
            if (lane == 0) {
                dme::mbar_arrive_expect_tx(&r.full_bar[rp.stage], uint32_t(16 * cols * 2));
                for (int rr = 0; rr < 16; ++rr) {
                    const size_t row = stream_row(EPI, a.N, a.rope.D, grp, rr);
                    dme::copy_tile_1d_stream(dst + size_t(rr) * rowb, static_cast<const char*>(a.W) + (row * size_t(K) + c0) * 2,
                                             uint32_t(cols * 2), &r.full_bar[rp.stage], pol);
                }
            }
            __syncwarp();
            ++rp.uses; if (++rp.stage == r.nstages) { rp.stage = 0; rp.phase ^= 1u; }
            after();
        }
    }
    return true;
}

// Consumer side of one product (the eight consumer warps, all 256 threads): X is in shared memory already
// (skinny_prologue).  ok is carried through: once a wait has given up the remaining stages are passed without
// arithmetic, every barrier is still reached.
template <typename T, int EPI, int MH>
__device__ __forceinline__ void stream_consume(const SkinnyArgs& a, const StreamRing& r, RingPos& rp, const T* xs, float (*red)[kSkinnyWarps][32][4 * MH],
                                               int slab_cols, int* status, int cta, int ncta, bool& ok, unsigned long long* best = nullptr) {
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = lane / 4, t4 = lane % 4;
    const int K = a.K, xstride = K + kSkinnyXPad;
    const int Mp = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : a.M <= 8 ? 8 : 16;
    const int slab = K < slab_cols ? K : slab_cols;
    const int nslab = (K + slab - 1) / slab;
    const int rowb = slab * 2 + 16;
    const int ngroups = stream_groups(EPI, a.N);
    const T* xrow = xs + size_t(g) * xstride + t4 * 16;
    int parity = 0;
    for (int grp = cta; grp < ngroups; grp += ncta, parity ^= 1) {
        // four accumulators per row half, one per 16-column step of a block: the products of a stage form
        // chains of nblk / 8 dependent MMAs instead of one chain through all of them
        float acc[MH][4][4];
        #pragma unroll
        for (int mh = 0; mh < MH; ++mh)
            #pragma unroll
            for (int s = 0; s < 4; ++s) { acc[mh][s][0] = acc[mh][s][1] = acc[mh][s][2] = acc[mh][s][3] = 0.f; }
        EpiAhead<MH> ahead;
        skinny_epilogue_fetch<T, EPI, 2, MH>(a, grp, threadIdx.x, ahead);
        for (int sl = 0; sl < nslab; ++sl) {
            if (ok && !dme::wait(&r.full_bar[rp.stage], rp.phase, status)) ok = false;
            const int c0 = sl * slab, cols = min(slab, K - c0);
            const int nblk = (cols + 63) / 64;
            const unsigned char* st = r.stages + size_t(rp.stage) * r.stage_bytes;
            if (ok && cols % (64 * kSkinnyWarps) == 0) {
                // whole blocks for every warp (the usual stage): nb blocks each, taken BB at a time with every
                // shared-memory load of the batch issued before its first MMA
                constexpr int BB = 4 / MH;
                const int nb = cols / (64 * kSkinnyWarps);
                const unsigned char* wrow_a = st + size_t(g) * rowb + t4 * 32;
                const unsigned char* wrow_b = st + size_t(g + 8) * rowb + t4 * 32;
                for (int b0 = 0; b0 < nb; b0 += BB) {                         // warp-uniform
                    uint4 wv[BB][4], xv[BB][MH][2];
                    #pragma unroll
                    for (int b = 0; b < BB; ++b) {
                        const int blk = warp + kSkinnyWarps * min(b0 + b, nb - 1);
                        const uint4* pa = reinterpret_cast<const uint4*>(wrow_a + blk * 128);
                        const uint4* pb = reinterpret_cast<const uint4*>(wrow_b + blk * 128);
                        wv[b][0] = pa[0]; wv[b][1] = pa[1]; wv[b][2] = pb[0]; wv[b][3] = pb[1];
                        #pragma unroll
                        for (int mh = 0; mh < MH; ++mh) {
                            xv[b][mh][0] = xv[b][mh][1] = make_uint4(0u, 0u, 0u, 0u);
                            if (g + 8 * mh < Mp) {
                                const uint4* xp = reinterpret_cast<const uint4*>(xrow + size_t(8 * mh) * xstride + c0 + blk * 64);
                                xv[b][mh][0] = xp[0]; xv[b][mh][1] = xp[1];
                            }
                        }
                    }
                    #pragma unroll
                    for (int b = 0; b < BB; ++b) {
                        if (b0 + b < nb) {
                            const uint32_t wA[8] = {wv[b][0].x, wv[b][0].y, wv[b][0].z, wv[b][0].w, wv[b][1].x, wv[b][1].y, wv[b][1].z, wv[b][1].w};
                            const uint32_t wB[8] = {wv[b][2].x, wv[b][2].y, wv[b][2].z, wv[b][2].w, wv[b][3].x, wv[b][3].y, wv[b][3].z, wv[b][3].w};
                            #pragma unroll
                            for (int mh = 0; mh < MH; ++mh) {
                                const uint32_t xw[8] = {xv[b][mh][0].x, xv[b][mh][0].y, xv[b][mh][0].z, xv[b][mh][0].w,
                                                        xv[b][mh][1].x, xv[b][mh][1].y, xv[b][mh][1].z, xv[b][mh][1].w};
                                #pragma unroll
                                for (int s = 0; s < 4; ++s) {
                                    const uint32_t af[4] = {wA[2 * s], wB[2 * s], wA[2 * s + 1], wB[2 * s + 1]};
                                    mma_16816<T>(acc[mh][s], af, xw[2 * s], xw[2 * s + 1]);
                                }
                            }
                        }
                    }
                }
            } else if (ok) {
                #pragma unroll 2
                for (int blk = warp; blk < nblk; blk += kSkinnyWarps) {       // warp-uniform
                    const bool live = blk * 64 + t4 * 16 < cols;
                    uint4 wa0 = make_uint4(0u, 0u, 0u, 0u), wa1 = wa0, wb0 = wa0, wb1 = wa0;
                    if (live) {
                        const uint4* pa = reinterpret_cast<const uint4*>(st + size_t(g) * rowb + (blk * 64 + t4 * 16) * 2);
                        const uint4* pb = reinterpret_cast<const uint4*>(st + size_t(g + 8) * rowb + (blk * 64 + t4 * 16) * 2);
                        wa0 = pa[0]; wa1 = pa[1]; wb0 = pb[0]; wb1 = pb[1];
                    }
                    const uint32_t wA[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
                    const uint32_t wB[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
                    #pragma unroll
                    for (int mh = 0; mh < MH; ++mh) {
                        uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
                        if (live && g + 8 * mh < Mp) {
                            const uint4* xp = reinterpret_cast<const uint4*>(xrow + size_t(8 * mh) * xstride + c0 + blk * 64);
                            xa = xp[0]; xb = xp[1];
                        }
                        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                        #pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            const uint32_t af[4] = {wA[2 * s], wB[2 * s], wA[2 * s + 1], wB[2 * s + 1]};
                            mma_16816<T>(acc[mh][s], af, xw[2 * s], xw[2 * s + 1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) dme::mbar_arrive(&r.empty_bar[rp.stage]);
            if (++rp.stage == r.nstages) { rp.stage = 0; rp.phase ^= 1u; }
        }
        #pragma unroll
        for (int mh = 0; mh < MH; ++mh)
            *reinterpret_cast<float4*>(&red[parity][warp][lane][4 * mh]) =
                make_float4((acc[mh][0][0] + acc[mh][1][0]) + (acc[mh][2][0] + acc[mh][3][0]), (acc[mh][0][1] + acc[mh][1][1]) + (acc[mh][2][1] + acc[mh][3][1]),
                            (acc[mh][0][2] + acc[mh][1][2]) + (acc[mh][2][2] + acc[mh][3][2]), (acc[mh][0][3] + acc[mh][1][3]) + (acc[mh][2][3] + acc[mh][3][3]));
        skinny_barrier();
        skinny_epilogue<T, EPI, 2, MH>(a, red[parity], grp, threadIdx.x, false, 0.f, best, &ahead);
    }
}

// ---- grid barrier over the consumer threads of all CTAs ---------------------------------------------
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u32(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
// Called by all kSkinnyThreads consumer threads.  `target` counts arrivals: it grows by the grid size per
// barrier.  Thread 0 arrives with a release (the CTA barrier before it orders the other threads' writes
// ahead of it), polls with relaxed loads and fences once the count is there.
__device__ __forceinline__ void mega_grid_barrier(unsigned* counter, unsigned& target, int* status) {
    target += gridDim.x;
    skinny_barrier();                                            // this CTA's writes of the phase are issued
    if (threadIdx.x == 0) {
        red_release_add_u32(counter, 1u);
        if (ld_relaxed_u32(counter) < target) {
            const uint64_t t0 = dme::global_timer_ns();
            for (;;) {
                bool there = false;
                #pragma unroll 1
                for (int i = 0; i < 64 && !there; ++i) there = ld_relaxed_u32(counter) >= target;
                if (there) break;
                if (*reinterpret_cast<volatile int*>(status) != 0) break;
                if (dme::global_timer_ns() - t0 > dme::kWaitLimitNs) { atomicExch(status, 1); break; }
            }
        }
        __threadfence();
    }
    skinny_barrier();
}

// ---- attention over the cache for the new token of every sequence ------------------------------------
// Partial softmax state of ONE query head in one warp: running maximum (log2 domain), sum, and the
// unnormalised output (DL columns per lane).  In memory: D floats of o, then m, then l.
template <int DL>
struct AttState {
    float m, l, o[DL];
};
template <int DL>
__device__ __forceinline__ void att_state_clear(AttState<DL>& s) {
    s.m = -INFINITY; s.l = 0.f;
    #pragma unroll
    for (int e = 0; e < DL; ++e) s.o[e] = 0.f;
}
template <int DL>
__device__ __forceinline__ void att_state_store(const AttState<DL>& s, float* slot, int lane) {
    constexpr int D = DL * 32;
    #pragma unroll
    for (int e = 0; e < DL; ++e) slot[lane * DL + e] = s.o[e];
    if (lane == 0) { slot[D] = s.m; slot[D + 1] = s.l; }
}
// s <- s merged with (m2, l2, o2)
template <int DL>
__device__ __forceinline__ void att_state_merge(AttState<DL>& s, float m2, float l2, const float (&o2)[DL]) {
    const float m = fmaxf(s.m, m2);
    const float a1 = s.m == -INFINITY ? 0.f : exp2f(s.m - m);
    const float a2 = m2 == -INFINITY ? 0.f : exp2f(m2 - m);
    s.l = s.l * a1 + l2 * a2;
    #pragma unroll
    for (int e = 0; e < DL; ++e) s.o[e] = s.o[e] * a1 + o2[e] * a2;
    s.m = m;
}

// How one layer's attention is cut up.  A unit is one (sequence, kv head, group of HG query heads, key split) and
// goes to one CTA; in the CTA warp w takes query head w % HG of the group and the 32-key chunks c with
// c % KS == w / HG (KS = 8 / HG).  HG: the fewest heads per CTA (1, 2 or 4, dividing the heads per kv head) that
// still gives every CTA at most one unit.  Key splits only when a warp would otherwise take more than 4 chunks,
// and then as many as keep one unit per CTA: every split is another partial state that EVERY CTA reads back in
// the output projection's prologue.
struct MegaAttPlan { int hg, nsplit, per; };
__device__ __forceinline__ MegaAttPlan mega_att_plan(const MegaParams& p, int n, int ncta) {
    const int G = p.nQH / p.nKVH;
    MegaAttPlan pl;
    pl.hg = G % 4 == 0 ? 4 : G % 2 == 0 ? 2 : 1;
    if (pl.hg > 1 && p.B * p.nKVH * (G / (pl.hg / 2)) <= ncta) pl.hg /= 2;
    const int KS = kSkinnyWarps / pl.hg, base_units = p.B * p.nKVH * (G / pl.hg);
    const int chunks = (n + 31) / 32;
    int smax = ncta / base_units;
    smax = smax < 1 ? 1 : smax > kMegaMaxSplits ? kMegaMaxSplits : smax;
    int cpu = (chunks + smax - 1) / smax;                        // chunks per unit
    cpu = cpu < 2 * KS ? 2 * KS : (cpu + KS - 1) / KS * KS;
    pl.nsplit = (chunks + cpu - 1) / cpu;
    pl.per = cpu * 32;
    return pl;
}

// One layer's attention: every (sequence, head, split) leaves its partial state in p.part; the output
// projection's prologue merges them.  n = keys in the cache (the new token's included).  scratch: shared
// memory, kSkinnyWarps * (2 D + 2) floats.  All kSkinnyThreads consumer threads call it; the warps of one head
// meet at a CTA barrier when KS > 1.
template <typename T, int HG, int DL>
__device__ __forceinline__ void mega_attention(const MegaParams& p, const MegaAttPlan& pl, int li, int n, float* scratch) {
    constexpr int D = DL * 32, KS = kSkinnyWarps / HG;
    const int G = p.nQH / p.nKVH, NHG = G / HG;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = warp % HG, sub = warp / HG;
    float* qs = scratch + warp * D;                              // this warp's query row
    float* slots = scratch + kSkinnyWarps * D;                   // [warp][D + 2]
    const int units = p.B * p.nKVH * NHG * pl.nsplit;
    const int W = (p.nQH + 2 * p.nKVH) * D;
    const T* kc = static_cast<const T*>(p.kcache) + size_t(li) * p.layer_cache_elems;
    const T* vc = static_cast<const T*>(p.vcache) + size_t(li) * p.layer_cache_elems;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int sp = u % pl.nsplit, bu = u / pl.nsplit;
        const int hq = bu % NHG, bk = bu / NHG;                  // bk = b * nKVH + kvh
        const int kvh = bk % p.nKVH, b = bk / p.nKVH;
        const int h = kvh * G + hq * HG + g;                     // query head
        const int k0 = sp * pl.per, k1 = min(n, k0 + pl.per);
        {   // q of this warp's head, as fp32, for broadcast reads
            const T* q = static_cast<const T*>(p.qkv) + size_t(b) * W + size_t(h) * D + lane * DL;
            #pragma unroll
            for (int e = 0; e < DL; ++e) qs[lane * DL + e] = to_float(q[e]);
            __syncwarp();
        }
        AttState<DL> st;
        att_state_clear<DL>(st);
        const T* kbase = kc + size_t(bk) * p.max_seq * D;
        const T* vbase = vc + size_t(bk) * p.max_seq * D;
        for (int kb = k0 + 32 * sub; kb < k1; kb += 32 * KS) {   // warp-uniform
            const int key = kb + lane, cnt = min(32, k1 - kb);
            const bool valid = key < k1;
            // every load of the chunk is issued before the first use: K row of this lane's key, and for each of
            // the chunk's keys this lane's DL columns of V
            uint4 kv[D / 8];
            const uint4* krow = reinterpret_cast<const uint4*>(kbase + size_t(valid ? key : k1 - 1) * D);
            #pragma unroll
            for (int c = 0; c < D / 8; ++c) kv[c] = krow[c];
            constexpr int VB = DL == 2 ? 32 : 16;                 // keys of V held in registers at a time
            float vv[VB][DL];
            auto load_v = [&](int j0) {
                #pragma unroll
                for (int j = 0; j < VB; ++j) {
                    const T* vrow = vbase + size_t(kb + min(j0 + j, cnt - 1)) * D + lane * DL;
                    if (DL == 2) {
                        const uint32_t r = *reinterpret_cast<const uint32_t*>(vrow);
                        const T* e2 = reinterpret_cast<const T*>(&r);
                        vv[j][0] = to_float(e2[0]); vv[j][1] = to_float(e2[1]);
                    } else {
                        const uint2 r = *reinterpret_cast<const uint2*>(vrow);
                        const T* e4 = reinterpret_cast<const T*>(&r);
                        #pragma unroll
                        for (int e = 0; e < DL; ++e) vv[j][e] = to_float(e4[e]);
                    }
                }
            };
            load_v(0);
            // ---- score of this lane's key ----
            float s0 = 0.f, s1 = 0.f;
            #pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const T* ke = reinterpret_cast<const T*>(&kv[c]);
                const float4 qa = *reinterpret_cast<const float4*>(qs + 8 * c);
                const float4 qb = *reinterpret_cast<const float4*>(qs + 8 * c + 4);
                s0 += to_float(ke[0]) * qa.x + to_float(ke[1]) * qa.y + to_float(ke[2]) * qa.z + to_float(ke[3]) * qa.w;
                s1 += to_float(ke[4]) * qb.x + to_float(ke[5]) * qb.y + to_float(ke[6]) * qb.z + to_float(ke[7]) * qb.w;
            }
            // ---- online softmax over the chunk ----
            const float sc = valid ? (s0 + s1) * p.scale_log2 : -INFINITY;
            const float m_new = fmaxf(st.m, wave::dpp::reduce_max(sc));      // finite: the chunk has a valid key
            const float pe = valid ? exp2f(sc - m_new) : 0.f;
            const float alpha = st.m == -INFINITY ? 0.f : exp2f(st.m - m_new);
            st.l = st.l * alpha + wave::dpp::reduce_sum(pe);
            st.m = m_new;
            // ---- o = o * alpha + p . V ----
            float o2[DL][2];
            #pragma unroll
            for (int e = 0; e < DL; ++e) { o2[e][0] = st.o[e] * alpha; o2[e][1] = 0.f; }
            #pragma unroll
            for (int j0 = 0; j0 < 32; j0 += VB) {
                if (j0 > 0) load_v(j0);
                #pragma unroll
                for (int j = 0; j < VB; ++j) {
                    const float pj = __shfl_sync(0xffffffffu, pe, j0 + j);   // 0 for the keys past the end
                    #pragma unroll
                    for (int e = 0; e < DL; ++e) o2[e][j & 1] += pj * vv[j][e];
                }
            }
            #pragma unroll
            for (int e = 0; e < DL; ++e) st.o[e] = o2[e][0] + o2[e][1];
        }
        __syncwarp();                                            // qs is free for the next unit
        if (KS > 1) {
            // the KS warps of one head meet in the head's first warp
            if (sub > 0) att_state_store<DL>(st, slots + warp * (D + 2), lane);
            skinny_barrier();
            if (sub == 0) {
                #pragma unroll 1
                for (int s2 = 1; s2 < KS; ++s2) {
                    const float* slot = slots + (s2 * HG + g) * (D + 2);
                    float o2[DL];
                    #pragma unroll
                    for (int e = 0; e < DL; ++e) o2[e] = slot[lane * DL + e];
                    att_state_merge<DL>(st, slot[D], slot[D + 1], o2);
                }
            }
            skinny_barrier();
        }
        if (sub == 0) att_state_store<DL>(st, p.part + (size_t(b * p.nQH + h) * kMegaMaxSplits + sp) * kMegaPartPad(D), lane);
    }
}

// Prologue of the output projection: X[b][h D + d] = the splits of (b, h) merged in split order and normalised,
// as 16-bit, straight into shared memory (forward.hpp's attention output, never stored in global memory).
// A thread takes 16 columns of one (sequence, head); the loads of up to 6 splits are in flight together.
template <typename T, int DL>
__device__ __forceinline__ void mega_attn_merge_prologue(const MegaParams& p, int nsplit, T* xs, int xstride, int Mp) {
    constexpr int D = DL * 32, CH = D / 16, MS = 6;
    const int items = p.B * p.nQH * CH;
    for (int it = threadIdx.x; it < items; it += kSkinnyThreads) {
        const int ch = it % CH, bh = it / CH;
        const int h = bh % p.nQH, b = bh / p.nQH;
        const float* base = p.part + size_t(bh) * kMegaMaxSplits * kMegaPartPad(D);
        float m = -INFINITY, l = 0.f, o[16];
        #pragma unroll
        for (int e = 0; e < 16; ++e) o[e] = 0.f;
        for (int s0 = 0; s0 < nsplit; s0 += MS) {
            float4 v[MS][4]; float m2[MS], l2[MS];
            #pragma unroll
            for (int s = 0; s < MS; ++s) {
                const bool live = s0 + s < nsplit;
                const float* slot = base + size_t(live ? s0 + s : s0) * kMegaPartPad(D);     // 16-byte aligned
                #pragma unroll
                for (int q = 0; q < 4; ++q) v[s][q] = *reinterpret_cast<const float4*>(slot + ch * 16 + 4 * q);
                m2[s] = live ? slot[D] : -INFINITY; l2[s] = live ? slot[D + 1] : 0.f;
            }
            #pragma unroll
            for (int s = 0; s < MS; ++s) {
                const float mn = fmaxf(m, m2[s]);
                const float a1 = m == -INFINITY ? 0.f : exp2f(m - mn);
                const float a2 = m2[s] == -INFINITY ? 0.f : exp2f(m2[s] - mn);
                l = l * a1 + l2[s] * a2;
                const float* vs = reinterpret_cast<const float*>(&v[s][0]);
                #pragma unroll
                for (int e = 0; e < 16; ++e) o[e] = o[e] * a1 + vs[e] * a2;
                m = mn;
            }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        uint4 w0, w1;
        w0.x = pack2<T>(o[0] * inv, o[1] * inv);   w0.y = pack2<T>(o[2] * inv, o[3] * inv);
        w0.z = pack2<T>(o[4] * inv, o[5] * inv);   w0.w = pack2<T>(o[6] * inv, o[7] * inv);
        w1.x = pack2<T>(o[8] * inv, o[9] * inv);   w1.y = pack2<T>(o[10] * inv, o[11] * inv);
        w1.z = pack2<T>(o[12] * inv, o[13] * inv); w1.w = pack2<T>(o[14] * inv, o[15] * inv);
        uint4* dst = reinterpret_cast<uint4*>(xs + size_t(b) * xstride + h * D + ch * 16);
        dst[0] = w0; dst[1] = w1;
    }
    const int K = p.nQH * D;
    for (int i = threadIdx.x; i < (Mp - p.B) * (K / 8); i += kSkinnyThreads)             // rows past the batch are zero
        *reinterpret_cast<uint4*>(xs + size_t(p.B + i / (K / 8)) * xstride + (i % (K / 8)) * 8) = make_uint4(0u, 0u, 0u, 0u);
    skinny_barrier();
}

// ---- the weight stream of one CTA as a sequence of stages ---------------------------------------------
// kind: 0 Q/K/V, 1 output, 2 gate/up, 3 down projection of layer li; 4 lm_head (after the last layer).
struct MegaCursor { int step, li, kind, grp, sl; };

__device__ __forceinline__ void mega_kind_shape(const MegaParams& p, int kind, int& N, int& K, int& epi) {
    switch (kind) {
        case 0:  N = (p.nQH + 2 * p.nKVH) * p.D; K = p.H; epi = EPI_ROPE; break;
        case 1:  N = p.H; K = p.nQH * p.D; epi = EPI_ACC32; break;
        case 2:  N = p.F; K = p.H; epi = EPI_SILU16; break;
        case 3:  N = p.H; K = p.F; epi = EPI_ACC32; break;
        default: N = p.V; K = p.H; epi = EPI_STORE32; break;
    }
}
__device__ __forceinline__ const void* mega_kind_weights(const MegaParams& p, const MegaLayer* layers, int li, int kind) {
    switch (kind) {
        case 0:  return layers[li].Wqkv;
        case 1:  return layers[li].Wo;
        case 2:  return layers[li].Wgu;
        case 3:  return layers[li].Wdown;
        default: return p.lm_head;
    }
}
// Moves c to the next product in which this CTA has a row group, from (and including) the product c names, when
// c.grp is past its groups.  false: the launch's stream is over.
__device__ __forceinline__ bool mega_cursor_settle(const MegaParams& p, MegaCursor& c, int cta) {
    for (;;) {
        if (c.step >= p.n_steps) return false;
        int N, K, epi;
        mega_kind_shape(p, c.kind, N, K, epi);
        if (c.grp < stream_groups(epi, N)) return true;
        c.grp = cta; c.sl = 0;
        if (c.kind == 4) { c.kind = 0; c.li = 0; ++c.step; }
        else if (c.kind == 3) { if (++c.li == p.n_layers) c.kind = 4; else c.kind = 0; }
        else ++c.kind;
    }
}
// L2 prefetch of the stage c names, then on to the next stage; called by all lanes of the producer warp, lanes
// 16..31 issue (one row each, or one run of 8 contiguous rows each).  false: nothing left.
__device__ __forceinline__ bool mega_prefetch_stage(const MegaParams& p, const MegaLayer* layers, MegaCursor& c, int cta, int ncta) {
    if (!mega_cursor_settle(p, c, cta)) return false;
    const int lane = threadIdx.x % 32;
    int N, K, epi;
    mega_kind_shape(p, c.kind, N, K, epi);
    const int slab = K < p.slab_cols ? K : p.slab_cols, nslab = (K + slab - 1) / slab;
    const int c0 = c.sl * slab, cols = min(slab, K - c0);
    const char* W = static_cast<const char*>(mega_kind_weights(p, layers, c.li, c.kind));
    if (nslab == 1) {
        if (lane == 16 || lane == 17) {                          // whole rows: a run of 8 consecutive rows is contiguous
            const int rr = (lane - 16) * 8;
            const size_t r0 = stream_row(epi, N, p.D, c.grp, rr), r7 = stream_row(epi, N, p.D, c.grp, rr + 7);
            dme::prefetch_l2(W + r0 * size_t(K) * 2, uint32_t((r7 - r0 + 1) * size_t(K) * 2));
        }
    } else if (lane >= 16) {
        dme::prefetch_l2(W + (stream_row(epi, N, p.D, c.grp, lane - 16) * size_t(K) + c0) * 2, uint32_t(cols * 2));
    }
    if (++c.sl == nslab) { c.sl = 0; c.grp += ncta; }
    return true;
}

// ---- the kernel -------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ SkinnyArgs mega_args_qkv(const MegaParams& p, const MegaLayer& L, int li, int pos, const int* ids) {
    SkinnyArgs a{};
    const int W = (p.nQH + 2 * p.nKVH) * p.D;
    a.M = p.B; a.eps = p.eps; a.W = L.Wqkv; a.X32 = p.hidden; a.norm_w = L.norm_attn; a.out = p.qkv; a.N = W; a.K = p.H; a.ldo = W;
    if (li == 0) { a.Xemb = p.embed; a.Xids = ids; }
    a.rope.bias = L.bqkv; a.rope.cos_t = p.cos_t; a.rope.sin_t = p.sin_t;
    a.rope.kcache = static_cast<T*>(p.kcache) + size_t(li) * p.layer_cache_elems;
    a.rope.vcache = static_cast<T*>(p.vcache) + size_t(li) * p.layer_cache_elems;
    a.rope.pos_dev = nullptr; a.rope.pos0 = pos; a.rope.nQH = p.nQH; a.rope.nKVH = p.nKVH; a.rope.D = p.D; a.rope.max_seq = p.max_seq;
    return a;
}
__device__ __forceinline__ SkinnyArgs mega_args_o(const MegaParams& p, const MegaLayer& L) {
    SkinnyArgs a{};
    const int qd = p.nQH * p.D;
    a.M = p.B; a.eps = p.eps; a.W = L.Wo; a.out = p.hidden; a.N = p.H; a.K = qd; a.ldo = p.H;     // X: mega_attn_merge_prologue
    return a;
}
__device__ __forceinline__ SkinnyArgs mega_args_gu(const MegaParams& p, const MegaLayer& L) {
    SkinnyArgs a{};
    a.M = p.B; a.eps = p.eps; a.W = L.Wgu; a.X32 = p.hidden; a.norm_w = L.norm_mlp; a.out = p.act; a.N = p.F; a.K = p.H; a.ldo = p.F;
    return a;
}
__device__ __forceinline__ SkinnyArgs mega_args_down(const MegaParams& p, const MegaLayer& L) {
    SkinnyArgs a{};
    a.M = p.B; a.eps = p.eps; a.W = L.Wdown; a.X16 = p.act; a.ldx = p.F; a.out = p.hidden; a.N = p.H; a.K = p.F; a.ldo = p.H;
    return a;
}
__device__ __forceinline__ SkinnyArgs mega_args_head(const MegaParams& p) {
    SkinnyArgs a{};
    a.M = p.B; a.eps = p.eps; a.W = p.lm_head; a.X32 = p.hidden; a.norm_w = p.final_norm; a.out = p.logits; a.N = p.V; a.K = p.H; a.ldo = p.V;
    return a;
}

template <typename T, int DL>
__global__ void __launch_bounds__(kSkinnyStreamThreads, 1)
decode_mega_kernel(const MegaParams p) {
    extern __shared__ __align__(128) unsigned char skinny_smem[];
    __shared__ float red[2][kSkinnyWarps][32][4];
    __shared__ __align__(16) float part_ss[kSkinnyWarps];
    __shared__ uint64_t bars[2 * kSkinnyMaxStages];
    __shared__ unsigned long long s_keys[kMegaMaxRows];
    __shared__ int s_ids[kMegaMaxRows];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int Mp = p.B <= 1 ? 1 : p.B <= 2 ? 2 : p.B <= 4 ? 4 : 8;
    T* xs = reinterpret_cast<T*>(skinny_smem);
    MegaLayer* layers = reinterpret_cast<MegaLayer*>(skinny_smem + p.x_bytes);       // the layer table, copied once
    StreamRing ring{skinny_smem + p.x_bytes + p.tab_bytes, p.stage_bytes, p.nstages, bars, bars + kSkinnyMaxStages};
    if (threadIdx.x == 0) stream_ring_init(ring);
    if (threadIdx.x < kMegaMaxRows) {
        s_keys[threadIdx.x] = 0ull;
        s_ids[threadIdx.x] = threadIdx.x < p.B ? p.ids_in[threadIdx.x] : 0;
    }
    for (int i = threadIdx.x; i < p.n_layers * int(sizeof(MegaLayer) / sizeof(void*)); i += blockDim.x)
        reinterpret_cast<const void**>(layers)[i] = reinterpret_cast<const void* const*>(p.layers)[i];
    __syncthreads();
    const int cta = blockIdx.x, ncta = gridDim.x;
    RingPos rp;

    if (warp == kSkinnyWarps) {
        // ---- producer warp: the weights of n_steps steps, in the consumers' order; an L2 prefetch runs p.ahead stages in front ----
        const uint64_t pol = dme::policy_evict_first();
        MegaCursor pc{0, 0, 0, cta, 0};
        bool more = true;
        for (int i = 0; i < p.ahead && more; ++i) more = mega_prefetch_stage(p, layers, pc, cta, ncta);
        auto after = [&]() { if (more && p.ahead > 0) more = mega_prefetch_stage(p, layers, pc, cta, ncta); };
        bool ok = true;
        for (int step = 0; step < p.n_steps && ok; ++step) {
            for (int li = 0; li < p.n_layers && ok; ++li) {
                const MegaLayer& L = layers[li];
                SkinnyArgs a = mega_args_qkv<T>(p, L, li, 0, nullptr);
                ok = stream_produce<T, EPI_ROPE>(a, ring, rp, p.slab_cols, p.status, pol, cta, ncta, after);
                a = mega_args_o(p, L);
                ok = ok && stream_produce<T, EPI_ACC32>(a, ring, rp, p.slab_cols, p.status, pol, cta, ncta, after);
                a = mega_args_gu(p, L);
                ok = ok && stream_produce<T, EPI_SILU16>(a, ring, rp, p.slab_cols, p.status, pol, cta, ncta, after);
                a = mega_args_down(p, L);
                ok = ok && stream_produce<T, EPI_ACC32>(a, ring, rp, p.slab_cols, p.status, pol, cta, ncta, after);
            }
            SkinnyArgs a = mega_args_head(p);
            ok = ok && stream_produce<T, EPI_STORE32>(a, ring, rp, p.slab_cols, p.status, pol, cta, ncta, after);
        }
        if (!ok && lane == 0) atomicExch(p.sticky, 1);
        return;
    }

    // ---- consumers ----
    bool ok = true;
    unsigned target = 0;
    const int pos0 = p.state[0], col0 = p.state[1];
    for (int step = 0; step < p.n_steps; ++step) {
        const int pos = min(pos0 + step, p.max_seq - 1), col = col0 + step;
        for (int li = 0; li < p.n_layers; ++li) {
            const MegaLayer& L = layers[li];
            {   // Q/K/V projection of the normalised hidden state; bias, RoPE, cache scatter
                const SkinnyArgs a = mega_args_qkv<T>(p, L, li, pos, s_ids);
                if (li == 0) {
                    // forward.hpp:174-183: the residual stream starts as the embedding rows, each CTA writing its share
                    const int total = p.B * p.H;
                    for (int i = cta * kSkinnyThreads + threadIdx.x; i < total; i += ncta * kSkinnyThreads) {
                        const int m = i / p.H, k = i % p.H;
                        p.hidden[i] = to_float(static_cast<const T*>(p.embed)[size_t(s_ids[m]) * p.H + k]);
                    }
                }
                if (li == 0) skinny_prologue<T, PRO_RMSNORM, true>(a, xs, part_ss, Mp, warp, lane);
                else         skinny_prologue<T, PRO_RMSNORM>(a, xs, part_ss, Mp, warp, lane);
                stream_consume<T, EPI_ROPE, 1>(a, ring, rp, xs, red, p.slab_cols, p.status, cta, ncta, ok);
            }
            mega_grid_barrier(p.bar, target, p.status);
            const MegaAttPlan att = mega_att_plan(p, pos + 1, ncta);
            if (att.hg == 1)      mega_attention<T, 1, DL>(p, att, li, pos + 1, reinterpret_cast<float*>(skinny_smem));
            else if (att.hg == 2) mega_attention<T, 2, DL>(p, att, li, pos + 1, reinterpret_cast<float*>(skinny_smem));
            else                  mega_attention<T, 4, DL>(p, att, li, pos + 1, reinterpret_cast<float*>(skinny_smem));
            mega_grid_barrier(p.bar, target, p.status);
            {   // output projection of the merged attention output, accumulated into the residual stream
                const SkinnyArgs a = mega_args_o(p, L);
                mega_attn_merge_prologue<T, DL>(p, att.nsplit, xs, a.K + kSkinnyXPad, Mp);
                stream_consume<T, EPI_ACC32, 1>(a, ring, rp, xs, red, p.slab_cols, p.status, cta, ncta, ok);
            }
            mega_grid_barrier(p.bar, target, p.status);
            {   // gate / up projection of the normalised hidden state, SiLU(gate) * up
                const SkinnyArgs a = mega_args_gu(p, L);
                skinny_prologue<T, PRO_RMSNORM>(a, xs, part_ss, Mp, warp, lane);
                stream_consume<T, EPI_SILU16, 1>(a, ring, rp, xs, red, p.slab_cols, p.status, cta, ncta, ok);
            }
            mega_grid_barrier(p.bar, target, p.status);
            {   // down projection, accumulated into the residual stream
                const SkinnyArgs a = mega_args_down(p, L);
                skinny_prologue<T, PRO_PLAIN>(a, xs, part_ss, Mp, warp, lane);
                stream_consume<T, EPI_ACC32, 1>(a, ring, rp, xs, red, p.slab_cols, p.status, cta, ncta, ok);
            }
            mega_grid_barrier(p.bar, target, p.status);
        }
        {   // final norm, lm_head, and the argmax key of this CTA's columns
            const SkinnyArgs a = mega_args_head(p);
            unsigned long long best[1] = {0ull};
            skinny_prologue<T, PRO_RMSNORM>(a, xs, part_ss, Mp, warp, lane);
            stream_consume<T, EPI_STORE32_BEST, 1>(a, ring, rp, xs, red, p.slab_cols, p.status, cta, ncta, ok, best);
            if (p.want_argmax) {
                if (threadIdx.x < 128) {
                    const int l = threadIdx.x % 32, c = threadIdx.x / 32;
                    const int m = 2 * (l % 4) + (c & 1);
                    if (m < p.B && best[0]) atomicMax(&s_keys[m], best[0]);
                }
                skinny_barrier();
                if (threadIdx.x < p.B && s_keys[threadIdx.x]) atomicMax(&p.keys[threadIdx.x], s_keys[threadIdx.x]);
            }
        }
        mega_grid_barrier(p.bar, target, p.status);
        if (p.want_argmax) {
            // every CTA reads the chosen ids (they are the next step's input); the last reader clears the keys
            if (threadIdx.x < p.B) {
                const unsigned long long k = __ldcg(&p.keys[threadIdx.x]);
                const int id = int(0xffffffffu - unsigned(k & 0xffffffffull));
                s_ids[threadIdx.x] = id >= 0 && id < p.V ? id : 0;
                s_keys[threadIdx.x] = 0ull;
                if (cta == 0) {
                    p.next_ids[threadIdx.x] = id;
                    if (p.tokens && col < p.tokens_stride) p.tokens[size_t(threadIdx.x) * p.tokens_stride + col] = id;
                }
            }
            skinny_barrier();
            if (threadIdx.x == 0) {
                __threadfence();
                if (atomicAdd(p.key_ticket, 1u) == unsigned(ncta - 1)) {
                    for (int m = 0; m < p.B; ++m) p.keys[m] = 0ull;
                    *p.key_ticket = 0u;
                    __threadfence();
                }
            }
        }
    }
    if (cta == 0 && threadIdx.x == 0) { p.state[0] = pos0 + p.n_steps; p.state[1] = col0 + p.n_steps; }
    if (!ok && lane == 0) atomicExch(p.sticky, 1);
}

} // namespace b200p
