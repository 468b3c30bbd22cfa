// ---------------------------------------------------------------------------
// prefill.cu -- FA2 prefill attention on the 5th-generation tensor cores.
//
// Stands in for fa_multiwave_kernel<D,W> behind cdna3::attn::prefill
// (cdna3-prims/include/cdna3/detail/fa_prefill_kernel.hpp:43-177,
//  cdna3-prims/include/cdna3/attention.hpp:86-109) and for the MFMA step of the
// reference's build order (research/flash-attention-mi300x/fa_mfma2.hip:63-217).
// Same semantics: GQA (kvhead = qhead / group), causal mask "key > query is
// masked", KV tiles past the diagonal skipped, scale 1/sqrt(D), fp32 softmax,
// 16-bit output, O / l with l > 0 guarded.
//
// The reference keeps S, P and O in LDS, one 16-row block per wave, and rescales
// O serially on lane 0.  Here a work item is 256 query rows of one (batch, head)
// as two 128-row tiles; one persistent CTA per SM (it takes all of the SM's shared
// and tensor memory) draws items from a device-wide counter, heaviest query blocks
// of a head first, and is warp-specialised:
//   warp 9        TMA producer: Q once, then K_j / V_j tiles ([128][D], 64-element
//                 boxes, 128-byte swizzle) into two mbarrier rings;
//   warp 8        MMA issuer (one thread): S_t = Q_t.K_j^T and O_t += P_t.V_j as
//                 tcgen05.mma with the accumulators in tensor memory; P_t is read
//                 straight from tensor memory (it overwrites S_t as 16-bit pairs);
//                 issue order PV_j^0, QK_{j+1}^0, PV_j^1, QK_{j+1}^1 so that one
//                 tile's softmax overlaps the other tile's matrix work;
//   warps 0-3/4-7 softmax for tile 0 / 1: one query row per thread (tcgen05.ld
//                 32x32b gives a thread its whole row, so row max and row sum need
//                 no cross-lane step at all), exp2 with the scale folded in, lazy
//                 rescaling of O (only when the running max grew by more than 2^8),
//                 final O / l and the store (swizzled staging tile + TMA store).
// All barrier phases run on from one item to the next, so the next item's Q, K_0 and
// first Q.K^T are in flight while the softmax warps normalise and store the previous
// item's O (measured per item: 18.5k cycles of fill, drain and launch with one CTA per
// item, 16.5k with persistent CTAs, on top of 3.5k per 128-key step).
// TMEM columns: S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [384,384+D).
// Compute-bound on the bf16 tensor pipe; K/V are re-read from L2 by the CTAs of
// the same (batch, kv head), which are adjacent in the grid.
//
// Every mbarrier wait is bounded; a wait that gives up raises the library's
// device status word and the CTA drains and frees its tensor memory.
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "attn_common.cuh"
#include "dme/dme_tma.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"
#include "mma_sync.cuh"

namespace b200p {

namespace {

constexpr int kBM = 128;                 // query rows per tile
constexpr int kBN = 128;                 // keys per tile
// RS = threads per query row in the softmax (1 in every instantiation).  Warps 0 .. 8*RS-1 are softmax
// warps (tile, lane quarter), the next warpgroup holds the MMA and the TMA warp.
constexpr int prefill_threads(int RS) { return (8 * RS + 4) * 32; }
constexpr float kLazyRescale = 8.0f;     // log2 units
// P is handed to the MMA warp in two parts: the first kFirstChunks 32-key chunks of a tile as soon as they are stored,
// then the rest; only the second part's P.V stands between the end of the softmax and the next Q.K^T.
// (Measured: 1, 2 or 3 chunks first make no difference beyond run-to-run noise.)
constexpr int kFirstChunks = 2;
// The debug instantiation (DBG, used by b200p_attn_prefill_debug only) writes the raw scores of the first
// tile to the debug buffer; the production instantiation does not carry that code.

template <int D> struct PrefillShape {
    static constexpr int SUB = D / 64;                         // 64-element boxes per row
    static constexpr int SUB_BYTES = kBM * 128;                // [128 rows][128 B]
    static constexpr int TILE_BYTES = SUB * SUB_BYTES;         // one Q / K / V tile
    static constexpr int KSTAGES = (D == 128) ? 2 : 4;
    static constexpr int VSTAGES = (D == 128) ? 2 : 4;
    static constexpr int OFF_Q = 0;
    static constexpr int OFF_K = 2 * TILE_BYTES;
    static constexpr int OFF_V = OFF_K + KSTAGES * TILE_BYTES;
    static constexpr int OFF_OUT = OFF_V + VSTAGES * TILE_BYTES;   // one [128 rows][128 B] staging tile per query tile (epilogue)
    static constexpr int OFF_BAR = OFF_OUT + 2 * SUB_BYTES;
    static constexpr int SMEM_BYTES = OFF_BAR + 1024;
};

struct PrefillParams {
    float* debug_s;            // optional: raw S of tile (0,0) of CTA (0,0,0), [128][128] fp32
    int* status;               // this launch's abort word: raised by a wait that gave up, polled by all its waits
    int* sticky;               // the library's sticky status word, raised at exit by a CTA that saw a failed wait
    int* work_counter;         // zero at launch: the CTAs draw the ids of their later work items from it
    int seqQ, seqK, nQH, nKVH, group, batch, causal;
    float scale_log2;
};

template <typename T> struct Fmt;
template <> struct Fmt<__half>        { static constexpr int id = 0; };
template <> struct Fmt<__nv_bfloat16> { static constexpr int id = 1; };

// One work item: 256 query rows (two 128-row tiles) of one (batch, head).  Items are numbered like the
// blocks of a (query block, head, batch) grid with the query block fastest and the heaviest (latest)
// query block first, so that items in flight at the same time share their (batch, KV head) in L2.
struct PrefillItem {
    int head, b, kvh, nmax;
    int q0[2], n[2];
};
__device__ __forceinline__ PrefillItem prefill_item(const PrefillParams& p, int id) {
    PrefillItem w;
    const int nqb = (p.seqQ + 2 * kBM - 1) / (2 * kBM);
    const int qb = nqb - 1 - id % nqb;
    w.head = (id / nqb) % p.nQH;
    w.b = id / (nqb * p.nQH);
    w.kvh = w.head / p.group;
    const int ntk = (p.seqK + kBN - 1) / kBN;
    #pragma unroll
    for (int t = 0; t < 2; ++t) {
        w.q0[t] = qb * 2 * kBM + t * kBM;
        if (w.q0[t] >= p.seqQ) w.n[t] = 0;
        else if (p.causal) w.n[t] = min(ntk, (w.q0[t] + kBM - 1) / kBN + 1);
        else w.n[t] = ntk;
    }
    w.nmax = max(w.n[0], w.n[1]);
    return w;
}

template <typename T, int D, int RS, bool DBG>
__global__ void __launch_bounds__(prefill_threads(RS), 1)
prefill_tc_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap mapQ,
                  const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                  const __grid_constant__ CUtensorMap mapO) {
    using Sh = PrefillShape<D>;
    constexpr int KST = Sh::KSTAGES, VST = Sh::VSTAGES;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Sh::OFF_BAR);
    uint64_t* q_full  = bars;                 // [1]
    uint64_t* k_full  = bars + 1;             // [KST]
    uint64_t* k_empty = k_full + KST;
    uint64_t* v_full  = k_empty + KST;        // [VST]
    uint64_t* v_empty = v_full + VST;
    uint64_t* s_full  = v_empty + VST;        // [2]
    uint64_t* p_half  = s_full + 2;           // [2 tiles][2 halves of P]
    uint64_t* o_done  = p_half + 4;           // [2]
    uint64_t* q_empty = o_done + 2;           // [1] the item's last Q.K^T has completed: Q may be overwritten
    uint64_t* o_free  = q_empty + 1;          // [2] the tile's epilogue has read O out of tensor memory
    uint64_t* item_full  = o_free + 2;        // [2] ring of work-item ids
    uint64_t* item_empty = item_full + 2;     // [2]
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_failed;
    __shared__ int s_item[2];

    constexpr int kMmaWarp = 8 * RS, kTmaWarp = 8 * RS + 1;
    constexpr int kItemReaders = 2 * kBM + 1;                  // every softmax thread + the MMA thread
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int nqb = (p.seqQ + 2 * kBM - 1) / (2 * kBM);
    const int total_items = nqb * p.nQH * p.batch;

    if (threadIdx.x == 0) {
        s_failed = 0;
        dme::mbar_init(q_full, 1); dme::mbar_init(q_empty, 1);
        for (int s = 0; s < KST; ++s) { dme::mbar_init(&k_full[s], 1); dme::mbar_init(&k_empty[s], 1); }
        for (int s = 0; s < VST; ++s) { dme::mbar_init(&v_full[s], 1); dme::mbar_init(&v_empty[s], 1); }
        for (int t = 0; t < 2; ++t) {
            dme::mbar_init(&s_full[t], 1); dme::mbar_init(&p_half[2 * t], kBM); dme::mbar_init(&p_half[2 * t + 1], kBM);
            dme::mbar_init(&o_done[t], 1); dme::mbar_init(&o_free[t], kBM);
            dme::mbar_init(&item_full[t], 1); dme::mbar_init(&item_empty[t], kItemReaders);
        }
        dme::mbar_init_fence();
    }
    if (warp == kMmaWarp) { tc::tmem_alloc(&s_tmem_base, 512); tc::tmem_relinquish(); }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem_base;
    const uint32_t sm_q = dme::smem_addr(smem + Sh::OFF_Q), sm_k = dme::smem_addr(smem + Sh::OFF_K), sm_v = dme::smem_addr(smem + Sh::OFF_V);

    // The CTA is persistent: it works through items until the launch's counter runs out.  The TMA thread
    // draws the ids (its own block index first, then gridDim.x + a device-wide atomic counter, i.e. the
    // order a hardware block scheduler would have used) and publishes them through a two-slot ring; the
    // other roles read them there.  All barrier phases run on across items, so the next item's Q, K_0 and
    // first Q.K^T are under way while the softmax warps still normalise and store the previous item's O.
    auto next_item = [&](int it) -> int {                      // consumer side: id of the CTA's it-th item, or -1
        if (!dme::wait(&item_full[it & 1], uint32_t((it >> 1) & 1), p.status)) return -2;
        const int id = *reinterpret_cast<volatile int*>(&s_item[it & 1]);
        dme::mbar_arrive(&item_empty[it & 1]);
        return id;
    };

    // Register budget: the softmax warpgroups hold a whole 128-column score row per thread, the MMA / TMA
    // warpgroup carries ring state, descriptors and the per-item bookkeeping; the three limits (multiples of 8) must
    // sum to no more than 3 x 168 = 504 (the launch allocation): 208 + 208 + 88.  Measured against 216 + 216 + 72:
    // 16 instead of 44 bytes of spills in the D = 128 kernel (they sit in the 72-register branch), +3 % throughput.
    // (Each role branch opens with its own setmaxnreg, so the compiler sees one limit per branch.)
    if (warp >= 8 * RS) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
      if (warp == kTmaWarp) {
        // ---------------------------------- TMA producer ----------------------------------
        if (lane == 0) {
            dme::prefetch_tensor_map(&mapQ); dme::prefetch_tensor_map(&mapK); dme::prefetch_tensor_map(&mapV);
            dme::Ring<KST> kr; dme::Ring<VST> vr;
            int kloads = 0, vloads = 0;
            bool ok = true;
            for (int it = 0; ok; ++it) {
                // draw and publish the item
                if (it >= 2 && !dme::wait(&item_empty[it & 1], uint32_t(((it >> 1) - 1) & 1), p.status)) { ok = false; break; }
                int id = it == 0 ? int(blockIdx.x) : int(gridDim.x) + atomicAdd(p.work_counter, 1);
                if (id >= total_items) id = -1;
                s_item[it & 1] = id;
                dme::mbar_arrive(&item_full[it & 1]);
                if (id < 0) break;
                const PrefillItem w = prefill_item(p, id);
                // Q: the previous item's last Q.K^T must be done with the buffer
                if (it >= 1 && !dme::wait(q_empty, uint32_t((it - 1) & 1), p.status)) { ok = false; break; }
                dme::mbar_arrive_expect_tx(q_full, uint32_t((w.n[0] > 0) + (w.n[1] > 0)) * Sh::TILE_BYTES);
                for (int t = 0; t < 2; ++t) if (w.n[t] > 0)
                    for (int sb = 0; sb < Sh::SUB; ++sb)
                        dme::copy_tile_4d(smem + Sh::OFF_Q + t * Sh::TILE_BYTES + sb * Sh::SUB_BYTES, &mapQ, sb * 64, w.q0[t], w.head, w.b, q_full);
                for (int j = 0; j < w.nmax; ++j) {
                    if (kloads >= KST && !dme::wait(&k_empty[kr.stage], kr.phase ^ 1u, p.status)) { ok = false; break; }
                    dme::mbar_arrive_expect_tx(&k_full[kr.stage], Sh::TILE_BYTES);
                    for (int sb = 0; sb < Sh::SUB; ++sb)
                        dme::copy_tile_4d(smem + Sh::OFF_K + kr.stage * Sh::TILE_BYTES + sb * Sh::SUB_BYTES, &mapK, sb * 64, j * kBN, w.kvh, w.b, &k_full[kr.stage]);
                    kr.advance(); ++kloads;
                    if (vloads >= VST && !dme::wait(&v_empty[vr.stage], vr.phase ^ 1u, p.status)) { ok = false; break; }
                    dme::mbar_arrive_expect_tx(&v_full[vr.stage], Sh::TILE_BYTES);
                    for (int sb = 0; sb < Sh::SUB; ++sb)
                        dme::copy_tile_4d(smem + Sh::OFF_V + vr.stage * Sh::TILE_BYTES + sb * Sh::SUB_BYTES, &mapV, sb * 64, j * kBN, w.kvh, w.b, &v_full[vr.stage]);
                    vr.advance(); ++vloads;
                }
            }
            if (!ok) atomicExch(&s_failed, 1);
        }
      } else if (warp == kMmaWarp) {
        // ---------------------------------- MMA issuer ------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::instr_desc_f16(kBM, kBN, Fmt<T>::id, 0, 0);
            constexpr uint32_t idesc_pv = tc::instr_desc_f16(kBM, D, Fmt<T>::id, 0, 1);
            // Descriptors differ from a per-tile base only in the 14-bit start-address field
            // (units of 16 bytes), so a k-step is one integer add of a compile-time constant on the base;
            // the k loops are unrolled so that the issue overhead per MMA stays far below its 64 cycles.
            const uint64_t q_base = tc::smem_desc_sw128(sm_q, 16, 1024);
            const uint64_t k_base = tc::smem_desc_sw128(sm_k, 16, 1024);
            const uint64_t v_base = tc::smem_desc_sw128(sm_v, Sh::SUB_BYTES, 1024);
            auto issue_qk = [&](int t, int kstage) {
                const uint64_t qd = q_base + uint64_t((t * Sh::TILE_BYTES) >> 4);
                const uint64_t kd = k_base + uint64_t((kstage * Sh::TILE_BYTES) >> 4);
                #pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off16 = (uint32_t(ks >> 2) * Sh::SUB_BYTES + uint32_t(ks & 3) * 32u) >> 4;
                    tc::mma_ss(tmem + t * kBN, qd + off16, kd + off16, idesc_qk, ks > 0);
                }
            };
            auto issue_pv = [&](int t, int vstage, bool first, int kk0, int kk1) {  // 16-key steps kk0 .. kk1-1 of the tile
                const uint64_t vd = v_base + uint64_t((vstage * Sh::TILE_BYTES) >> 4);
                #pragma unroll
                for (int kk = kk0; kk < kk1; ++kk)
                    tc::mma_ts(tmem + 256 + t * 128, tmem + t * kBN + kk * 8, vd + uint64_t(kk * (2048 >> 4)),
                               idesc_pv, !(first && kk == 0));
            };
            dme::Ring<KST> kr; dme::Ring<VST> vr;
            int cs0 = 0, cs1 = 0;          // steps of tile 0 / 1 in earlier items: phase of s_full / p_half
            int co0 = 0, co1 = 0;          // earlier items in which the tile had work: phase of o_done / o_free
            bool ok = true;
            for (int it = 0; ok; ++it) {
                const int id = next_item(it);
                if (id < 0) { ok = id != -2; break; }
                const PrefillItem w = prefill_item(p, id);
                const int nmax = w.nmax, n0 = w.n[0], n1 = w.n[1];
                ok = dme::wait(q_full, uint32_t(it & 1), p.status);
                if (ok) ok = dme::wait(&k_full[kr.stage], kr.phase, p.status);
                if (!ok) break;
                tc::fence_after_sync();
                if (n0 > 0) { issue_qk(0, kr.stage); tc::commit(&s_full[0]); }
                if (n1 > 0) { issue_qk(1, kr.stage); tc::commit(&s_full[1]); }
                tc::commit(&k_empty[kr.stage]);
                kr.advance();
                if (nmax == 1) tc::commit(q_empty);
                // one tile's share of step j: P.V over the two halves of P as they arrive, then the next Q.K^T
                auto tile_step = [&](auto tc_t, int j, int nt, int cst, int cot) -> bool {
                    constexpr int t = decltype(tc_t)::value;
                    if (j >= nt) return true;
                    if (!dme::wait(&p_half[2 * t], uint32_t((cst + j) & 1), p.status)) return false;
                    // the first P.V of an item overwrites O_t: the previous item's epilogue must have read it
                    if (j == 0 && cot > 0 && !dme::wait(&o_free[t], uint32_t((cot - 1) & 1), p.status)) return false;
                    tc::fence_after_sync();
                    issue_pv(t, vr.stage, j == 0, 0, 2 * kFirstChunks);   // the first hand-off's keys while the softmax finishes the rest
                    if (!dme::wait(&p_half[2 * t + 1], uint32_t((cst + j) & 1), p.status)) return false;
                    tc::fence_after_sync();
                    issue_pv(t, vr.stage, j == 0, 2 * kFirstChunks, kBN / 16);
                    if (j + 1 < nt) { issue_qk(t, kr.stage); tc::commit(&s_full[t]); }
                    else tc::commit(&o_done[t]);
                    return true;
                };
                for (int j = 0; j < nmax && ok; ++j) {
                    ok = dme::wait(&v_full[vr.stage], vr.phase, p.status);
                    if (ok && j + 1 < nmax) ok = dme::wait(&k_full[kr.stage], kr.phase, p.status);
                    if (!ok) break;
                    ok = tile_step(std::integral_constant<int, 0>{}, j, n0, cs0, co0);
                    if (ok) ok = tile_step(std::integral_constant<int, 1>{}, j, n1, cs1, co1);
                    if (!ok) break;
                    tc::commit(&v_empty[vr.stage]);
                    vr.advance();
                    if (j + 1 < nmax) {
                        tc::commit(&k_empty[kr.stage]); kr.advance();
                        if (j + 2 == nmax) tc::commit(q_empty);           // that was the item's last Q.K^T
                    }
                }
                cs0 += n0; cs1 += n1; co0 += n0 > 0; co1 += n1 > 0;
            }
            if (!ok) atomicExch(&s_failed, 1);
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // ---------------------------------- softmax warps ---------------------------------
        // One thread owns a whole 128-key score row.  (Two threads per row, 64 keys each with a shared-memory
        // exchange of the row maxima, was measured at 502 vs 944 TFLOP/s and is not kept.)
        constexpr int CW = kBN / RS;                           // score columns per thread
        constexpr int OW = D / RS;                             // output columns per thread
        const int t = warp / (4 * RS);                        // query tile
        const int half = (warp / 4) % RS;                     // column half of this thread
        const int r = (warp % 4) * 32 + lane;                 // row inside the tile = TMEM lane
        const uint32_t lane_base = uint32_t(32 * (warp % 4)) << 16;
        const uint32_t tS = tmem + lane_base + uint32_t(t * kBN);
        const uint32_t tO = tmem + lane_base + 256u + uint32_t(t * 128) + uint32_t(half * OW);
        int cs = 0, co = 0;                                    // as in the MMA thread, for this tile
        bool ok = true;
        // The tile's 128 threads meet at named barrier 2 + t in the epilogue, so they leave this loop TOGETHER: whether a
        // thread's waits of an item all succeeded is and-reduced over the warpgroup (a barrier every one of them reaches,
        // once per item) before anyone acts on it.
        auto all_of_tile = [&](bool mine) -> bool {
            uint32_t r_;
            asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbarrier.cta.red.and.pred p, %2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(r_) : "r"(uint32_t(mine)), "r"(2 + t) : "memory");
            return r_ != 0;
        };
        auto tile_sync = [&]() { asm volatile("bar.sync %0, 128;" :: "r"(2 + t) : "memory"); };
        const bool issuer = r == 0;                            // issues and tracks this tile's output stores
        unsigned char* stage = smem + Sh::OFF_OUT + t * Sh::SUB_BYTES;
        if (issuer) dme::prefetch_tensor_map(&mapO);
        for (int it = 0;; ++it) {
          const int id = next_item(it);
          if (id < 0) { ok = all_of_tile(id != -2); break; }   // -1: the launch's items are used up (the same value in every thread)
          const PrefillItem w = prefill_item(p, id);
          const int q0t = t ? w.q0[1] : w.q0[0], nt = t ? w.n[1] : w.n[0];     // no arrays indexed at run time
          const int o_b = w.b, o_head = w.head;
          const int row = q0t + r;
          float m_used = -INFINITY, l = 0.f;
          for (int j = 0; j < nt; ++j) {
            if (!dme::wait(&s_full[t], uint32_t((cs + j) & 1), p.status)) { ok = false; break; }
            tc::fence_after_sync();
            const bool need_mask = (p.causal && j * kBN + kBN - 1 > q0t) || (j * kBN + kBN > p.seqK);
            // columns (of this thread's range) <= col_limit are live
            const int col_limit = min(p.causal ? row : 0x7fffffff, p.seqK - 1) - j * kBN - half * CW;
            // ---- this thread's part of the score row into registers (one wait for all loads) ------------
            uint32_t sv[CW];
            #pragma unroll
            for (int c = 0; c < CW / 32; ++c) tc::ld_32x32b_x32(tS + half * CW + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[c * 32]));
            tc::wait_ld();
            if (DBG && p.debug_s && j == 0 && t == 0 && id == 0) {
                #pragma unroll
                for (int i = 0; i < CW; ++i) p.debug_s[r * kBN + half * CW + i] = __uint_as_float(sv[i]);
            }
            if (need_mask) {
                #pragma unroll
                for (int i = 0; i < CW; ++i) if (i > col_limit) sv[i] = 0xff800000u;       // -inf
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // 3-input max
            #pragma unroll
            for (int i = 0; i < CW; i += 8) {
                #pragma unroll
                for (int u = 0; u < 4; ++u) mx4[u] = max3(mx4[u], __uint_as_float(sv[i + 2 * u]), __uint_as_float(sv[i + 2 * u + 1]));
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = mx * p.scale_log2;
            float alpha = 1.f;
            if (m_new > m_used + kLazyRescale) { alpha = fast_exp2(m_used - m_new); m_used = m_new; }
            // ---- rescale O when some row of this warp moved its max (never on the first tile) ----
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                #pragma unroll
                for (int c = 0; c < OW / 32; ++c) {
                    uint32_t v[32];
                    tc::ld_32x32b_x32(tO + c * 32, v);
                    tc::wait_ld();
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tc::st_32x32b_x32(tO + c * 32, v);
                }
                tc::wait_st();
            }
            // ---- P = exp2(S * scale - m) as 16-bit pairs over the front of S.  Each half of the keys is handed
            // to the MMA warp as soon as it is stored; the row sum is taken after the hand-off. ----
            const float neg_m = -m_used;
            #pragma unroll
            for (int c = 0; c < CW / 32; ++c) {
                uint32_t pk[16];
                #pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float s0 = __uint_as_float(sv[c * 32 + 2 * i]), s1 = __uint_as_float(sv[c * 32 + 2 * i + 1]);
                    const float2 e = exp2_pair(s0, s1, p.scale_log2, neg_m);
                    sv[c * 32 + 2 * i] = __float_as_uint(e.x); sv[c * 32 + 2 * i + 1] = __float_as_uint(e.y);
                    pk[i] = pack2<T>(e.x, e.y);
                }
                tc::st_32x32b_x16(tS + (half * CW) / 2 + c * 16, pk);
                const int key_chunk = half * (CW / 32) + c;                   // 32-key chunk of the tile: 0..3
                if (key_chunk == kFirstChunks - 1 || key_chunk == 3) {
                    tc::wait_st();
                    tc::fence_before_sync();
                    dme::mbar_arrive(&p_half[2 * t + (key_chunk == 3)]);
                }
            }
            float la[4] = {0.f, 0.f, 0.f, 0.f};
            #pragma unroll
            for (int i = 0; i < CW; i += 4) {
                #pragma unroll
                for (int u = 0; u < 4; ++u) la[u] += __uint_as_float(sv[i + u]);
            }
            l = l * alpha + ((la[0] + la[1]) + (la[2] + la[3]));
          }
          // ---- epilogue: O / l -> 16-bit, through a swizzled staging tile and TMA stores (64 columns at a time).  O is taken
          // into registers first and the tile's tensor memory released, so the next item's P.V does not wait for the stores.
          if (ok && nt > 0) ok = dme::wait(&o_done[t], uint32_t(co & 1), p.status);
          ok = all_of_tile(ok);
          if (!ok) break;
          if (nt > 0) {
            tc::fence_after_sync();
            uint32_t v[OW];
            #pragma unroll
            for (int c = 0; c < OW / 32; ++c) tc::ld_32x32b_x32(tO + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
            tc::wait_ld();
            tc::fence_before_sync();
            dme::mbar_arrive(&o_free[t]);
            const float inv = l > 0.f ? 1.f / l : 1.f;
            #pragma unroll
            for (int hb = 0; hb < D / 64; ++hb) {
                if (issuer) dme::store_wait_read<0>();           // the previous store from this staging tile has read it out
                tile_sync();
                #pragma unroll
                for (int ch = 0; ch < 8; ++ch) {                 // row r, 16-byte chunk ch, 128-byte swizzle
                    const int c0 = hb * 64 + ch * 8;
                    uint4 o4;
                    o4.x = pack2<T>(__uint_as_float(v[c0 + 0]) * inv, __uint_as_float(v[c0 + 1]) * inv);
                    o4.y = pack2<T>(__uint_as_float(v[c0 + 2]) * inv, __uint_as_float(v[c0 + 3]) * inv);
                    o4.z = pack2<T>(__uint_as_float(v[c0 + 4]) * inv, __uint_as_float(v[c0 + 5]) * inv);
                    o4.w = pack2<T>(__uint_as_float(v[c0 + 6]) * inv, __uint_as_float(v[c0 + 7]) * inv);
                    *reinterpret_cast<uint4*>(stage + swz128(r, ch)) = o4;
                }
                dme::fence_proxy_async_smem();
                tile_sync();
                if (issuer) {                                    // rows past seqQ are clipped by the tensor map
                    dme::store_tile_4d(&mapO, hb * 64, q0t, o_head, o_b, stage);
                    dme::store_commit();
                }
            }
          }
          cs += nt; co += nt > 0;
        }
        if (issuer) dme::store_wait_all();
        if (!ok) atomicExch(&s_failed, 1);
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    if (warp == kMmaWarp) tc::tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && s_failed) atomicExch(p.sticky, 1);
}

template <typename T, int D, int RS>
int launch_prefill_rs(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                   const b200p_attn_strides& s, float* debug_s, cudaStream_t st) {
    using Sh = PrefillShape<D>;
    const CUtensorMapDataType dt = dtype == B200P_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap mq, mk, mv;
    const uint64_t qd[4] = {uint64_t(D), uint64_t(c->seqQ), uint64_t(c->nQHeads), uint64_t(c->batch)};
    const uint64_t qs[3] = {uint64_t(s.q_seq) * 2, uint64_t(s.q_head) * 2, uint64_t(s.q_batch) * 2};
    const uint64_t kd[4] = {uint64_t(D), uint64_t(c->seqK), uint64_t(c->nKVHeads), uint64_t(c->batch)};
    const uint64_t ks[3] = {uint64_t(s.k_seq) * 2, uint64_t(s.k_head) * 2, uint64_t(s.k_batch) * 2};
    const uint64_t vs[3] = {uint64_t(s.v_seq) * 2, uint64_t(s.v_head) * 2, uint64_t(s.v_batch) * 2};
    const uint32_t box[4] = {64, 128, 1, 1};
    cudaError_t e = make_tensor_map(&mq, dt, 4, Q, qd, qs, box, Swizzle::B128);
    if (e == cudaSuccess) e = make_tensor_map(&mk, dt, 4, K, kd, ks, box, Swizzle::B128);
    if (e == cudaSuccess) e = make_tensor_map(&mv, dt, 4, V, kd, vs, box, Swizzle::B128);
    CUtensorMap mo;
    const uint64_t os[3] = {uint64_t(s.o_seq) * 2, uint64_t(s.o_head) * 2, uint64_t(s.o_batch) * 2};
    if (e == cudaSuccess) e = make_tensor_map(&mo, dt, 4, O, qd, os, box, Swizzle::B128);
    if (e != cudaSuccess) return int(e);

    const bool dbg = debug_s != nullptr;
    auto kern = dbg ? prefill_tc_kernel<T, D, RS, true> : prefill_tc_kernel<T, D, RS, false>;
    static bool attr_set[64][2] = {};
    int dev = 0; cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev][dbg]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Sh::SMEM_BYTES);
        if (e != cudaSuccess) return int(e);
        attr_set[dev][dbg] = true;
    }
    PrefillParams p{};
    p.debug_s = debug_s;
    p.sticky = device_status_ptr();
    LaunchSlot slot{};
    if (!p.sticky) return B200P_E_NO_DEVICE;
    if (int se = take_launch_slot(st, &slot)) return se;       // work counter and abort word of this launch, cleared on its stream
    p.status = slot.abort; p.work_counter = slot.work;
    p.seqQ = c->seqQ; p.seqK = c->seqK; p.nQH = c->nQHeads; p.nKVH = c->nKVHeads; p.group = c->nQHeads / c->nKVHeads;
    p.batch = c->batch; p.causal = c->causal;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(D));
    // One persistent CTA per SM (the kernel takes all of an SM's shared and tensor memory), or one CTA per
    // work item when the knob's bit 1 is set.
    const long long items = (long long)((c->seqQ + 2 * kBM - 1) / (2 * kBM)) * c->nQHeads * c->batch;
    if (items > 0x7fffffffLL / 2) return B200P_E_RANGE;
    const int sms = sm_count();
    const bool one_per_item = (tuning(KNOB_PREFILL_VARIANT, 0) & 2) != 0;
    dim3 grid(unsigned(one_per_item || items < sms ? items : sms), 1, 1);
    kern<<<grid, prefill_threads(RS), Sh::SMEM_BYTES, st>>>(p, mq, mk, mv, mo);
    return launched();
}

template <typename T, int D>
int launch_prefill(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                   const b200p_attn_strides& s, float* debug_s, cudaStream_t st) {
    return launch_prefill_rs<T, D, 1>(Q, K, V, O, c, dtype, s, debug_s, st);
}

} // namespace

int prefill_dispatch_strided(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                             const b200p_attn_strides* strides, float* debug_s, cudaStream_t st);

int prefill_dispatch(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                     float* debug_s, cudaStream_t st) {
    return prefill_dispatch_strided(Q, K, V, O, c, dtype, nullptr, debug_s, st);
}

int prefill_dispatch_strided(const void* Q, const void* K, const void* V, void* O, const b200p_prefill_cfg* c, int dtype,
                             const b200p_attn_strides* strides, float* debug_s, cudaStream_t st) {
    if (!c) return B200P_E_NULL;
    if (dtype != B200P_F16 && dtype != B200P_BF16) return B200P_E_DTYPE;
    if (c->D != 64 && c->D != 128) return B200P_E_DIM;                        // attention.hpp:105-107
    if (c->nQHeads <= 0 || c->nKVHeads <= 0 || c->nQHeads % c->nKVHeads != 0) return B200P_E_DIM;
    if (c->seqQ <= 0 || c->seqK <= 0 || c->batch <= 0) return B200P_E_LENGTH;
    if (c->nQHeads > 65535 || c->batch > 65535) return B200P_E_RANGE;
    if (!Q || !K || !V || !O) return B200P_E_NULL;
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16)) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    b200p_attn_strides s;
    if (strides) {
        s = *strides;
        // TMA needs 16-byte multiples for every stride; the output rows are written with 16-byte stores
        const long long all[12] = {s.q_seq, s.q_head, s.q_batch, s.k_seq, s.k_head, s.k_batch,
                                   s.v_seq, s.v_head, s.v_batch, s.o_seq, s.o_head, s.o_batch};
        for (long long v : all) if (v <= 0 || (v * 2) % 16 != 0) return B200P_E_ALIGN;
    } else {                                                   // the reference's dense head-major layout
        const long long D = c->D;
        s.q_seq = D; s.q_head = (long long)c->seqQ * D; s.q_batch = (long long)c->nQHeads * c->seqQ * D;
        s.k_seq = D; s.k_head = (long long)c->seqK * D; s.k_batch = (long long)c->nKVHeads * c->seqK * D;
        s.v_seq = s.k_seq; s.v_head = s.k_head; s.v_batch = s.k_batch;
        s.o_seq = s.q_seq; s.o_head = s.q_head; s.o_batch = s.q_batch;
    }
    if (dtype == B200P_F16)
        return c->D == 128 ? launch_prefill<__half, 128>(Q, K, V, O, c, dtype, s, debug_s, st)
                           : launch_prefill<__half, 64>(Q, K, V, O, c, dtype, s, debug_s, st);
    return c->D == 128 ? launch_prefill<__nv_bfloat16, 128>(Q, K, V, O, c, dtype, s, debug_s, st)
                       : launch_prefill<__nv_bfloat16, 64>(Q, K, V, O, c, dtype, s, debug_s, st);
}

} // namespace b200p

using namespace b200p;

extern "C" int b200p_attn_prefill(const void* Q, const void* K, const void* V, void* O,
                                  const b200p_prefill_cfg* cfg, int dtype, b200p_stream_t stream) {
    return prefill_dispatch(Q, K, V, O, cfg, dtype, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int b200p_attn_prefill_strided(const void* Q, const void* K, const void* V, void* O,
                                          const b200p_prefill_cfg* cfg, int dtype, const b200p_attn_strides* strides,
                                          b200p_stream_t stream) {
    if (!strides) return B200P_E_NULL;
    return prefill_dispatch_strided(Q, K, V, O, cfg, dtype, strides, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int b200p_attn_prefill_debug(const void* Q, const void* K, const void* V, void* O,
                                        const b200p_prefill_cfg* cfg, int dtype, float* raw_scores,
                                        b200p_stream_t stream) {
    return prefill_dispatch(Q, K, V, O, cfg, dtype, raw_scores, static_cast<cudaStream_t>(stream));
}
