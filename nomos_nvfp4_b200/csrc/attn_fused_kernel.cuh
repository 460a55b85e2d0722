// Device side of the fused split-K attention over the packed quantised KV ring
// (sm_100a).  See attn_fused.cu for the host side and the overall description.
#pragma once

#include <type_traits>

#include <cuda.h>             // CUtensorMap (type only: the encoder is resolved at run time)
#include <cooperative_groups.h>
#include <math_constants.h>

#include "common.cuh"
#include "kv_rows.cuh"
#include "launch.h"

namespace nomos {
namespace fused {

// Tile parameters (overridable at build time for tuning).  One query-row tile (decode, up to 8
// rows of a GQA group) needs ~130 registers per thread and runs 12 warps per SM; three tiles
// (verify, up to 24 rows) keep 96 fp32 accumulators per thread and run 8.
#ifndef NOMOS_NWARP
#define NOMOS_NWARP 12
#endif
#ifndef NOMOS_NWARP_MULTI
#define NOMOS_NWARP_MULTI 8
#endif
#ifndef NOMOS_NSTAGE
#define NOMOS_NSTAGE 2
#endif

constexpr int TILE = 32;                 // tokens per warp tile
constexpr int NSTAGE = NOMOS_NSTAGE;     // tile stages per warp
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float M_INIT = -1.0e30f;       // finite "minus infinity" for the running max
constexpr int Q_FIX_MAX = 32639;         // 127 * 256 + 127: two int8 limbs, hi in [-127,127], lo in [-128,127]
constexpr float P_FIX = 65535.0f;        // probabilities reach the tensor core as 16-bit fixed point (two u8 limbs)
constexpr float LAZY_MAX = 8.0f;         // base-2 slack before the running softmax reference is moved
constexpr float RND_MAGIC = 8388608.0f;  // 2^23: adding it leaves round-to-nearest(x) in the low mantissa bits

// Wide heads are cut into head-dim slices in one of two ways.
// QS > 1 (the default for head_dim 256 / 512): QS warps of a CTA -- a "quad" -- take every tile TOGETHER.  Warp j of
//   the quad owns dims [j HD/QS, (j+1) HD/QS): it streams only those byte columns of the K and V rows (and of the
//   block scales), computes the partial logits of its dims, the quad adds the partials up through shared memory (one
//   named barrier per tile), every warp works out the same softmax weights, and warp j accumulates its slice of the
//   output.  K and V leave HBM once and every product is computed once; per warp the loop is the head_dim 128 loop.
// DS > 1 (kept for comparison): the PV product is split over DS CTAs that each compute the full QK (all of K is read
//   by every slice, from L2 after the first) and hold HD / DS output dims.
template <int FMT, int HD, int MT, int DS = 1, int QS = 1>
struct Cfg {
    static_assert(DS == 1 || QS == 1, "one way of slicing at a time");
    static constexpr int QSL = QS;
    static constexpr int HDK = HD / QS;                                       // dims whose QK partial a warp computes
    static constexpr int HDV = HD / (DS * QS);                                // output dims of a warp
    static constexpr int ROWB = (FMT == KV_I8) ? HD : HD / 2;                 // cache bytes per token row
    static constexpr int ROWBK = ROWB / QS;                                   // bytes of a K row a warp reads
    static constexpr int ROWBV = ROWB / (DS * QS);                            // bytes of a V row a warp reads
    static constexpr int CHUNKS = ROWB / 16;                                  // 16-byte chunks per row
    static constexpr int CHUNKSK = ROWBK / 16;
    static constexpr int CHUNKSV = ROWBV / 16;
    static constexpr int NBLK = HD / 32;
    static constexpr int NBLKK = NBLK / QS;
    static constexpr int NBLKV = HDV / 32;
    static constexpr int SCB = (FMT == KV_I4B32) ? NBLK * 2 : 4;              // scale bytes per token in the cache
    static constexpr int SCBW = (FMT == KV_I4B32) ? NBLKK * 2 : 4;            // scale bytes per token a warp keeps
    static constexpr int KV_BYTES = TILE * ROWBK;                             // K tile (slice)
    static constexpr int V_BYTES = TILE * ROWBV;                              // V tile (slice)
    static constexpr int ST_BYTES = KV_BYTES + V_BYTES;                       // tiles of one stage
    static constexpr int SC_BYTES = TILE * SCBW;
    static_assert(ROWBK >= 64 && ROWBK % 64 == 0 && HDK % 128 == 0, "a K slice is whole 128-dim groups");
    static constexpr int STAGE_BYTES = ST_BYTES + 2 * SC_BYTES;
    static constexpr int NSLOT = 8 * MT;                                      // query rows (row x group head) per CTA
    static constexpr int NT = HDV / 8;                                        // PV N tiles (8 output dims each)
    static_assert(ROWBV >= 64 && ROWBV % 64 == 0, "a V slice is copied in 64-byte column groups");
    static constexpr int Q_BYTES = 2 * NSLOT * HD;                            // two limbs
    static constexpr int SLOT_BYTES = NSLOT * 16 + NSLOT * NBLK * 4;          // qscale, lo, hi, pad; 8*sum(q) per block
    // warps per CTA: as many as the register file and ~200 KB of pipeline memory allow
    static constexpr int NW_REG = (MT == 1 && HDV <= 256) ? NOMOS_NWARP : NOMOS_NWARP_MULTI;
    static constexpr int XCH_WARP_BYTES = QS > 1 ? 2 * MT * 8 * 32 * 4 : 0;  // a warp's share of the quads' partial-logit buffers
    static constexpr int NW_MEM = (200 * 1024) / (NSTAGE * STAGE_BYTES + XCH_WARP_BYTES);
    static constexpr int NW_MIN = NW_REG < NW_MEM ? NW_REG : (NW_MEM < 1 ? 1 : NW_MEM);
    static constexpr int NW = (NW_MIN / QS) * QS;                            // whole quads
    static constexpr int NQ = NW / QS;                                       // tile streams per CTA
    static_assert(NW >= QS, "a CTA holds at least one quad");
    static constexpr int APPEND_BYTES = NW * (ROWB + 64);                     // per warp: one quantised row + its scales
    // Shared-memory map: [K/V tiles of every warp and stage | scales | query limbs | slot
    // constants | append scratch | mbarriers].  The tile region starts on a 1024-byte boundary
    // (what the TMA swizzle patterns are defined against) and is reused for the merges.
    static constexpr int TILES_BYTES = NW * NSTAGE * ST_BYTES;
    static constexpr int SCALES_BYTES = NW * NSTAGE * 2 * SC_BYTES;
    static constexpr int MERGE_BYTES = NW * NSLOT * (HDV + 2) * 4;
    static constexpr int REGION0_BYTES = ((TILES_BYTES > MERGE_BYTES ? TILES_BYTES : MERGE_BYTES) + 15) / 16 * 16;
    // cluster merge: the CTA's own merged rows [NSLOT][HD+2] sit behind the warps' rows, where the other CTAs of the
    // cluster read them through distributed shared memory
    static constexpr int CPART_OFF = (MERGE_BYTES + 15) / 16 * 16;
    static constexpr bool CLUSTER_OK = DS == 1 && CPART_OFF + NSLOT * (HD + 2) * 4 <= REGION0_BYTES;
    static constexpr int BAR_BYTES = NW * NSTAGE * 8;
    static constexpr int XCH_BYTES = NW * XCH_WARP_BYTES;                      // partial logits: [quad][tile parity][warp of the quad][MT*8][32 lanes] fp32
    static constexpr int SMEM_BYTES = 1024 + REGION0_BYTES + SCALES_BYTES + Q_BYTES + SLOT_BYTES + APPEND_BYTES + BAR_BYTES + XCH_BYTES;
    static_assert(SMEM_BYTES <= 232448, "shared memory budget of a CTA");
    // Rows of 64 / 128 bytes map one-to-one onto the TMA 64B / 128B swizzle patterns, which are
    // the XOR layouts swz_chunk() defines; wider rows stay on the cp.async path.
    static constexpr bool TMA_OK = (ROWB == 64 || ROWB == 128) && DS == 1 && QS == 1;
};

// Tensor maps of the K and V byte planes: {row bytes, nkv * cache_cap rows, batch}.
struct TmaMaps {
    CUtensorMap k, v;
};

struct KParams {
    const uint8_t *q;
    const uint8_t *k_cache, *v_cache, *k_scales, *v_scales;
    uint8_t *out;
    float *partial;          // workspace partials or exported partials: [split][grow][HD+2]
    int write_partial;       // 1: write (o, M, l) to partial; 0: write normalised out
    int export_nat;          // 1: partial m is exported in natural-log units
    int q_type, out_type;
    int S, nh, nkv, kvg, cache_hd, cache_cap, win_start, klen, window;
    int tile0, ntiles, tiles_per_split, row_groups, grows;
    float qk_scale_log2;     // softmax_scale * log2(e)
    // in-kernel split merge: the last CTA of a (batch, kv head, row group) unit to finish merges
    unsigned long long *counters;   // one word per unit: (tag << 16) | arrivals, see merge_splits_in_kernel; nullptr = no in-kernel merge
    int splits;
    int arrivals;                   // CTAs per unit that arrive before the merge: splits x head-dim slices
    int coop_merge;                 // K > 0: the last K CTAs of a unit to arrive each merge a share of the unit's rows once all have arrived (the whole
                                    //    grid is resident at once, so waiting for the others cannot starve them)
    int cluster_merge;              // 1: the splits of a unit are the CTAs of one thread-block cluster; they merge through
                                    //    distributed shared memory (no partials in device memory, no arrival word)
    float *partial_export;          // optional exported (o, m, l) per row, m in natural-log units
    int early_rows;                 // window rows [0, early_rows) may be read before griddepcontrol.wait
    int kv_read_once;               // 1: every cache byte is read by exactly one CTA of the launch (tile copies are marked evict-first in L2)
    // fused quantize-on-write: the last n_new keys of the window are given as fp32 rows
    const float *new_k, *new_v;     // [n_new][nkv][HD], row stride new_stride elements; nullptr = none
    uint8_t *k_cache_w, *v_cache_w, *k_scales_w, *v_scales_w;   // writable aliases of the cache
    int n_new, new_stride, new_base_pos;
    long q_batch_stride, kv_batch_stride, scale_batch_stride, out_batch_stride;
    const int *block_table;  // paged caches (tcgen05 kernel): [batch][max_pages] page of each 128-key tile; nullptr = contiguous
    const int *seq_lens;     // paged caches: keys of each sequence
    int max_pages;
    // sequence-sharded decode across GPUs (peer_world > 1): the CTA that merges a unit's splits pushes the unit's
    // (o, m, l) rows into every peer's mailbox, waits for the peers' rows in its own and writes the final output
    float *peer_rows[8];                // rank g's mailbox rows [2 step slots][world][grows][HD+2], as mapped in this process
    unsigned long long *peer_flags[8];  // rank g's arrival stamps [2][world][grows]: the step number once the row is complete
    int peer_rank, peer_world;
    unsigned long long peer_seq;        // step number, the same on every rank, never 0
    unsigned long long peer_timeout_ns; // how long a CTA waits for a peer's rows before it gives up (fault bit 2)
    unsigned int kvg_magic;  // ceil(2^32 / kvg), 0 for kvg == 1: idx / kvg = umulhi(idx, kvg_magic)
    int use_tma;             // bit 0: whole tiles come by TMA; bit 1: their scales by bulk copy
    int dry_pass;            // 1: the whole grid is resident at once, so a CTA may start before its stream predecessor is done
    unsigned int *fault;     // sticky device word: bit 0 = a tile never arrived within the wait limit (mma.sync kernel),
                             // bit 1 = a hand-off of the tcgen05 kernel ran out of time, bit 2 = a peer's partial never arrived
};

// idx / kvg for the small non-negative indices used here, without the division routine.
__device__ __forceinline__ int div_kvg(const KParams &p, int idx) {
    return p.kvg_magic ? (int)__umulhi((unsigned)idx, p.kvg_magic) : idx;
}

// Query elements are read through L2 only (ld.global.cg): the warming pass reads them before the
// stream-order wait, while the stream predecessor may still be writing them, and the pass that
// counts must not find such a line in the L1 or in the read-only path.
__device__ __forceinline__ float load_q(const uint8_t *q, int q_type, long idx) {
    return q_type == ET_BF16 ? __uint_as_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short *>(q) + idx) << 16)
                             : __ldcg(reinterpret_cast<const float *>(q) + idx);
}

// D(16x8,s32) = A(16x32,u8,row) * B(32x8,s8,col), no accumulator input.
__device__ __forceinline__ void mma_u8s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}


__device__ __forceinline__ void mma_u8u8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}

// ---- TMA and mbarrier wrappers (every copy targets this CTA only)
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// One attempt; the hardware may keep the thread suspended (no issue slots used) for up to the
// hinted time before it answers.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(200000u)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity to complete; gives up after about two seconds.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) return false;
    }
}
// Starts the fetch of a tensor map into the descriptor cache ahead of its first use.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(map)) : "memory");
}
// One 32-row box of a {bytes, rows, batch} byte tensor into shared memory.
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap *map, int row, int batch, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(dst),
        "l"(reinterpret_cast<unsigned long long>(map)), "r"(0), "r"(row), "r"(batch), "r"(bar)
        : "memory");
}
// The same copy for bytes that this launch reads exactly once (the cache rows of a decode call): marked evict-first
// in L2, so that a hundred megabytes of them do not push out what the launch does come back to -- its own code, the
// query, the split partials -- or what the next kernel in the stream needs.
__device__ __forceinline__ void tma_load_tile_once(uint32_t dst, const CUtensorMap *map, int row, int batch, uint32_t bar) {
    asm volatile(
        "{\n"
        ".reg .b64 pol;\n"
        "createpolicy.fractional.L2::evict_first.b64 pol, 1.0;\n"
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], pol;\n"
        "}\n" ::"r"(dst),
        "l"(reinterpret_cast<unsigned long long>(map)), "r"(0), "r"(row), "r"(batch), "r"(bar)
        : "memory");
}
// A whole 16-byte cp.async, evict-first in L2 when `once`.
__device__ __forceinline__ void cp_async16_hint(uint32_t dst, const void *src, bool once) {
    if (once) {
        asm volatile(
            "{\n"
            ".reg .b64 pol;\n"
            "createpolicy.fractional.L2::evict_first.b64 pol, 1.0;\n"
            "cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, pol;\n"
            "}\n" ::"r"(dst),
            "l"(src)
            : "memory");
    } else {
        cp_async16(dst, src, 16);
    }
}
// Contiguous bytes (16-byte aligned both sides, size a multiple of 16) into shared memory.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

}  // namespace fused
}  // namespace nomos

namespace nomos {
namespace fused {

__device__ __forceinline__ unsigned long long arrive_add(unsigned long long *ctr) {
    unsigned long long old;
    asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], 1;\n" : "=l"(old) : "l"(ctr) : "memory");
    return old;
}

// Small merges (the common decode case: at most 32 splits, one (row, dim) element per thread).  Thread
// `tid` does the whole merge of its element by itself: its row's (m, l) of every split (the same
// addresses for the 128 threads of a row) and its own partial outputs are all requested at once, one
// round trip to L2, and the weights are worked out redundantly per thread -- no staging, no barrier.
// The capacity (unrolled loads; clamped instead of predicated so that they batch) follows the number of
// splits.  Not inlined: it runs once, in the one CTA per unit that arrives last.  (Having an idle warp run it
// ahead of time to warm the instruction caches was tried: the merge itself got no faster -- it waits on
// L2, not on its code -- and the decode call 1.2 us slower.)
struct SmallMergeArgs {
    const float *partial;      // split 0 of the workspace partials
    float *partial_export;     // merged (o, m, l) rows instead of normalised outputs, or nullptr
    uint8_t *out;
    long rstride;              // floats between two splits
    long out_batch_stride;
    int G, S, nh, kvg, out_type;
    unsigned int kvg_magic;
    int b, kvh, first, nrows;  // batch element, KV head, first slot of the row group, its valid slots
};
template <int HD>
__device__ __noinline__ void merge_small(const SmallMergeArgs a, int tid) {
    if (tid >= a.nrows * HD) return;
    const int sl = tid / HD, d = tid - sl * HD;
    const int idx = a.first + sl;
    const int r = a.kvg_magic ? (int)__umulhi((unsigned)idx, a.kvg_magic) : idx;
    const int hrow = r * a.nh + a.kvh * a.kvg + (idx - r * a.kvg);
    const long grow = (long)a.b * a.S * a.nh + hrow;
    const float *base = a.partial + (size_t)grow * (HD + 2);
    const int G = a.G;
    auto run = [&](auto cap_tag) {
        constexpr int GC = decltype(cap_tag)::value;
        float2 ml[GC];
        float o[GC];
#pragma unroll
        for (int i = 0; i < GC; ++i) {
            const float *row = base + (size_t)min(i, G - 1) * a.rstride;
            ml[i] = __ldcg(reinterpret_cast<const float2 *>(row + HD));
            o[i] = __ldcg(row + d);
        }
        float m = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < GC; ++i) {
            ml[i].x = (i < G && ml[i].y > 0.0f) ? ml[i].x : -CUDART_INF_F;    // a split that saw no key, or a clamped repeat
            m = fmaxf(m, ml[i].x);
        }
        if (m == -CUDART_INF_F) m = 0.0f;            // no split saw a key for this row: weights are all 0
        float l = 0.0f, a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int i = 0; i < GC; ++i) {
            const float w = ex2f(ml[i].x - m);
            l = fmaf(w, ml[i].y, l);
            if (i & 1) a1 = fmaf(w, o[i], a1); else a0 = fmaf(w, o[i], a0);
        }
        const float acc = a0 + a1;
        if (a.partial_export) {
            a.partial_export[(size_t)grow * (HD + 2) + d] = acc;
            if (d == 0) {
                a.partial_export[(size_t)grow * (HD + 2) + HD] = l > 0.0f ? m * LN2 : 0.0f;
                a.partial_export[(size_t)grow * (HD + 2) + HD + 1] = l;
            }
        } else {
            const float v = l > 0.0f ? acc / l : 0.0f;
            const long oi = a.b * a.out_batch_stride + (long)hrow * HD + d;
            if (a.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(a.out)[oi] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(a.out)[oi] = v;
        }
    };
    if (G <= 8) run(std::integral_constant<int, 8>{});
    else if (G <= 16) run(std::integral_constant<int, 16>{});
    else if (G <= 24) run(std::integral_constant<int, 24>{});
    else run(std::integral_constant<int, 32>{});
}
// Merges of more elements than threads with at most 12 splits (speculative verify: 18 rows x 128 dims,
// 9 splits).  Same idea as merge_small, no staging and no barrier.  A thread takes four pairs of dims
// per round (partial rows are 8-byte aligned) and requests all their splits' outputs at once; the 32
// lanes of a warp hold consecutive pairs of ONE row (a row is HD/2 pairs, a multiple of 32), so the
// row's weights are worked out across the warp -- lane k fetches (m, l) of split k, two warp reductions
// give the reference and the denominator -- and handed round by shuffle.  Up to 52 independent loads per
// thread, one round trip to L2 per round; verify needs a single round.
// [begin, end) restricts the call to a share of the unit's pairs (both multiples of 32: a warp's pairs share a row).
template <int HD, int GC, int EL = 4>
__device__ __noinline__ void merge_medium(const SmallMergeArgs a, int tid, int nthr, int begin = 0, int end = 1 << 30) {
    constexpr int HP = HD / 2;
    static_assert(HP % 32 == 0 && GC <= 32, "a warp's pairs share a row; one lane per split");
    const int total = min(end, a.nrows * HP), G = a.G, lane = tid & 31;
#pragma unroll 1
    for (int e0 = begin + tid; e0 < total; e0 += EL * nthr) {
        const float *base[EL];
        long grow[EL];
        int hrow[EL], dd[EL];
        float2 v[EL][GC], ml[EL];
#pragma unroll
        for (int j = 0; j < EL; ++j) {
            const int e = min(e0 + j * nthr, total - 1);
            const int sl = e / HP;
            dd[j] = 2 * (e - sl * HP);
            const int idx = a.first + sl;
            const int r = a.kvg_magic ? (int)__umulhi((unsigned)idx, a.kvg_magic) : idx;
            hrow[j] = r * a.nh + a.kvh * a.kvg + (idx - r * a.kvg);
            grow[j] = (long)a.b * a.S * a.nh + hrow[j];
            base[j] = a.partial + (size_t)grow[j] * (HD + 2);
        }
#pragma unroll
        for (int j = 0; j < EL; ++j) {
            ml[j] = __ldcg(reinterpret_cast<const float2 *>(base[j] + (size_t)min(lane, G - 1) * a.rstride + HD));
#pragma unroll
            for (int k = 0; k < GC; ++k)
                v[j][k] = __ldcg(reinterpret_cast<const float2 *>(base[j] + (size_t)min(k, G - 1) * a.rstride + dd[j]));
        }
#pragma unroll
        for (int j = 0; j < EL; ++j) {
            const float mk = (lane < G && ml[j].y > 0.0f) ? ml[j].x : -CUDART_INF_F;   // a split that saw no key, or no split
            float m = warp_max(mk);
            if (m == -CUDART_INF_F) m = 0.0f;
            const float wk = ex2f(mk - m);
            float l = wk * ml[j].y;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            float ox = 0.0f, oy = 0.0f;
#pragma unroll
            for (int k = 0; k < GC; ++k) {
                const float w = __shfl_sync(0xffffffffu, wk, k);          // 0 from lanes past the last split
                ox = fmaf(w, v[j][k].x, ox);
                oy = fmaf(w, v[j][k].y, oy);
            }
            if (e0 + j * nthr >= total) continue;
            if (a.partial_export) {
                float *pe = a.partial_export + (size_t)grow[j] * (HD + 2);
                *reinterpret_cast<float2 *>(pe + dd[j]) = make_float2(ox, oy);
                if (dd[j] == 0) *reinterpret_cast<float2 *>(pe + HD) = make_float2(l > 0.0f ? m * LN2 : 0.0f, l);
            } else {
                const float vx = l > 0.0f ? ox / l : 0.0f, vy = l > 0.0f ? oy / l : 0.0f;
                const long oi = a.b * a.out_batch_stride + (long)hrow[j] * HD + dd[j];
                if (a.out_type == ET_BF16) *reinterpret_cast<__nv_bfloat162 *>(reinterpret_cast<__nv_bfloat16 *>(a.out) + oi) = __floats2bfloat162_rn(vx, vy);
                else *reinterpret_cast<float2 *>(reinterpret_cast<float *>(a.out) + oi) = make_float2(vx, vy);
            }
        }
    }
}
// A unit's merge arguments; true when it takes the small path.
template <int NSLOT, int HD, int NTHR>
__device__ __forceinline__ bool small_merge_args(const KParams &p, int b, int kvh, int rg, SmallMergeArgs &a) {
    a.partial = p.partial; a.partial_export = p.partial_export; a.out = p.out;
    a.rstride = (long)p.grows * (HD + 2); a.out_batch_stride = p.out_batch_stride;
    a.G = p.splits; a.S = p.S; a.nh = p.nh; a.kvg = p.kvg; a.out_type = p.out_type; a.kvg_magic = p.kvg_magic;
    a.b = b; a.kvh = kvh; a.first = rg * NSLOT; a.nrows = min(NSLOT, p.S * p.kvg - rg * NSLOT);
    return p.counters != nullptr && p.splits <= 32 && a.nrows * HD <= NTHR;
}

// The barrier-free merges: runs the one that fits the unit, if any.
template <int NSLOT, int HD, int NTHR>
__device__ __forceinline__ bool merge_without_staging(const KParams &p, int b, int kvh, int rg, int tid, int nthr) {
    SmallMergeArgs sa;
    if (small_merge_args<NSLOT, HD, NTHR>(p, b, kvh, rg, sa)) {
        merge_small<HD>(sa, tid);
        return true;
    }
    if (p.counters == nullptr) return false;
    // outputs and exported partials must take 8-byte stores for the paired path
    const bool al8 = ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.partial_export)) & 7) == 0 &&
                     (p.out_batch_stride & 3) == 0;
    if (p.splits > 12 || !al8) return false;
    if (p.splits <= 4) merge_medium<HD, 4>(sa, tid, nthr);
    else if (p.splits <= 8) merge_medium<HD, 8>(sa, tid, nthr);
    else merge_medium<HD, 12>(sa, tid, nthr);
    return true;
}

// In-kernel merge across the splits of one (batch, KV head, row group) unit, called by every
// thread of a CTA after its partial (o, m, l) rows are stored.  The last CTA of the unit to
// arrive merges the unit's rows; the others return.  `scratch` is shared memory the CTA no
// longer needs, at least 8 * NSLOT * splits bytes.
// One arrival on a tagged counter word; returns how many have arrived including this one, or -1 if the word could
// not be brought under the tag within the try limit.  The word is (tag << 16 | round bit << 15 | arrivals): the CTA
// that closes a round leaves it tagged with zero arrivals, so the common case is a single atomic add.  The round bit
// is what the cooperative merge's waiters watch: the last arrival of a round flips it (and zeroes the count in the
// same store), so "everybody has arrived" needs no second word and nobody has to reset anything afterwards.  A word without the tag has never
// been used by this library (the workspace is caller-owned and arrives uninitialised): the add went to garbage, and
// the arrivals that find garbage install a tagged word with compare-and-swap, which only fails when another arrival
// made progress.
constexpr unsigned long long ARRIVE_TAG = 0x6e6f6d6f7341ull;
__device__ __forceinline__ int tagged_arrive(unsigned long long *ctr, int *round_bit = nullptr) {
    unsigned long long old = arrive_add(ctr);
    const auto done = [&](unsigned long long o) {
        if (round_bit) *round_bit = (int)((o >> 15) & 1ull);
        return (int)(o & 0x7fffull) + 1;
    };
    if ((old >> 16) == ARRIVE_TAG) return done(old);
    for (int tries = 0; tries < (1 << 16); ++tries) {            // bounded: gives up rather than spin forever
        const unsigned long long cur = *reinterpret_cast<volatile unsigned long long *>(ctr);
        if ((cur >> 16) == ARRIVE_TAG) {
            old = arrive_add(ctr);
            if ((old >> 16) == ARRIVE_TAG) return done(old);
        } else {
            __threadfence();          // rare path: plain fences around the compare-and-swap
            const bool won = atomicCAS(ctr, cur, (ARRIVE_TAG << 16) | 1ull) == cur;
            __threadfence();
            if (won) { if (round_bit) *round_bit = 0; return 1; }
        }
    }
    return -1;
}
__device__ __forceinline__ void st_release_gpu(unsigned long long *addr, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;\n" ::"l"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long *addr) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];\n" : "=l"(v) : "l"(addr) : "memory");
    return v;
}

// Cooperative merge: CTA number `share` of the G that make up a unit merges pairs [share * per, (share + 1) * per) of
// the unit's nrows * HD / 2 output pairs, instead of the last CTA merging all of them through one SM (84 KB of
// partials for a verify call, 600 KB for a 512-wide head).  A warp takes EL pairs at a time; lane k fetches split k's
// (m, l) and partial outputs of those pairs (a second round for splits 32..63), so every load of the warp is in
// flight at once; the reference, the denominator and the sums are warp reductions.
template <int HD>
__device__ __noinline__ void merge_coop(const SmallMergeArgs a, int share, int nshares, int tid, int nthr) {
    constexpr int EL = 4, HP = HD / 2;
    const int G = a.G, lane = tid & 31, warp = tid >> 5, nwarp = nthr >> 5;
    const int total = a.nrows * HP;
    const int per = (total + nshares - 1) / nshares;
    const int begin = share * per, end = min(total, begin + per);
#pragma unroll 1
    for (int e0 = begin + warp * EL; e0 < end; e0 += nwarp * EL) {
        float2 ml[2][EL], v[2][EL];
        long grow[EL];
        int hrow[EL], dd[EL];
#pragma unroll
        for (int j = 0; j < EL; ++j) {
            const int e = min(e0 + j, end - 1);
            const int sl = e / HP;
            dd[j] = 2 * (e - sl * HP);
            const int idx = a.first + sl;
            const int r = a.kvg_magic ? (int)__umulhi((unsigned)idx, a.kvg_magic) : idx;
            hrow[j] = r * a.nh + a.kvh * a.kvg + (idx - r * a.kvg);
            grow[j] = (long)a.b * a.S * a.nh + hrow[j];
        }
#pragma unroll
        for (int rd = 0; rd < 2; ++rd) {
            const int k = min(lane + 32 * rd, G - 1);
            if (rd == 1 && G <= 32) break;
#pragma unroll
            for (int j = 0; j < EL; ++j) {
                const float *row = a.partial + (size_t)k * a.rstride + (size_t)grow[j] * (HD + 2);
                ml[rd][j] = __ldcg(reinterpret_cast<const float2 *>(row + HD));
                v[rd][j] = __ldcg(reinterpret_cast<const float2 *>(row + dd[j]));
            }
        }
#pragma unroll
        for (int j = 0; j < EL; ++j) {
            float mk[2], m = -CUDART_INF_F;
#pragma unroll
            for (int rd = 0; rd < 2; ++rd) {
                const bool live = (rd == 0 || G > 32) && lane + 32 * rd < G && ml[rd][j].y > 0.0f;   // a split that saw a key
                mk[rd] = live ? ml[rd][j].x : -CUDART_INF_F;
                m = fmaxf(m, mk[rd]);
            }
            m = warp_max(m);
            if (m == -CUDART_INF_F) m = 0.0f;
            float l = 0.0f, ox = 0.0f, oy = 0.0f;
#pragma unroll
            for (int rd = 0; rd < 2; ++rd) {
                if (rd == 1 && G <= 32) break;
                const float w = ex2f(mk[rd] - m);                  // 0 for dead lanes
                l = fmaf(w, ml[rd][j].y, l);
                ox = fmaf(w, v[rd][j].x, ox);
                oy = fmaf(w, v[rd][j].y, oy);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                l += __shfl_xor_sync(0xffffffffu, l, o);
                ox += __shfl_xor_sync(0xffffffffu, ox, o);
                oy += __shfl_xor_sync(0xffffffffu, oy, o);
            }
            if (lane != 0 || e0 + j >= end) continue;
            if (a.partial_export) {
                float *pe = a.partial_export + (size_t)grow[j] * (HD + 2);
                *reinterpret_cast<float2 *>(pe + dd[j]) = make_float2(ox, oy);
                if (dd[j] == 0) *reinterpret_cast<float2 *>(pe + HD) = make_float2(l > 0.0f ? m * LN2 : 0.0f, l);
            } else {
                const float vx = l > 0.0f ? ox / l : 0.0f, vy = l > 0.0f ? oy / l : 0.0f;
                const long oi = a.b * a.out_batch_stride + (long)hrow[j] * HD + dd[j];
                if (a.out_type == ET_BF16) *reinterpret_cast<__nv_bfloat162 *>(reinterpret_cast<__nv_bfloat16 *>(a.out) + oi) = __floats2bfloat162_rn(vx, vy);
                else *reinterpret_cast<float2 *>(reinterpret_cast<float *>(a.out) + oi) = make_float2(vx, vy);
            }
        }
    }
}

// The cooperative form of the unit merge, out of line (it runs once per CTA; p is the kernels' __grid_constant__
// parameter block).  The last K = p.coop_merge CTAs of the unit to arrive each merge 1/K of its rows: a CTA that
// arrives earlier leaves at once (its SM is free for the next launch), one of the K waits -- with a time limit --
// until the last arrival has flipped the word's round bit, merges its share and leaves.  The whole grid is resident at once (host-checked), so the CTAs waited for are running.
template <int NSLOT, int HD, int NTHR>
__device__ __noinline__ void coop_merge_unit(const KParams &p, int b, int kvh, int rg) {
    __shared__ int s_go, s_share;
    unsigned long long *ctr = p.counters + ((size_t)blockIdx.z * gridDim.y + blockIdx.y);
    const int K = min(p.coop_merge, p.arrivals);
    __syncthreads();                      // all partial stores of this CTA are issued
    if (threadIdx.x == 0) {
        int round = 0;
        const int arrived = tagged_arrive(ctr, &round);
        s_share = arrived - (p.arrivals - K) - 1;
        bool all = arrived == p.arrivals;
        if (all) {
            // the last arrival closes the round: count back to zero, round bit flipped, in one release store (its
            // acquire-release arrival has seen every other CTA's partial rows; the waiters acquire this store)
            st_release_gpu(ctr, (ARRIVE_TAG << 16) | ((unsigned long long)(round ^ 1) << 15));
        } else if (s_share >= 0) {
            unsigned long long t0, t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            for (;;) {
                const unsigned long long cur = ld_acquire_gpu(ctr);
                if ((cur >> 16) == ARRIVE_TAG && (int)((cur >> 15) & 1ull) != round) { all = true; break; }
                __nanosleep(100);
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                if (t1 - t0 > 1000000000ull) { atomicOr(p.fault, 1u); break; }
            }
        }
        s_go = (s_share >= 0 && all) ? 1 : 0;
    }
    __syncthreads();
    if (!s_go) return;
    SmallMergeArgs sa;
    small_merge_args<NSLOT, HD, NTHR>(p, b, kvh, rg, sa);
    if (p.splits <= 12) {
        // few splits: the no-staging merge of verify calls on this CTA's share of the pairs, one pair per thread and
        // round (shares are whole warps' worth of pairs, so a warp's pairs still share a row)
        const int total = sa.nrows * (HD / 2);
        const int per = ((total + K - 1) / K + 31) / 32 * 32;
        const int begin = s_share * per, end = min(total, begin + per);
        if (p.splits <= 4) merge_medium<HD, 4, 1>(sa, threadIdx.x, NTHR, begin, end);
        else if (p.splits <= 8) merge_medium<HD, 8, 1>(sa, threadIdx.x, NTHR, begin, end);
        else if (p.splits <= 10) merge_medium<HD, 10, 1>(sa, threadIdx.x, NTHR, begin, end);
        else merge_medium<HD, 12, 1>(sa, threadIdx.x, NTHR, begin, end);
    } else {
        merge_coop<HD>(sa, s_share, K, threadIdx.x, NTHR);
    }
}

// Returns true in the CTA that merged the unit's rows (the last one to arrive).
template <int NSLOT, int HD, int NTHR, int GB = 8>
__device__ __forceinline__ bool merge_unit_splits(const KParams &p, uint8_t *scratch, int b, int kvh, int rg) {
    if (p.counters == nullptr) return false;
    if (p.coop_merge) {                   // (no single CTA then holds the unit's merged rows)
        coop_merge_unit<NSLOT, HD, NTHR>(p, b, kvh, rg);
        return false;
    }

    // ------------------------------------------- in-kernel merge across the splits
    // Arrival counting without a zeroed workspace (see the tag below).
    __shared__ int s_last;
    __syncthreads();                      // all partial stores of this CTA are issued
    if (threadIdx.x == 0) {
        // The arrival is one acquire-release atomic at GPU scope: release makes the whole CTA's partial
        // stores (ordered before it by the barrier above) visible before the count, acquire orders the
        // merging CTA's loads (all its threads, through the barrier below) after every other arrival.
        unsigned long long *ctr = p.counters + ((size_t)blockIdx.z * gridDim.y + blockIdx.y);
        const int arrived = tagged_arrive(ctr);
        if (arrived == p.arrivals) *ctr = ARRIVE_TAG << 16;             // clean for the next launch on this workspace
        s_last = (arrived == p.arrivals);
    }
    __syncthreads();
    if (!s_last) return false;
    // The last CTA of the unit merges its rows.  Phase A stages every split's (m, l) in shared
    // memory; phase B (a warp per row) turns them into weights 2^(m_i - m*) and the merged
    // denominator; phase C gives each thread (row, dim) elements and streams the splits' partial
    // outputs from L2 with many independent loads in flight.
    const int G = p.splits;
    float *ms = reinterpret_cast<float *>(scratch);      // [NSLOT][G]  m of each split, then its weight
    float *ls = ms + NSLOT * G;                          // [NSLOT][G]  l of each split
    __shared__ float s_mstar[NSLOT], s_lstar[NSLOT];
    const int first = rg * NSLOT;
    const int nrows = min(NSLOT, p.S * p.kvg - first);   // valid slots of this row group
    const size_t rstride = (size_t)p.grows * (HD + 2);
    auto grow_of = [&](int sl) {
        const int idx = first + sl;
        const int r = div_kvg(p, idx);
        return ((long)b * p.S + r) * p.nh + kvh * p.kvg + (idx - r * p.kvg);
    };
    // (m, l) of every split -> shared memory; then a warp per row: weights 2^(m_i - m*) and the merged denominator
    auto stage_weights = [&]() {
        for (int e = threadIdx.x; e < nrows * G; e += NTHR) {
            const int sl = e / G, i = e - sl * G;
            const float *pr = p.partial + (size_t)i * rstride + (size_t)grow_of(sl) * (HD + 2);
            const float2 ml = __ldcg(reinterpret_cast<const float2 *>(pr + HD));     // (m, l): 8-byte aligned, one round trip
            ls[sl * G + i] = ml.y;
            ms[sl * G + i] = ml.y > 0.0f ? ml.x : -CUDART_INF_F;
        }
        __syncthreads();
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int sl = warp; sl < nrows; sl += NTHR / 32) {
            float m = -CUDART_INF_F;
            for (int i = lane; i < G; i += 32) m = fmaxf(m, ms[sl * G + i]);
            m = warp_max(m);
            if (m == -CUDART_INF_F) m = 0.0f;            // no split saw a key for this row: weights are all 0
            float lp = 0.0f;
            for (int i = lane; i < G; i += 32) {
                const float w = ex2f(ms[sl * G + i] - m);
                lp = fmaf(w, ls[sl * G + i], lp);
                ms[sl * G + i] = w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lp += __shfl_xor_sync(0xffffffffu, lp, o);
            if (lane == 0) { s_mstar[sl] = m; s_lstar[sl] = lp; }
        }
        __syncthreads();
    };
    auto emit_ml = [&](int sl, int d, float o, float mstar, float lstar) {
        const long grow = grow_of(sl);
        if (p.partial_export) {
            p.partial_export[(size_t)grow * (HD + 2) + d] = o;
            if (d == 0) {
                p.partial_export[(size_t)grow * (HD + 2) + HD] = lstar > 0.0f ? mstar * LN2 : 0.0f;
                p.partial_export[(size_t)grow * (HD + 2) + HD + 1] = lstar;
            }
        } else {
            const float v = lstar > 0.0f ? o / lstar : 0.0f;
            const int idx = first + sl;
            const int r = div_kvg(p, idx);
            const long oi = b * p.out_batch_stride + ((long)r * p.nh + kvh * p.kvg + (idx - r * p.kvg)) * HD + d;
            if (p.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[oi] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(p.out)[oi] = v;
        }
    };
    auto emit = [&](int sl, int d, float o) { emit_ml(sl, d, o, s_mstar[sl], s_lstar[sl]); };
    if (merge_without_staging<NSLOT, HD, NTHR>(p, b, kvh, rg, threadIdx.x, NTHR)) return true;
    // General case: a thread takes EL pairs of dims at a time (partial rows are 8-byte aligned) and
    // up to GBW splits of each, every load of such a batch issued before the first use (clamped
    // instead of predicated, so they batch freely); the first batch is requested before the (m, l)
    // staging barrier, like above.  GBW follows the number of splits so that up to twelve take a
    // single round trip to L2.
    constexpr int EL = 4, HP = HD / 2;
    const int total = nrows * HP;
    auto general = [&](auto gbw_tag) {
        constexpr int GBW = decltype(gbw_tag)::value;
        const float *base[EL];
        int sl[EL];
        float2 v[EL][GBW];
        auto setup = [&](int e0) {
#pragma unroll
            for (int j = 0; j < EL; ++j) {
                const int e = min(e0 + j * NTHR, total - 1);
                sl[j] = e / HP;
                base[j] = p.partial + (size_t)grow_of(sl[j]) * (HD + 2) + 2 * (e - sl[j] * HP);
            }
        };
        auto issue = [&](int i0) {
#pragma unroll
            for (int j = 0; j < EL; ++j)
#pragma unroll
                for (int k = 0; k < GBW; ++k)
                    v[j][k] = __ldcg(reinterpret_cast<const float2 *>(base[j] + (size_t)min(i0 + k, G - 1) * rstride));
        };
        int e0 = threadIdx.x;
        setup(e0);
        issue(0);
        stage_weights();
        for (bool first_round = true; e0 < total; e0 += EL * NTHR, first_round = false) {
            if (!first_round) { setup(e0); issue(0); }
            float2 o[EL];
#pragma unroll
            for (int j = 0; j < EL; ++j) o[j] = make_float2(0.0f, 0.0f);
            for (int i0 = 0;;) {
#pragma unroll
                for (int j = 0; j < EL; ++j)
#pragma unroll
                    for (int k = 0; k < GBW; ++k) {
                        const float w = i0 + k < G ? ms[sl[j] * G + i0 + k] : 0.0f;
                        o[j].x = fmaf(w, v[j][k].x, o[j].x);
                        o[j].y = fmaf(w, v[j][k].y, o[j].y);
                    }
                i0 += GBW;
                if (i0 >= G) break;
                issue(i0);
            }
#pragma unroll
            for (int j = 0; j < EL; ++j) {
                const int e = e0 + j * NTHR;
                if (e < total) {
                    const int d = 2 * (e - sl[j] * HP);
                    emit(sl[j], d, o[j].x);
                    emit(sl[j], d + 1, o[j].y);
                }
            }
        }
    };
    if (G <= 4) general(std::integral_constant<int, 4>{});
    else if (G <= 8) general(std::integral_constant<int, 8>{});
    else general(std::integral_constant<int, 12>{});
    return true;
}

// ---- sequence shards on several GPUs: exchange of the merged rows through peer memory
__device__ __forceinline__ void st_release_sys(unsigned long long *addr, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;\n" ::"l"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *addr) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(addr) : "memory");
    return v;
}

// Called by every thread of the CTA that merged a unit's splits into this rank's own mailbox rows
// (p.partial_export points at them; m in natural-log units).  Three steps, one launch, no collective library:
//   1. push: the unit's rows are copied into the same place of every peer's mailbox with plain stores to
//      peer-mapped memory (NVLink), then each row's stamp is released at system scope with the step number;
//   2. wait: thread (peer, row) polls this rank's own mailbox for the peer's stamp of this step, for at most
//      peer_timeout_ns; a peer that never shows up raises fault bit 2 and the CTA returns without an output;
//   3. merge: the world's rows of each query row are combined exactly like split partials and normalised.
// Mailboxes have two step slots (step & 1): a rank can be at most one step ahead of a peer it exchanged with,
// so the slot a push overwrites was consumed two steps ago.  Nothing here is multicast, and no thread waits
// without a limit.
// (p is the kernels' __grid_constant__ parameter block: its address can be handed to this out-of-line function
// without the compiler keeping a per-thread copy of it.)
template <int NSLOT, int HD, int NTHR>
__device__ __noinline__ void peer_exchange_and_merge(const KParams &p, int b, int kvh, int rg) {
    __shared__ int s_peer_ok;
    const int G = p.peer_world, me = p.peer_rank, tid = threadIdx.x;
    const int slot = (int)(p.peer_seq & 1ull);
    const int first = rg * NSLOT;
    const int nrows = min(NSLOT, p.S * p.kvg - first);
    const size_t blk = (size_t)p.grows * (HD + 2);                   // floats of one (slot, source rank) block
    auto grow_of = [&](int sl) {
        const int idx = first + sl;
        const int r = p.kvg_magic ? (int)__umulhi((unsigned)idx, p.kvg_magic) : idx;
        return ((long)b * p.S + r) * p.nh + kvh * p.kvg + (idx - r * p.kvg);
    };
    if (tid == 0) s_peer_ok = 1;
    __syncthreads();                                                 // this CTA's merged rows are written
    // ---- 1. push
    constexpr int RP = (HD + 2) / 2;                                 // float2 per row
    const int per_peer = nrows * RP;
    for (int e = tid; e < per_peer * (G - 1); e += NTHR) {
        const int gi = e / per_peer, rem = e - gi * per_peer;
        const int g = gi + (gi >= me ? 1 : 0);
        const int sl = rem / RP, c = rem - sl * RP;
        const size_t off = ((size_t)slot * G + me) * blk + (size_t)grow_of(sl) * (HD + 2) + 2 * c;
        const float2 v = __ldcg(reinterpret_cast<const float2 *>(p.peer_rows[me] + off));
        *reinterpret_cast<float2 *>(p.peer_rows[g] + off) = v;
    }
    // The stamps are released at system scope by the threads that write them; the CTA barrier in front orders every
    // thread's row stores before them (release is cumulative over what the barrier made visible to the releasing
    // thread), so no thread pays for a system-wide fence of its own.
    __syncthreads();
    for (int e = tid; e < nrows * (G - 1); e += NTHR) {
        const int gi = e / nrows, sl = e - gi * nrows;
        const int g = gi + (gi >= me ? 1 : 0);
        st_release_sys(p.peer_flags[g] + ((size_t)slot * G + me) * p.grows + grow_of(sl), p.peer_seq);
    }
    // ---- 2. wait
    for (int e = tid; e < nrows * (G - 1); e += NTHR) {
        const int gi = e / nrows, sl = e - gi * nrows;
        const int g = gi + (gi >= me ? 1 : 0);
        const unsigned long long *f = p.peer_flags[me] + ((size_t)slot * G + g) * p.grows + grow_of(sl);
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        bool seen = ld_acquire_sys(f) == p.peer_seq;
        while (!seen) {
#pragma unroll 1
            for (int k = 0; k < 16 && !seen; ++k) { __nanosleep(40); seen = ld_acquire_sys(f) == p.peer_seq; }
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (!seen && t1 - t0 > p.peer_timeout_ns) break;
        }
        if (!seen) { s_peer_ok = 0; atomicOr(p.fault, 4u); }
    }
    __syncthreads();
    if (!s_peer_ok) return;
    // ---- 3. merge the world's rows (rank me's own rows included) and write the normalised output
    for (int e = tid; e < nrows * HD; e += NTHR) {
        const int sl = e / HD, d = e - sl * HD;
        const long grow = grow_of(sl);
        const float *base = p.peer_rows[me] + (size_t)slot * G * blk + (size_t)grow * (HD + 2);
        float m = -CUDART_INF_F;
        float mg[8], lg[8], og[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float *row = base + (size_t)min(g, G - 1) * blk;
            const float2 ml = __ldcg(reinterpret_cast<const float2 *>(row + HD));
            og[g] = __ldcg(row + d);
            lg[g] = g < G ? ml.y : 0.0f;
            mg[g] = (g < G && ml.y > 0.0f) ? ml.x * LOG2E : -CUDART_INF_F;       // exported m is in natural-log units
            m = fmaxf(m, mg[g]);
        }
        if (m == -CUDART_INF_F) m = 0.0f;
        float l = 0.0f, acc = 0.0f;
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float w = ex2f(mg[g] - m);
            l = fmaf(w, lg[g], l);
            acc = fmaf(w, og[g], acc);
        }
        const float v = l > 0.0f ? acc / l : 0.0f;
        const int idx = first + sl;
        const int r = p.kvg_magic ? (int)__umulhi((unsigned)idx, p.kvg_magic) : idx;
        const long oi = b * p.out_batch_stride + ((long)r * p.nh + kvh * p.kvg + (idx - r * p.kvg)) * HD + d;
        if (p.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[oi] = __float2bfloat16_rn(v);
        else reinterpret_cast<float *>(p.out)[oi] = v;
    }
}

// In-kernel tail of every attention CTA: the split merge and, on a sequence-sharded call, the exchange with the
// other GPUs' shards.
// The split merge when a unit's splits are the CTAs of one thread-block cluster (grid x = splits = cluster x).
// Every CTA has left its own merged rows (o[HD], m, l per slot, base-2 m) at `cpart` in its shared memory; after the
// cluster barrier CTA r takes dims [r * per, r * per + per) of every slot, reads the G rows' (m, l) and its dims
// from the peers' shared memory, and writes the normalised output.  A second cluster barrier keeps every CTA's
// shared memory alive until all have read it.  Both are hardware barriers over CTAs that are co-scheduled by
// construction (a cluster starts as a whole); no CTA leaves the kernel before them.
template <int NSLOT, int HD, int NTHR>
__device__ __noinline__ void cluster_merge_unit(const KParams &p, float *cpart, int b, int kvh, int rg) {
    namespace cg = cooperative_groups;
    cg::cluster_group cl = cg::this_cluster();
    const int G = (int)cl.num_blocks(), R = (int)cl.block_rank();
    cl.sync();
    const int first = rg * NSLOT;
    const int nrows = min(NSLOT, p.S * p.kvg - first);
    const int per = (HD + G - 1) / G;
    for (int item = threadIdx.x; item < nrows * per; item += NTHR) {
        const int sl = item / per, d = R * per + (item - sl * per);
        if (d >= HD) continue;
        float mi[16], li[16], oi[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i < G) {
                const float *row = cl.map_shared_rank(cpart, i) + (size_t)sl * (HD + 2);
                mi[i] = row[HD]; li[i] = row[HD + 1]; oi[i] = row[d];
            } else {
                mi[i] = 0.0f; li[i] = 0.0f; oi[i] = 0.0f;
            }
        }
        float m = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            mi[i] = li[i] > 0.0f ? mi[i] : -CUDART_INF_F;              // a split that saw no key (or no such split)
            m = fmaxf(m, mi[i]);
        }
        if (m == -CUDART_INF_F) m = 0.0f;
        float l = 0.0f, o = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float w = ex2f(mi[i] - m);
            l = fmaf(w, li[i], l);
            o = fmaf(w, oi[i], o);
        }
        const int idx = first + sl;
        const int r = div_kvg(p, idx);
        const float v = l > 0.0f ? o / l : 0.0f;
        const long oidx = b * p.out_batch_stride + ((long)r * p.nh + kvh * p.kvg + (idx - r * p.kvg)) * HD + d;
        if (p.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[oidx] = __float2bfloat16_rn(v);
        else reinterpret_cast<float *>(p.out)[oidx] = v;
    }
    cl.sync();
}

template <int NSLOT, int HD, int NTHR, int GB = 8>
__device__ __forceinline__ void merge_splits_in_kernel(const KParams &p, uint8_t *scratch, int b, int kvh, int rg) {
    const bool merged = merge_unit_splits<NSLOT, HD, NTHR, GB>(p, scratch, b, kvh, rg);
    if (merged && p.peer_world > 1) peer_exchange_and_merge<NSLOT, HD, NTHR>(p, b, kvh, rg);
}

template <int FMT, int HD, int MT, int DS = 1, int QS = 1>
__global__ void __launch_bounds__(Cfg<FMT, HD, MT, DS, QS>::NW * 32)
    attn_fused_kernel(const __grid_constant__ KParams p, const __grid_constant__ TmaMaps tm) {
    using C = Cfg<FMT, HD, MT, DS, QS>;
    constexpr int HDV = C::HDV;
    constexpr int NWARP = C::NW;
    constexpr int NQ = C::NQ;                 // tile streams of the CTA: one per warp, or one per quad of QS warps
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *pipe = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // K/V tiles [NW][NSTAGE][2]
    uint8_t *sc_region = pipe + C::REGION0_BYTES;                                  // scales  [NW][NSTAGE][2]
    uint8_t *qreg = sc_region + C::SCALES_BYTES;
    int8_t *q_limbs = reinterpret_cast<int8_t *>(qreg);                        // [2][NSLOT][HD]
    float *slot_qscale = reinterpret_cast<float *>(qreg + C::Q_BYTES);         // [NSLOT]
    int *slot_lo = reinterpret_cast<int *>(qreg + C::Q_BYTES + C::NSLOT * 4);
    int *slot_hi = reinterpret_cast<int *>(qreg + C::Q_BYTES + C::NSLOT * 8);
    int *slot_qsum = reinterpret_cast<int *>(qreg + C::Q_BYTES + C::NSLOT * 16);   // [NSLOT][NBLK]
    uint8_t *append_scratch = qreg + C::Q_BYTES + C::SLOT_BYTES;                  // [NW][ROWB + 64]
    const uint32_t bars_u32 = smem_u32(append_scratch + C::APPEND_BYTES);         // [NW][NSTAGE] mbarriers
    float *xch_region = reinterpret_cast<float *>(append_scratch + C::APPEND_BYTES + C::BAR_BYTES);   // quads' partial logits

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int quad = warp / QS, wj = warp % QS;                                     // tile stream of this warp, its slice in the quad
    const int split = blockIdx.x / DS, dsl = blockIdx.x % DS, kvh = blockIdx.y;     // dsl: head-dim slice of this CTA
    const int b = blockIdx.z / p.row_groups, rg = blockIdx.z % p.row_groups;

    // ------------------------------------------------------------ tile schedule
    const int tile_begin = p.tile0 + split * p.tiles_per_split;
    const int tile_end = min(p.tile0 + p.ntiles, tile_begin + p.tiles_per_split);
    const int my_first = tile_begin + quad;
    const int my_count = my_first < tile_end ? (tile_end - my_first + NQ - 1) / NQ : 0;

    const int row_stride = (FMT == KV_I8) ? p.cache_hd : p.cache_hd / 2;   // bytes between consecutive token rows
    const uint8_t *kbase = p.k_cache + b * p.kv_batch_stride + (size_t)kvh * p.cache_cap * (size_t)row_stride + wj * C::ROWBK;
    const uint8_t *vbase = p.v_cache + b * p.kv_batch_stride + (size_t)kvh * p.cache_cap * (size_t)row_stride + (dsl * QS + wj) * C::ROWBV;
    constexpr int SC_SLICE = (FMT == KV_I4B32) ? C::SCBW : 0;                // block scales are sliced with the dims, row scales are not
    const uint8_t *ksbase = p.k_scales + b * p.scale_batch_stride + (size_t)kvh * p.cache_cap * C::SCB + wj * SC_SLICE;
    const uint8_t *vsbase = p.v_scales + b * p.scale_batch_stride + (size_t)kvh * p.cache_cap * C::SCB + wj * SC_SLICE;

    uint8_t *my_pipe = pipe + warp * NSTAGE * C::ST_BYTES;           // stage s: K tile, V tile (slice)
    uint8_t *my_sc = sc_region + warp * NSTAGE * 2 * C::SC_BYTES;    // stage s: K scales, V scales
    const uint32_t my_pipe_u32 = smem_u32(my_pipe), my_sc_u32 = smem_u32(my_sc);
    const uint32_t my_bar_u32 = bars_u32 + warp * NSTAGE * 8;
    const int ring0 = p.win_start % p.cache_cap;

    // TMA path: one lane requests a whole tile (two tensor copies + two bulk copies of scales)
    // against the stage's mbarrier; the warp waits on the barrier's phase.  tma_mask marks the
    // stages whose current tile came that way, phase_bits their barrier parity.
    uint32_t tma_mask = 0, phase_bits = 0;
    if constexpr (C::TMA_OK) {
        if (p.use_tma && lane == 0) {
#pragma unroll
            for (int s = 0; s < NSTAGE; ++s) mbar_init(my_bar_u32 + 8 * s, 1);
            fence_mbar_init();
        }
        __syncwarp();
    }

    // Copy geometry: per cp.async instruction the warp covers 8 rows x 64 bytes; lane = (row r, chunk c0).
    constexpr int HPASS = C::CHUNKSK / 4;                    // 64-byte column groups per row (of this warp's K slice)
    const int cr = lane >> 2, cc0 = lane & 3;
    const size_t lane_goff = (size_t)cr * row_stride + cc0 * 16;
    uint32_t lane_soff[HPASS];
#pragma unroll
    for (int h = 0; h < HPASS; ++h) lane_soff[h] = cr * C::ROWBK + swz_chunk<C::ROWBK>(cr, cc0 + 4 * h) * 16;
    constexpr int HPASSV = C::CHUNKSV / 4;
    uint32_t lane_soffv[HPASSV];
#pragma unroll
    for (int h = 0; h < HPASSV; ++h) lane_soffv[h] = cr * C::ROWBV + swz_chunk<C::ROWBV>(cr, cc0 + 4 * h) * 16;

    // one token's scale bytes (4: fp32 row scale; 2 per block of 32 for the block-32 layout)
    auto copy_scales = [&](uint32_t dst, const uint8_t *src, bool ok) {
        if constexpr (C::SCBW == 4) cp_async4(dst, src, ok ? 4 : 0);
        else if constexpr (C::SCBW == 8) cp_async8(dst, src, ok ? 8 : 0);
        else {
#pragma unroll
            for (int o = 0; o < C::SCBW; o += 16) cp_async16(dst + o, src + o, ok ? 16 : 0);
        }
    };
    auto issue = [&](int it) {
        if (it < my_count) {
            const int tok0 = (my_first + it * NQ) * TILE;
            const int stg = it % NSTAGE;
            const uint32_t st = my_pipe_u32 + stg * C::ST_BYTES;
            const uint32_t ss = my_sc_u32 + stg * 2 * C::SC_BYTES;
            int slot0 = ring0 + tok0;
            slot0 = slot0 >= p.cache_cap ? slot0 - p.cache_cap : slot0;          // klen <= cache_cap (host-checked)
            const bool whole = slot0 + TILE <= p.cache_cap && tok0 + TILE <= p.klen;
            tma_mask &= ~(1u << stg);
            if (C::TMA_OK && p.use_tma && whole) {
                // the 32 rows are contiguous in the ring and inside the window: one box per plane
                const bool bulk_sc = (p.use_tma & 2) && ((slot0 * C::SCB) & 15) == 0;
                fence_proxy_async();          // earlier generic-proxy accesses of the stage precede the copies
                __syncwarp();
                if (lane == 0) {
                    const uint32_t bar = my_bar_u32 + 8 * stg;
                    mbar_expect_tx(bar, 2 * C::KV_BYTES + (bulk_sc ? 2 * C::SC_BYTES : 0));
                    if (p.kv_read_once) {
                        tma_load_tile_once(st, &tm.k, kvh * p.cache_cap + slot0, b, bar);
                        tma_load_tile_once(st + C::KV_BYTES, &tm.v, kvh * p.cache_cap + slot0, b, bar);
                    } else {
                        tma_load_tile(st, &tm.k, kvh * p.cache_cap + slot0, b, bar);
                        tma_load_tile(st + C::KV_BYTES, &tm.v, kvh * p.cache_cap + slot0, b, bar);
                    }
                    if (bulk_sc) {
                        bulk_load(ss, ksbase + (size_t)slot0 * C::SCB, C::SC_BYTES, bar);
                        bulk_load(ss + C::SC_BYTES, vsbase + (size_t)slot0 * C::SCB, C::SC_BYTES, bar);
                    }
                }
                if (!bulk_sc) {
                    const size_t sg = (size_t)(slot0 + lane) * C::SCB;
                    copy_scales(ss + lane * C::SCBW, ksbase + sg, true);
                    copy_scales(ss + C::SC_BYTES + lane * C::SCBW, vsbase + sg, true);
                }
                tma_mask |= 1u << stg;
            } else if (whole) {
                // cp.async path: 16-byte coalesced copies into the same swizzled layout (evict-first in L2 when the
                // launch reads every cache byte once; only where this is the regular path, the wide heads)
                const uint8_t *gk = kbase + (size_t)slot0 * row_stride + lane_goff;
                const uint8_t *gv = vbase + (size_t)slot0 * row_stride + lane_goff;
                const bool once = !C::TMA_OK && p.kv_read_once;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int h = 0; h < HPASS; ++h)
                        cp_async16_hint(st + lane_soff[h] + 8 * i * C::ROWBK, gk + (size_t)(8 * i) * row_stride + 64 * h, once);
#pragma unroll
                    for (int h = 0; h < HPASSV; ++h)
                        cp_async16_hint(st + C::KV_BYTES + lane_soffv[h] + 8 * i * C::ROWBV, gv + (size_t)(8 * i) * row_stride + 64 * h, once);
                }
                const size_t sg = (size_t)(slot0 + lane) * C::SCB;
                copy_scales(ss + lane * C::SCBW, ksbase + sg, true);
                copy_scales(ss + C::SC_BYTES + lane * C::SCBW, vsbase + sg, true);
            } else {
                // ragged tile: wraps the ring or runs past the window; rows past the end are zero-filled
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = tok0 + cr + 8 * i;
                    int slot = ring0 + tok;
                    slot = slot >= p.cache_cap ? slot - p.cache_cap : slot;
                    const bool ok = tok < p.klen;
                    const size_t go = (size_t)(ok ? slot : 0) * row_stride + cc0 * 16;
#pragma unroll
                    for (int h = 0; h < HPASS; ++h) cp_async16(st + lane_soff[h] + 8 * i * C::ROWBK, kbase + go + 64 * h, ok ? 16 : 0);
#pragma unroll
                    for (int h = 0; h < HPASSV; ++h)
                        cp_async16(st + C::KV_BYTES + lane_soffv[h] + 8 * i * C::ROWBV, vbase + go + 64 * h, ok ? 16 : 0);
                }
                const int tok = tok0 + lane;
                int slot = ring0 + tok;
                slot = slot >= p.cache_cap ? slot - p.cache_cap : slot;
                const bool ok = tok < p.klen;
                const size_t sg = (size_t)(ok ? slot : 0) * C::SCB;
                copy_scales(ss + lane * C::SCBW, ksbase + sg, ok);
                copy_scales(ss + C::SC_BYTES + lane * C::SCBW, vsbase + sg, ok);
            }
        }
        cp_async_commit();
    };

    // Programmatic dependent launch.  This grid may have been set up while its predecessor in
    // the stream was still running: wait for the predecessor's memory (the query, freshly
    // appended cache rows, the shared split workspace) before the first global access.  Then let
    // the split-merge grid be set up right away; it blocks the same way until this grid is done.
    // Cache rows the caller declared settled (not written by the stream predecessor) are requested
    // before that wait, so the pipeline fill overlaps the predecessor's tail.
    int early_n = 0;
    while (early_n < NSTAGE - 1 && early_n < my_count && (my_first + early_n * NQ + 1) * TILE <= p.early_rows) issue(early_n++);
    // ------------------------------------------- fused quantize-on-write of the new keys
    // The newest n_new keys arrive as fp32 rows.  A warp quantises one (row, plane) with the row codec
    // of the append kernels (bit for bit) into its scratch row [codes | scales]; for row group 0 and
    // head-dim slice 0 -- so exactly once per KV head -- it also copies bytes and scales into the
    // ring for later calls.  Returns the block-32 row's cached q8 scale (unused otherwise).
    auto quantize_new = [&](int i, int kv, uint8_t *scr, bool store) {
        const float *src = (kv ? p.new_v : p.new_k) + ((size_t)b * p.n_new + i) * p.new_stride + kvh * HD;
        const size_t crow = (size_t)kvh * p.cache_cap + (size_t)((p.new_base_pos + i) % p.cache_cap);
        float q8s = 0.0f;
        if constexpr (FMT == KV_I8) {
            quant_row_i8_cg(src, HD, HD, reinterpret_cast<int8_t *>(scr), reinterpret_cast<float *>(scr + C::ROWB), lane);
        } else if constexpr (FMT == KV_I4) {
            const float sc = quant_row_i4<true>(src, HD, HD, scr, nullptr, lane);
            if (lane == 0) *reinterpret_cast<float *>(scr + C::ROWB) = sc;
        } else {
            q8s = quant_row_i4_block32<true>(src, HD, scr, reinterpret_cast<__half *>(scr + C::ROWB), lane);
        }
        __syncwarp();
        if (rg == 0 && dsl == 0 && store) {
            uint8_t *g_rows = (kv ? p.v_cache_w : p.k_cache_w) + b * p.kv_batch_stride + crow * row_stride;
            uint8_t *g_sc = (kv ? p.v_scales_w : p.k_scales_w) + b * p.scale_batch_stride;
            // the row, zero-padded to the cache row width like the append kernels do (block-32 rows are never wider)
            const int row_chunks = (FMT == KV_I4B32) ? C::CHUNKS : row_stride / 16;
            for (int c = lane; c < row_chunks; c += 32)
                reinterpret_cast<uint4 *>(g_rows)[c] = c < C::CHUNKS ? reinterpret_cast<const uint4 *>(scr)[c] : make_uint4(0, 0, 0, 0);
            if constexpr (FMT == KV_I4B32) {
                if (lane < C::NBLK) reinterpret_cast<uint16_t *>(g_sc)[crow * C::NBLK + lane] = reinterpret_cast<const uint16_t *>(scr + C::ROWB)[lane];
                if (lane == 0) reinterpret_cast<float *>(g_sc + (size_t)p.nkv * p.cache_cap * C::NBLK * 2)[crow] = q8s;
            } else {
                if (lane == 0) reinterpret_cast<float *>(g_sc)[crow] = *reinterpret_cast<const float *>(scr + C::ROWB);
            }
        }
    };
    // A single new row (decode) is quantised NOW, while the first tiles and the query are in flight, by two
    // warps (K and V) of the CTA that owns its tile, so that the codec's global round trips are off the path
    // of the warp that will use the row; the CTA barrier after the query prologue publishes the scratch rows.
    const int new_tile = (p.klen - 1) / TILE;                             // tile of the newest key
    const bool early_new = p.new_k != nullptr && p.n_new == 1 && NWARP >= 2 && new_tile >= tile_begin && new_tile < tile_end;
    const int new_owner = early_new ? (new_tile - tile_begin) % NWARP : -1;
    const int new_helper = early_new ? (new_owner + 1) % NWARP : -1;

    // The query preparation (and the early quantisation of a single new row) runs twice.  The first pass
    // starts before the stream-order wait, on whatever the buffers hold at that moment, and its results are
    // thrown away (only shared-memory scratch is written): it brings this straight-line code into the
    // instruction caches while the CTA would otherwise idle behind its predecessor -- every launch streams far
    // more than L2 holds, so code a CTA runs once is otherwise fetched from device memory.
#pragma unroll 1
    // (a grid of several waves would only pay for the first pass; not compiled in for 512-wide heads, where the
    // pass is long and measured a loss)
    for (int pass = (HD <= 256 && p.dry_pass) ? 0 : 1; pass < 2; ++pass) {
        if (pass == 1) {
            pdl_wait();
            pdl_launch_dependents();
        }
        // ------------------------------------------------------------ Q prologue
        // Slot sl of this CTA = local row index rg*NSLOT + sl = (query row r, group head j).
        // The query loads go out first, then the first cache tiles are requested, so the (tiny) query
        // is not queued behind megabytes of prefetch and the pipeline fill overlaps its preparation.
        constexpr int QITER = (C::NSLOT + NWARP - 1) / NWARP;
        float qx[QITER][HD / 32];
    #pragma unroll
        for (int qi = 0; qi < QITER; ++qi) {
            const int sl = warp + qi * NWARP;
            const int idx = rg * C::NSLOT + sl;
            const int r = div_kvg(p, idx), j = idx - r * p.kvg;
            const bool valid = sl < C::NSLOT && r < p.S;
    #pragma unroll
            for (int i = 0; i < HD / 32; ++i)
                qx[qi][i] = valid ? load_q(p.q, p.q_type, b * p.q_batch_stride + ((long)r * p.nh + kvh * p.kvg + j) * HD + lane + 32 * i) : 0.0f;
        }
        if (pass == 1)
            for (int s = early_n; s < NSTAGE - 1; ++s) issue(s);
        if (warp == new_owner) quantize_new(0, 0, append_scratch + warp * (C::ROWB + 64), pass == 1);
        if (warp == new_helper) quantize_new(0, 1, append_scratch + warp * (C::ROWB + 64), pass == 1);

        // Each row becomes 16-bit fixed point: q ~= sq * (256*hi + lo), hi/lo int8.
    #pragma unroll
        for (int qi = 0; qi < QITER; ++qi) {
            const int sl = warp + qi * NWARP;
            if (sl >= C::NSLOT) break;
            const int idx = rg * C::NSLOT + sl;
            const int r = div_kvg(p, idx);
            const bool valid = r < p.S;
            float amax = 0.0f;
    #pragma unroll
            for (int i = 0; i < HD / 32; ++i) amax = fmaxf(amax, fabsf(qx[qi][i]));
            amax = warp_max(amax);
            const float sq = amax > 0.0f ? amax * (1.0f / (float)Q_FIX_MAX) : 1.0f;
            const float inv = rcpf(sq);
            int qblk[HD / 32];
    #pragma unroll
            for (int i = 0; i < HD / 32; ++i) {
                qblk[i] = 0;
                int qf = __float2int_rn(qx[qi][i] * inv);
                qf = max(-Q_FIX_MAX, min(Q_FIX_MAX, qf));
                const int hi = (qf + 128) >> 8;
                const int lo = qf - (hi << 8);
                int pos = lane + 32 * i;
                if constexpr (FMT != KV_I8) {
                    // int4 tiles hand element 32b+8t+2j+par of a row to MMA k slot 16*par+4t+j of step b
                    pos = 32 * i + ((lane & 1) << 4) + ((lane >> 3) << 2) + ((lane >> 1) & 3);
                    int bs = qf;                                        // sum of the block's fixed-point values
                    bs = __reduce_add_sync(0xffffffffu, bs);           // one instruction per block instead of five shuffle rounds
                    qblk[i] = bs;
                }
                // rows are stored with their 16-byte chunks XOR-swizzled by the slot index, so that the
                // ldmatrix that builds an A fragment (8 slots x one chunk) is free of bank conflicts
                const int spos = ((((pos >> 4) ^ (sl & 7)) << 4) | (pos & 15));
                q_limbs[sl * HD + spos] = (int8_t)hi;
                q_limbs[(C::NSLOT + sl) * HD + spos] = (int8_t)lo;
            }
            if constexpr (FMT != KV_I8) {
                if (lane == 0) {
                    int tot = 0;
    #pragma unroll
                    for (int i = 0; i < HD / 32; ++i) tot += qblk[i];
    #pragma unroll
                    for (int i = 0; i < HD / 32; ++i) slot_qsum[sl * C::NBLK + i] = 8 * ((FMT == KV_I4 && QS == 1) ? tot : qblk[i]);
                }
            }
            if (lane == 0) {
                const int hi_b = valid ? p.klen - (p.S - 1 - r) : 0;
                slot_qscale[sl] = valid ? sq * p.qk_scale_log2 : 0.0f;
                slot_hi[sl] = hi_b;
                slot_lo[sl] = (valid && p.window > 0) ? max(0, hi_b - p.window) : 0;
            }
        }
        if (pass == 0) __syncwarp();
    }
    __syncthreads();

    float qscale[MT];
    int lo_b[MT], hi_b[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        qscale[mt] = slot_qscale[mt * 8 + g];
        lo_b[mt] = slot_lo[mt * 8 + g];
        hi_b[mt] = slot_hi[mt * 8 + g];
    }
    // Q A-fragments (rows g = high limb, rows g+8 = low limb of slot g): registers for
    // one M tile, re-read from shared memory otherwise.
    constexpr bool Q_IN_REGS = (MT == 1) && (C::HDK <= 256);
    constexpr int KS0_STEP = C::HDK / 32;            // k steps (32 dims) of this warp's slice; its first global step is wj * KS0_STEP
    uint32_t qa[Q_IN_REGS ? C::HDK / 32 : 1][4];
    // A fragment of k step ks for M tile mt in one ldmatrix.x4: matrices = (high limb, chunk 2ks),
    // (low limb, chunk 2ks), (high, 2ks+1), (low, 2ks+1) of slots 8mt..8mt+7  ->  a0, a1, a2, a3.
    const uint32_t q_u32 = smem_u32(q_limbs);
    auto load_qa = [&](uint32_t(&a)[4], int mt, int ks) {
        const int slot = mt * 8 + (lane & 7);
        const int limb = (lane >> 3) & 1;
        const int ch = 2 * ks + (lane >> 4);
        ldmatrix_x4(a, q_u32 + (limb * C::NSLOT + slot) * HD + ((ch ^ (slot & 7)) << 4));
    };
    if constexpr (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < C::HDK / 32; ++ks) load_qa(qa[ks], 0, wj * KS0_STEP + ks);
    }
    // ks counts the k steps of this warp's slice
    auto get_qa = [&](uint32_t(&a)[4], int mt, int ks) {
        if constexpr (Q_IN_REGS) {
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = qa[ks][i];
        } else {
            load_qa(a, mt, wj * KS0_STEP + ks);
        }
    };

    // ------------------------------------------------------------ running state
    float M[MT], l[MT];
    float acc[MT][C::NT][2];              // [slot tile][8-dim tile][2 dims] of slot g
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        M[mt] = M_INIT; l[mt] = 0.0f;
#pragma unroll
        for (int nt = 0; nt < C::NT; ++nt) { acc[mt][nt][0] = 0.0f; acc[mt][nt][1] = 0.0f; }
    }
    int lo_max = 0, hi_min = 0x7fffffff;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
        if (hi_b[mt] > 0) { lo_max = max(lo_max, lo_b[mt]); hi_min = min(hi_min, hi_b[mt]); }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        lo_max = max(lo_max, __shfl_xor_sync(0xffffffffu, lo_max, o));
        hi_min = min(hi_min, __shfl_xor_sync(0xffffffffu, hi_min, o));
    }

    for (int it = 0; it < my_count; ++it) {
        issue(it + NSTAGE - 1);
        const int stg = it % NSTAGE;
        cp_async_wait<NSTAGE - 1>();
        if constexpr (C::TMA_OK) {
            if ((tma_mask >> stg) & 1u) {
                if (!mbar_wait_bounded(my_bar_u32 + 8 * stg, (phase_bits >> stg) & 1u) && lane == 0) atomicOr(p.fault, 1u);
                phase_bits ^= 1u << stg;
            }
        }
        __syncwarp();

        const int tok0 = (my_first + it * NQ) * TILE;
        const uint32_t st = my_pipe_u32 + stg * C::ST_BYTES;
        const bool need_mask = (tok0 + TILE > hi_min) || (tok0 < lo_max);
        const uint8_t *ksm = my_sc + stg * 2 * C::SC_BYTES;         // K scales of the tile, token-major
        const uint8_t *vsm = ksm + C::SC_BYTES;                     // V scales

        // ------------------------------------------- new keys of this tile
        // Overwrite the rows the copy engine fetched for the new keys' slots with their quantised form
        // (from the scratch rows filled in the prologue, or quantised here when there are several).
        if (p.new_k != nullptr && tok0 + TILE > p.klen - p.n_new) {
            auto patch = [&](int r, int kv, const uint8_t *scr) {
                uint8_t *tile_rows = my_pipe + stg * C::ST_BYTES + kv * C::KV_BYTES;          // fused append runs with DS == 1 only
                uint8_t *tile_sc = my_sc + (stg * 2 + kv) * C::SC_BYTES + r * C::SCB;
                if (lane < C::CHUNKS)
                    *reinterpret_cast<uint4 *>(tile_rows + r * C::ROWB + swz_chunk<C::ROWB>(r, lane) * 16) =
                        *reinterpret_cast<const uint4 *>(scr + lane * 16);
                if (lane < C::SCB / 2)
                    reinterpret_cast<uint16_t *>(tile_sc)[lane] = reinterpret_cast<const uint16_t *>(scr + C::ROWB)[lane];
                __syncwarp();
            };
            if (early_new) {
                const int r = p.klen - 1 - tok0;
                patch(r, 0, append_scratch + new_owner * (C::ROWB + 64));
                patch(r, 1, append_scratch + new_helper * (C::ROWB + 64));
            } else {
                uint8_t *scr = append_scratch + warp * (C::ROWB + 64);
                for (int i = 0; i < p.n_new; ++i) {
                    const int wi = p.klen - p.n_new + i;                 // window index of new key i
                    if (wi < tok0 || wi >= tok0 + TILE) continue;
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {
                        quantize_new(i, kv, scr, true);
                        patch(wi - tok0, kv, scr);
                    }
                }
            }
        }

        // --------------------------------------------------------------- QK
        // Base-2 logits s2[mt][n][e] of slot (mt, g) against token 8n+2t+e.  The MMA rows g / g+8
        // carry the high / low limb of the slot's query, the columns 2t, 2t+1 the two tokens.
        float s2[MT][4][2];
        if constexpr (FMT == KV_I8) {
            int c[MT][4][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) c[mt][n][i] = 0;
#pragma unroll
            for (int half = 0; half < C::HDK / 64; ++half) {
                uint32_t kb[4][4];        // K bytes of the four 8-token groups, chunks 4half..4half+3
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const int row = 8 * n + (lane & 7);
                    const int ch = 4 * half + (lane >> 3);
                    ldmatrix_x4(kb[n], st + row * C::ROWBK + swz_chunk<C::ROWBK>(row, ch) * 16);
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int k2 = 0; k2 < 2; ++k2) {
                        uint32_t a[4];
                        get_qa(a, mt, 2 * half + k2);
#pragma unroll
                        for (int n = 0; n < 4; ++n) mma_s8s8(c[mt][n], a, kb[n][2 * k2], kb[n][2 * k2 + 1]);
                    }
            }
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const float2 kk = *reinterpret_cast<const float2 *>(ksm + (8 * n + 2 * t) * 4);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    s2[mt][n][0] = (float)(c[mt][n][0] * 256 + c[mt][n][2]) * (qscale[mt] * kk.x);
                    s2[mt][n][1] = (float)(c[mt][n][1] * 256 + c[mt][n][3]) * (qscale[mt] * kk.y);
                }
            }
        } else {
            // int4: a 16-byte chunk holds one block of 32 values; low nibbles (even elements) feed
            // MMA k slots 0-15, high nibbles k slots 16-31, both as biased unsigned bytes q+8.  The
            // bias is removed exactly with 8 * sum(q limbs), precomputed per slot (and block).
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                int c[MT][4];
                float sblk[MT][2];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) c[mt][i] = 0;
                    sblk[mt][0] = 0.0f; sblk[mt][1] = 0.0f;
                }
#pragma unroll
                for (int grp = 0; grp < C::HDK / 128; ++grp) {
                    uint32_t kr[4];
                    const int row = 8 * n + (lane & 7);
                    const int ch = 4 * grp + (lane >> 3);
                    ldmatrix_x4(kr, st + row * C::ROWBK + swz_chunk<C::ROWBK>(row, ch) * 16);
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const int blk = 4 * grp + m;
                        const uint32_t lo = lop3_and_xor(kr[m], 0x0f0f0f0fu, 0x08080808u);
                        const uint32_t hi = lop3_and_xor(kr[m] >> 4, 0x0f0f0f0fu, 0x08080808u);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            uint32_t a[4];
                            get_qa(a, mt, blk);
                            if constexpr (FMT == KV_I4) {
                                mma_s8u8(c[mt], a, lo, hi);
                            } else {
                                int cb[4] = {0, 0, 0, 0};
                                mma_s8u8(cb, a, lo, hi);
                                // fp16 block scales of tokens 8n+2t and 8n+2t+1
                                const int bias = slot_qsum[(mt * 8 + g) * C::NBLK + wj * C::NBLKK + blk];
                                const float f0 = __half2float(*reinterpret_cast<const __half *>(ksm + ((8 * n + 2 * t) * C::NBLKK + blk) * 2));
                                const float f1 = __half2float(*reinterpret_cast<const __half *>(ksm + ((8 * n + 2 * t + 1) * C::NBLKK + blk) * 2));
                                sblk[mt][0] = fmaf((float)(cb[0] * 256 + cb[2] - bias), f0, sblk[mt][0]);
                                sblk[mt][1] = fmaf((float)(cb[1] * 256 + cb[3] - bias), f1, sblk[mt][1]);
                            }
                        }
                    }
                }
                if constexpr (FMT == KV_I4) {
                    const float2 kk = *reinterpret_cast<const float2 *>(ksm + (8 * n + 2 * t) * 4);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        int bias = slot_qsum[(mt * 8 + g) * C::NBLK];                // 8 * sum over the whole row ...
                        if constexpr (QS > 1) {                                      // ... or over this warp's blocks
                            bias = 0;
#pragma unroll
                            for (int bk = 0; bk < C::NBLKK; ++bk) bias += slot_qsum[(mt * 8 + g) * C::NBLK + wj * C::NBLKK + bk];
                        }
                        s2[mt][n][0] = (float)(c[mt][0] * 256 + c[mt][2] - bias) * (qscale[mt] * kk.x);
                        s2[mt][n][1] = (float)(c[mt][1] * 256 + c[mt][3] - bias) * (qscale[mt] * kk.y);
                    }
                } else {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        s2[mt][n][0] = sblk[mt][0] * qscale[mt];
                        s2[mt][n][1] = sblk[mt][1] * qscale[mt];
                    }
                }
            }
        }
        if constexpr (QS > 1) {
            // ---- the quad adds up its partial logits.  Every warp writes its 8 MT values per lane, the quad meets at its
            // named barrier (one per tile; the buffer alternates with the tile's parity, so the next tile's writes cannot
            // overtake a warp still reading), and every warp sums the QS partials in the same order: the four warps hold
            // bit-identical logits, hence identical softmax references, weights and denominators.
            float *xq = xch_region + (size_t)((quad * 2 + (it & 1)) * QS) * (MT * 8 * 32);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int e = 0; e < 2; ++e) xq[(wj * MT * 8 + (mt * 4 + n) * 2 + e) * 32 + lane] = s2[mt][n][e];
            asm volatile("bar.sync %0, %1;\n" ::"r"(1 + quad), "n"(QS * 32) : "memory");
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        float acc_s = 0.0f;
#pragma unroll
                        for (int jj = 0; jj < QS; ++jj) acc_s += xq[(jj * MT * 8 + (mt * 4 + n) * 2 + e) * 32 + lane];
                        s2[mt][n][e] = acc_s;
                    }
        }
        if (need_mask) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int tok = tok0 + 8 * n + 2 * t + j;
                        if (tok < lo_b[mt] || tok >= hi_b[mt]) s2[mt][n][j] = -CUDART_INF_F;
                    }
        }

        // ------------------------------------------------ softmax weights, 16-bit fixed point
        // w = 2^(s - tile max) * v_scale, divided by the tile's largest w, is rounded to u16 and
        // split into two u8 limbs for the tensor core; F carries the tile's weight into the fp32
        // running sums.  Block-32 caches have one v_scale per (token, block of 32 dims).
        constexpr int NVB = (FMT == KV_I4B32) ? C::NBLKV : 1;             // V scale blocks of this CTA's slice
        float vsc[4][2][NVB];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            if constexpr (FMT == KV_I4B32) {
#pragma unroll
                for (int e = 0; e < 2; ++e)
#pragma unroll
                    for (int vb = 0; vb < NVB; ++vb)
                        vsc[n][e][vb] = __half2float(*reinterpret_cast<const __half *>(vsm + ((8 * n + 2 * t + e) * C::NBLKK + (QS > 1 ? 0 : dsl * C::NBLKV) + vb) * 2));
            } else {
                const float2 vv = *reinterpret_cast<const float2 *>(vsm + (8 * n + 2 * t) * 4);
                vsc[n][0][0] = vv.x; vsc[n][1][0] = vv.y;
            }
        }
        uint32_t pa[MT][NVB][4];          // A fragments of the PV MMA: a0/a2 = high limbs, a1/a3 = low limbs
        int ubias[MT][NVB];               // int4 only: 8 * sum of the u16 weights (removes the +8 nibble bias)
        float F[MT];
        float alpha[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int n = 0; n < 4; ++n) mx = fmaxf(mx, fmaxf(s2[mt][n][0], s2[mt][n][1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            // The running reference only moves when the tile maximum exceeds it by more than 2^8:
            // weights are normalised per tile anyway, so a stale reference costs no precision (the
            // tile weight is at most 2^8 larger) and the fp32 sums are rescaled a handful of times
            // per call instead of once per tile.
            const float m_new = mx > M[mt] + LAZY_MAX ? mx : M[mt];
            const bool empty = mx == -CUDART_INF_F;                 // every token of the tile is masked for this slot
            const float mx_safe = empty ? 0.0f : mx;
            const float tile_w = empty ? 0.0f : ex2f(mx - m_new);
            alpha[mt] = ex2f(M[mt] - m_new);
            if (__any_sync(0xffffffffu, m_new != M[mt])) {
#pragma unroll
                for (int nt = 0; nt < C::NT; ++nt) { acc[mt][nt][0] *= alpha[mt]; acc[mt][nt][1] *= alpha[mt]; }
            }
            M[mt] = m_new;
            float pe[4][2];
            float lsum = 0.0f, wmax = 0.0f;
#pragma unroll
            for (int n = 0; n < 4; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    pe[n][e] = ex2f(s2[mt][n][e] - mx_safe);
                    lsum += pe[n][e];
#pragma unroll
                    for (int vb = 0; vb < NVB; ++vb) wmax = fmaxf(wmax, pe[n][e] * vsc[n][e][vb]);
                }
            wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, 1));
            wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, 2));
            const float inv = wmax > 0.0f ? P_FIX * rcpf(wmax) : 0.0f;
            F[mt] = tile_w * wmax * (1.0f / P_FIX);
            l[mt] = fmaf(tile_w, lsum, l[mt] * alpha[mt]);
#pragma unroll
            for (int vb = 0; vb < NVB; ++vb) {
                uint32_t pk[4];
                int usum = 0;
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const uint32_t f0 = __float_as_uint(fmaf(pe[n][0] * vsc[n][0][vb], inv, RND_MAGIC));
                    const uint32_t f1 = __float_as_uint(fmaf(pe[n][1] * vsc[n][1][vb], inv, RND_MAGIC));
                    pk[n] = prmt(f0, f1, 0x5410u);                  // two u16
                    if constexpr (FMT != KV_I8) usum += (int)(f0 & 0xffffu) + (int)(f1 & 0xffffu);
                }
                pa[mt][vb][0] = prmt(pk[0], pk[1], 0x7531u);
                pa[mt][vb][1] = prmt(pk[0], pk[1], 0x6420u);
                pa[mt][vb][2] = prmt(pk[2], pk[3], 0x7531u);
                pa[mt][vb][3] = prmt(pk[2], pk[3], 0x6420u);
                if constexpr (FMT != KV_I8) {
                    usum += __shfl_xor_sync(0xffffffffu, usum, 1);
                    usum += __shfl_xor_sync(0xffffffffu, usum, 2);
                    ubias[mt][vb] = 8 * usum;
                } else {
                    ubias[mt][vb] = 0;
                }
            }
        }
        // --------------------------------------------------------------- PV
        // One MMA spans the whole 32-token tile: A = weight limbs (rows g / g+8 = high / low),
        // B = V bytes transposed by ldmatrix.trans + byte permutes; the int32 result is exact.
        const uint32_t vst = st + C::KV_BYTES;
        if constexpr (FMT == KV_I8) {
#pragma unroll
            for (int ch = 0; ch < HDV / 16; ++ch) {
                uint32_t vr[4];           // vr[o]: tokens 8o+2t, 8o+2t+1 x dims 16ch+2g, 16ch+2g+1
                ldmatrix_x4_trans(vr, vst + lane * C::ROWBV + swz_chunk<C::ROWBV>(lane, ch) * 16);
                const uint32_t be0 = prmt(vr[0], vr[1], 0x6420u), bo0 = prmt(vr[0], vr[1], 0x7531u);
                const uint32_t be1 = prmt(vr[2], vr[3], 0x6420u), bo1 = prmt(vr[2], vr[3], 0x7531u);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    int d4[4];
                    mma_u8s8_zero(d4, pa[mt][0][0], pa[mt][0][1], pa[mt][0][2], pa[mt][0][3], be0, be1);
                    acc[mt][2 * ch][0] = fmaf((float)(d4[0] * 256 + d4[2]), F[mt], acc[mt][2 * ch][0]);
                    acc[mt][2 * ch][1] = fmaf((float)(d4[1] * 256 + d4[3]), F[mt], acc[mt][2 * ch][1]);
                    mma_u8s8_zero(d4, pa[mt][0][0], pa[mt][0][1], pa[mt][0][2], pa[mt][0][3], bo0, bo1);
                    acc[mt][2 * ch + 1][0] = fmaf((float)(d4[0] * 256 + d4[2]), F[mt], acc[mt][2 * ch + 1][0]);
                    acc[mt][2 * ch + 1][1] = fmaf((float)(d4[1] * 256 + d4[3]), F[mt], acc[mt][2 * ch + 1][1]);
                }
            }
        } else {
#pragma unroll
            for (int ch = 0; ch < HDV / 32; ++ch) {         // packed chunk ch = block ch = dims 32ch..32ch+31 of the slice
                uint32_t vr[4];           // vr[o]: tokens 8o+2t, 8o+2t+1 x packed bytes 16ch+2g, 16ch+2g+1
                ldmatrix_x4_trans(vr, vst + lane * C::ROWBV + swz_chunk<C::ROWBV>(lane, ch) * 16);
                uint32_t pb[2][2];        // [byte 2g | 2g+1][tokens 0-15 | 16-31]: one packed byte of four tokens
                pb[0][0] = prmt(vr[0], vr[1], 0x6420u); pb[1][0] = prmt(vr[0], vr[1], 0x7531u);
                pb[0][1] = prmt(vr[2], vr[3], 0x6420u); pb[1][1] = prmt(vr[2], vr[3], 0x7531u);
                constexpr int VBI = (FMT == KV_I4B32) ? 1 : 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {               // element 4g+e of the block: byte e/2, nibble e%2
                    const uint32_t b0 = lop3_and_xor((e & 1) ? pb[e >> 1][0] >> 4 : pb[e >> 1][0], 0x0f0f0f0fu, 0x08080808u);
                    const uint32_t b1 = lop3_and_xor((e & 1) ? pb[e >> 1][1] >> 4 : pb[e >> 1][1], 0x0f0f0f0fu, 0x08080808u);
                    const int nt = 4 * ch + e;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const int vb = VBI * ch;
                        int d4[4];
                        mma_u8u8_zero(d4, pa[mt][vb][0], pa[mt][vb][1], pa[mt][vb][2], pa[mt][vb][3], b0, b1);
                        acc[mt][nt][0] = fmaf((float)(d4[0] * 256 + d4[2] - ubias[mt][vb]), F[mt], acc[mt][nt][0]);
                        acc[mt][nt][1] = fmaf((float)(d4[1] * 256 + d4[3] - ubias[mt][vb]), F[mt], acc[mt][nt][1]);
                    }
                }
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    // ---------------------------------------------------- merge warps in shared
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        l[mt] += __shfl_xor_sync(0xffffffffu, l[mt], 1);
        l[mt] += __shfl_xor_sync(0xffffffffu, l[mt], 2);
    }
    __syncthreads();                      // every warp is done with its pipeline memory
    float *mbuf = reinterpret_cast<float *>(pipe);          // [NWARP][NSLOT][HDV+2]
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float *r0 = mbuf + ((size_t)warp * C::NSLOT + mt * 8 + g) * (HDV + 2);
        // only the rows of real query rows are stored (a decode call fills 2 of a group's 8 slots): with all eight
        // rows, 130 floats apart, every store of the warp took four shared-memory wavefronts
        if (div_kvg(p, rg * C::NSLOT + mt * 8 + g) >= p.S) continue;
#pragma unroll
        for (int nt = 0; nt < C::NT; ++nt) {
            // this thread has MMA columns 2t, 2t+1 of n tile nt.  int8: column c of tile nt is
            // dim 16*(nt/2) + 2c + (nt&1); int4: dim 32*(nt/4) + 4c + (nt&3).
            if constexpr (FMT == KV_I8) {
                const int d0 = 16 * (nt >> 1) + 4 * t + (nt & 1);
                r0[d0] = acc[mt][nt][0];
                r0[d0 + 2] = acc[mt][nt][1];
            } else {
                const int d0 = 32 * (nt >> 2) + 8 * t + (nt & 3);
                r0[d0] = acc[mt][nt][0];
                r0[d0 + 4] = acc[mt][nt][1];
            }
        }
        if (t == 0) { r0[HDV] = M[mt]; r0[HDV + 1] = l[mt]; }
    }
    __syncthreads();

    // One warp per slot (slots warp, warp + NWARP, ...), its lanes over the dims, a rolled loop over the tile streams:
    // a few dozen instructions.  (This runs once per CTA and is fetched cold; unrolled over the streams and spread
    // over all threads it took 1.2 to 1.7 us.)
    for (int sl = warp; sl < C::NSLOT; sl += NWARP) {
        const int idx = rg * C::NSLOT + sl;
        const int r = div_kvg(p, idx), j = idx - r * p.kvg;
        if (r >= p.S) continue;
        // one (m, l, o) per tile stream: the warps of a quad hold the same (m, l) and different dims; lane w holds stream w's pair
        const float *row_ml = mbuf + ((size_t)(min(lane, NQ - 1) * QS) * C::NSLOT + sl) * (HDV + 2) + HDV;
        const float mw = lane < NQ ? row_ml[0] : M_INIT, lw = lane < NQ ? row_ml[1] : 0.0f;
        const float mstar = warp_max(mw);
        const float wg = lane < NQ ? ex2f(mw - mstar) : 0.0f;
        constexpr int NDQ = HDV * QS / 32;                     // dims of this CTA per lane
        float o[NDQ], lstar = 0.0f;
#pragma unroll
        for (int i = 0; i < NDQ; ++i) o[i] = 0.0f;
#pragma unroll                                         // (every stream's loads in flight: rolled up the loop took 0.8 us)
        for (int w = 0; w < NQ; ++w) {
            const float ww = __shfl_sync(0xffffffffu, wg, w);
            lstar = fmaf(ww, __shfl_sync(0xffffffffu, lw, w), lstar);
#pragma unroll
            for (int i = 0; i < NDQ; ++i) {
                const int dq = lane + 32 * i, sj = dq / HDV, d = dq - sj * HDV;   // slice of the quad that holds the dim, dim inside the slice
                o[i] = fmaf(ww, mbuf[((size_t)(w * QS + sj) * C::NSLOT + sl) * (HDV + 2) + d], o[i]);
            }
        }
        const long grow = ((long)b * p.S + r) * p.nh + kvh * p.kvg + j;
        if (p.write_partial) {
            float *dst = (C::CLUSTER_OK && p.cluster_merge) ? reinterpret_cast<float *>(pipe + C::CPART_OFF) + (size_t)sl * (HD + 2)
                                                            : p.partial + ((size_t)split * p.grows + grow) * (HD + 2);
#pragma unroll
            for (int i = 0; i < NDQ; ++i) dst[dsl * HDV * QS + lane + 32 * i] = o[i];
            if (lane == 0 && dsl == 0) {                        // every slice computes the same (m, l)
                dst[HD] = p.export_nat ? mstar * LN2 : mstar;
                dst[HD + 1] = lstar;
            }
        } else {
            const long oi = b * p.out_batch_stride + ((long)r * p.nh + kvh * p.kvg + j) * HD + dsl * HDV * QS;
#pragma unroll
            for (int i = 0; i < NDQ; ++i) {
                const float v = lstar > 0.0f ? o[i] / lstar : 0.0f;
                if (p.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[oi + lane + 32 * i] = __float2bfloat16_rn(v);
                else reinterpret_cast<float *>(p.out)[oi + lane + 32 * i] = v;
            }
        }
    }
    if constexpr (C::CLUSTER_OK) {
        if (p.cluster_merge) {
            cluster_merge_unit<C::NSLOT, HD, NWARP * 32>(p, reinterpret_cast<float *>(pipe + C::CPART_OFF), b, kvh, rg);
            return;
        }
    }
    merge_splits_in_kernel<C::NSLOT, HD, NWARP * 32>(p, pipe, b, kvh, rg);
}

// Merge G partial triples per row.  partials [G][rows][hd+2] = (o.., m, l); m in log2
// units when nat == 0 (in-library split partials), natural-log units when nat == 1.
// One CTA per row: the weights 2^(m_i - m*) are computed once into shared memory.
constexpr int MERGE_MAX_G = 1024;
__global__ void __launch_bounds__(128) merge_kernel(const float *partials, int G, int rows, int hd, void *out, int out_type,
                                                     int nat, float *partial_out) {
    __shared__ float wgt[MERGE_MAX_G];
    __shared__ float red[8];
    pdl_wait();                           // no-op unless launched as a programmatic dependent
    pdl_launch_dependents();              // a following attention grid may start streaming its cache now
    const int row = blockIdx.x, tid = threadIdx.x;
    const float unit = nat ? LOG2E : 1.0f;
    const size_t rstride = (size_t)rows * (hd + 2);
    const float *base = partials + (size_t)row * (hd + 2);
    float mloc = -CUDART_INF_F;
    for (int i = tid; i < G; i += 128) {
        const float li = base[i * rstride + hd + 1];
        const float mi = base[i * rstride + hd] * unit;
        wgt[i] = li > 0.0f ? mi : -CUDART_INF_F;
        mloc = fmaxf(mloc, wgt[i]);
    }
    mloc = warp_max(mloc);
    if ((tid & 31) == 0) red[tid >> 5] = mloc;
    __syncthreads();
    const float mstar = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    float lloc = 0.0f;
    for (int i = tid; i < G; i += 128) {
        const float w = wgt[i] == -CUDART_INF_F ? 0.0f : ex2f(wgt[i] - mstar);
        lloc += w * base[i * rstride + hd + 1];
        wgt[i] = w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, o);
    if ((tid & 31) == 0) red[4 + (tid >> 5)] = lloc;
    __syncthreads();
    const float lstar = red[4] + red[5] + red[6] + red[7];
    for (int d = tid; d < hd; d += 128) {
        float o = 0.0f;
        for (int i = 0; i < G; ++i) o = fmaf(wgt[i], base[i * rstride + d], o);
        if (partial_out) {
            partial_out[(size_t)row * (hd + 2) + d] = o;
        } else {
            const float v = lstar > 0.0f ? o / lstar : 0.0f;
            if (out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(out)[(size_t)row * hd + d] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(out)[(size_t)row * hd + d] = v;
        }
    }
    if (partial_out && tid == 0) {
        partial_out[(size_t)row * (hd + 2) + hd] = lstar > 0.0f ? mstar * LN2 : 0.0f;   // exported m: natural log
        partial_out[(size_t)row * (hd + 2) + hd + 1] = lstar;
    }
}

}  // namespace fused
}  // namespace nomos
