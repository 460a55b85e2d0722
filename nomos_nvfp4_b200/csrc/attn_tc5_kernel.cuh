// Decode / verify attention over the int8 KV cache on the fifth-generation tensor cores
// (tcgen05 + tensor memory), head_dim 128, sm_100a.  The host side (plan, tensor maps, launch)
// is in attn_fused.cu.
//
// The contraction is laid out so that the 128-row M dimension of tcgen05.mma is always full,
// however few query rows there are:
//   QK:  S^T[128 keys x N] = K_tile[128 keys x 128 B] (A, K-major, exactly the bytes TMA wrote)
//                            x Qlimbs[N x 128 B]      (B, K-major)
//   PV:  O^T[128 dims x N] = V_tile^T[128 dims x 128 keys] (A, MN-major: the same [key][dim]
//                            bytes TMA wrote, read transposed by the tensor core)
//                            x Plimbs[N x 128 keys]   (B, K-major)
// N = 2 x (padded slots): column s holds the high limb of slot s (a query row x group head),
// column NSP+s the low limb, for the 16-bit fixed-point query and the 16-bit fixed-point softmax
// weights alike, so every product is an exact int32.
// Accumulators live in tensor memory: a softmax warp reads the TMEM lanes 32(w%4)..32(w%4)+31,
// i.e. thread = one key of the tile for S^T, thread = one output dim for O^T.
//
// Roles: groups of four softmax warps (128 threads = the 128 TMEM lanes), then one warp whose lane
// 0 is the TMA producer and one whose lane 0 issues the MMAs.  Up to eight slots: one group, two
// S/P/O buffers, two CTAs per SM (two more warps only help in the split merge).  More slots
// (speculative verify): NOMOS_TC5_NG groups take the CTA's tiles in turn -- group g owns tiles g,
// g+NG, ... with all their slots, keeps its own running reference, denominators and output sums,
// and the groups are merged in shared memory at the end -- over four S/P/O buffers, so that one
// group's dependent chain (TMEM load, maxima, weights, P store, O read-back) overlaps the others'.
// Optional in the same launch: quantize-on-write of up to NEW_MAX new rows (a softmax warp
// overwrites the rows TMA fetched), and paged caches (a tile is a page of 128 keys looked up in a
// block table).  Every wait is an mbarrier wait with a time limit; a wait
// that runs out raises the CTA's abort flag and a bit in the device fault word, every role leaves
// its loop, tensor memory is freed and the CTA exits.
#pragma once

#include "attn_fused_kernel.cuh"
#include "kv_rows.cuh"

namespace nomos {
namespace tc5 {

using fused::KParams;
using fused::LOG2E;
using fused::LN2;
using fused::M_INIT;
using fused::Q_FIX_MAX;
using fused::P_FIX;
using fused::LAZY_MAX;
using fused::RND_MAGIC;

constexpr int KT = 128;                      // keys per tile = M of the QK MMA
constexpr int HD = 128;                      // head dim = M of the PV MMA
constexpr int TILE_BYTES = KT * HD;          // one K or V tile (int8)
constexpr int SCALE_BYTES = KT * 4;          // one tile's fp32 row scales
constexpr float LG2_VS_MIN = -64.0f;
constexpr int NEW_MAX = 8;                   // most rows one call may quantise on the way in
constexpr int MAX_PAGED_TILES = 256;         // paged caches: most tiles (pages) one CTA walks
#ifndef NOMOS_TC5_NG
#define NOMOS_TC5_NG 2                       // softmax warp groups (tiles in flight) when a CTA serves more than eight slots
#endif
#ifndef NOMOS_TC5_WIDE_FROM
#define NOMOS_TC5_WIDE_FROM 9                // slots from which a CTA runs several groups, one CTA per SM; below: one group, two CTAs per SM
#endif


template <int NS>
struct Cfg {
    static constexpr int NSP = (NS + 7) / 8 * 8;                     // slots padded to the MMA's N granularity
    static constexpr int N = 2 * NSP;
    static constexpr bool WIDE = NS >= NOMOS_TC5_WIDE_FROM;
    static constexpr int NSTG = WIDE ? 5 : 3;                        // 3 stages: two CTAs per SM
    static constexpr int MIN_CTAS = WIDE ? 1 : 2;
    static constexpr int NG = WIDE ? NOMOS_TC5_NG : 1;               // softmax warp groups; group g owns tiles g, g+NG, ...
    static constexpr int NB = WIDE ? 4 : 2;                          // buffers of S^T, P and O^T (tile i uses buffer i % NB)
    static constexpr int LAG = NG;                                   // the issuer sends PV(i - LAG) after QK(i)
    static constexpr int TMEM_COLS = 128 * NB;                       // S buffers, then O buffers, 64 columns each
    static constexpr int NSW = 4 * NG;                               // softmax warps; then the TMA warp, then the MMA warp
    static constexpr int NTHREADS = NG == 1 ? 256 : 32 * (NSW + 2);
    static_assert(NS % 2 == 0 && NS <= 32 && N <= 64, "a buffer is 64 TMEM columns; lane s of a warp keeps slot s's reference");
    static_assert(LAG < NB && TMEM_COLS <= 512 && NG <= 3, "S buffer i % NB is rewritten NB tiles later, after p_ready(i) was seen");
    static constexpr int QP_BYTES = N * 128;                         // Q limbs, or one buffer of P limbs
    static constexpr int OFF_SCALES = NSTG * 2 * TILE_BYTES;
    static constexpr int OFF_Q = OFF_SCALES + NSTG * 2 * SCALE_BYTES;
    static constexpr int OFF_P = OFF_Q + QP_BYTES;
    static constexpr int OFF_XCH = OFF_P + NB * QP_BYTES;            // [NG][2][NSP][4] warp maxima
    static constexpr int OFF_SLOT = OFF_XCH + NG * 2 * NSP * 16;     // qscale[NSP], lo[NSP], hi[NSP]: query scale, first and one-past-last key of each slot
    static constexpr int OFF_SLOTC = (OFF_SLOT + NSP * 12 + 15) / 16 * 16;   // per softmax warp: NSP x (max, weight, alpha, -)
    static constexpr int OFF_BAR = OFF_SLOTC + NSW * NSP * 16;
    static constexpr int NBAR = 2 * NSTG + 4 * NB + 1 + 2 * NG + 2;  // full, empty; s_ready, p_ready, o_ready, o_free (per buffer); q_ready; xch (x2 per group); patched (x2)
    static constexpr int MRG_BYTES = NG * (2 * NS * HD + 2 * NSP) * 4;   // the groups' sums for their merge, over the tile stages
    static_assert(MRG_BYTES <= NSTG * 2 * TILE_BYTES, "group merge scratch reuses the tile stages");
    static constexpr int OFF_MISC = (OFF_BAR + NBAR * 8 + 15) / 16 * 16;   // tmem base, abort flag
    static constexpr int OFF_NEW = OFF_MISC + 16;                    // quantize-on-write: [NEW_MAX][K, V] rows of codes + scale
    static constexpr int OFF_NEWSC = OFF_NEW + 2 * NEW_MAX * (128 + 16);   // scales of the new rows [2][NEW_MAX]
    static constexpr int OFF_PAGES = OFF_NEWSC + 2 * NEW_MAX * 4;    // paged caches: page of each of this CTA's tiles
    static constexpr int SMEM_BYTES = 1024 + OFF_PAGES + MAX_PAGED_TILES * 4;
    static_assert(OFF_NEW % 16 == 0, "row scratch is copied in 16-byte chunks");
    static_assert(SMEM_BYTES + 1024 <= 232448 / MIN_CTAS - (MIN_CTAS > 1 ? 1024 : 0), "shared memory budget of an SM (227 KB per CTA, 228 KB in all)");
    static_assert(OFF_BAR % 8 == 0, "mbarriers need 8-byte alignment");
    static_assert(OFF_Q % 1024 == 0 && QP_BYTES % 1024 == 0, "operand tiles sit on swizzle-pattern boundaries");
};

struct TmaMaps4 {
    CUtensorMap k, v;        // {row bytes, nkv * cache_cap rows, batch}, box {128 B, 128 rows, 1}, 128B swizzle
    CUtensorMap ks, vs;      // {nkv * cache_cap fp32, batch}, box {128, 1}
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
                 "l"(reinterpret_cast<unsigned long long>(map)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(base), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem], int8 operands, int32 accumulate; issued by one thread.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// This warp's 32 TMEM lanes x COUNT consecutive 32-bit columns: thread t gets lane t's row.
template <int COUNT>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, int (&r)[COUNT]) {
    static_assert(COUNT == 2 || COUNT == 4 || COUNT == 8, "column count");
    if constexpr (COUNT == 2)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr));
    else if constexpr (COUNT == 4)
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                     : "r"(taddr));
    else
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "r"(taddr));
}
// hi * 2^SH + lo as a float, |hi|, |lo| < 2^22.  int -> float on the integer and FMA pipes: x + 1.5 * 2^23
// read as a float, minus 1.5 * 2^23 (the conversion instruction itself measured much slower here: it shares
// the quarter-rate unit with ex2).
template <int SH>
__device__ __forceinline__ float limbs2f(int hi, int lo) {
    const float fh = __int_as_float(hi + 0x4B400000) - 12582912.0f, fl = __int_as_float(lo + 0x4B400000) - 12582912.0f;
    return fmaf(fh, (float)(1 << SH), fl);
}
// Warp-wide maximum of a float in one instruction (sm_100a).
__device__ __forceinline__ float redux_max(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;\n" : "=f"(r) : "f"(v));
    return r;
}

// Shared-memory matrix descriptors (sm_100 format: version 1, 128-byte swizzle, 8-row groups of
// 128-byte rows 1024 bytes apart).  K-major: rows = M/N index, the 128 bytes of a row = K.
// MN-major: the 128 bytes of a row = 128 consecutive M indices, rows = K index.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: int32 accumulate, M = 128, given N, operand signedness and A major-ness.
__device__ __forceinline__ uint32_t make_idesc(int n, bool a_signed, bool b_signed, bool a_mn_major) {
    return (2u << 4) | ((a_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
           ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

// Bounded mbarrier wait shared by all roles of a CTA: false = gave up (own time limit of about a
// second, or another role already raised the abort flag).
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int *fault) {
    if (fused::mbar_try_wait(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
#pragma unroll 1
        for (int k = 0; k < 32; ++k)                     // try_wait itself suspends the thread for a while
            if (fused::mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 1000000000ull) {
            *abort_flag = 1;
            atomicOr(fault, 2u);
            return false;
        }
    }
}

// Window geometry in slot space.  The keys of the window [tbase, klen) live in up to two runs of
// consecutive ring slots; tiles are 128 slots, the first of a run starting at a multiple of four
// slots (16-byte rule of the scale copies), so a tile's first rows may precede the run.
struct TileGeo {
    int slot0;      // ring slot of the tile's row 0
    int t0;         // window index of row 0 (may be negative or below tbase)
    int t_lo, t_hi; // rows with window index in [t_lo, t_hi) belong to the tile
};
struct WindowGeo {
    int ring0, len_a, a0, n_a, tbase, klen;
    __device__ __forceinline__ TileGeo tile(int j) const {
        TileGeo g;
        if (j < n_a) {
            g.slot0 = a0 + j * KT;
            g.t0 = tbase + g.slot0 - ring0;
            g.t_lo = tbase;
            g.t_hi = tbase + len_a;
        } else {
            g.slot0 = (j - n_a) * KT;
            g.t0 = tbase + len_a + g.slot0;
            g.t_lo = tbase + len_a;
            g.t_hi = klen;
        }
        return g;
    }
};

// The end of a CTA that ran several softmax groups: their sums, staged in shared memory (layout below),
// are merged per slot and stored.  Short rolled loops, kept out of line (they run once per CTA).
//   mrg [NG][NS][128 dims] output sums | lsm [NG][NS][128 keys] denominators per key row |
//   rsm [NG][NSP] running references   | lfs [NG][NSP] denominators
struct TailArgs {
    float *partial;            // this split's partial rows (row 0 of the batch), or nullptr: write normalised outputs
    uint8_t *out;
    long out_batch_stride;
    int export_nat, out_type, S, nh, kvg;
    unsigned int kvg_magic;
    int b, kvh, slot0, nvalid; // batch element, KV head, first slot of the row group, its valid slots
};
template <int NS, int NSP, int NG, int NSW>
__device__ __noinline__ void group_denominators(float *stage, int warp, int lane) {
    const float *lsm = stage + NG * NS * HD;
    float *lfs = stage + NG * NS * HD + NG * NS * KT + NG * NSP;
#pragma unroll 1
    for (int idx = warp; idx < NG * NS; idx += NSW) {                 // a warp per (group, slot)
        const float4 v = reinterpret_cast<const float4 *>(lsm + idx * KT)[lane];
        float t = (v.x + v.y) + (v.z + v.w);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) lfs[(idx / NS) * NSP + idx % NS] = t;
    }
}
template <int NS, int NSP, int NG>
__device__ __noinline__ void group_outputs(const TailArgs a, const float *stage, int grp, int kr) {
    const float *mrg = stage, *rsm = stage + NG * NS * HD + NG * NS * KT, *lfs = rsm + NG * NSP;
    // common reference = the largest, sums rescaled by 2^(own - common); thread (group, dim) takes slots
    // group, group + NG, ...
#pragma unroll 1
    for (int s = grp; s < a.nvalid; s += NG) {
        float rmax = rsm[s];
#pragma unroll
        for (int gg = 1; gg < NG; ++gg) rmax = fmaxf(rmax, rsm[gg * NSP + s]);
        float o = 0.0f, l = 0.0f;
#pragma unroll
        for (int gg = 0; gg < NG; ++gg) {
            const float w = ex2f(rsm[gg * NSP + s] - rmax);          // a group without tiles has sums 0 and the initial reference
            o = fmaf(mrg[(gg * NS + s) * HD + kr], w, o);
            l = fmaf(lfs[gg * NSP + s], w, l);
        }
        const int idx = a.slot0 + s;
        const int r = a.kvg_magic ? (int)__umulhi((unsigned)idx, a.kvg_magic) : idx;
        const int hrow = r * a.nh + a.kvh * a.kvg + (idx - r * a.kvg);          // row within the batch element
        if (a.partial) {
            float *pr = a.partial + (size_t)(a.b * a.S * a.nh + hrow) * (HD + 2) + kr;
            pr[0] = o;
            if (kr == 0) {
                pr[HD] = a.export_nat ? rmax * LN2 : rmax;
                pr[HD + 1] = l;
            }
        } else {
            const float v = l > 0.0f ? o / l : 0.0f;
            const long oi = a.b * a.out_batch_stride + (long)hrow * HD + kr;
            if (a.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(a.out)[oi] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(a.out)[oi] = v;
        }
    }
}

template <int NS>
__global__ void __launch_bounds__(Cfg<NS>::NTHREADS, Cfg<NS>::MIN_CTAS)
    attn_tc5_kernel(const __grid_constant__ KParams p, const __grid_constant__ TmaMaps4 tm) {
    using C = Cfg<NS>;
    constexpr int NSP = C::NSP, NSTG = C::NSTG;
    constexpr int NG = C::NG, NB = C::NB, LAG = C::LAG, NSW = C::NSW, NTHREADS = C::NTHREADS;
    constexpr int NSG = NS;                          // slots per softmax thread: all of the CTA's
    constexpr int CH = NSG % 8 == 0 ? 8 : NSG % 4 == 0 ? 4 : 2;      // slots per TMEM load
    constexpr int NCH = NSG / CH;
    constexpr uint32_t TMEM_O = 64 * NB;             // first column of the O^T buffers

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sm_u32 = smem_u32(sm);
    float *slot_qscale = reinterpret_cast<float *>(sm + C::OFF_SLOT);      // base-2 logit per unit of the integer dot product and of the key's scale
    int *slot_lo = reinterpret_cast<int *>(sm + C::OFF_SLOT + NSP * 4);
    int *slot_hi = reinterpret_cast<int *>(sm + C::OFF_SLOT + NSP * 8);
    float *xch_all = reinterpret_cast<float *>(sm + C::OFF_XCH);            // [NG][2][NSP][4]
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(sm + C::OFF_MISC);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + C::OFF_MISC + 4);
    const uint32_t bar0 = sm_u32 + C::OFF_BAR;
    auto bar_full = [&](int s) { return bar0 + 8 * s; };
    auto bar_empty = [&](int s) { return bar0 + 8 * (NSTG + s); };
    auto bar_s_ready = [&](int i) { return bar0 + 8 * (2 * NSTG + i); };
    auto bar_p_ready = [&](int i) { return bar0 + 8 * (2 * NSTG + NB + i); };
    auto bar_o_ready = [&](int i) { return bar0 + 8 * (2 * NSTG + 2 * NB + i); };
    auto bar_o_free = [&](int i) { return bar0 + 8 * (2 * NSTG + 3 * NB + i); };
    const uint32_t bar_q_ready = bar0 + 8 * (2 * NSTG + 4 * NB);
    auto bar_xch = [&](int g, int i) { return bar0 + 8 * (2 * NSTG + 4 * NB + 1 + 2 * g + i); };
    // the new keys are the window's last ones, so at most the CTA's last two tiles hold any: each of
    // those has a barrier of its own, used once
    auto bar_patched = [&](int k) { return bar0 + 8 * (2 * NSTG + 4 * NB + 1 + 2 * NG + k); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int b = blockIdx.z / p.row_groups, rg = blockIdx.z % p.row_groups;

    // ------------------------------------------------------------ window and tile schedule
    WindowGeo wg;
    wg.tbase = p.tile0;                               // first window index any query row needs
    wg.klen = p.klen;
    wg.ring0 = (p.win_start + wg.tbase) % p.cache_cap;
    wg.len_a = min(p.klen - wg.tbase, p.cache_cap - wg.ring0);
    wg.a0 = wg.ring0 & ~3;
    wg.n_a = (wg.ring0 + wg.len_a - wg.a0 + KT - 1) / KT;
    const int tile_begin = split * p.tiles_per_split;
    int tile_end = min(p.ntiles, tile_begin + p.tiles_per_split);
    int my_n = max(0, tile_end - tile_begin);
    const int row_base = kvh * p.cache_cap;          // this head's first row in the {rows} dimension of the maps
    // Paged caches (block_table != nullptr): the sequence's tile j lives in page block_table[b][j] of the
    // pools, a page holding 128 rows of every KV head; its length comes from seq_lens[b].  Set below, after
    // the stream-order wait (both arrays may have been written by the preceding kernel).
    const bool paged = p.block_table != nullptr;
    int *page_ids = reinterpret_cast<int *>(sm + C::OFF_PAGES);
    // fused quantize-on-write: the last n_new keys of the window arrive as fp32 rows with this call
    const int new_lo = p.new_k ? p.klen - p.n_new : 0x7fffffff;      // window index of the first new key
    auto tile_has_new = [&](const TileGeo &g) { return min(g.t0 + KT, g.t_hi) > new_lo; };
    // which of the two "patched" barriers CTA tile i uses (only asked for tiles with new keys)
    auto patch_index = [&](int i) { return (i >= 1 && tile_has_new(wg.tile(tile_begin + i - 1))) ? 1 : 0; };
    // fp32 row scales ride TMA when every tile's first scale sits on a 16-byte boundary; otherwise
    // each softmax thread fetches its key's two scales one tile ahead with plain loads
    const bool scales_by_tma = (p.use_tma & 2) != 0;

    // ------------------------------------------------------------ set-up
    if (threadIdx.x == 0) {
        *abort_flag = 0;
#pragma unroll
        for (int s = 0; s < NSTG; ++s) { fused::mbar_init(bar_full(s), 1); fused::mbar_init(bar_empty(s), 1); }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            fused::mbar_init(bar_s_ready(i), 1);
            fused::mbar_init(bar_p_ready(i), 128);
            fused::mbar_init(bar_o_ready(i), 1);
            fused::mbar_init(bar_o_free(i), 128);
        }
#pragma unroll
        for (int g = 0; g < NG; ++g) { fused::mbar_init(bar_xch(g, 0), 128); fused::mbar_init(bar_xch(g, 1), 128); }
        fused::mbar_init(bar_q_ready, 128 * NG);
        fused::mbar_init(bar_patched(0), 32);
        fused::mbar_init(bar_patched(1), 32);
        fused::fence_mbar_init();
    }
    if (warp == NSW + 1 && lane == 0) {
        fused::prefetch_tensormap(&tm.k); fused::prefetch_tensormap(&tm.v);
        if (scales_by_tma) { fused::prefetch_tensormap(&tm.ks); fused::prefetch_tensormap(&tm.vs); }
    }
    if (warp == NSW) {
        tmem_alloc(sm_u32 + C::OFF_MISC, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: every thread waits for the stream predecessor before it lets
    // this grid's own dependents be scheduled.  The producer thread first requests the tiles the
    // caller declared settled, and the softmax warps first run their query preparation once on
    // whatever the query buffer holds (see below); both wait further down.
    const bool dry_first = !paged && warp < NSW && p.dry_pass;
    if (!((warp == NSW && lane == 0) || dry_first) || paged) {
        fused::pdl_wait();
        fused::pdl_launch_dependents();
    }
    if (paged) {
        const int len = p.seq_lens[b];
        wg.klen = len; wg.ring0 = 0; wg.a0 = 0; wg.len_a = len;
        wg.n_a = (len + KT - 1) / KT;
        tile_end = min(wg.n_a, tile_begin + p.tiles_per_split);
        my_n = max(0, tile_end - tile_begin);
        for (int i = threadIdx.x; i < my_n; i += NTHREADS) page_ids[i] = p.block_table[(size_t)b * p.max_pages + tile_begin + i];
        __syncthreads();
    }

    auto make_tail_args = [&]() {
        TailArgs t;
        t.partial = p.write_partial ? p.partial + ((size_t)split * p.grows) * (HD + 2) : nullptr;
        t.out = p.out; t.out_batch_stride = p.out_batch_stride;
        t.export_nat = p.export_nat; t.out_type = p.out_type; t.S = p.S; t.nh = p.nh;
        t.kvg = p.kvg; t.kvg_magic = p.kvg_magic;
        t.b = b; t.kvh = kvh; t.slot0 = rg * NS; t.nvalid = min(NS, p.S * p.kvg - rg * NS);
        return t;
    };

    if (warp == NSW) {
        // =========================================================== TMA producer
        if (lane == 0) {
            bool waited = paged;
            for (int i = 0; i < my_n; ++i) {
                const int st = i % NSTG;
                const TileGeo g = wg.tile(tile_begin + i);
                const int row0 = paged ? (page_ids[i] * p.nkv + kvh) * KT : row_base + g.slot0;   // first row of the tile in the maps
                // rows the caller declared settled may be requested before the stream predecessor is done
                if (!waited && g.t0 + KT > p.early_rows) { fused::pdl_wait(); fused::pdl_launch_dependents(); waited = true; }
                if (i >= NSTG && !wait_or_abort(bar_empty(st), ((i / NSTG) - 1) & 1, abort_flag, p.fault)) break;
                const uint32_t kdst = sm_u32 + st * 2 * TILE_BYTES;
                const uint32_t sdst = sm_u32 + C::OFF_SCALES + st * 2 * SCALE_BYTES;
                fused::mbar_expect_tx(bar_full(st), 2 * TILE_BYTES + (scales_by_tma ? 2 * SCALE_BYTES : 0));
                const int bc = paged ? 0 : b;                    // the pools are one plane for all sequences
                if (p.kv_read_once) {            // evict-first in L2: the launch does not come back to these bytes
                    fused::tma_load_tile_once(kdst, &tm.k, row0, bc, bar_full(st));
                    fused::tma_load_tile_once(kdst + TILE_BYTES, &tm.v, row0, bc, bar_full(st));
                } else {
                    fused::tma_load_tile(kdst, &tm.k, row0, bc, bar_full(st));
                    fused::tma_load_tile(kdst + TILE_BYTES, &tm.v, row0, bc, bar_full(st));
                }
                if (scales_by_tma) {
                    tma_load_2d(sdst, &tm.ks, row0, bc, bar_full(st));
                    tma_load_2d(sdst + SCALE_BYTES, &tm.vs, row0, bc, bar_full(st));
                }
            }
            if (!waited) { fused::pdl_wait(); fused::pdl_launch_dependents(); }
        }
        __syncwarp();
    } else if (warp == NSW + 1) {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(C::N, true, true, false);
            const uint32_t idesc_pv = make_idesc(C::N, true, false, true);
            const uint64_t qdesc = smem_desc_sw128(sm_u32 + C::OFF_Q);
            bool go = wait_or_abort(bar_q_ready, 0, abort_flag, p.fault);
            for (int i = 0; go && i < my_n + LAG; ++i) {
                if (i < my_n) {
                    // S^T[i % NB] = K_i x Q^T.  The buffer's previous reader (tile i-NB) was done before
                    // p_ready(i-NB), which this thread observed when it issued PV(i-NB), LAG < NB rounds later.
                    const int st = i % NSTG, bf = i % NB;
                    if (!wait_or_abort(bar_full(st), (i / NSTG) & 1, abort_flag, p.fault)) break;
                    if (tile_has_new(wg.tile(tile_begin + i))) {      // a softmax warp overwrites the new keys' rows first
                        if (!wait_or_abort(bar_patched(patch_index(i)), 0, abort_flag, p.fault)) break;
                    }
                    tc_fence_after();
                    const uint64_t kdesc = smem_desc_sw128(sm_u32 + st * 2 * TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < HD / 32; ++k)      // 32 bytes of K per instruction: +32 B on both operands
                        umma_i8(tmem_base + 64 * bf, kdesc + 2 * k, qdesc + 2 * k, idesc_qk, k > 0);
                    umma_commit(bar_s_ready(bf));
                }
                if (i >= LAG) {
                    // O^T[j % NB] = V_j^T x P_j^T
                    const int j = i - LAG, st = j % NSTG, bf = j % NB;
                    if (!wait_or_abort(bar_p_ready(bf), (j / NB) & 1, abort_flag, p.fault)) break;
                    if (j >= NB && !wait_or_abort(bar_o_free(bf), ((j - NB) / NB) & 1, abort_flag, p.fault)) break;
                    tc_fence_after();
                    const uint64_t vdesc = smem_desc_sw128(sm_u32 + st * 2 * TILE_BYTES + TILE_BYTES);
                    const uint64_t pdesc = smem_desc_sw128(sm_u32 + C::OFF_P + bf * C::QP_BYTES);
#pragma unroll
                    for (int k = 0; k < KT / 32; ++k)      // 32 keys per instruction: 4 row groups of V (+4096 B), +32 B of P
                        umma_i8(tmem_base + TMEM_O + 64 * bf, vdesc + 256 * k, pdesc + 2 * k, idesc_pv, k > 0);
                    umma_commit(bar_o_ready(bf));
                    umma_commit(bar_empty(st));
                }
            }
        }
        __syncwarp();
    } else if (warp < NSW) {
        // =========================================================== softmax warps
        const int grp = warp >> 2, wq = warp & 3;        // group, and the TMEM lane quarter this warp may read
        const int kr = threadIdx.x & 127;                // key row of S^T, output dim of O^T
        float *xch = xch_all + grp * 2 * NSP * 4;        // this group's [2][NSP][4] exchange area
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(32 * wq) << 16);
        auto wait_warp = [&](uint32_t bar, uint32_t parity) {
            return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag, p.fault)) != 0;
        };
        // byte (row, col) of a K-major operand tile with 128-byte rows, 128B-swizzled
        auto at = [](int row, int col) { return (row >> 3) * 1024 + (row & 7) * 128 + ((((col >> 4) ^ (row & 7)) << 4) | (col & 15)); };

        const float *gks = reinterpret_cast<const float *>(p.k_scales + b * p.scale_batch_stride);
        const float *gvs = reinterpret_cast<const float *>(p.v_scales + b * p.scale_batch_stride);
        const int last_row = p.nkv * p.cache_cap - 1;
        float ks_next = 0.0f, vs_next = 1.0f;
        auto fetch_scales = [&](int i) {
            if (!scales_by_tma && i < my_n) {
                const int row = min(row_base + wg.tile(tile_begin + i).slot0 + kr, last_row);   // rows past the cache are masked anyway
                ks_next = __ldcg(gks + row);                 // through L2: the newest rows' scales may have been written
                vs_next = __ldcg(gvs + row);                 // by the stream predecessor after the warming pass read them
            }
        };
        // The query preparation runs twice.  The first pass starts before the stream-order wait, on
        // whatever the query (and new-row) buffers hold at that moment, and its results are thrown away:
        // it only brings this straight-line code into the instruction caches while the CTA would otherwise
        // idle behind its predecessor, so that the pass that counts, after the wait, is not fetched cold
        // (measured: about 3 us less on the verify kernel).  Nothing but shared-memory scratch is written
        // in the first pass.
        float lsum[NSG], acc[NSG];                       // denominators and output sums over this group's tiles, every slot
        int lo_max = 0, hi_min = 0x7fffffff;             // keys in [lo_max, hi_min) are visible to every query row
#pragma unroll 1
        for (int pass = dry_first ? 0 : 1; pass < 2; ++pass) {
            if (pass == 1 && dry_first) {
                fused::pdl_wait();
                fused::pdl_launch_dependents();
            }
            fetch_scales(grp);                               // in flight while the query rows are prepared
            // ---- query rows -> two int8 limbs each (16-bit fixed point: q ~= sq * (256 hi + lo)).
            // A warp prepares slots warp, warp+4, ...; all their loads are issued before the first use.
            constexpr int QPW = (NSP + NSW - 1) / NSW;
            uint32_t qraw[QPW][HD / 32];
            {
                long qoff[QPW];
    #pragma unroll
                for (int k = 0; k < QPW; ++k) {
                    const int idx = rg * NS + warp + NSW * k;
                    const int r = fused::div_kvg(p, idx), j = idx - r * p.kvg;
                    const bool valid = warp + NSW * k < NS && r < p.S;
                    qoff[k] = b * p.q_batch_stride + (valid ? ((long)r * p.nh + kvh * p.kvg + j) * HD : (long)(kvh * p.kvg) * HD) + lane;
                }
                // raw bits first, conversions afterwards: every load is in flight before the first use.  The loads go
                // through L2 only (ld.global.cg, never the read-only path): the warming pass reads the query while the
                // stream predecessor (e.g. the producer epilogue rewriting it in place) may still be running.
                if (p.q_type == ET_BF16) {
    #pragma unroll
                    for (int k = 0; k < QPW; ++k)
    #pragma unroll
                        for (int i = 0; i < HD / 32; ++i) qraw[k][i] = (uint32_t)__ldcg(reinterpret_cast<const uint16_t *>(p.q) + qoff[k] + 32 * i) << 16;
                } else {
    #pragma unroll
                    for (int k = 0; k < QPW; ++k)
    #pragma unroll
                        for (int i = 0; i < HD / 32; ++i) qraw[k][i] = __ldcg(reinterpret_cast<const uint32_t *>(p.q) + qoff[k] + 32 * i);
                }
            }
            // ---- fused quantize-on-write, early: while the query and the first tiles are in flight, the softmax
            // warps of the CTA that owns the tile(s) of the new keys quantise the fp32 rows with the row codec of
            // the append kernels (bit for bit) into scratch rows, one (row, plane) per warp at a time, and -- row
            // group 0 only, so once per KV head -- copy bytes and scale into the ring for later calls.
            const bool cta_has_new = p.new_k != nullptr && my_n > 0 && tile_has_new(wg.tile(tile_end - 1));
            if (cta_has_new) {
                float *new_sc = reinterpret_cast<float *>(sm + C::OFF_NEWSC);
                for (int pidx = warp; pidx < 2 * p.n_new; pidx += NSW) {
                    const int n = pidx >> 1, kv = pidx & 1;
                    uint8_t *scr = sm + C::OFF_NEW + pidx * 144;
                    const float *src = (kv ? p.new_v : p.new_k) + ((size_t)b * p.n_new + n) * p.new_stride + kvh * HD;
                    quant_row_i8_cg(src, HD, HD, reinterpret_cast<int8_t *>(scr), reinterpret_cast<float *>(scr + 128), lane);
                    __syncwarp();
                    const float sc_row = *reinterpret_cast<const float *>(scr + 128);
                    if (lane == 0) new_sc[kv * NEW_MAX + n] = sc_row;
                    if (rg == 0 && pass == 1) {
                        const size_t crow = (size_t)row_base + (size_t)((p.new_base_pos + n) % p.cache_cap);
                        uint8_t *g_rows = (kv ? p.v_cache_w : p.k_cache_w) + b * p.kv_batch_stride + crow * p.cache_hd;
                        float *g_sc = reinterpret_cast<float *>((kv ? p.v_scales_w : p.k_scales_w) + b * p.scale_batch_stride) + crow;
                        if (lane < 8) reinterpret_cast<uint4 *>(g_rows)[lane] = reinterpret_cast<const uint4 *>(scr)[lane];
                        if (lane == 0) *g_sc = sc_row;
                    }
                }
            }
            float qx[QPW][HD / 32];
    #pragma unroll
            for (int k = 0; k < QPW; ++k) {
                const int idx = rg * NS + warp + NSW * k;
                const bool valid = warp + NSW * k < NS && fused::div_kvg(p, idx) < p.S;
    #pragma unroll
                for (int i = 0; i < HD / 32; ++i) qx[k][i] = valid ? __uint_as_float(qraw[k][i]) : 0.0f;
            }
    #pragma unroll
            for (int k = 0; k < QPW; ++k) {
                const int sl = warp + NSW * k;
                if (sl >= NSP) break;
                const int idx = rg * NS + sl;
                const int r = fused::div_kvg(p, idx);
                const bool valid = sl < NS && r < p.S;
                float amax = 0.0f;
    #pragma unroll
                for (int i = 0; i < HD / 32; ++i) amax = fmaxf(amax, fabsf(qx[k][i]));
                amax = warp_max(amax);
                const float sq = amax > 0.0f ? amax * (1.0f / (float)Q_FIX_MAX) : 1.0f;   // each row its own scale
                const float inv = rcpf(sq);
    #pragma unroll
                for (int i = 0; i < HD / 32; ++i) {
                    int qf = __float2int_rn(qx[k][i] * inv);
                    qf = max(-Q_FIX_MAX, min(Q_FIX_MAX, qf));
                    const int hi = (qf + 128) >> 8, lo = qf - (hi << 8);
                    sm[C::OFF_Q + at(sl, lane + 32 * i)] = (uint8_t)(int8_t)hi;
                    sm[C::OFF_Q + at(NSP + sl, lane + 32 * i)] = (uint8_t)(int8_t)lo;
                }
                if (lane == 0) {
                    const int hi_b = valid ? wg.klen - (p.S - 1 - r) : 0;
                    slot_qscale[sl] = valid ? sq * p.qk_scale_log2 : 0.0f;
                    slot_hi[sl] = hi_b;
                    slot_lo[sl] = (valid && p.window > 0) ? max(0, hi_b - p.window) : 0;
                }
            }
            // the limbs are read by the tensor core (async proxy).  Not in the warming pass: with tile copies in
            // flight the fence takes as long as they do (measured +1 us on the decode call).
            if (pass == 1) fused::fence_proxy_async();
            // every softmax warp's slot constants are visible (and the scratch may be rewritten by the next pass)
            asm volatile("bar.sync 1, %0;\n" ::"n"(32 * NSW) : "memory");
            lo_max = 0; hi_min = 0x7fffffff;
#pragma unroll
            for (int s = 0; s < NSG; ++s) {
                lsum[s] = 0.0f; acc[s] = 0.0f;
                if (slot_hi[s] > 0) { lo_max = max(lo_max, slot_lo[s]); hi_min = min(hi_min, slot_hi[s]); }
            }
        }
        mbar_arrive(bar_q_ready);                        // the MMA issuer starts on the first tile
        bool alive = wait_warp(bar_q_ready, 0);

        // The loops below are written phase by phase over all slots (loads, then arithmetic, then
        // stores) so that the slots' independent instruction chains overlap: each scheduler of the
        // SM runs a single softmax warp and has nothing else to hide latencies with.
        float r_lane = M_INIT;                                // running reference of slot `lane` (lanes < NSG)
        float fw_lane = 0.0f;                                 // same lane: what a unit of the previous tile's O^T is worth
        float4 *my_consts = reinterpret_cast<float4 *>(sm + C::OFF_SLOTC) + warp * NSP;
        // O^T of tile j: add the exact int32 sums with the tile's weight fe[slot]
        auto epilogue = [&](int j, const float (&fe)[NSG]) -> bool {
            const int bf = j % NB;
            if (!wait_warp(bar_o_ready(bf), (j / NB) & 1)) return false;
            tc_fence_after();
            int oh[NCH][CH], ol[NCH][CH];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                tmem_ld<CH>(tmem_lane + TMEM_O + 64 * bf + CH * c, oh[c]);
                tmem_ld<CH>(tmem_lane + TMEM_O + 64 * bf + NSP + CH * c, ol[c]);
            }
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
                for (int e = 0; e < CH; ++e)      // each limb sum is below 128 * 255 * 127 < 2^22: the combination fits an int
                    acc[c * CH + e] = fmaf(limbs2f<8>(oh[c][e], ol[c][e]), fe[c * CH + e], acc[c * CH + e]);
            tc_fence_before();
            mbar_arrive(bar_o_free(bf));
            return true;
        };

        int last_done = -1;                              // this group's last tile whose P was handed to the tensor core
        for (int i = grp; alive && i < my_n; i += NG) {
            const int st = i % NSTG, bf = i % NB;
            const int b2 = (i / NG) & 1, xph = ((i / NG) >> 1) & 1;      // exchange buffer and its barrier's phase: per own tile
            const TileGeo g = wg.tile(tile_begin + i);
            const float ks_ld = ks_next, vs_ld = vs_next;
            fetch_scales(i + NG);
            if (!wait_warp(bar_full(st), (i / NSTG) & 1)) { alive = false; break; }
            const float *sc = reinterpret_cast<const float *>(sm + C::OFF_SCALES + st * 2 * SCALE_BYTES);
            const int t = g.t0 + kr;
            const bool row_ok = t >= g.t_lo && t < g.t_hi;
            const bool need_mask = g.t0 < max(g.t_lo, lo_max) || g.t0 + KT > min(g.t_hi, hi_min);
            float ks = scales_by_tma ? sc[kr] : ks_ld;
            float vs_raw = scales_by_tma ? sc[KT + kr] : vs_ld;
            if (tile_has_new(g)) {
                // ---- new keys of this tile: warp 0 overwrites the rows TMA fetched for their slots with the
                // codes quantised in the prologue; the MMA issuer waits for this.
                const uint32_t bar_pt = bar_patched(patch_index(i));
                if (wq == 0) {
                    for (int n = 0; n < p.n_new; ++n) {
                        const int wi = new_lo + n;                        // window index of new key n
                        if (wi < max(g.t0, g.t_lo) || wi >= min(g.t0 + KT, g.t_hi)) continue;
                        const int r = wi - g.t0;
#pragma unroll
                        for (int kv = 0; kv < 2; ++kv) {
                            const uint8_t *scr = sm + C::OFF_NEW + (2 * n + kv) * 144;
                            uint8_t *tile_rows = sm + st * 2 * TILE_BYTES + kv * TILE_BYTES;
                            if (lane < 8)
                                *reinterpret_cast<uint4 *>(tile_rows + (r >> 3) * 1024 + (r & 7) * 128 + ((lane ^ (r & 7)) << 4)) =
                                    *reinterpret_cast<const uint4 *>(scr + lane * 16);
                        }
                    }
                    fused::fence_proxy_async();                          // the tensor core reads the patched rows
                    mbar_arrive(bar_pt);
                }
                if (!wait_warp(bar_pt, 0)) { alive = false; break; }
                if (t >= new_lo && row_ok) {
                    const float *new_sc = reinterpret_cast<const float *>(sm + C::OFF_NEWSC);
                    ks = new_sc[t - new_lo];
                    vs_raw = new_sc[NEW_MAX + t - new_lo];
                }
            }
            const float vs = row_ok ? fmaxf(vs_raw, 5.421011e-20f) : 1.0f;   // floor 2^-64: keeps 1/vs finite
            const float lvs = lg2f(vs), rvs = row_ok ? rcpf(vs) : 0.0f;
            if (!wait_warp(bar_s_ready(bf), (i / NB) & 1)) { alive = false; break; }
            tc_fence_after();
            int sh[NCH][CH], sl_[NCH][CH];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                tmem_ld<CH>(tmem_lane + 64 * bf + CH * c, sh[c]);
                tmem_ld<CH>(tmem_lane + 64 * bf + NSP + CH * c, sl_[c]);
            }
            tmem_wait_ld();
            // u = base-2 logit + log2(v_scale): 2^(u - max u) is the key's weight on the V bytes relative
            // to the tile's largest, the quantity that goes to the tensor core as 16-bit fixed point
            float u[NSG];
#pragma unroll
            for (int s = 0; s < NSG; ++s)         // limb sums are below 128 * 128 * 127 < 2^22: the combination fits an int
                u[s] = fmaf(limbs2f<8>(sh[s / CH][s % CH], sl_[s / CH][s % CH]), slot_qscale[s] * ks, lvs);
            if (need_mask) {
#pragma unroll
                for (int s = 0; s < NSG; ++s) {
                    const bool ok = row_ok && t >= slot_lo[s] && t < slot_hi[s];
                    u[s] = ok ? u[s] : -CUDART_INF_F;
                }
            }
            // tile maximum per slot: one warp-wide max each, exchanged through shared memory;
            // lane s carries slot s's value to a single store
            float mine = 0.0f;
#pragma unroll
            for (int s = 0; s < NSG; ++s) {
                const float wm = redux_max(u[s]);
                mine = lane == s ? wm : mine;
            }
            if (lane < NSG) xch[(b2 * NSP + lane) * 4 + wq] = mine;
            mbar_arrive(bar_xch(grp, b2));
            if (!wait_warp(bar_xch(grp, b2), xph)) { alive = false; break; }
            // Per-slot constants of the tile are the same for every key: lane s of each warp works them
            // out for slot s (the running reference R of that slot lives in that lane) and the warp
            // shares them through shared memory, instead of every thread repeating them for every slot.
            // The reference only moves when the tile maximum exceeds it by more than 2^8 (weights are
            // normalised per tile, so a stale reference costs no precision): either it stays (alpha = 1,
            // tile weight 2^d) or it moves to the tile maximum (tile weight 1, alpha = 2^-d).
            bool moved = false;
            if (lane < NSG) {
                const float4 m4 = *reinterpret_cast<const float4 *>(xch + (b2 * NSP + lane) * 4);
                const float umax = fmaxf(fmaxf(m4.x, m4.y), fmaxf(m4.z, m4.w));
                const float d = umax - r_lane;                           // -inf when every key of the tile is masked
                moved = d > LAZY_MAX;
                const float e = ex2f(moved ? -d : d);
                r_lane = moved ? umax : r_lane;
                const float tw = moved ? 1.0f : e;                      // weight of this tile's sums against the reference
                const float alpha = moved ? e : 1.0f;                   // what the sums so far are rescaled by
                my_consts[lane] = make_float4(umax == -CUDART_INF_F ? 0.0f : umax, tw, alpha, fw_lane * alpha);
                fw_lane = tw * (1.0f / P_FIX);
            }
            const bool any_moved = __any_sync(0xffffffffu, moved);
            __syncwarp();
            if (any_moved) {
#pragma unroll
                for (int s = 0; s < NSG; ++s) {
                    const float alpha = my_consts[s].z;
                    lsum[s] *= alpha; acc[s] *= alpha;
                }
            }
            float fe[NSG];                                               // weight of the previous tile's O^T units
            uint32_t fx[NSG];
#pragma unroll
            for (int s = 0; s < NSG; ++s) {
                const float4 c = my_consts[s];                           // (tile max or 0, tile weight, alpha, previous tile's unit weight)
                const float w = ex2f(u[s] - c.x);                        // in [0, 1]
                fe[s] = c.w;
                lsum[s] = fmaf(w * c.y, rvs, lsum[s]);                   // 2^(logit - R): the softmax denominator
                fx[s] = __float_as_uint(fmaf(w, P_FIX, RND_MAGIC));
            }
            __syncwarp();                                                // my_consts is rewritten next tile
            // byte (row s, key kr) of the 128B-swizzled P tile: the row picks the 1024-byte group and the
            // line in it, and flips bits 4..6 of the key
            uint8_t *pt = sm + C::OFF_P + bf * C::QP_BYTES;
#pragma unroll
            for (int s = 0; s < NSG; ++s) {
                const int off = (s >> 3) * 1024 + (s & 7) * 128 + (kr ^ ((s & 7) << 4));
                pt[off] = (uint8_t)(fx[s] >> 8);
                pt[off + NSP * 128] = (uint8_t)fx[s];                    // low limbs: NSP rows (a multiple of 8) further down
            }
            fused::fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar_p_ready(bf));
            if (last_done >= 0 && !epilogue(last_done, fe)) { alive = false; break; }
            last_done = i;
        }
        if (alive && last_done >= 0) {
            float fe[NSG];
            if (lane < NSG) my_consts[lane].w = fw_lane;
            __syncwarp();
#pragma unroll
            for (int s = 0; s < NSG; ++s) fe[s] = my_consts[s].w;
            alive = epilogue(last_done, fe);
        }

        const int nvalid = min(NS, p.S * p.kvg - rg * NS);
        float *pbase = p.partial + ((size_t)split * p.grows) * (HD + 2) + kr;
        // one slot's row of this thread's dim: the partial (sum, reference, denominator) or the final output
        auto put_row = [&](int s, float a, float rs, float l) {
            const int idx = rg * NS + s;
            const int r = fused::div_kvg(p, idx);
            const int hrow = r * p.nh + kvh * p.kvg + (idx - r * p.kvg);          // row within the batch element
            if (p.write_partial) {
                float *pr = pbase + (size_t)(b * p.S * p.nh + hrow) * (HD + 2);
                pr[0] = a;
                if (kr == 0) {
                    pr[HD] = p.export_nat ? rs * LN2 : rs;
                    pr[HD + 1] = l;
                }
            } else {
                const float v = l > 0.0f ? a / l : 0.0f;
                const long oi = b * p.out_batch_stride + (long)hrow * HD + kr;
                if (p.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[oi] = __float2bfloat16_rn(v);
                else reinterpret_cast<float *>(p.out)[oi] = v;
            }
        };
        if constexpr (NG == 1) {
            // ---- denominators: sum the per-key partial sums over the 128 threads
            float *lred = xch;                               // [NSP][4] sums, then [NSP][4] references (element 0)
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int s = 0; s < NSG; ++s) lsum[s] += __shfl_xor_sync(0xffffffffu, lsum[s], o);
            float mine_l = 0.0f;
#pragma unroll
            for (int s = 0; s < NSG; ++s) mine_l = lane == s ? lsum[s] : mine_l;
            if (lane < NSG) lred[lane * 4 + wq] = mine_l;
            if (lane < NSG && wq == 0) lred[(NSP + lane) * 4] = r_lane;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");                 // the four softmax warps
            // ---- outputs: this thread owns dim kr of every slot
#pragma unroll
            for (int s = 0; s < NSG; ++s) {
                if (s < nvalid) {
                    const float4 l4 = *reinterpret_cast<const float4 *>(lred + s * 4);
                    put_row(s, acc[s], lred[(NSP + s) * 4], (l4.x + l4.y) + (l4.z + l4.w));
                }
            }
        } else {
            // Every group has seen its last O^T, so every MMA of the CTA has completed and every tile has
            // landed: the tile stages are free to carry the groups' sums.  What follows runs once per CTA,
            // so it is written as short rolled loops over shared memory rather than unrolled over the slots.
            asm volatile("bar.sync 1, %0;\n" ::"n"(32 * NSW) : "memory");
            float *mrg = reinterpret_cast<float *>(sm);                       // [NG][NS][128 dims] output sums
            float *lsm = mrg + NG * NS * HD;                                  // [NG][NS][128 keys] denominators per key row
            float *rsm = lsm + NG * NS * KT;                                  // [NG][NSP] running references
            float *lfs = rsm + NG * NSP;                                      // [NG][NSP] denominators
#pragma unroll
            for (int s = 0; s < NSG; ++s) {
                mrg[(grp * NS + s) * HD + kr] = acc[s];
                lsm[(grp * NS + s) * KT + kr] = lsum[s];
            }
            if (wq == 0 && lane < NSG) rsm[grp * NSP + lane] = r_lane;
            asm volatile("bar.sync 1, %0;\n" ::"n"(32 * NSW) : "memory");
            group_denominators<NS, NSP, NG, NSW>(mrg, warp, lane);
            asm volatile("bar.sync 1, %0;\n" ::"n"(32 * NSW) : "memory");
            group_outputs<NS, NSP, NG>(make_tail_args(), mrg, grp, kr);
        }
    }

    // ------------------------------------------------------------ tear-down
    tc_fence_before();
    __syncthreads();
    if (warp == NSW) tmem_dealloc(tmem_base, C::TMEM_COLS);
    fused::merge_splits_in_kernel<NS, HD, NTHREADS, 8>(p, sm, b, kvh, rg);
}

}  // namespace tc5
}  // namespace nomos
