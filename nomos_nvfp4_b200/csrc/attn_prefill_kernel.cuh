// Query-major flash prefill over the int8 KV cache on the fifth-generation tensor cores (tcgen05 + tensor
// memory), head_dim 128, sm_100a.  The host side (eligibility, tensor maps, launch) is in attn_fused.cu.
//
// Replaces the reference's square / prefix batched prefill attention
//   lib/attention_gpu_int8.mojo:804-887 (int8), lib/batched_attn_gpu.mojo:448-666 (fp32 / bf16 twins)
// which materialise an [nkv, S*kvg, key_len] score matrix in device memory (the reference's own note on the
// "real fix": lib/engine_prefill.mojo:145; the cap it forces on prompts: pyhost/serve.py:41-64).  Nothing of size
// S x key_len exists here: a CTA owns 128 query rows and walks the key tiles they may attend.
//
// One CTA = 128 query rows of ONE KV head: 128 / kvg consecutive query positions x the kvg query heads of the
// group (position-major, so causal bounds are monotone in the row index), against key tiles of 128 keys.
//   S[128 rows x 128 keys]  = Qlimb[128 x 128 B] (A, K-major, int8) x K_tile[128 keys x 128 B]^T (B, K-major, int8)
//                             once per query limb, kind::i8, int32 accumulators S_hi and S_lo in tensor memory.
//                             B is the K bytes exactly as TMA wrote them; the query is a 16-bit fixed point per row
//                             (two int8 limbs), so the integer dot product is exact.
//   O[128 rows x 128 dims] += Plimb[128 x 128 keys] (A, K-major, fp16) x V16[128 keys x 128 dims] (B, MN-major, fp16)
//                             once per weight limb, kind::f16, one fp32 accumulator in tensor memory across all tiles.
//                             V16 holds the int8 CODES of V (exact in fp16), converted by four "dequant" warps; the
//                             softmax weight times the value's row scale is split into fp16 hi + lo, so the weights
//                             carry 22 bits.  (With single fp16 weights the result sat 0.7e-3 x RMS from exact
//                             arithmetic at the median and 2e-3 in the tail over a few thousand rows -- the rounding
//                             of P does not average out against the row's RMS -- which is the accuracy bar itself.)
// The row scales are applied in fp32 by the softmax threads: the key's to the logit, the value's to the weight.
// The cache stays int8 in device memory and on the way in: TMA boxes of 128 rows x 128 bytes, one tensor map per
// plane over this GPU's own memory, no cluster, nothing multicast.
//
// Roles (640 threads): warps 0-15 softmax -- query row r = TMEM lane r is shared by four threads, lane r % 32 of warps
// r / 32 + 4 q, q = 0..3 (all may read that lane quarter), each taking 32 of the tile's 128 keys: four warps per
// scheduler hide each other's latencies (one warp per scheduler measured 0.16 instructions per cycle, two 0.34), the
// row maximum crosses the four through shared memory once per tile; warps 16-17 dequant (a thread converts two key rows
// of the V tile), warp 18 lane 0 TMA producer (+ TMEM allocation), warp 19 lane 0 MMA issuer.  The softmax threads pull
// S into registers and release it at once, so QK of tile i+1 runs while they work on tile i; O stays in tensor memory across tiles and is rescaled in
// place only when a row's running maximum moves by more than 2^8 (a handful of times per row).  Every wait is an
// mbarrier wait with a time limit; a wait that runs out raises the CTA's abort flag and bit 1 of the device fault
// word, every role leaves its loop, tensor memory is freed and the CTA exits.
#pragma once

#include "attn_tc5_kernel.cuh"

namespace nomos {
namespace pf {

using fused::LOG2E;
using tc5::wait_or_abort;

constexpr int KT = 128;                       // keys per tile
constexpr int HD = 128;                       // head dim
constexpr int MR = 128;                       // query rows per CTA
constexpr int RAW_TILE = KT * HD;             // int8 tile as TMA writes it (16 KB)
constexpr int H_TILE = KT * HD * 2;           // fp16 operand tile (32 KB) = two 64-column blocks of 16 KB
constexpr int H_BLOCK = 16384;
constexpr float M_INIT = -1.0e30f;
constexpr float LAZY = 8.0f;                  // base-2 slack before a row's running maximum is moved

constexpr int OFF_RAW = 0;                    // [2 stages][K, V] int8 as TMA writes them
constexpr int OFF_V16 = 2 * 2 * RAW_TILE;     // 65536: V codes as fp16
constexpr int OFF_Q8 = OFF_V16 + H_TILE;      // query limbs: high, then low ([128 rows x 128 B] int8 each)
constexpr int OFF_P16 = OFF_Q8 + 2 * RAW_TILE;   // weight limbs: high, then low (fp16 operand tiles)
constexpr int OFF_BAR = OFF_P16 + 2 * H_TILE; // 196608
constexpr int NBAR = 16;
constexpr int OFF_MISC = OFF_BAR + NBAR * 8;  // tmem base, abort flag
constexpr int OFF_SC = OFF_MISC + 64;         // [2 stages][K scales | V scales] fp32, 128 each, bulk-copied with the tile
constexpr int TPR = 4;                        // softmax threads per query row
constexpr int KPT = KT / TPR;                 // keys of a tile (and dims of Q / O) per softmax thread
constexpr int NSOFT = TPR * MR;               // softmax threads
constexpr int W_DEQ = NSOFT / 32;             // first of the two dequant warps; then the TMA producer, then the MMA issuer
constexpr int W_TMA = W_DEQ + 2, W_MMA = W_DEQ + 3;
constexpr int OFF_XCH = OFF_SC + 2 * 2 * KT * 4;        // [3][TPR][128 rows] fp32: row maxima by tile parity; region 2: query maxima, then denominators
constexpr int SMEM_BYTES = 1024 + OFF_XCH + 3 * TPR * 128 * 4;
constexpr int NTHREADS = NSOFT + 128;
static_assert(KPT == 32, "a softmax thread moves one 32-column block of tensor memory per limb");
constexpr int TMEM_COLS = 512;                // S_hi at column 0, S_lo at 128, O at 256
constexpr int Q_FIX_MAX = fused::Q_FIX_MAX;   // 16-bit fixed-point query, two int8 limbs
static_assert(OFF_V16 % 1024 == 0 && OFF_Q8 % 1024 == 0 && OFF_P16 % 1024 == 0, "operand tiles sit on swizzle-pattern boundaries");
static_assert(OFF_SC % 16 == 0, "bulk copies land on 16-byte boundaries");
static_assert(SMEM_BYTES <= 232448, "shared memory budget of a CTA");

struct PParams {
    const uint8_t *q;
    uint8_t *out;
    const float *k_scales, *v_scales;         // fp32 row scales [batch][nkv][cache_cap]
    int q_type, out_type;
    int S, nh, nkv, kvg, cache_cap;
    int row0;                                 // cache slot of key index 0 of the array (win_start; the window does not wrap)
    int key_len;                              // keys of the array
    int d0;                                   // query row s may attend key indices <= d0 + s (d0 may be negative)
    int window;                               // > 0: and no key index below d0 + s - window + 1
    int pos_per_cta;                          // 128 / kvg
    int q_blocks;
    int scales_vec;                           // 1: a tile's scales start on a 16-byte boundary (vector loads)
    float q_scale;                            // softmax_scale * log2(e)
    long q_batch_stride, out_batch_stride, scale_batch_stride;
    unsigned int *fault;
};

struct PMaps {
    CUtensorMap k, v;                         // {row bytes, nkv * cache_cap rows, batch}, box {128 B, 128 rows, 1}, 128B swizzle
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor for kind::f16: fp32 accumulate, fp16 A and B, M = 128, given N; B may be MN-major.
__device__ __forceinline__ uint32_t make_idesc_f16(int n, bool b_mn_major) {
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}
// This warp's 32 TMEM lanes x 32 consecutive 32-bit columns: thread t gets lane t's row.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&r)[32]) {
    uint32_t u[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]),
          "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]), "=r"(u[17]), "=r"(u[18]),
          "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]), "=r"(u[25]), "=r"(u[26]), "=r"(u[27]),
          "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __uint_as_float(u[i]);
}
__device__ __forceinline__ void tmem_ld16i(uint32_t taddr, int (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
        "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
        "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
        "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15])),
        "r"(__float_as_uint(r[16])), "r"(__float_as_uint(r[17])), "r"(__float_as_uint(r[18])), "r"(__float_as_uint(r[19])),
        "r"(__float_as_uint(r[20])), "r"(__float_as_uint(r[21])), "r"(__float_as_uint(r[22])), "r"(__float_as_uint(r[23])),
        "r"(__float_as_uint(r[24])), "r"(__float_as_uint(r[25])), "r"(__float_as_uint(r[26])), "r"(__float_as_uint(r[27])),
        "r"(__float_as_uint(r[28])), "r"(__float_as_uint(r[29])), "r"(__float_as_uint(r[30])), "r"(__float_as_uint(r[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in an fp16 operand tile: two blocks of 64 columns,
// each [128 rows x 128 bytes] in the 128-byte swizzle pattern (8-row groups 1024 bytes apart).
__device__ __forceinline__ int h_off(int row, int chunk) {
    return (chunk >> 3) * H_BLOCK + (row >> 3) * 1024 + (row & 7) * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}
// Four int8 codes -> the same four integers as fp16.  The bytes become 1024 + (code + 128) as fp16 bit patterns
// (0x6400 | u8); subtracting 1152 is exact.
__device__ __forceinline__ void cvt4(uint32_t codes, uint32_t &lo, uint32_t &hi) {
    const uint32_t u = codes ^ 0x80808080u;
    const uint32_t p0 = prmt(u, 0x64646464u, 0x4140u);       // bytes (u0, 0x64, u1, 0x64) -> halves 1024+u0, 1024+u1
    const uint32_t p1 = prmt(u, 0x64646464u, 0x4342u);
    const __half2 bias = __float2half2_rn(1152.0f);
    const __half2 c0 = __hsub2(*reinterpret_cast<const __half2 *>(&p0), bias);
    const __half2 c1 = __hsub2(*reinterpret_cast<const __half2 *>(&p1), bias);
    lo = *reinterpret_cast<const uint32_t *>(&c0);
    hi = *reinterpret_cast<const uint32_t *>(&c1);
}

__global__ void __launch_bounds__(NTHREADS, 1) attn_prefill_kernel(const __grid_constant__ PParams p, const __grid_constant__ PMaps tm) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sm_u32 = smem_u32(sm);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(sm + OFF_MISC);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + OFF_MISC + 4);
    float *xch = reinterpret_cast<float *>(sm + OFF_XCH);              // [3][TPR][128]
    const uint32_t bar0 = sm_u32 + OFF_BAR;
    auto bar_raw_full = [&](int s) { return bar0 + 8 * s; };            // TMA -> dequant and MMA (tx bytes)
    auto bar_raw_empty = [&](int s) { return bar0 + 8 * (2 + s); };     // dequant warps (V converted) + commit after QK (1) + softmax warps (scales used) -> TMA
    const uint32_t bar_v16_full = bar0 + 8 * 4;                         // dequant warps -> MMA
    const uint32_t bar_v16_empty = bar0 + 8 * 5;                        // commit after PV -> dequant
    const uint32_t bar_s_full = bar0 + 8 * 6;                           // commit after QK -> softmax
    const uint32_t bar_s_empty = bar0 + 8 * 7;                          // softmax warps: S is in registers -> MMA
    const uint32_t bar_p_full = bar0 + 8 * 8;                           // softmax warps -> MMA
    const uint32_t bar_o_done = bar0 + 8 * 9;                           // commit after PV -> softmax
    const uint32_t bar_q_ready = bar0 + 8 * 10;                         // softmax warps -> MMA
    const uint32_t bar_xch = bar0 + 8 * 11;                             // softmax warps: the threads of every row have written their exchange slots

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy blocks (late query positions: the most key tiles) are scheduled first
    const int qb = p.q_blocks - 1 - blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int s_first = qb * p.pos_per_cta;
    const int s_last = min(p.S, s_first + p.pos_per_cta) - 1;

    // key range of the block: from the first row's lower bound to the last row's upper bound
    const int hi_blk = min(p.d0 + s_last, p.key_len - 1);
    const int lo_blk = p.window > 0 ? max(0, p.d0 + s_first - p.window + 1) : 0;
    const int tile_lo = lo_blk / KT;
    const int n_tiles = hi_blk >= lo_blk ? hi_blk / KT - tile_lo + 1 : 0;
    const int map_row0 = kvh * p.cache_cap + p.row0;                   // row of key index 0 in the tensor maps

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        fused::mbar_init(bar_raw_full(0), 1); fused::mbar_init(bar_raw_full(1), 1);
        fused::mbar_init(bar_raw_empty(0), NSOFT / 32 + 3); fused::mbar_init(bar_raw_empty(1), NSOFT / 32 + 3);
        fused::mbar_init(bar_v16_full, 2); fused::mbar_init(bar_v16_empty, 1);
        fused::mbar_init(bar_s_full, 1); fused::mbar_init(bar_s_empty, NSOFT / 32);
        fused::mbar_init(bar_p_full, NSOFT / 32); fused::mbar_init(bar_o_done, 1);
        fused::mbar_init(bar_q_ready, NSOFT / 32);
        fused::mbar_init(bar_xch, NSOFT / 32);
        fused::fence_mbar_init();
    }
    // the scale stages start as zeros: a partial copy at the end of the key array then leaves finite values behind
    for (int e = threadIdx.x; e < 2 * 2 * KT; e += NTHREADS) reinterpret_cast<float *>(sm + OFF_SC)[e] = 0.0f;
    fused::fence_proxy_async();
    if (warp == W_MMA && lane == 0) { fused::prefetch_tensormap(&tm.k); fused::prefetch_tensormap(&tm.v); }
    if (warp == W_TMA) {
        tc5::tmem_alloc(sm_u32 + OFF_MISC, TMEM_COLS);
        tc5::tmem_relinquish();
    }
    tc5::tc_fence_before();
    __syncthreads();
    tc5::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    fused::pdl_wait();                         // the query and the cache rows may come from the stream predecessor
    fused::pdl_launch_dependents();

    if (warp == W_TMA) {
        // =========================================================== TMA producer
        if (lane == 0) {
            for (int i = 0; i < n_tiles; ++i) {
                const int st = i & 1;
                if (i >= 2 && !wait_or_abort(bar_raw_empty(st), ((i >> 1) - 1) & 1, abort_flag, p.fault)) break;
                const uint32_t dst = sm_u32 + OFF_RAW + st * 2 * RAW_TILE;
                const int row = map_row0 + (tile_lo + i) * KT;
                // the tile's fp32 row scales ride along as two bulk copies (whole 16-byte units inside the key array)
                const int t0 = (tile_lo + i) * KT;
                const uint32_t sc_bytes = p.scales_vec ? (uint32_t)(min(KT, p.key_len - t0) & ~3) * 4u : 0u;
                fused::mbar_expect_tx(bar_raw_full(st), 2 * RAW_TILE + 2 * sc_bytes);
                fused::tma_load_tile(dst, &tm.k, row, b, bar_raw_full(st));
                fused::tma_load_tile(dst + RAW_TILE, &tm.v, row, b, bar_raw_full(st));
                if (sc_bytes) {
                    const size_t so = b * (p.scale_batch_stride / 4) + (size_t)kvh * p.cache_cap + p.row0 + t0;
                    fused::bulk_load(sm_u32 + OFF_SC + st * 2 * KT * 4, p.k_scales + so, sc_bytes, bar_raw_full(st));
                    fused::bulk_load(sm_u32 + OFF_SC + st * 2 * KT * 4 + KT * 4, p.v_scales + so, sc_bytes, bar_raw_full(st));
                }
            }
        }
        __syncwarp();
    } else if (warp == W_MMA) {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = tc5::make_idesc(KT, true, true, false);
            const uint32_t idesc_pv = make_idesc_f16(HD, true);
            const uint64_t qdesc[2] = {tc5::smem_desc_sw128(sm_u32 + OFF_Q8), tc5::smem_desc_sw128(sm_u32 + OFF_Q8 + RAW_TILE)};
            const uint64_t pdesc[2] = {tc5::smem_desc_sw128(sm_u32 + OFF_P16), tc5::smem_desc_sw128(sm_u32 + OFF_P16 + H_TILE)};
            // B of PV, MN-major: the two 64-dim blocks of V16 are one operand, the second H_BLOCK bytes after the first
            // (leading-dimension offset); key groups of 8 rows stay 1024 bytes apart
            const uint64_t vdesc = (tc5::smem_desc_sw128(sm_u32 + OFF_V16) & ~(0x3fffull << 16)) | ((uint64_t)(H_BLOCK >> 4) << 16);
            bool go = n_tiles > 0 && wait_or_abort(bar_q_ready, 0, abort_flag, p.fault);
            for (int i = 0; go && i <= n_tiles; ++i) {
                if (i < n_tiles) {
                    // S_hi / S_lo = Qlimb x K_i^T straight off the bytes TMA wrote: per limb 4 steps of 32 dims (32 bytes)
                    const int st = i & 1;
                    if (!wait_or_abort(bar_raw_full(st), (i >> 1) & 1, abort_flag, p.fault)) break;
                    if (i >= 1 && !wait_or_abort(bar_s_empty, (i - 1) & 1, abort_flag, p.fault)) break;
                    tc5::tc_fence_after();
                    const uint64_t kdesc = tc5::smem_desc_sw128(sm_u32 + OFF_RAW + st * 2 * RAW_TILE);
#pragma unroll
                    for (int limb = 0; limb < 2; ++limb)
#pragma unroll
                        for (int k = 0; k < HD / 32; ++k)
                            tc5::umma_i8(tmem_base + 128 * limb, qdesc[limb] + 2 * k, kdesc + 2 * k, idesc_qk, k > 0);
                    tc5::umma_commit(bar_s_full);
                    tc5::umma_commit(bar_raw_empty(st));
                }
                if (i >= 1) {
                    // O += Phi_j x V_j + Plo_j x V_j: per weight limb 8 steps of 16 keys against all 128 dims (an instruction
                    // costs the issuing thread about a hundred cycles whatever its size: few and large)
                    // (A: 32 bytes inside a 64-key block, then the next block; B: 16 rows of the MN-major V blocks = 2048 bytes)
                    const int j = i - 1;
                    if (!wait_or_abort(bar_v16_full, j & 1, abort_flag, p.fault)) break;
                    if (!wait_or_abort(bar_p_full, j & 1, abort_flag, p.fault)) break;
                    tc5::tc_fence_after();
#pragma unroll
                    for (int limb = 0; limb < 2; ++limb)
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const uint64_t a_adv = (uint64_t)((k >> 2) * (H_BLOCK >> 4) + (k & 3) * 2);
                            const uint64_t b_adv = (uint64_t)(k * (2048 >> 4));
                            umma_f16(tmem_base + 256, pdesc[limb] + a_adv, vdesc + b_adv, idesc_pv, (j > 0 || limb > 0 || k > 0) ? 1u : 0u);
                        }
                    tc5::umma_commit(bar_v16_empty);
                    tc5::umma_commit(bar_o_done);
                }
            }
        }
        __syncwarp();
    } else if (warp >= W_DEQ) {
        // =========================================================== dequant warps: a thread converts key rows t, t + 64 of the V tile
        const int t = threadIdx.x - NSOFT;
        for (int i = 0; i < n_tiles; ++i) {
            const int st = i & 1;
            const uint8_t *raw = sm + OFF_RAW + st * 2 * RAW_TILE + RAW_TILE;
            if (!__all_sync(0xffffffffu, wait_or_abort(bar_raw_full(st), (i >> 1) & 1, abort_flag, p.fault))) break;
            if (i >= 1 && !__all_sync(0xffffffffu, wait_or_abort(bar_v16_empty, (i - 1) & 1, abort_flag, p.fault))) break;
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int r = t + 64 * rr;
#pragma unroll
                for (int c = 0; c < 8; ++c) {                          // 16 codes per step -> two 16-byte chunks of fp16
                    const uint4 x = *reinterpret_cast<const uint4 *>(raw + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
                    uint4 y0, y1;
                    cvt4(x.x, y0.x, y0.y); cvt4(x.y, y0.z, y0.w);
                    cvt4(x.z, y1.x, y1.y); cvt4(x.w, y1.z, y1.w);
                    *reinterpret_cast<uint4 *>(sm + OFF_V16 + h_off(r, 2 * c)) = y0;
                    *reinterpret_cast<uint4 *>(sm + OFF_V16 + h_off(r, 2 * c + 1)) = y1;
                }
            }
            fused::fence_proxy_async();
            __syncwarp();
            if (lane == 0) { tc5::mbar_arrive(bar_v16_full); tc5::mbar_arrive(bar_raw_empty(st)); }
        }
    } else {
        // =========================================================== softmax warps: four threads per query row
        const int qt = warp >> 2;                                      // which 32 keys of a tile (and which 32 dims of Q / O) this thread takes
        const int r = 32 * (warp & 3) + lane;                          // query row = TMEM lane
        const int s = s_first + r / p.kvg, j = r - (r / p.kvg) * p.kvg;
        const bool valid = r < p.pos_per_cta * p.kvg && s < p.S;
        const int hi_r = valid ? min(p.d0 + s, p.key_len - 1) : -1;                     // inclusive
        const int lo_r = (valid && p.window > 0) ? max(0, p.d0 + s - p.window + 1) : 0;
        const uint32_t tmem_lane = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16);
        auto wait_warp = [&](uint32_t bar, uint32_t parity) {
            return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag, p.fault)) != 0;
        };
        // Meeting point of the softmax threads: an mbarrier with the same time limit as every other wait (a
        // hardware barrier would wait forever for a warp that had given up).  false = abandoned.
        // One arrival per warp: the warp's stores and fences are ordered before it by the warp barrier.
        auto warp_arrive = [&](uint32_t bar) {
            __syncwarp();
            if (lane == 0) tc5::mbar_arrive(bar);
        };
        uint32_t xphase = 0;
        auto pair_sync = [&]() {
            warp_arrive(bar_xch);
            const bool ok = wait_warp(bar_xch, xphase);
            xphase ^= 1u;
            return ok;
        };
        // ---- the query row -> 16-bit fixed point of its own maximum, two int8 limbs (q ~= sq * (256 hi + lo)),
        // stored K-major in the 128-byte swizzle pattern; this thread converts dims 32 qt .. 32 qt + 31
        float qscale_r;                          // base-2 logit per unit of the integer dot product and of the key's scale
        {
            const long qoff = b * p.q_batch_stride + ((long)(valid ? s : 0) * p.nh + kvh * p.kvg + (valid ? j : 0)) * HD + KPT * qt;
            float x[KPT];
#pragma unroll
            for (int c = 0; c < KPT / 8; ++c) {
                if (p.q_type == ET_BF16) {
                    const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(p.q) + qoff) + c);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) { x[8 * c + 2 * e] = __uint_as_float(w[e] << 16); x[8 * c + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
                } else {
                    const float4 v0 = __ldcg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.q) + qoff) + 2 * c);
                    const float4 v1 = __ldcg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.q) + qoff) + 2 * c + 1);
                    x[8 * c] = v0.x; x[8 * c + 1] = v0.y; x[8 * c + 2] = v0.z; x[8 * c + 3] = v0.w;
                    x[8 * c + 4] = v1.x; x[8 * c + 5] = v1.y; x[8 * c + 6] = v1.z; x[8 * c + 7] = v1.w;
                }
            }
            float amax = 0.0f;
#pragma unroll
            for (int d = 0; d < KPT; ++d) amax = fmaxf(amax, fabsf(x[d]));
            xch[(2 * TPR + qt) * 128 + r] = amax;
            pair_sync();
#pragma unroll
            for (int o = 1; o < TPR; ++o) amax = fmaxf(amax, xch[(2 * TPR + ((qt + o) & (TPR - 1))) * 128 + r]);
            const float sq = (valid && amax > 0.0f) ? amax * (1.0f / (float)Q_FIX_MAX) : 1.0f;
            const float inv = 1.0f / sq;
            qscale_r = valid ? sq * p.q_scale : 0.0f;
#pragma unroll
            for (int c = 0; c < KPT / 16; ++c) {                       // 16 dims per 16-byte chunk
                uint32_t wh[4], wl[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    uint32_t ph = 0, pl = 0;
#pragma unroll
                    for (int bb = 0; bb < 4; ++bb) {
                        int qf = valid ? __float2int_rn(x[16 * c + 4 * e + bb] * inv) : 0;
                        qf = max(-Q_FIX_MAX, min(Q_FIX_MAX, qf));
                        const int hi = (qf + 128) >> 8, lo = qf - (hi << 8);
                        ph |= (uint32_t)(hi & 0xff) << (8 * bb);
                        pl |= (uint32_t)(lo & 0xff) << (8 * bb);
                    }
                    wh[e] = ph; wl[e] = pl;
                }
                const int off = (r >> 3) * 1024 + (r & 7) * 128 + ((((KPT / 16) * qt + c) ^ (r & 7)) << 4);
                *reinterpret_cast<uint4 *>(sm + OFF_Q8 + off) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                *reinterpret_cast<uint4 *>(sm + OFF_Q8 + RAW_TILE + off) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            }
            fused::fence_proxy_async();
            warp_arrive(bar_q_ready);
        }
        // fp32 row scales of the keys, read per tile by every thread (the same 1 KB for the whole CTA: L1 hits)
        const float *gks = p.k_scales + b * (p.scale_batch_stride / 4) + (size_t)kvh * p.cache_cap + p.row0;
        const float *gvs = p.v_scales + b * (p.scale_batch_stride / 4) + (size_t)kvh * p.cache_cap + p.row0;
        float m = M_INIT, l = 0.0f;              // running maximum of the row (its threads agree), this thread's share of the denominator
        bool alive = true;
        for (int i = 0; alive && i < n_tiles; ++i) {
            const int t0 = (tile_lo + i) * KT + KPT * qt;              // first key of this thread's share of the tile
            // rows outside [lo_r, hi_r] see nothing of the key (a select, never a multiply); decided per warp, so that
            // whole tiles in the middle of every row's range carry no masking instructions at all
            const bool need_mask = __any_sync(0xffffffffu, t0 < lo_r || t0 + KPT - 1 > hi_r);
            const int st = i & 1;
            // scales of this thread's keys: in shared memory when they could ride the bulk copies (the copy covers whole
            // 16-byte units inside the key array: a ragged tail is read from global memory), else from global memory
            const bool whole = p.scales_vec && (((tile_lo + i) * KT + (min(KT, p.key_len - (tile_lo + i) * KT) & ~3)) >= t0 + KPT);
            const float *sks = reinterpret_cast<const float *>(sm + OFF_SC + st * 2 * KT * 4) + KPT * qt - t0;      // used when `whole`
            const float *svs = reinterpret_cast<const float *>(sm + OFF_SC + st * 2 * KT * 4 + KT * 4) + KPT * qt - t0;
            const int tl = p.key_len - 1;
            if (!wait_warp(bar_raw_full(st), (i >> 1) & 1)) { alive = false; break; }   // the scales have landed
            if (!wait_warp(bar_s_full, i & 1)) { alive = false; break; }
            tc5::tc_fence_after();
            float sv[KPT];                                             // base-2 logits of this row against its 32 keys
            float tmax = -CUDART_INF_F;
#pragma unroll
            for (int c = 0; c < KPT / 16; ++c) {                       // 16 columns of each limb at a time: registers
                int sh[16], sl[16];
                tmem_ld16i(tmem_lane + KPT * qt + 16 * c, sh);
                tmem_ld16i(tmem_lane + 128 + KPT * qt + 16 * c, sl);
                tc5::tmem_wait_ld();
#pragma unroll
                for (int e4 = 0; e4 < 16; e4 += 4) {
                    float4 k4;
                    if (whole) {
                        k4 = *reinterpret_cast<const float4 *>(sks + t0 + 16 * c + e4);
                    } else {
                        k4 = make_float4(gks[min(t0 + 16 * c + e4, tl)], gks[min(t0 + 16 * c + e4 + 1, tl)], gks[min(t0 + 16 * c + e4 + 2, tl)],
                                         gks[min(t0 + 16 * c + e4 + 3, tl)]);
                    }
                    const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // limb sums are below 128 * 128 * 127 < 2^22: 256 hi + lo fits an int, one rounding in the conversion
                        float u = (float)(sh[e4 + e] * 256 + sl[e4 + e]) * (qscale_r * kk[e]);
                        if (need_mask) {
                            const int t = t0 + 16 * c + e4 + e;
                            u = (t >= lo_r && t <= hi_r) ? u : -CUDART_INF_F;
                        }
                        sv[16 * c + e4 + e] = u;
                        tmax = fmaxf(tmax, u);
                    }
                }
            }
            tc5::tc_fence_before();
            warp_arrive(bar_s_empty);                                  // S is in registers: QK of the next tile may overwrite it
            // the row's tile maximum: its threads meet through shared memory (double-buffered by tile parity)
            xch[((i & 1) * TPR + qt) * 128 + r] = tmax;
            if (!pair_sync()) { alive = false; break; }
#pragma unroll
            for (int o = 1; o < TPR; ++o) tmax = fmaxf(tmax, xch[((i & 1) * TPR + ((qt + o) & (TPR - 1))) * 128 + r]);
            // the running maximum only moves when the tile exceeds it by more than 2^8: the weights stay below 2^8 and
            // the accumulator in tensor memory is rescaled a handful of times per row instead of once per tile
            const bool moved = tmax > m + LAZY;
            const float m_new = moved ? tmax : m;
            const float alpha = moved ? ex2f(m - m_new) : 1.0f;
            m = m_new;
            // P is single-buffered and O lives in tensor memory: both wait for the previous tile's PV product
            if (i >= 1 && !wait_warp(bar_o_done, (i - 1) & 1)) { alive = false; break; }
            if (i >= 1 && __any_sync(0xffffffffu, moved)) {            // this thread rescales its 32 dims of O
                tc5::tc_fence_after();
                float o[32];
                tmem_ld32(tmem_lane + 256 + KPT * qt, o);
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] *= alpha;
                tmem_st32(tmem_lane + 256 + KPT * qt, o);
                tmem_wait_st();
            }
            // weights of this thread's 32 keys = chunks 4 qt .. 4 qt + 3 of the P tiles: weight x value scale as fp16 hi + lo
            float lsum0 = 0.0f, lsum1 = 0.0f;
#pragma unroll
            for (int e8 = 0; e8 < KPT; e8 += 8) {
                float vv[8];
                if (whole) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(svs + t0 + e8);
                    const float4 b4 = *reinterpret_cast<const float4 *>(svs + t0 + e8 + 4);
                    vv[0] = a4.x; vv[1] = a4.y; vv[2] = a4.z; vv[3] = a4.w; vv[4] = b4.x; vv[5] = b4.y; vv[6] = b4.z; vv[7] = b4.w;
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) vv[e] = gvs[min(t0 + e8 + e, tl)];
                }
                uint32_t wh[4], wl[4];
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float p0 = ex2f(sv[e8 + e] - m), p1 = ex2f(sv[e8 + e + 1] - m);
                    lsum0 += p0; lsum1 += p1;
                    const float w0 = p0 * vv[e], w1 = p1 * vv[e + 1];
                    const __half2 h = __floats2half2_rn(w0, w1);
                    const __half2 hl = __floats2half2_rn(w0 - __low2float(h), w1 - __high2float(h));
                    wh[e >> 1] = *reinterpret_cast<const uint32_t *>(&h);
                    wl[e >> 1] = *reinterpret_cast<const uint32_t *>(&hl);
                }
                const int chunk = (KPT / 8) * qt + (e8 >> 3);          // 16-byte chunk (8 keys) of the row
                *reinterpret_cast<uint4 *>(sm + OFF_P16 + h_off(r, chunk)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                *reinterpret_cast<uint4 *>(sm + OFF_P16 + H_TILE + h_off(r, chunk)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            }
            l = fmaf(l, alpha, lsum0 + lsum1);
            fused::fence_proxy_async();
            tc5::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                tc5::mbar_arrive(bar_raw_empty(st));                   // done with the stage's scales
                tc5::mbar_arrive(bar_p_full);
            }
        }
        // ---- output: O / l (rows without any key are exact zeros, lib/batched_attn_gpu.mojo:329-409); this thread
        // writes dims 32 qt .. 32 qt + 31 of its row
        if (alive && n_tiles > 0) alive = wait_warp(bar_o_done, (n_tiles - 1) & 1);
        if (alive) {
            xch[(2 * TPR + qt) * 128 + r] = l;
            alive = pair_sync();
#pragma unroll
            for (int o = 1; o < TPR; ++o) l += xch[(2 * TPR + ((qt + o) & (TPR - 1))) * 128 + r];
        }
        if (alive) {
            tc5::tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const long oi = b * p.out_batch_stride + ((long)(valid ? s : 0) * p.nh + kvh * p.kvg + (valid ? j : 0)) * HD + KPT * qt;
            float o[32];
            if (n_tiles > 0) {
                tmem_ld32(tmem_lane + 256 + KPT * qt, o);
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = 0.0f;
            }
            if (valid) {
                if (p.out_type == ET_BF16) {
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.out) + oi);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(o[8 * q4 + 2 * e] * inv, o[8 * q4 + 2 * e + 1] * inv);
                            w[e] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        dst[q4] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
                    float4 *dst = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + oi);
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        dst[q4] = make_float4(o[4 * q4] * inv, o[4 * q4 + 1] * inv, o[4 * q4 + 2] * inv, o[4 * q4 + 3] * inv);
                }
            }
        }
    }

    // ------------------------------------------------------------ tear-down
    tc5::tc_fence_before();
    __syncthreads();
    if (warp == W_TMA) tc5::tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace pf
}  // namespace nomos
