// Split-K flash-decoding attention over the PACKED quantised KV ring (sm_100a).
//
// Replaces, in one launch (+ a tiny merge when the sequence is split), what the
// reference does per layer with 5-7 launches: window reader -> int8/bf16 scratch
// (lib/kv_cache_quant.mojo:221-249,708-800,925-953), QK (lib/attention_gpu_int8.mojo:48-91
// or cuBLAS, lib/attention_gpu.mojo:231-238), row softmax (lib/softmax_gpu_mojo.mojo:37-134)
// and PV (lib/attention_gpu_int8.mojo:94-137 / lib/attention_gpu.mojo:241-248), and for
// S>1 the multirow verify kernels (lib/attention_gpu_int8.mojo:322-584).
//
// Work decomposition
//   grid = (splits, nkv, batch * row_groups); one CTA streams one KV head's chunk of
//   the window and serves every query row of the GQA group from the same bytes.
//   Each warp owns a private 3-stage cp.async ring of 32-token tiles (16-byte
//   coalesced global->shared copies, no CTA barrier in the main loop).
// Arithmetic (per warp tile)
//   QK:  int8 tensor-core MMA m16n8k32.  A = the query rows as two int8 limbs of a
//        15-bit fixed point (rows g / g+8 of the M tile = high / low limb of slot g),
//        B = the K bytes exactly as stored (ldmatrix from the swizzled tile).  The
//        int32 result is exact; one fp32 multiply per (token, slot) applies
//        q_scale * k_scale.  int4 caches feed the same MMA as biased unsigned
//        nibbles with an exact integer correction.
//   softmax: online, base-2, in the C-fragment registers; row max over the tile by
//        two xor-shuffles.
//   PV:  fp16 tensor-core MMA m16n8k16 with fp32 accumulators.  A = p * v_scale in
//        fp16 (the C fragment of QK is already in A-fragment order), B = V bytes
//        transposed by ldmatrix.trans and widened to fp16 exactly (magic-number
//        byte->half expansion, no integer->float conversion instructions).
// The un-normalised (m, l, o) of every warp are merged in shared memory, then
// across splits by merge_kernel (or exported for the multi-GPU all-gather).
#include <math_constants.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "launch.h"

namespace nomos {

namespace {

constexpr int TILE = 32;        // tokens per warp tile
constexpr int NSTAGE = 3;       // cp.async stages per warp
constexpr int NWARP = 2;        // warps per CTA
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float P_OFFSET = 14.0f;      // p * v_scale is kept <= 2^14 so fp16 never underflows usefully
constexpr float M_INIT = -1.0e30f;     // finite "minus infinity" for the running max
constexpr int Q_FIX_MAX = 16256;       // 127 * 128: two int8 limbs, hi in [-127,127], lo in [-64,63]

template <int FMT, int HD, int MT>
struct Cfg {
    static constexpr int ROWB = (FMT == KV_I8) ? HD : HD / 2;                 // cache bytes per token row
    static constexpr int CHUNKS = ROWB / 16;                                  // 16-byte chunks per row
    static constexpr int NBLK = HD / 32;
    static constexpr int SCB = (FMT == KV_I4B32) ? NBLK * 2 : 4;              // scale bytes per token
    static constexpr int KV_BYTES = TILE * ROWB;
    static constexpr int SC_BYTES = TILE * SCB;
    static constexpr int STAGE_BYTES = 2 * KV_BYTES + 2 * SC_BYTES;
    static constexpr int NSLOT = 8 * MT;                                      // query rows (row x group head) per CTA
    static constexpr int MTP = (MT + 1) / 2;                                  // PV M tiles
    static constexpr int NT = HD / 8;                                         // PV N tiles
    static constexpr int Q_BYTES = 2 * NSLOT * HD;                            // two limbs
    static constexpr int SLOT_BYTES = NSLOT * 16;                             // qscale, lo, hi, pad
    static constexpr int PIPE_BYTES = NWARP * NSTAGE * STAGE_BYTES;
    static constexpr int MERGE_BYTES = NWARP * NSLOT * (HD + 2) * 4;
    static constexpr int SMEM_BYTES = Q_BYTES + SLOT_BYTES + (PIPE_BYTES > MERGE_BYTES ? PIPE_BYTES : MERGE_BYTES);
};

struct KParams {
    const uint8_t *q;
    const uint8_t *k_cache, *v_cache, *k_scales, *v_scales;
    uint8_t *out;
    float *partial;          // workspace partials or exported partials: [split][grow][HD+2]
    int write_partial;       // 1: write (o, M, l) to partial; 0: write normalised out
    int export_nat;          // 1: partial m is exported in natural-log units with the offset removed
    int q_type, out_type;
    int S, nh, nkv, kvg, cache_hd, cache_cap, win_start, klen, window;
    int tile0, ntiles, tiles_per_split, row_groups, grows;
    float qk_scale_log2;     // softmax_scale * log2(e)
    long q_batch_stride, kv_batch_stride, scale_batch_stride, out_batch_stride;
};

__device__ __forceinline__ float load_q(const uint8_t *q, int q_type, long idx) {
    return q_type == ET_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(q)[idx])
                             : reinterpret_cast<const float *>(q)[idx];
}

// fp16 m16n8k16 MMA that only produces rows 0-7 (a1 = a3 = 0): used when the PV M
// tile has a single QK M tile behind it, so rows 8-15 cost no registers.
__device__ __forceinline__ void mma_f16_top(float &d0, float &d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float x2, x3;
    const uint32_t z = 0u;
    const float zf = 0.0f;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};\n"
                 : "+f"(d0), "+f"(d1), "=f"(x2), "=f"(x3)
                 : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1), "f"(zf));
}

template <int FMT, int HD, int MT>
__global__ void __launch_bounds__(NWARP * 32) attn_fused_kernel(const KParams p) {
    using C = Cfg<FMT, HD, MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    int8_t *q_limbs = reinterpret_cast<int8_t *>(smem);                        // [2][NSLOT][HD]
    float *slot_qscale = reinterpret_cast<float *>(smem + C::Q_BYTES);         // [NSLOT]
    int *slot_lo = reinterpret_cast<int *>(smem + C::Q_BYTES + C::NSLOT * 4);
    int *slot_hi = reinterpret_cast<int *>(smem + C::Q_BYTES + C::NSLOT * 8);
    uint8_t *pipe = smem + C::Q_BYTES + C::SLOT_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int b = blockIdx.z / p.row_groups, rg = blockIdx.z % p.row_groups;

    // ------------------------------------------------------------ Q prologue
    // Slot sl of this CTA = local row index rg*NSLOT + sl = (query row r, group head j).
    for (int sl = warp; sl < C::NSLOT; sl += NWARP) {
        const int idx = rg * C::NSLOT + sl;
        const int r = idx / p.kvg, j = idx % p.kvg;
        const bool valid = r < p.S;
        float x[HD / 32];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < HD / 32; ++i) {
            x[i] = valid ? load_q(p.q, p.q_type, b * p.q_batch_stride + ((long)r * p.nh + kvh * p.kvg + j) * HD + lane + 32 * i) : 0.0f;
            amax = fmaxf(amax, fabsf(x[i]));
        }
        amax = warp_max(amax);
        const float sq = amax > 0.0f ? amax / (float)Q_FIX_MAX : 1.0f;
        const float inv = 1.0f / sq;
#pragma unroll
        for (int i = 0; i < HD / 32; ++i) {
            int qf = __float2int_rn(x[i] * inv);
            qf = max(-Q_FIX_MAX, min(Q_FIX_MAX, qf));
            const int hi = (qf + 64) >> 7;
            const int lo = qf - (hi << 7);
            const int d = lane + 32 * i;
            int pos = d;
            if constexpr (FMT != KV_I8) {
                // int4 tiles deliver element 32b+8t+2j+par in MMA k slot par*16+4t+j.
                const int blk = d >> 5, w = d & 31;
                pos = (blk << 5) + ((w & 1) << 4) + ((w >> 3) << 2) + ((w >> 1) & 3);
            }
            q_limbs[sl * HD + pos] = (int8_t)hi;
            q_limbs[(C::NSLOT + sl) * HD + pos] = (int8_t)lo;
        }
        if (lane == 0) {
            const int hi_b = valid ? p.klen - (p.S - 1 - r) : 0;
            slot_qscale[sl] = valid ? sq * p.qk_scale_log2 : 0.0f;
            slot_hi[sl] = hi_b;
            slot_lo[sl] = (valid && p.window > 0) ? max(0, hi_b - p.window) : 0;
        }
    }
    __syncthreads();

    // per-thread slot constants: slot (mt, g)
    float qscale[MT];
    int lo_b[MT], hi_b[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        qscale[mt] = slot_qscale[mt * 8 + g];
        lo_b[mt] = slot_lo[mt * 8 + g];
        hi_b[mt] = slot_hi[mt * 8 + g];
    }
    // Q A-fragments: kept in registers for a single M tile, re-read from shared otherwise.
    constexpr bool Q_IN_REGS = (MT == 1) && (HD <= 256);
    uint32_t qa[Q_IN_REGS ? HD / 32 : 1][4];
    auto load_qa = [&](uint32_t(&a)[4], int mt, int ks) {
        const int8_t *hi_row = q_limbs + (mt * 8 + g) * HD + ks * 32 + 4 * t;
        const int8_t *lo_row = hi_row + C::NSLOT * HD;
        a[0] = *reinterpret_cast<const uint32_t *>(hi_row);
        a[1] = *reinterpret_cast<const uint32_t *>(lo_row);
        a[2] = *reinterpret_cast<const uint32_t *>(hi_row + 16);
        a[3] = *reinterpret_cast<const uint32_t *>(lo_row + 16);
    };
    if constexpr (Q_IN_REGS) {
#pragma unroll
        for (int ks = 0; ks < HD / 32; ++ks) load_qa(qa[ks], 0, ks);
    }

    // ------------------------------------------------------------ tile schedule
    const int tile_begin = p.tile0 + split * p.tiles_per_split;
    const int tile_end = min(p.tile0 + p.ntiles, tile_begin + p.tiles_per_split);
    const int my_first = tile_begin + warp;
    const int my_count = my_first < tile_end ? (tile_end - my_first + NWARP - 1) / NWARP : 0;

    const uint8_t *kbase = p.k_cache + b * p.kv_batch_stride + (size_t)kvh * p.cache_cap * (size_t)(FMT == KV_I8 ? p.cache_hd : p.cache_hd / 2);
    const uint8_t *vbase = p.v_cache + b * p.kv_batch_stride + (size_t)kvh * p.cache_cap * (size_t)(FMT == KV_I8 ? p.cache_hd : p.cache_hd / 2);
    const uint8_t *ksbase = p.k_scales + b * p.scale_batch_stride + (size_t)kvh * p.cache_cap * C::SCB;
    const uint8_t *vsbase = p.v_scales + b * p.scale_batch_stride + (size_t)kvh * p.cache_cap * C::SCB;
    const int row_stride = (FMT == KV_I8) ? p.cache_hd : p.cache_hd / 2;

    uint8_t *my_pipe = pipe + warp * NSTAGE * C::STAGE_BYTES;
    const uint32_t my_pipe_u32 = smem_u32(my_pipe);
    const int ring0 = p.win_start % p.cache_cap;

    auto issue = [&](int it) {
        if (it < my_count) {
            const int tok0 = (my_first + it * NWARP) * TILE;
            const uint32_t st = my_pipe_u32 + (it % NSTAGE) * C::STAGE_BYTES;
            // K and V rows: lane copies chunk (lane % CHUNKS) of rows (lane / CHUNKS) + i * (32 / CHUNKS)
            constexpr int ROWS_PER_PASS = 32 / (C::CHUNKS > 32 ? 32 : C::CHUNKS);
            constexpr int CH_PASSES = C::CHUNKS > 32 ? C::CHUNKS / 32 : 1;
#pragma unroll
            for (int i = 0; i < TILE / ROWS_PER_PASS; ++i) {
                const int row = (C::CHUNKS >= 32 ? 0 : lane / C::CHUNKS) + i * ROWS_PER_PASS;
                const int tok = tok0 + row;
                int slot = ring0 + tok;
                slot = slot >= p.cache_cap ? slot - p.cache_cap : slot;       // klen <= cache_cap (checked on the host)
                const int nbytes = tok < p.klen ? 16 : 0;
                const size_t goff = (size_t)(tok < p.klen ? slot : 0) * row_stride;
#pragma unroll
                for (int cp = 0; cp < CH_PASSES; ++cp) {
                    const int c = (C::CHUNKS >= 32 ? lane : lane % C::CHUNKS) + cp * 32;
                    const uint32_t soff = row * C::ROWB + swz_chunk<C::ROWB>(row, c) * 16;
                    cp_async16(st + soff, kbase + goff + c * 16, nbytes);
                    cp_async16(st + C::KV_BYTES + soff, vbase + goff + c * 16, nbytes);
                }
            }
            {   // scales: lane <-> token
                const int tok = tok0 + lane;
                int slot = ring0 + tok;
                slot = slot >= p.cache_cap ? slot - p.cache_cap : slot;
                const bool ok = tok < p.klen;
                const size_t goff = (size_t)(ok ? slot : 0) * C::SCB;
                const uint32_t sk = st + 2 * C::KV_BYTES + lane * C::SCB;
                const uint32_t sv = sk + C::SC_BYTES;
                if constexpr (C::SCB == 4) {
                    cp_async4(sk, ksbase + goff, ok ? 4 : 0);
                    cp_async4(sv, vsbase + goff, ok ? 4 : 0);
                } else if constexpr (C::SCB == 8) {
                    cp_async8(sk, ksbase + goff, ok ? 8 : 0);
                    cp_async8(sv, vsbase + goff, ok ? 8 : 0);
                } else {
#pragma unroll
                    for (int o = 0; o < C::SCB; o += 16) {
                        cp_async16(sk + o, ksbase + goff + o, ok ? 16 : 0);
                        cp_async16(sv + o, vsbase + goff + o, ok ? 16 : 0);
                    }
                }
            }
        }
        cp_async_commit();
    };

    // ------------------------------------------------------------ running state
    float M[MT], l[MT];
    float acc[C::MTP][C::NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) { M[mt] = M_INIT; l[mt] = 0.0f; }
#pragma unroll
    for (int pm = 0; pm < C::MTP; ++pm)
#pragma unroll
        for (int nt = 0; nt < C::NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[pm][nt][i] = 0.0f;

    int lo_max = 0, hi_min = 0x7fffffff;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        if (hi_b[mt] > 0) { lo_max = max(lo_max, lo_b[mt]); hi_min = min(hi_min, hi_b[mt]); }
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        lo_max = max(lo_max, __shfl_xor_sync(0xffffffffu, lo_max, o));
        hi_min = min(hi_min, __shfl_xor_sync(0xffffffffu, hi_min, o));
    }

#pragma unroll
    for (int s = 0; s < NSTAGE - 1; ++s) issue(s);

    for (int it = 0; it < my_count; ++it) {
        issue(it + NSTAGE - 1);
        cp_async_wait<NSTAGE - 1>();
        __syncwarp();

        const int tok0 = (my_first + it * NWARP) * TILE;
        const uint32_t st = my_pipe_u32 + (it % NSTAGE) * C::STAGE_BYTES;
        const uint8_t *stp = my_pipe + (it % NSTAGE) * C::STAGE_BYTES;
        const bool need_mask = (tok0 + TILE > hi_min) || (tok0 < lo_max);

        // --------------------------------------------------------------- QK
        float s2[MT][4][2];
        float vs[4][2];           // V scale of my 8 tokens (row-scale formats)
        if constexpr (FMT == KV_I8) {
            int c[MT][4][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int n = 0; n < 4; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) c[mt][n][i] = 0;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
#pragma unroll
                for (int half = 0; half < HD / 64; ++half) {
                    uint32_t kb[4];
                    const int row = 8 * n + (lane & 7);
                    const int ch = 4 * half + (lane >> 3);
                    ldmatrix_x4(kb, st + row * C::ROWB + swz_chunk<C::ROWB>(row, ch) * 16);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        if constexpr (Q_IN_REGS) {
                            mma_s8s8(c[mt][n], qa[2 * half], kb[0], kb[1]);
                            mma_s8s8(c[mt][n], qa[2 * half + 1], kb[2], kb[3]);
                        } else {
                            uint32_t a[4];
                            load_qa(a, mt, 2 * half);
                            mma_s8s8(c[mt][n], a, kb[0], kb[1]);
                            load_qa(a, mt, 2 * half + 1);
                            mma_s8s8(c[mt][n], a, kb[2], kb[3]);
                        }
                    }
                }
            }
            const float *ksm = reinterpret_cast<const float *>(stp + 2 * C::KV_BYTES);
            const float *vsm = reinterpret_cast<const float *>(stp + 2 * C::KV_BYTES + C::SC_BYTES);
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                const float2 kk = *reinterpret_cast<const float2 *>(ksm + 8 * n + 2 * t);
                const float2 vv = *reinterpret_cast<const float2 *>(vsm + 8 * n + 2 * t);
                vs[n][0] = vv.x; vs[n][1] = vv.y;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    s2[mt][n][0] = (float)(c[mt][n][0] * 128 + c[mt][n][2]) * (qscale[mt] * kk.x);
                    s2[mt][n][1] = (float)(c[mt][n][1] * 128 + c[mt][n][3]) * (qscale[mt] * kk.y);
                }
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

        // ---------------------------------------------------- online softmax
        float vmax = 0.0f;
#pragma unroll
        for (int n = 0; n < 4; ++n) vmax = fmaxf(vmax, fmaxf(vs[n][0], vs[n][1]));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 1));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, 2));
        const float lgv = lg2f(vmax);
        float rvs[4][2];          // 1 / v_scale (0 for the zero-filled rows past the end of the window)
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int j = 0; j < 2; ++j) rvs[n][j] = vs[n][j] > 0.0f ? __frcp_rn(vs[n][j]) : 0.0f;

        uint32_t pa[MT][2][2];      // [mt][kstep][a0|a2]: fp16x2 of p * v_scale
        bool rescale = false;
        float alpha[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int n = 0; n < 4; ++n) mx = fmaxf(mx, fmaxf(s2[mt][n][0], s2[mt][n][1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(M[mt], mx + lgv);
            alpha[mt] = ex2f(M[mt] - m_new);
            rescale |= (m_new != M[mt]);
            M[mt] = m_new;
            const float sub = m_new - P_OFFSET;
            // p * v_scale goes to the tensor core in fp16.  The softmax denominator is
            // accumulated from those ROUNDED values (divided back by v_scale), so the
            // rounding acts as a perturbation of normalised weights and cancels for a
            // dominant key instead of showing up as an absolute error of the output.
            float lsum = 0.0f;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const int n = 2 * ks + hf;
                    const uint32_t pk = pack_f16x2(ex2f(s2[mt][n][0] - sub) * vs[n][0], ex2f(s2[mt][n][1] - sub) * vs[n][1]);
                    pa[mt][ks][hf] = pk;
                    const float2 pr = __half22float2(*reinterpret_cast<const __half2 *>(&pk));
                    lsum = fmaf(pr.x, rvs[n][0], lsum);
                    lsum = fmaf(pr.y, rvs[n][1], lsum);
                }
            l[mt] = l[mt] * alpha[mt] + lsum;
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int pm = 0; pm < C::MTP; ++pm)
#pragma unroll
                for (int nt = 0; nt < C::NT; ++nt) {
                    acc[pm][nt][0] *= alpha[2 * pm];
                    acc[pm][nt][1] *= alpha[2 * pm];
                    if (2 * pm + 1 < MT) {
                        acc[pm][nt][2] *= alpha[2 * pm + 1 < MT ? 2 * pm + 1 : 0];
                        acc[pm][nt][3] *= alpha[2 * pm + 1 < MT ? 2 * pm + 1 : 0];
                    }
                }
        }

        // --------------------------------------------------------------- PV
        if constexpr (FMT == KV_I8) {
            const uint32_t vst = st + C::KV_BYTES;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
                for (int cpair = 0; cpair < HD / 32; ++cpair) {
                    uint32_t vr[4];
                    const int mi = lane >> 3;
                    const int row = 16 * ks + 8 * (mi & 1) + (lane & 7);
                    const int ch = 2 * cpair + (mi >> 1);
                    ldmatrix_x4_trans(vr, vst + row * C::ROWB + swz_chunk<C::ROWB>(row, ch) * 16);
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const uint32_t x0 = vr[2 * cc] ^ 0x80808080u, x1 = vr[2 * cc + 1] ^ 0x80808080u;
                        const uint32_t be0 = hsub2_u32(prmt(x0, 0x64646464u, 0x4240u), 0x64806480u);
                        const uint32_t be1 = hsub2_u32(prmt(x1, 0x64646464u, 0x4240u), 0x64806480u);
                        const uint32_t bo0 = hsub2_u32(prmt(x0, 0x64646464u, 0x4341u), 0x64806480u);
                        const uint32_t bo1 = hsub2_u32(prmt(x1, 0x64646464u, 0x4341u), 0x64806480u);
                        const int nte = 2 * (2 * cpair + cc);
#pragma unroll
                        for (int pm = 0; pm < C::MTP; ++pm) {
                            if (2 * pm + 1 < MT) {
                                mma_f16(acc[pm][nte], pa[2 * pm][ks][0], pa[2 * pm + 1 < MT ? 2 * pm + 1 : 0][ks][0],
                                        pa[2 * pm][ks][1], pa[2 * pm + 1 < MT ? 2 * pm + 1 : 0][ks][1], be0, be1);
                                mma_f16(acc[pm][nte + 1], pa[2 * pm][ks][0], pa[2 * pm + 1 < MT ? 2 * pm + 1 : 0][ks][0],
                                        pa[2 * pm][ks][1], pa[2 * pm + 1 < MT ? 2 * pm + 1 : 0][ks][1], bo0, bo1);
                            } else {
                                mma_f16_top(acc[pm][nte][0], acc[pm][nte][1], pa[2 * pm][ks][0], pa[2 * pm][ks][1], be0, be1);
                                mma_f16_top(acc[pm][nte + 1][0], acc[pm][nte + 1][1], pa[2 * pm][ks][0], pa[2 * pm][ks][1], bo0, bo1);
                            }
                        }
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
    float *mbuf = reinterpret_cast<float *>(pipe);          // [NWARP][NSLOT][HD+2]
#pragma unroll
    for (int pm = 0; pm < C::MTP; ++pm)
#pragma unroll
        for (int nt = 0; nt < C::NT; ++nt) {
            // n tile nt holds d = 16*(nt/2) + 2*col + (nt&1); this thread has cols 2t, 2t+1
            const int d0 = 16 * (nt >> 1) + 4 * t + (nt & 1);
            float *r0 = mbuf + ((size_t)warp * C::NSLOT + (2 * pm) * 8 + g) * (HD + 2);
            r0[d0] = acc[pm][nt][0];
            r0[d0 + 2] = acc[pm][nt][1];
            if (2 * pm + 1 < MT) {
                float *r1 = r0 + 8 * (HD + 2);
                r1[d0] = acc[pm][nt][2];
                r1[d0 + 2] = acc[pm][nt][3];
            }
        }
    if (t == 0) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float *r0 = mbuf + ((size_t)warp * C::NSLOT + mt * 8 + g) * (HD + 2);
            r0[HD] = M[mt];
            r0[HD + 1] = l[mt];
        }
    }
    __syncthreads();

    for (int sl = 0; sl < C::NSLOT; ++sl) {
        const int idx = rg * C::NSLOT + sl;
        const int r = idx / p.kvg, j = idx % p.kvg;
        if (r >= p.S) break;
        float mstar = M_INIT;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) mstar = fmaxf(mstar, mbuf[((size_t)w * C::NSLOT + sl) * (HD + 2) + HD]);
        float wgt[NWARP], lstar = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) {
            const float *rw = mbuf + ((size_t)w * C::NSLOT + sl) * (HD + 2);
            wgt[w] = ex2f(rw[HD] - mstar);
            lstar += wgt[w] * rw[HD + 1];
        }
        const long grow = ((long)b * p.S + r) * p.nh + kvh * p.kvg + j;
        for (int d = threadIdx.x; d < HD; d += NWARP * 32) {
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < NWARP; ++w) o += wgt[w] * mbuf[((size_t)w * C::NSLOT + sl) * (HD + 2) + d];
            if (p.write_partial) {
                p.partial[((size_t)split * p.grows + grow) * (HD + 2) + d] = o;
            } else {
                const float v = lstar > 0.0f ? o / lstar : 0.0f;
                const long oi = b * p.out_batch_stride + ((long)r * p.nh + kvh * p.kvg + j) * HD + d;
                if (p.out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(p.out)[oi] = __float2bfloat16_rn(v);
                else reinterpret_cast<float *>(p.out)[oi] = v;
            }
        }
        if (p.write_partial && threadIdx.x == 0) {
            float *pr = p.partial + ((size_t)split * p.grows + grow) * (HD + 2);
            pr[HD] = p.export_nat ? (mstar - P_OFFSET) * LN2 : mstar;
            pr[HD + 1] = lstar;
        }
    }
}

// Merge G partial triples per row.  partials [G][rows][HD+2]; m in log2 units when
// nat == 0 (in-kernel split partials), natural-log units when nat == 1 (exported).
__global__ void merge_kernel(const float *partials, int G, int rows, int hd, void *out, int out_type, int nat,
                             float *partial_out) {
    const int row = blockIdx.x;
    const float unit = nat ? LOG2E : 1.0f;
    float mstar = -CUDART_INF_F;
    for (int i = 0; i < G; ++i) {
        const float *pr = partials + ((size_t)i * rows + row) * (hd + 2);
        if (pr[hd + 1] > 0.0f) mstar = fmaxf(mstar, pr[hd] * unit);
    }
    float lstar = 0.0f;
    for (int i = 0; i < G; ++i) {
        const float *pr = partials + ((size_t)i * rows + row) * (hd + 2);
        if (pr[hd + 1] > 0.0f) lstar += ex2f(pr[hd] * unit - mstar) * pr[hd + 1];
    }
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.0f;
        for (int i = 0; i < G; ++i) {
            const float *pr = partials + ((size_t)i * rows + row) * (hd + 2);
            if (pr[hd + 1] > 0.0f) o += ex2f(pr[hd] * unit - mstar) * pr[d];
        }
        if (partial_out) {
            partial_out[(size_t)row * (hd + 2) + d] = o;
        } else {
            const float v = lstar > 0.0f ? o / lstar : 0.0f;
            if (out_type == ET_BF16) reinterpret_cast<__nv_bfloat16 *>(out)[(size_t)row * hd + d] = __float2bfloat16_rn(v);
            else reinterpret_cast<float *>(out)[(size_t)row * hd + d] = v;
        }
    }
    if (partial_out && threadIdx.x == 0) {
        // exported partials carry m in natural-log units, offset removed
        partial_out[(size_t)row * (hd + 2) + hd] = lstar > 0.0f ? (nat ? mstar * LN2 : (mstar - P_OFFSET) * LN2) : 0.0f;
        partial_out[(size_t)row * (hd + 2) + hd + 1] = lstar;
    }
}

// ------------------------------------------------------------------ host side

struct DeviceInfo { int sm_count = 0; };
static DeviceInfo device_info() {
    static DeviceInfo cached[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev].sm_count == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev].sm_count = n > 0 ? n : 148;
    }
    return cached[dev];
}

struct Plan {
    int mt, row_groups, tile0, ntiles, splits, tiles_per_split, grows;
};

template <int FMT, int HD, int MT>
static int kernel_occupancy() {
    static int occ[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (occ[dev] == 0) {
        using C = Cfg<FMT, HD, MT>;
        cudaFuncSetAttribute(attn_fused_kernel<FMT, HD, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        int n = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_fused_kernel<FMT, HD, MT>, NWARP * 32, C::SMEM_BYTES);
        occ[dev] = n > 0 ? n : 1;
    }
    return occ[dev];
}

static int pick_mt(int slots) { return slots <= 8 ? 1 : 3; }

static Plan make_plan(const AttnArgs &a, int occupancy, int hd) {
    Plan pl;
    const int slots = a.S * a.kvg;
    pl.mt = pick_mt(slots);
    pl.row_groups = (slots + 8 * pl.mt - 1) / (8 * pl.mt);
    // first window index any row needs
    int j_begin = 0;
    if (a.window > 0) j_begin = std::max(0, (a.klen - (a.S - 1)) - a.window);
    pl.tile0 = j_begin / TILE;
    pl.ntiles = (a.klen + TILE - 1) / TILE - pl.tile0;
    pl.grows = a.batch * a.S * a.nh;
    const int units = a.nkv * a.batch * pl.row_groups;
    const int slots_gpu = device_info().sm_count * occupancy;
    int best = 1;
    if (a.force_splits > 0) {
        best = std::min(a.force_splits, pl.ntiles);
    } else {
        // cost ~ waves * (tiles per warp) + a small charge per split for the merge
        double best_cost = 1e30;
        int max_splits = std::min(pl.ntiles, 512);
        if (a.fit_splits_to_ws) {
            const long per_split = (long)pl.grows * (hd + 2) * 4;
            max_splits = (int)std::max<long>(1, std::min<long>(max_splits, a.workspace ? a.ws_bytes / per_split : 0));
        }
        for (int n = 1; n <= max_splits; ++n) {
            const int tps = (pl.ntiles + n - 1) / n;
            const int n_eff = (pl.ntiles + tps - 1) / tps;
            if (n_eff != n) continue;
            const int per_warp = (tps + NWARP - 1) / NWARP;
            const long ctas = (long)units * n;
            const long waves = (ctas + slots_gpu - 1) / slots_gpu;
            const double cost = (double)waves * (per_warp + 1.5) + 0.02 * n;
            if (cost < best_cost) { best_cost = cost; best = n; }
        }
    }
    pl.tiles_per_split = (pl.ntiles + best - 1) / best;
    pl.splits = (pl.ntiles + pl.tiles_per_split - 1) / pl.tiles_per_split;
    return pl;
}

template <int FMT, int HD, int MT>
static int launch_inst(cudaStream_t st, const AttnArgs &a, bool query_ws, long *ws_needed) {
    using C = Cfg<FMT, HD, MT>;
    const int occ = kernel_occupancy<FMT, HD, MT>();
    const Plan pl = make_plan(a, occ, HD);
    const long need = pl.splits > 1 ? (long)pl.splits * pl.grows * (HD + 2) * 4 : 0;
    if (query_ws) { *ws_needed = need; return NOMOS_OK; }
    if (need > a.ws_bytes || (need > 0 && a.workspace == nullptr)) {
        set_error("attention workspace too small: need %ld bytes, have %ld", need, a.ws_bytes);
        return NOMOS_ECAPACITY;
    }
    KParams p;
    p.q = static_cast<const uint8_t *>(a.q);
    p.k_cache = static_cast<const uint8_t *>(a.k_cache);
    p.v_cache = static_cast<const uint8_t *>(a.v_cache);
    p.k_scales = static_cast<const uint8_t *>(a.k_scales);
    p.v_scales = static_cast<const uint8_t *>(a.v_scales);
    p.out = static_cast<uint8_t *>(a.out);
    const bool direct_export = (pl.splits == 1 && a.partial_out != nullptr);
    p.partial = direct_export ? a.partial_out : static_cast<float *>(a.workspace);
    p.write_partial = (pl.splits > 1 || direct_export) ? 1 : 0;
    p.export_nat = direct_export ? 1 : 0;
    p.q_type = a.q_type; p.out_type = a.out_type;
    p.S = a.S; p.nh = a.nh; p.nkv = a.nkv; p.kvg = a.kvg; p.cache_hd = a.cache_hd; p.cache_cap = a.cache_cap;
    p.win_start = a.win_start; p.klen = a.klen; p.window = a.window;
    p.tile0 = pl.tile0; p.ntiles = pl.ntiles; p.tiles_per_split = pl.tiles_per_split;
    p.row_groups = pl.row_groups; p.grows = pl.grows;
    p.qk_scale_log2 = a.softmax_scale * LOG2E;
    p.q_batch_stride = a.q_batch_stride; p.kv_batch_stride = a.kv_batch_stride;
    p.scale_batch_stride = a.scale_batch_stride; p.out_batch_stride = a.out_batch_stride;
    dim3 grid(pl.splits, a.nkv, a.batch * pl.row_groups);
    attn_fused_kernel<FMT, HD, MT><<<grid, NWARP * 32, C::SMEM_BYTES, st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("attn_fused launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    if (pl.splits > 1) {
        merge_kernel<<<pl.grows, 128, 0, st>>>(static_cast<const float *>(a.workspace), pl.splits, pl.grows, HD, a.out,
                                               a.out_type, 0, a.partial_out);
        e = cudaGetLastError();
        if (e != cudaSuccess) { set_error("merge launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    }
    return NOMOS_OK;
}

template <int FMT, int HD>
static int dispatch_mt(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    return pick_mt(a.S * a.kvg) == 1 ? launch_inst<FMT, HD, 1>(st, a, q, ws) : launch_inst<FMT, HD, 3>(st, a, q, ws);
}

static int dispatch(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    if (a.kv_fmt != KV_I8) { set_error("kv_fmt %d not built yet", a.kv_fmt); return NOMOS_EUNSUPPORTED; }
    switch (a.l_hd) {
        case 128: return dispatch_mt<KV_I8, 128>(st, a, q, ws);
        default: set_error("head_dim %d unsupported (128)", a.l_hd); return NOMOS_EUNSUPPORTED;
    }
}

}  // namespace

long attn_workspace_bytes(const AttnArgs &a) {
    long ws = 0;
    const int rc = dispatch(nullptr, a, true, &ws);
    return rc == NOMOS_OK ? ws : (long)rc;
}

int launch_attn_fused(cudaStream_t st, const AttnArgs &a) { return dispatch(st, a, false, nullptr); }

int launch_merge_partials(cudaStream_t st, const float *partials, int G, int rows, int l_hd, void *out, int out_type) {
    merge_kernel<<<rows, 128, 0, st>>>(partials, G, rows, l_hd, out, out_type, 1, nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("merge launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

int launch_merge_partials_log2(cudaStream_t st, const float *partials, int G, int rows, int l_hd, float *out) {
    merge_kernel<<<rows, 128, 0, st>>>(partials, G, rows, l_hd, out, ET_F32, 0, nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("merge launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

}  // namespace nomos
