// Row quantizers of the KV cache (one warp per row), shared by the append kernels and by the
// fused attention kernel's quantize-on-write.  Every rounding step is an explicit
// round-to-nearest intrinsic, so the bytes do not depend on FMA contraction settings.
// Reference arithmetic: lib/kv_cache_quant.mojo:33-40, 170-193 (int8), 338-365 (int4 row scale),
// 536-578 (int4 block-32).
#pragma once

#include "common.cuh"

namespace nomos {

template <typename SrcT>
__device__ __forceinline__ float load_as_f32(const SrcT *p);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
// CG = true reads a source row through L2 only (ld.global.cg).  The attention kernels quantise new rows once
// before their stream-order wait (a warming pass whose results are discarded) and once after it: the second
// read must not be served from a line the first one left in L1.
template <bool CG>
__device__ __forceinline__ float load_src(const float *p) {
    if constexpr (CG) return __ldcg(p);
    else return *p;
}

// scale = amax/127 (0 -> 1), code = round_away(x * (1/scale)); pad [l_hd, row_w) with 0.
template <typename SrcT>
__device__ __forceinline__ void quant_row_i8(const SrcT *src, int l_hd, int row_w, int8_t *dst, float *scale_out, int lane) {
    float amax = 0.0f;
    for (int i = lane; i < l_hd; i += 32) amax = fmaxf(amax, fabsf(load_as_f32(src + i)));
    amax = warp_max(amax);
    float scale = __fdiv_rn(amax, 127.0f);
    if (scale == 0.0f) scale = 1.0f;
    if (lane == 0) *scale_out = scale;
    const float inv = __fdiv_rn(1.0f, scale);
    for (int j = lane; j < row_w; j += 32)
        dst[j] = (j < l_hd) ? static_cast<int8_t>(round_away_clamp(__fmul_rn(load_as_f32(src + j), inv), 127)) : int8_t(0);
}

// The same codec for fp32 rows read through L2 only (see load_src).
__device__ __forceinline__ void quant_row_i8_cg(const float *src, int l_hd, int row_w, int8_t *dst, float *scale_out, int lane) {
    float amax = 0.0f;
    for (int i = lane; i < l_hd; i += 32) amax = fmaxf(amax, fabsf(__ldcg(src + i)));
    amax = warp_max(amax);
    float scale = __fdiv_rn(amax, 127.0f);
    if (scale == 0.0f) scale = 1.0f;
    if (lane == 0) *scale_out = scale;
    const float inv = __fdiv_rn(1.0f, scale);
    for (int j = lane; j < row_w; j += 32)
        dst[j] = (j < l_hd) ? static_cast<int8_t>(round_away_clamp(__fmul_rn(__ldcg(src + j), inv), 127)) : int8_t(0);
}

// Row-scale int4: scale = amax/7 (0 -> 1), reciprocal multiply, nibble pack
// (even element low).  If view != nullptr the signed codes are also written as an
// int8 row of width row_w (the "q8 view" of the verify route).
template <bool CG = false>
__device__ __forceinline__ float quant_row_i4(const float *src, int l_hd, int row_w, uint8_t *dst, int8_t *view, int lane) {
    float amax = 0.0f;
    for (int i = lane; i < l_hd; i += 32) amax = fmaxf(amax, fabsf(load_src<CG>(src + i)));
    amax = warp_max(amax);
    float scale = __fdiv_rn(amax, 7.0f);
    if (scale == 0.0f) scale = 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    for (int jb = lane; jb < row_w / 2; jb += 32) {
        const int j0 = 2 * jb, j1 = j0 + 1;
        const int q0 = (j0 < l_hd) ? round_away_clamp(__fmul_rn(load_src<CG>(src + j0), inv), 7) : 0;
        const int q1 = (j1 < l_hd) ? round_away_clamp(__fmul_rn(load_src<CG>(src + j1), inv), 7) : 0;
        dst[jb] = static_cast<uint8_t>((q0 & 0xF) | ((q1 & 0xF) << 4));
        if (view) { view[j0] = (int8_t)q0; if (j1 < row_w) view[j1] = (int8_t)q1; }
    }
    return scale;
}

// Block-32 int4: per 32 values s = amax/7 (1 if amax == 0) narrowed to fp16; codes
// divide by the widened fp16 value (a true division).  Returns the per-row q8
// scale max_b(sf_b*7)/127 (1 if 0).  Lane i < 16 packs elements (2i, 2i+1) of
// each block.
template <bool CG = false>
__device__ __forceinline__ float quant_row_i4_block32(const float *src, int l_hd, uint8_t *dst, __half *scales16, int lane) {
    const int nblocks = (l_hd + 31) / 32;
    float row_recon = 0.0f;
    for (int b = 0; b < nblocks; ++b) {
        const int d = b * 32 + lane;
        const float x = (d < l_hd) ? load_src<CG>(src + d) : 0.0f;
        const float a = warp_max(fabsf(x));
        const float s = (a > 0.0f) ? __fdiv_rn(a, 7.0f) : 1.0f;
        const __half s16 = __float2half_rn(s);
        const float sf = __half2float(s16);
        row_recon = fmaxf(row_recon, __fmul_rn(sf, 7.0f));
        if (lane == 0) scales16[b] = s16;
        const int q = (d < l_hd) ? round_away_clamp(__fdiv_rn(x, sf), 7) : 0;
        const int q_hi = __shfl_down_sync(0xffffffffu, q, 1);
        if ((lane & 1) == 0) dst[d >> 1] = static_cast<uint8_t>((q & 0xF) | ((q_hi & 0xF) << 4));
    }
    return (row_recon > 0.0f) ? __fdiv_rn(row_recon, 127.0f) : 1.0f;
}

}  // namespace nomos
