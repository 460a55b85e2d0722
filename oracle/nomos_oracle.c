/*
 * nomos_oracle.c -- CPU restatement of the quantized-KV attention path of
 * lightofbaldr/nomos-nvfp4 (Mojo GPU kernels), used ONLY as a checker.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Nothing in the shipped
 * library links, imports or calls it; the parity tests, the smoke check and the
 * benchmark's CPU-baseline leg are its only users.
 *
 * PARITY STATUS: "parity unpinned" at the byte level.  The reference ships no
 * golden KV bytes/scales and its toolchain (Mojo) cannot run where this file is
 * built, so the restatement assumes IEEE-754 binary32 div/mul/add with no FMA
 * contraction, round-to-nearest-even fp16/bf16 narrowing, and truncating
 * float->int casts.  It IS pinned against every property the reference's own
 * tests hold for this path: the nibble identities of tools/parity_attn_int4.mojo,
 * the codec tolerance of tools/kv_quant_test.mojo and the A/B properties of the
 * nomos_debug_kv_* probes in nomos_ffi.mojo (see tests/).
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 *
 * Every function names the reference file:line it follows (paths relative to
 * the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ helpers */

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* bf16 <-> fp32.  Narrowing is round-to-nearest-even, the semantics of a Mojo
 * `.cast[DType.bfloat16]()` (lib/kv_cache_quant.mojo:97, lib/cast_gpu_mojo.mojo:16-27). */
static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* fp16 <-> fp32 through the compiler's IEEE half type (RNE). */
static inline uint16_t f32_to_f16(float f) { _Float16 h = (_Float16)f; uint16_t u; memcpy(&u, &h, 2); return u; }
static inline float f16_to_f32(uint16_t u) { _Float16 h; memcpy(&h, &u, 2); return (float)h; }

/* Round half away from zero by adding +-0.5 IN BINARY32 and truncating, then
 * clamp to the symmetric range.  lib/kv_cache_quant.mojo:33-40 (int8) and
 * :301-308 (int4).  Note 0.49999997f + 0.5f == 1.0f in binary32. */
static inline int round_away_clamp(float x, int lim) {
    volatile float y = (x >= 0.0f) ? (x + 0.5f) : (x - 0.5f);
    int r = (int)y;
    if (r > lim) r = lim;
    if (r < -lim) r = -lim;
    return r;
}

static inline float row_absmax(const float *x, int n) {
    float a = 0.0f;
    for (int i = 0; i < n; ++i) { float v = fabsf(x[i]); if (v > a) a = v; }
    return a;
}

/* Two's-complement nibble -> signed value in [-8,7].
 * lib/kv_cache_quant.mojo:761-763; identity (n^8)-8 from tools/parity_attn_int4.mojo:27-34. */
static inline int nib_sext(int nib) { return nib >= 8 ? nib - 16 : nib; }
static inline int i4_at(const uint8_t *row, int d) {
    int b = row[d >> 1];
    return nib_sext((d & 1) ? ((b >> 4) & 0xF) : (b & 0xF));
}

/* round-half-to-even to integer, the assumed meaning of Mojo's `round` in
 * q_to_i8 (lib/attention_gpu_int8.mojo:43-45); then the symmetric clamp (:35-40). */
static inline int q_to_i8(float x, float scale) {
    float r = nearbyintf(x / scale);   /* default rounding mode = nearest-even */
    int q = (int)r;
    if (q > 127) q = 127;
    if (q < -127) q = -127;
    return q;
}

/* ----------------------------------------------------- K1: standalone codec */

/* lib/kv_cache_quant.mojo:43-82 -- bf16 [n_rows, dim] -> int8 + fp32 row scale. */
ORC_API void orc_quant_kv_i8(const uint16_t *in_bf16, int8_t *out_i8, float *out_scales,
                             int n_rows, int dim) {
    for (int r = 0; r < n_rows; ++r) {
        const uint16_t *src = in_bf16 + (size_t)r * dim;
        float amax = 0.0f;
        for (int i = 0; i < dim; ++i) { float v = fabsf(bf16_to_f32(src[i])); if (v > amax) amax = v; }
        float scale = amax / 127.0f;
        if (scale == 0.0f) scale = 1.0f;
        out_scales[r] = scale;
        float inv = 1.0f / scale;
        for (int i = 0; i < dim; ++i)
            out_i8[(size_t)r * dim + i] = (int8_t)round_away_clamp(bf16_to_f32(src[i]) * inv, 127);
    }
}

/* lib/kv_cache_quant.mojo:85-97 */
ORC_API void orc_dequant_kv_i8(const int8_t *in_i8, const float *in_scales, uint16_t *out_bf16,
                               int n_rows, int dim) {
    for (int r = 0; r < n_rows; ++r)
        for (int i = 0; i < dim; ++i) {
            size_t k = (size_t)r * dim + i;
            out_bf16[k] = f32_to_bf16((float)in_i8[k] * in_scales[r]);
        }
}

/* ------------------------------------------------ K2: int8 quantize-on-write */

/* One (token, head) row: absmax/127 scale, multiply by the reciprocal, zero pad
 * to cache_hd.  lib/kv_cache_quant.mojo:170-193. */
static void put_row_i8(const float *x, int l_hd, int cache_hd, int8_t *dst, float *scale_out) {
    float scale = row_absmax(x, l_hd) / 127.0f;
    if (scale == 0.0f) scale = 1.0f;
    *scale_out = scale;
    float inv = 1.0f / scale;
    for (int j = 0; j < cache_hd; ++j)
        dst[j] = (j < l_hd) ? (int8_t)round_away_clamp(x[j] * inv, 127) : (int8_t)0;
}

/* lib/kv_cache_quant.mojo:144-218,252-271.  Ring slot = (base_pos+s) % cache_cap. */
ORC_API void orc_append_quant_kv_i8(const float *src_k, const float *src_v,
                                    int8_t *dst_k, int8_t *dst_v, float *k_scales, float *v_scales,
                                    int n_s, int nkv, int l_hd, int l_kvd, int cache_cap,
                                    int cache_hd, int base_pos) {
    for (int s = 0; s < n_s; ++s)
        for (int h = 0; h < nkv; ++h) {
            size_t src = (size_t)s * l_kvd + (size_t)h * l_hd;
            size_t row = (size_t)h * cache_cap + (size_t)((base_pos + s) % cache_cap);
            put_row_i8(src_k + src, l_hd, cache_hd, dst_k + row * cache_hd, k_scales + row);
            put_row_i8(src_v + src, l_hd, cache_hd, dst_v + row * cache_hd, v_scales + row);
        }
}

/* ---------------------------------------- K3: int4, one fp32 scale per row */

/* lib/kv_cache_quant.mojo:338-365: amax/7, reciprocal multiply, clamp +-7,
 * even element -> low nibble, odd element -> high nibble.  Optionally returns
 * the unpacked codes (used by the q8-view twin, :454-464). */
static void put_row_i4(const float *x, int l_hd, int cache_hd, uint8_t *dst, float *scale_out,
                       int8_t *codes_out /* cache_hd entries or NULL */) {
    float scale = row_absmax(x, l_hd) / 7.0f;
    if (scale == 0.0f) scale = 1.0f;
    *scale_out = scale;
    float inv = 1.0f / scale;
    int hc = cache_hd / 2;
    for (int jb = 0; jb < hc; ++jb) {
        int j0 = 2 * jb, j1 = j0 + 1;
        int q0 = (j0 < l_hd) ? round_away_clamp(x[j0] * inv, 7) : 0;
        int q1 = (j1 < l_hd) ? round_away_clamp(x[j1] * inv, 7) : 0;
        dst[jb] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
        if (codes_out) { codes_out[j0] = (int8_t)q0; if (j1 < cache_hd) codes_out[j1] = (int8_t)q1; }
    }
}

/* ------------------------- K4: int4 with one fp16 scale per 32 (block-32) */

/* lib/kv_cache_quant.mojo:536-578.  Per block: s = amax/7 (1.0 if amax == 0),
 * narrowed to fp16 and widened back; codes use a TRUE DIVISION by that value.
 * Also returns the cached per-row q8 scale max_b(sf_b*7)/127 (1.0 if 0). */
static float put_row_i4_block32(const float *x, int l_hd, uint8_t *dst, uint16_t *scales16) {
    int nblocks = (l_hd + 31) / 32;
    float row_recon = 0.0f;
    for (int b = 0; b < nblocks; ++b) {
        float a = 0.0f;
        for (int i = 0; i < 32; ++i) {
            int d = b * 32 + i;
            float v = (d < l_hd) ? fabsf(x[d]) : 0.0f;
            if (v > a) a = v;
        }
        float s = (a > 0.0f) ? (a / 7.0f) : 1.0f;
        uint16_t s16 = f32_to_f16(s);
        float sf = f16_to_f32(s16);
        float recon = sf * 7.0f;
        if (recon > row_recon) row_recon = recon;
        scales16[b] = s16;
        for (int lane = 0; lane < 16; ++lane) {
            int d0 = b * 32 + 2 * lane, d1 = d0 + 1;
            int q0 = (d0 < l_hd) ? round_away_clamp(x[d0] / sf, 7) : 0;
            int q1 = (d1 < l_hd) ? round_away_clamp(x[d1] / sf, 7) : 0;
            dst[d0 / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
        }
    }
    return (row_recon > 0.0f) ? (row_recon / 127.0f) : 1.0f;
}

/* lib/kv_cache_quant.mojo:803-836 (dispatch), :311-394 (row scale), :502-578 (block-32).
 * For scale_blocks > 1 the scale buffer is [nkv,cache_cap,nblocks] fp16 followed at byte
 * offset nkv*cache_cap*nblocks*2 by [nkv,cache_cap] fp32 q8 row scales (:529-534). */
ORC_API void orc_append_quant_kv_i4(const float *src_k, const float *src_v,
                                    uint8_t *dst_k, uint8_t *dst_v, void *k_scales, void *v_scales,
                                    int n_s, int nkv, int l_hd, int l_kvd, int cache_cap,
                                    int cache_hd, int base_pos, int scale_blocks) {
    int hc = cache_hd / 2;
    int nblocks = (l_hd + 31) / 32;
    for (int s = 0; s < n_s; ++s)
        for (int h = 0; h < nkv; ++h) {
            size_t src = (size_t)s * l_kvd + (size_t)h * l_hd;
            size_t row = (size_t)h * cache_cap + (size_t)((base_pos + s) % cache_cap);
            if (scale_blocks > 1) {
                uint16_t *k16 = (uint16_t *)k_scales, *v16 = (uint16_t *)v_scales;
                float *kq8 = (float *)((char *)k_scales + (size_t)nkv * cache_cap * nblocks * 2);
                float *vq8 = (float *)((char *)v_scales + (size_t)nkv * cache_cap * nblocks * 2);
                kq8[row] = put_row_i4_block32(src_k + src, l_hd, dst_k + row * hc, k16 + row * nblocks);
                vq8[row] = put_row_i4_block32(src_v + src, l_hd, dst_v + row * hc, v16 + row * nblocks);
            } else {
                put_row_i4(src_k + src, l_hd, cache_hd, dst_k + row * hc, (float *)k_scales + row, NULL);
                put_row_i4(src_v + src, l_hd, cache_hd, dst_v + row * hc, (float *)v_scales + row, NULL);
            }
        }
}

/* ------------------------------------ K5: append + publish an int8 "view" */

/* lib/kv_cache_quant.mojo:839-882 (dispatch), :397-497 (row scale: the view row is
 * the int4 code itself, view scale = the /7 scale), :581-689 (block-32: the view is
 * rebuilt from the stored nibbles: trunc((q4*sf)/q8s +- 0.5)).  View row index is
 * h*q8_pitch + (base_pos+s) -- absolute, NOT a ring slot. */
ORC_API void orc_append_quant_kv_i4_with_q8(const float *src_k, const float *src_v,
                                            uint8_t *dst_k, uint8_t *dst_v, void *k_scales, void *v_scales,
                                            int8_t *k_q8, int8_t *v_q8, float *k_q8_scales, float *v_q8_scales,
                                            int n_s, int nkv, int l_hd, int l_kvd, int cache_cap,
                                            int cache_hd, int base_pos, int q8_pitch, int scale_blocks) {
    int hc = cache_hd / 2;
    int nblocks = (l_hd + 31) / 32;
    for (int s = 0; s < n_s; ++s)
        for (int h = 0; h < nkv; ++h) {
            int apos = base_pos + s;
            size_t src = (size_t)s * l_kvd + (size_t)h * l_hd;
            size_t row = (size_t)h * cache_cap + (size_t)(apos % cache_cap);
            size_t vrow = (size_t)h * q8_pitch + (size_t)apos;
            for (int kv = 0; kv < 2; ++kv) {
                const float *x = (kv ? src_v : src_k) + src;
                uint8_t *dst = (kv ? dst_v : dst_k) + row * hc;
                void *scales = kv ? v_scales : k_scales;
                int8_t *view = (kv ? v_q8 : k_q8) + vrow * cache_hd;
                float *view_scale = (kv ? v_q8_scales : k_q8_scales) + vrow;
                if (scale_blocks > 1) {
                    uint16_t *s16 = (uint16_t *)scales + row * nblocks;
                    float *q8c = (float *)((char *)scales + (size_t)nkv * cache_cap * nblocks * 2);
                    float q8s = put_row_i4_block32(x, l_hd, dst, s16);
                    q8c[row] = q8s;
                    *view_scale = q8s;
                    for (int d = 0; d < l_hd; ++d) {
                        float sf = f16_to_f32(s16[d / 32]);
                        view[d] = (int8_t)round_away_clamp(((float)i4_at(dst, d) * sf) / q8s, 127);
                    }
                } else {
                    float sc;
                    put_row_i4(x, l_hd, cache_hd, dst, &sc, view);
                    ((float *)scales)[row] = sc;
                    *view_scale = sc;
                }
            }
        }
}

/* ---------------------------------------------------- K6-K9: window readers */

/* All readers map linear window index j in [0,klen) of head h to ring row
 * h*cache_cap + (win_start+j) % cache_cap and write linear row h*pitch + j
 * (pitch is the argument the reference calls max_seq).  lib/kv_cache_quant.mojo:239-249. */

/* lib/kv_cache_quant.mojo:221-249,274-290 */
ORC_API void orc_dequant_kv_i8_layer(const int8_t *src, const float *scales, uint16_t *dst_bf16,
                                     int nkv, int klen, int cache_hd, int pitch, int cache_cap, int win_start) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < nkv; ++h)
        for (int j = 0; j < klen; ++j) {
            size_t sr = (size_t)h * cache_cap + (size_t)((win_start + j) % cache_cap);
            size_t dr = (size_t)h * pitch + j;
            for (int d = 0; d < cache_hd; ++d)
                dst_bf16[dr * cache_hd + d] = f32_to_bf16((float)src[sr * cache_hd + d] * scales[sr]);
        }
}

/* lib/kv_cache_quant.mojo:739-800,885-918.  Block-32 reader computes
 * nblocks from cache_hd (:798), the writer from l_hd (:528). */
ORC_API void orc_dequant_kv_i4_layer(const uint8_t *src, const void *scales, uint16_t *dst_bf16,
                                     int nkv, int klen, int cache_hd, int pitch, int cache_cap,
                                     int win_start, int scale_blocks) {
    int hc = cache_hd / 2, nblocks = (cache_hd + 31) / 32;
    for (int h = 0; h < nkv; ++h)
        for (int j = 0; j < klen; ++j) {
            size_t sr = (size_t)h * cache_cap + (size_t)((win_start + j) % cache_cap);
            size_t dr = (size_t)h * pitch + j;
            for (int d = 0; d < cache_hd; ++d) {
                float q = (float)i4_at(src + sr * hc, d);
                float sc = (scale_blocks > 1)
                    ? f16_to_f32(((const uint16_t *)scales)[sr * nblocks + d / 32])
                    : ((const float *)scales)[sr];
                dst_bf16[dr * cache_hd + d] = f32_to_bf16(q * sc);
            }
        }
}

/* lib/kv_cache_quant.mojo:925-989 (row scale: lossless widen + copied scale) and
 * :708-736 (block-32: re-round onto the cached per-row q8 scale, which sits
 * nkv*cache_cap*scale_blocks*2 bytes into the scale buffer, :967). */
ORC_API void orc_dequant_kv_i4_to_q8_layer(const uint8_t *src, const void *scales, int8_t *dst_i8,
                                           float *dst_scale, int nkv, int klen, int cache_hd, int pitch,
                                           int cache_cap, int win_start, int scale_blocks) {
    int hc = cache_hd / 2, nblocks = (cache_hd + 31) / 32;
    const float *q8c = (const float *)((const char *)scales + (size_t)nkv * cache_cap * scale_blocks * 2);
    for (int h = 0; h < nkv; ++h)
        for (int j = 0; j < klen; ++j) {
            size_t sr = (size_t)h * cache_cap + (size_t)((win_start + j) % cache_cap);
            size_t dr = (size_t)h * pitch + j;
            for (int d = 0; d < cache_hd; ++d) {
                int q4 = i4_at(src + sr * hc, d);
                if (scale_blocks > 1) {
                    float bs = f16_to_f32(((const uint16_t *)scales)[sr * nblocks + d / 32]);
                    dst_i8[dr * cache_hd + d] = (int8_t)round_away_clamp(((float)q4 * bs) / q8c[sr], 127);
                } else {
                    dst_i8[dr * cache_hd + d] = (int8_t)q4;
                }
            }
            dst_scale[dr] = (scale_blocks > 1) ? q8c[sr] : ((const float *)scales)[sr];
        }
}

/* lib/kv_cache_quant.mojo:692-705 (defined in the reference, no caller). */
ORC_API void orc_block32_i4_q8_scales(const uint16_t *scales, float *dst_scale, int nkv, int klen,
                                      int nblocks, int pitch, int cache_cap, int win_start) {
    for (int h = 0; h < nkv; ++h)
        for (int j = 0; j < klen; ++j) {
            size_t sr = (size_t)h * cache_cap + (size_t)((win_start + j) % cache_cap);
            float am = 0.0f;
            for (int b = 0; b < nblocks; ++b) {
                float s = f16_to_f32(scales[sr * nblocks + b]) * 7.0f;
                if (s > am) am = s;
            }
            dst_scale[(size_t)h * pitch + j] = (am > 0.0f) ? am / 127.0f : 1.0f;
        }
}

/* --------------------------------------------- K10/K11: fp32 / bf16 appends */

/* lib/attention_gpu.mojo:87-106: nkv rows of l_hd floats to (kvh*max_seq + cl)*cache_hd. */
ORC_API void orc_append_kv_fp32(float *k_cache, float *v_cache, const float *k_new, const float *v_new,
                                int nkv, int l_hd, int cache_hd, int max_seq, int cl) {
    for (int h = 0; h < nkv; ++h) {
        size_t dst = ((size_t)h * max_seq + cl) * cache_hd;
        memcpy(k_cache + dst, k_new + (size_t)h * l_hd, (size_t)l_hd * 4);
        memcpy(v_cache + dst, v_new + (size_t)h * l_hd, (size_t)l_hd * 4);
    }
}

/* lib/batched_attn_gpu.mojo:55-102 (and the per-token twin lib/attention_gpu.mojo:136-162). */
ORC_API void orc_append_kv_batched_bf16(const float *src_k, const float *src_v, uint16_t *dst_k, uint16_t *dst_v,
                                        int n_s, int nkv, int l_hd, int l_kvd, int max_seq, int cache_hd,
                                        int base_pos) {
    for (int s = 0; s < n_s; ++s)
        for (int h = 0; h < nkv; ++h)
            for (int d = 0; d < l_hd; ++d) {
                size_t so = (size_t)s * l_kvd + (size_t)h * l_hd + d;
                size_t dofs = ((size_t)h * max_seq + (size_t)(base_pos + s)) * cache_hd + d;
                dst_k[dofs] = f32_to_bf16(src_k[so]);
                dst_v[dofs] = f32_to_bf16(src_v[so]);
            }
}

/* ------------------------------------------------------------ row softmax */

/* lib/softmax_gpu_mojo.mojo:37-134: max, exp(x-max) with running sum, multiply
 * by the reciprocal of the sum.  Summation order on the GPU is a tree; here it is
 * sequential, which only matters at the ulp level. */
static void softmax_row(float *x, int n) {
    float m = -3.4e38f;
    for (int i = 0; i < n; ++i) if (x[i] > m) m = x[i];
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) { x[i] = expf(x[i] - m); sum += x[i]; }
    float inv = 1.0f / sum;
    for (int i = 0; i < n; ++i) x[i] *= inv;
}

/* ------------------------- A3/A4: int8 attention with re-quantised Q and P */

/* Scores of one query row against keys [0,klen) at base row `krow0`.
 * lib/attention_gpu_int8.mojo:68-90: per 32-dim block, dq = amax/127 (1.0 if 0),
 * q8 = clamp(round(q/dq)), int32 dot, acc += dq * k_scale * float(isum). */
static void qk_row_int8(const float *q, const int8_t *k_i8, const float *k_scale, size_t krow0,
                        int klen, int l_hd, int cache_hd, float *scores) {
    int nqb = (l_hd + 31) / 32;
    float dq[64];
    int8_t q8[2048];
    for (int b = 0; b < nqb; ++b) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) { int d = b * 32 + i; if (d < l_hd) { float a = fabsf(q[d]); if (a > amax) amax = a; } }
        dq[b] = (amax > 0.0f) ? amax / 127.0f : 1.0f;
        for (int i = 0; i < 32; ++i) { int d = b * 32 + i; if (d < l_hd) q8[d] = (int8_t)q_to_i8(q[d], dq[b]); }
    }
    for (int t = 0; t < klen; ++t) {
        const int8_t *kr = k_i8 + (krow0 + t) * cache_hd;
        float acc = 0.0f;
        for (int b = 0; b < nqb; ++b) {
            int32_t isum = 0;
            for (int i = 0; i < 32; ++i) { int d = b * 32 + i; if (d < l_hd) isum += (int32_t)q8[d] * (int32_t)kr[d]; }
            acc += dq[b] * k_scale[krow0 + t] * (float)isum;
        }
        scores[t] = acc;
    }
}

/* lib/attention_gpu_int8.mojo:114-136: per 32-key block (anchored at key 0 of the
 * row's range), dp = max|p*vs|/127 (1.0 if 0), p8 = clamp(round(w/dp)), int32
 * dot with V, acc += dp * float(isum). */
static void pv_row_int8(const float *p, const int8_t *v_i8, const float *v_scale, size_t vrow0,
                        int klen, int l_hd, int cache_hd, float *out) {
    int nkb = (klen + 31) / 32;
    for (int d = 0; d < l_hd; ++d) out[d] = 0.0f;
    for (int b = 0; b < nkb; ++b) {
        float amax = 0.0f;
        int8_t p8[32];
        int n = 0;
        for (int i = 0; i < 32; ++i) {
            int t = b * 32 + i;
            if (t < klen) { float w = p[t] * v_scale[vrow0 + t]; float a = fabsf(w); if (a > amax) amax = a; n = i + 1; }
        }
        float dp = (amax > 0.0f) ? amax / 127.0f : 1.0f;
        for (int i = 0; i < n; ++i) { int t = b * 32 + i; p8[i] = (int8_t)q_to_i8(p[t] * v_scale[vrow0 + t], dp); }
        for (int d = 0; d < l_hd; ++d) {
            int32_t isum = 0;
            for (int i = 0; i < n; ++i) isum += (int32_t)p8[i] * (int32_t)v_i8[(vrow0 + b * 32 + i) * cache_hd + d];
            out[d] += dp * (float)isum;
        }
    }
}

/* lib/attention_gpu_int8.mojo:598-631.  scores is caller scratch [nh, seq_len]. */
ORC_API void orc_attn_decode_int8(const float *q, const int8_t *k_i8, const int8_t *v_i8,
                                  const float *k_scale, const float *v_scale, float *scores, float *out,
                                  int nh, int nkv, int l_hd, int cache_hd, int max_seq, int seq_len, int kvg) {
    (void)nkv;
    if (nh <= 0 || seq_len <= 0) return;
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < nh; ++h) {
        size_t row0 = (size_t)(h / kvg) * max_seq;
        float *sc = scores + (size_t)h * seq_len;
        qk_row_int8(q + (size_t)h * l_hd, k_i8, k_scale, row0, seq_len, l_hd, cache_hd, sc);
        softmax_row(sc, seq_len);
        pv_row_int8(sc, v_i8, v_scale, row0, seq_len, l_hd, cache_hd, out + (size_t)h * l_hd);
    }
}

/* lib/attention_gpu_int8.mojo:634-708 (kernels :322-584).  Row r attends absolute
 * keys [lo, apos], apos = query_base_pos + r, lo = max(0, apos-window+1) if window>0. */
ORC_API void orc_attn_multirow_int8(const float *q_b, float *scores, float *out, const int8_t *k_i8,
                                    const int8_t *v_i8, const float *k_scale, const float *v_scale,
                                    int nh, int nkv, int l_hd, int cache_hd, int max_seq, int S,
                                    int score_stride, int kvg, int window, int query_base_pos) {
    (void)nkv;
    if (nh <= 0 || S <= 0 || score_stride <= 0) return;
#pragma omp parallel for schedule(dynamic)
    for (int rh = 0; rh < S * nh; ++rh) {
        int r = rh / nh, h = rh % nh;
        int apos = query_base_pos + r;
        int lo = (window > 0 && apos - window + 1 > 0) ? apos - window + 1 : 0;
        int klen = apos + 1 - lo;
        if (klen <= 0) continue;
        size_t row0 = (size_t)(h / kvg) * max_seq + lo;
        float *sc = scores + (size_t)rh * score_stride;
        qk_row_int8(q_b + (size_t)rh * l_hd, k_i8, k_scale, row0, klen, l_hd, cache_hd, sc);
        softmax_row(sc, klen);
        pv_row_int8(sc, v_i8, v_scale, row0, klen, l_hd, cache_hd, out + (size_t)rh * l_hd);
    }
}

/* Valid key range of query row s for the batched/prefix softmax.
 * lib/batched_attn_gpu.mojo:176-183 (square) and :314-326 (prefix). */
static void prefix_bounds(int s, int key_len, int window, int query_base_pos, int key_base_pos,
                          int *lo_out, int *hi_out) {
    int q_abs = query_base_pos + s;
    int hi = q_abs - key_base_pos;
    if (hi >= key_len) hi = key_len - 1;
    int lo_abs = 0;
    if (window > 0 && q_abs - window + 1 > 0) lo_abs = q_abs - window + 1;
    int lo = lo_abs - key_base_pos;
    if (lo < 0) lo = 0;
    *lo_out = lo; *hi_out = hi;
}

/* Masked softmax over [lo,hi], exact zeros elsewhere; an empty range zeroes the
 * row.  lib/batched_attn_gpu.mojo:329-409. */
static void softmax_row_masked(float *x, int n, int lo, int hi) {
    if (hi < lo) { for (int i = 0; i < n; ++i) x[i] = 0.0f; return; }
    softmax_row(x + lo, hi - lo + 1);
    for (int i = 0; i < lo; ++i) x[i] = 0.0f;
    for (int i = hi + 1; i < n; ++i) x[i] = 0.0f;
}

/* lib/attention_gpu_int8.mojo:844-887 (prefix) and, with key_len=S and both
 * bases 0, :804-841 (square).  q_b/out are [S, nh, l_hd]; scores scratch is
 * [nkv, S*kvg, key_len]; PV blocks are anchored at key 0 of the shared range. */
ORC_API void orc_attn_prefix_batched_int8(const float *q_b, float *scores, float *out, const int8_t *k_i8,
                                          const int8_t *v_i8, const float *k_scale, const float *v_scale,
                                          int nh, int nkv, int l_hd, int cache_hd, int max_seq, int S,
                                          int key_len, int kvg, int window, int query_base_pos, int key_base_pos) {
    (void)nh;
#pragma omp parallel for schedule(dynamic)
    for (int row = 0; row < nkv * S * kvg; ++row) {
        int kvh = row / (S * kvg), r = row % (S * kvg), s = r / kvg, g = r % kvg;
        int h = kvh * kvg + g;
        size_t row0 = (size_t)kvh * max_seq;
        float *sc = scores + (size_t)row * key_len;
        int lo, hi;
        qk_row_int8(q_b + ((size_t)s * nkv * kvg + h) * l_hd, k_i8, k_scale, row0, key_len, l_hd, cache_hd, sc);
        prefix_bounds(s, key_len, window, query_base_pos, key_base_pos, &lo, &hi);
        softmax_row_masked(sc, key_len, lo, hi);
        pv_row_int8(sc, v_i8, v_scale, row0, key_len, l_hd, cache_hd, out + ((size_t)s * nkv * kvg + h) * l_hd);
    }
}

/* --------------------- A1/A2/A7/A8: fp32 and bf16-operand attention (cuBLAS) */

/* lib/attention_gpu.mojo:165-204 (fp32) and :207-248 (bf16 operands, fp32
 * accumulate, fp32 softmax, P narrowed to bf16).  kv_is_bf16 selects the cache
 * element type; for the bf16 route Q and P are narrowed as the reference's casts
 * do.  Accumulation order inside cuBLAS is unspecified; sequential fp32 here. */
ORC_API void orc_attn_decode_dense(const float *q, const void *k_cache, const void *v_cache, float *scores,
                                   float *out, int nh, int nkv, int l_hd, int cache_hd, int max_seq,
                                   int seq_len, int kvg, int kv_is_bf16) {
    (void)nkv;
    if (nh <= 0 || seq_len <= 0) return;
#pragma omp parallel for schedule(dynamic)
    for (int h = 0; h < nh; ++h) {
        size_t row0 = (size_t)(h / kvg) * max_seq;
        float *sc = scores + (size_t)h * seq_len;
        float qb[2048];
        for (int d = 0; d < l_hd; ++d) {
            float qv = q[(size_t)h * l_hd + d];
            qb[d] = kv_is_bf16 ? bf16_to_f32(f32_to_bf16(qv)) : qv;     /* Q narrowed once (lib/attention_gpu.mojo:230) */
        }
        for (int t = 0; t < seq_len; ++t) {
            float acc = 0.0f;
            size_t base = (row0 + t) * cache_hd;
            if (kv_is_bf16) { const uint16_t *kr = (const uint16_t *)k_cache + base; for (int d = 0; d < l_hd; ++d) acc += qb[d] * bf16_to_f32(kr[d]); }
            else { const float *kr = (const float *)k_cache + base; for (int d = 0; d < l_hd; ++d) acc += qb[d] * kr[d]; }
            sc[t] = acc;
        }
        softmax_row(sc, seq_len);
        float *o = out + (size_t)h * l_hd;
        for (int d = 0; d < l_hd; ++d) o[d] = 0.0f;
        for (int t = 0; t < seq_len; ++t) {                              /* per output element: keys in order */
            size_t base = (row0 + t) * cache_hd;
            float pt = kv_is_bf16 ? bf16_to_f32(f32_to_bf16(sc[t])) : sc[t];   /* P narrowed (:240) */
            if (kv_is_bf16) { const uint16_t *vr = (const uint16_t *)v_cache + base; for (int d = 0; d < l_hd; ++d) o[d] += pt * bf16_to_f32(vr[d]); }
            else { const float *vr = (const float *)v_cache + base; for (int d = 0; d < l_hd; ++d) o[d] += pt * vr[d]; }
        }
    }
}

/* lib/batched_attn_gpu.mojo:499-548 (fp32) / :613-666 (bf16); the square forms
 * (:448-496, :558-610) are key_len=S with both bases 0. */
ORC_API void orc_attn_prefix_batched_dense(const float *q_b, const void *k_cache, const void *v_cache,
                                           float *scores, float *out, int nh, int nkv, int l_hd, int cache_hd,
                                           int max_seq, int S, int key_len, int kvg, int window,
                                           int query_base_pos, int key_base_pos, int kv_is_bf16) {
    (void)nh;
#pragma omp parallel for schedule(dynamic)
    for (int row = 0; row < nkv * S * kvg; ++row) {
        int kvh = row / (S * kvg), r = row % (S * kvg), s = r / kvg, g = r % kvg;
        int h = kvh * kvg + g;
        size_t row0 = (size_t)kvh * max_seq;
        const float *qr = q_b + ((size_t)s * nkv * kvg + h) * l_hd;
        float *sc = scores + (size_t)row * key_len;
        int lo, hi;
        for (int t = 0; t < key_len; ++t) {
            float acc = 0.0f;
            for (int d = 0; d < l_hd; ++d) {
                size_t ki = (row0 + t) * cache_hd + d;
                if (kv_is_bf16) acc += bf16_to_f32(f32_to_bf16(qr[d])) * bf16_to_f32(((const uint16_t *)k_cache)[ki]);
                else acc += qr[d] * ((const float *)k_cache)[ki];
            }
            sc[t] = acc;
        }
        prefix_bounds(s, key_len, window, query_base_pos, key_base_pos, &lo, &hi);
        softmax_row_masked(sc, key_len, lo, hi);
        float *o = out + ((size_t)s * nkv * kvg + h) * l_hd;
        for (int d = 0; d < l_hd; ++d) {
            float acc = 0.0f;
            for (int t = 0; t < key_len; ++t) {
                size_t vi = (row0 + t) * cache_hd + d;
                if (kv_is_bf16) acc += bf16_to_f32(f32_to_bf16(sc[t])) * bf16_to_f32(((const uint16_t *)v_cache)[vi]);
                else acc += sc[t] * ((const float *)v_cache)[vi];
            }
            o[d] = acc;
        }
    }
}

/* ------------------------------------------------ the parity gate: O-exact */

/* Exact-dequant attention over the PACKED ring cache, double accumulation.
 *   kv_fmt 0: int8 + fp32 row scale        (lib/kv_cache_quant.mojo:248)
 *   kv_fmt 1: int4 + fp32 row scale        (:764)
 *   kv_fmt 2: int4 + fp16 scale per 32     (:799-800)
 * Row r of S attends absolute positions [lo_r, query_base_pos + r] with
 * lo_r = max(win_lo, query_base_pos + r - window + 1) when window > 0 else win_lo;
 * position p lives in ring slot p % cache_cap.  The score is multiplied by
 * softmax_scale before the softmax (1.0 reproduces the reference, which applies
 * none: lib/attention_gpu_int8.mojo:8-9).  q and out are [S, nh, l_hd].
 * If partial != NULL it receives per (row, head) the triple (m, l, o[l_hd])
 * un-normalised, laid out [S*nh, l_hd+2] = o.., m, l -- the quantity the
 * sequence-sharded multi-GPU merge exchanges. */
static inline double kv_elem(const void *cache, const void *scales, int kv_fmt, size_t row, int d,
                             int cache_hd, int nblocks) {
    if (kv_fmt == 0) return (double)((const int8_t *)cache)[row * cache_hd + d] * (double)((const float *)scales)[row];
    int q = i4_at((const uint8_t *)cache + row * (cache_hd / 2), d);
    if (kv_fmt == 1) return (double)q * (double)((const float *)scales)[row];
    return (double)q * (double)f16_to_f32(((const uint16_t *)scales)[row * nblocks + d / 32]);
}

ORC_API void orc_attn_exact(const float *q, const void *k_cache, const void *v_cache, const void *k_scales,
                            const void *v_scales, float *out, double *partial, int kv_fmt, int nh, int nkv,
                            int l_hd, int cache_hd, int cache_cap, int S, int kvg, int window,
                            int query_base_pos, int win_lo, double softmax_scale) {
    (void)nkv;
    int nblocks = (l_hd + 31) / 32;
#pragma omp parallel for schedule(dynamic)
    for (int rh = 0; rh < S * nh; ++rh) {
        int r = rh / nh, h = rh % nh, kvh = h / kvg;
        int apos = query_base_pos + r;
        int lo = win_lo;
        if (window > 0 && apos - window + 1 > lo) lo = apos - window + 1;
        int klen = apos + 1 - lo;
        float *o = out + (size_t)rh * l_hd;
        if (klen <= 0) { for (int d = 0; d < l_hd; ++d) o[d] = 0.0f; continue; }
        double *sc = (double *)malloc(sizeof(double) * (size_t)klen);
        double *acc = (double *)calloc((size_t)l_hd, sizeof(double));
        const float *qr = q + (size_t)rh * l_hd;
        double m = -INFINITY;
        for (int t = 0; t < klen; ++t) {
            size_t row = (size_t)kvh * cache_cap + (size_t)((lo + t) % cache_cap);
            double s = 0.0;
            for (int d = 0; d < l_hd; ++d) s += (double)qr[d] * kv_elem(k_cache, k_scales, kv_fmt, row, d, cache_hd, nblocks);
            sc[t] = s * softmax_scale;
            if (sc[t] > m) m = sc[t];
        }
        double l = 0.0;
        for (int t = 0; t < klen; ++t) {
            size_t row = (size_t)kvh * cache_cap + (size_t)((lo + t) % cache_cap);
            double p = exp(sc[t] - m);
            l += p;
            for (int d = 0; d < l_hd; ++d) acc[d] += p * kv_elem(v_cache, v_scales, kv_fmt, row, d, cache_hd, nblocks);
        }
        for (int d = 0; d < l_hd; ++d) o[d] = (float)(acc[d] / l);
        if (partial) {
            double *pp = partial + (size_t)rh * (l_hd + 2);
            for (int d = 0; d < l_hd; ++d) pp[d] = acc[d];
            pp[l_hd] = m; pp[l_hd + 1] = l;
        }
        free(sc); free(acc);
    }
}

/* Merge G partial triples per row into a normalised output: the associative
 * (m, l, o) combine the sequence-sharded path performs after its all-gather.
 * partials is [G, rows, l_hd+2]. */
ORC_API void orc_merge_partials(const double *partials, float *out, int G, int rows, int l_hd) {
    for (int r = 0; r < rows; ++r) {
        double m = -INFINITY;
        for (int g = 0; g < G; ++g) {
            const double *pp = partials + ((size_t)g * rows + r) * (l_hd + 2);
            if (pp[l_hd + 1] > 0.0 && pp[l_hd] > m) m = pp[l_hd];
        }
        double l = 0.0;
        for (int g = 0; g < G; ++g) {
            const double *pp = partials + ((size_t)g * rows + r) * (l_hd + 2);
            if (pp[l_hd + 1] > 0.0) l += exp(pp[l_hd] - m) * pp[l_hd + 1];
        }
        for (int d = 0; d < l_hd; ++d) {
            double a = 0.0;
            for (int g = 0; g < G; ++g) {
                const double *pp = partials + ((size_t)g * rows + r) * (l_hd + 2);
                if (pp[l_hd + 1] > 0.0) a += exp(pp[l_hd] - m) * pp[d];
            }
            out[(size_t)r * l_hd + d] = (l > 0.0) ? (float)(a / l) : 0.0f;
        }
    }
}

/* fp32 -> bf16 RNE on a buffer (lib/cast_gpu_mojo.mojo:16-27). */
ORC_API void orc_f32_to_bf16(const float *in, uint16_t *out, long n) {
    for (long i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}

ORC_API int orc_version(void) { return 1; }
