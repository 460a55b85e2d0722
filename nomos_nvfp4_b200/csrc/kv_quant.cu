// Quantize-on-write KV cache codecs and the window readers (sm_100a).
//
// One warp owns one (token, KV head) row, as in the reference, but several rows
// share a thread block and the int8/int4 row loops are unrolled over the row so
// the two reductions (K and V) overlap.  Every rounding step is spelled with an
// explicit round-to-nearest intrinsic so the bytes do not depend on the
// compiler's contraction choices; the file is also built with -fmad=false.
//
// Reference operators restated here (paths relative to the reference root):
//   lib/kv_cache_quant.mojo:43-131   standalone int8 codec
//   lib/kv_cache_quant.mojo:144-290  int8 append + window reader
//   lib/kv_cache_quant.mojo:311-689  int4 appends (row scale, block-32, q8 views)
//   lib/kv_cache_quant.mojo:708-989  int4 window readers
//   lib/attention_gpu.mojo:87-162, lib/batched_attn_gpu.mojo:55-102  fp32/bf16 appends
#include "common.cuh"
#include "kv_rows.cuh"
#include "launch.h"

namespace nomos {

constexpr int ROWS_PER_BLOCK = 4;   // warps per block in the append kernels

// ------------------------------------------------------------- int8 row codec

__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
quant_i8_rows_kernel(const __nv_bfloat16 *in, int8_t *out, float *scales, int n_rows, int dim) {
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    quant_row_i8(in + (size_t)r * dim, dim, dim, out + (size_t)r * dim, scales + r, threadIdx.x & 31);
}

__global__ void dequant_i8_rows_kernel(const int8_t *in, const float *scales, __nv_bfloat16 *out, long n, int dim) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) out[idx] = __float2bfloat16_rn(__fmul_rn((float)in[idx], scales[idx / dim]));
}

__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
append_i8_kernel(const float *src_k, const float *src_v, int8_t *dst_k, int8_t *dst_v, float *k_scales,
                 float *v_scales, int n_s, int nkv, int l_hd, int l_kvd, int cache_cap, int cache_hd, int base_pos) {
    const int w = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (w >= n_s * nkv) return;
    const int lane = threadIdx.x & 31;
    const int h = w % nkv, s = w / nkv;
    const size_t src = (size_t)s * l_kvd + (size_t)h * l_hd;
    const size_t row = (size_t)h * cache_cap + (size_t)((base_pos + s) % cache_cap);
    quant_row_i8(src_k + src, l_hd, cache_hd, dst_k + row * cache_hd, k_scales + row, lane);
    quant_row_i8(src_v + src, l_hd, cache_hd, dst_v + row * cache_hd, v_scales + row, lane);
}

// Paged int8 caches: one new row per sequence, at position positions[b] of sequence b, i.e. row
// positions[b] % 128 of page block_table[b][positions[b] / 128]; a page holds 128 rows of every KV head.
__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32)
append_paged_i8_kernel(const float *src_k, const float *src_v, int8_t *k_pool, int8_t *v_pool, float *ks_pool, float *vs_pool,
                       const int *block_table, const int *positions, int batch, int nkv, int l_hd, int l_kvd, int max_pages) {
    const int w = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (w >= batch * nkv) return;
    const int lane = threadIdx.x & 31;
    const int h = w % nkv, b = w / nkv;
    const int pos = positions[b];
    const int page = block_table[(size_t)b * max_pages + pos / 128];
    const size_t row = ((size_t)page * nkv + h) * 128 + (size_t)(pos % 128);
    const size_t src = (size_t)b * l_kvd + (size_t)h * l_hd;
    quant_row_i8(src_k + src, l_hd, l_hd, k_pool + row * l_hd, ks_pool + row, lane);
    quant_row_i8(src_v + src, l_hd, l_hd, v_pool + row * l_hd, vs_pool + row, lane);
}

// ------------------------------------------------------------- int4 row codecs

struct AppendI4Args {
    const float *src_k, *src_v;
    uint8_t *dst_k, *dst_v;
    void *k_scales, *v_scales;
    int8_t *k_q8, *v_q8;           // optional int8 views (nullptr = plain append)
    float *k_q8_scales, *v_q8_scales;
    int n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, q8_pitch, scale_blocks;
};

__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32) append_i4_kernel(AppendI4Args a) {
    const int w = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (w >= a.n_s * a.nkv) return;
    const int lane = threadIdx.x & 31;
    const int h = w % a.nkv, s = w / a.nkv;
    const int apos = a.base_pos + s;
    const size_t src = (size_t)s * a.l_kvd + (size_t)h * a.l_hd;
    const size_t row = (size_t)h * a.cache_cap + (size_t)(apos % a.cache_cap);
    const size_t vrow = (size_t)h * a.q8_pitch + (size_t)apos;
    const int hc = a.cache_hd / 2;
    const int nblocks = (a.l_hd + 31) / 32;
#pragma unroll
    for (int kv = 0; kv < 2; ++kv) {
        const float *x = (kv ? a.src_v : a.src_k) + src;
        uint8_t *dst = (kv ? a.dst_v : a.dst_k) + row * hc;
        void *scales = kv ? a.v_scales : a.k_scales;
        int8_t *view = kv ? a.v_q8 : a.k_q8;
        float *view_scale = kv ? a.v_q8_scales : a.k_q8_scales;
        if (a.scale_blocks > 1) {
            __half *s16 = reinterpret_cast<__half *>(scales) + row * nblocks;
            float *q8c = reinterpret_cast<float *>(reinterpret_cast<char *>(scales) + (size_t)a.nkv * a.cache_cap * nblocks * 2);
            const float q8s = quant_row_i4_block32(x, a.l_hd, dst, s16, lane);
            if (lane == 0) { q8c[row] = q8s; if (view) view_scale[vrow] = q8s; }
            if (view) {
                // Rebuild the int8 view from the bytes and fp16 scales just stored, the
                // way the block-32 -> q8 reader does later (multiply, then divide).
                __syncwarp();
                for (int d = lane; d < a.l_hd; d += 32) {
                    const int byte = dst[d >> 1];
                    const int q4 = nib_sext((d & 1) ? (byte >> 4) & 0xF : byte & 0xF);
                    const float sf = __half2float(s16[d >> 5]);
                    view[vrow * a.cache_hd + d] =
                        (int8_t)round_away_clamp(__fdiv_rn(__fmul_rn((float)q4, sf), q8s), 127);
                }
            }
        } else {
            const float sc = quant_row_i4(x, a.l_hd, a.cache_hd, dst, view ? view + vrow * a.cache_hd : nullptr, lane);
            if (lane == 0) { reinterpret_cast<float *>(scales)[row] = sc; if (view) view_scale[vrow] = sc; }
        }
    }
}

// ------------------------------------------------------------- window readers
// Linear window index j of head h reads ring row h*cache_cap + (win_start+j) % cache_cap
// and writes linear row h*pitch + j.  One thread converts 8 consecutive elements.

enum ReaderMode { RD_I8_BF16 = 0, RD_I4_BF16 = 1, RD_I4B32_BF16 = 2, RD_I4_Q8 = 3, RD_I4B32_Q8 = 4 };

template <int MODE>
__global__ void window_reader_kernel(const void *src, const void *scales, void *dst, float *dst_scale, int nkv, int klen,
                                     int cache_hd, int pitch, int cache_cap, int win_start, int scale_blocks) {
    const int groups = cache_hd / 8;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)nkv * klen * groups) return;
    const int gcol = (int)(idx % groups);
    const long t = idx / groups;
    const int j = (int)(t % klen), h = (int)(t / klen);
    const size_t sr = (size_t)h * cache_cap + (size_t)((win_start + j) % cache_cap);
    const size_t dr = (size_t)h * pitch + j;
    const int d0 = gcol * 8;
    int q[8];
    if constexpr (MODE == RD_I8_BF16) {
        const int2 w = *reinterpret_cast<const int2 *>(static_cast<const int8_t *>(src) + sr * cache_hd + d0);
#pragma unroll
        for (int i = 0; i < 4; ++i) { q[i] = (int8_t)(w.x >> (8 * i)); q[4 + i] = (int8_t)(w.y >> (8 * i)); }
    } else {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(src) + sr * (cache_hd / 2) + d0 / 2);
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = nib_sext((w >> (4 * i)) & 0xF);
    }
    const int nblocks = (cache_hd + 31) / 32;                 // the reader derives it from cache_hd
    float sc;
    if constexpr (MODE == RD_I4B32_BF16 || MODE == RD_I4B32_Q8)
        sc = __half2float(static_cast<const __half *>(scales)[sr * nblocks + d0 / 32]);
    else
        sc = static_cast<const float *>(scales)[sr];
    if constexpr (MODE == RD_I8_BF16 || MODE == RD_I4_BF16 || MODE == RD_I4B32_BF16) {
        __nv_bfloat16 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(__fmul_rn((float)q[i], sc));
        *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(dst) + dr * cache_hd + d0) = *reinterpret_cast<uint4 *>(o);
    } else {
        int8_t o[8];
        if constexpr (MODE == RD_I4_Q8) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (int8_t)q[i];
            if (gcol == 0) dst_scale[dr] = sc;
        } else {
            const float *q8c = reinterpret_cast<const float *>(static_cast<const char *>(scales) + (size_t)nkv * cache_cap * scale_blocks * 2);
            const float qs = q8c[sr];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = (int8_t)round_away_clamp(__fdiv_rn(__fmul_rn((float)q[i], sc), qs), 127);
            if (gcol == 0) dst_scale[dr] = qs;
        }
        *reinterpret_cast<int2 *>(static_cast<int8_t *>(dst) + dr * cache_hd + d0) = *reinterpret_cast<int2 *>(o);
    }
}

// ------------------------------------------------------- fp32 / bf16 appends

template <typename DstT>
__global__ void append_dense_kernel(const float *src_k, const float *src_v, DstT *dst_k, DstT *dst_v, int n_s, int nkv,
                                    int l_hd, int l_kvd, int max_seq, int cache_hd, int base_pos) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_s * nkv * l_hd) return;
    const int d = (int)(idx % l_hd);
    const long rem = idx / l_hd;
    const int h = (int)(rem % nkv), s = (int)(rem / nkv);
    const size_t so = (size_t)s * l_kvd + (size_t)h * l_hd + d;
    const size_t dofs = ((size_t)h * max_seq + (size_t)(base_pos + s)) * cache_hd + d;
    if constexpr (sizeof(DstT) == 2) {
        dst_k[dofs] = __float2bfloat16_rn(src_k[so]);
        dst_v[dofs] = __float2bfloat16_rn(src_v[so]);
    } else {
        dst_k[dofs] = src_k[so];
        dst_v[dofs] = src_v[so];
    }
}

// ------------------------------------------------------------------ launchers

static inline int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("%s: %s", what, cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}
static inline unsigned blocks_for(long n, int per) { return (unsigned)((n + per - 1) / per); }

int launch_quant_i8(cudaStream_t st, const void *in_bf16, void *out_i8, void *out_scales, int n_rows, int dim) {
    quant_i8_rows_kernel<<<blocks_for(n_rows, ROWS_PER_BLOCK), ROWS_PER_BLOCK * 32, 0, st>>>(
        static_cast<const __nv_bfloat16 *>(in_bf16), static_cast<int8_t *>(out_i8), static_cast<float *>(out_scales), n_rows, dim);
    return check_launch("nomos_kv_quant_i8");
}

int launch_dequant_i8(cudaStream_t st, const void *in_i8, const void *in_scales, void *out_bf16, int n_rows, int dim) {
    const long n = (long)n_rows * dim;
    dequant_i8_rows_kernel<<<blocks_for(n, 256), 256, 0, st>>>(static_cast<const int8_t *>(in_i8),
                                                                static_cast<const float *>(in_scales),
                                                                static_cast<__nv_bfloat16 *>(out_bf16), n, dim);
    return check_launch("nomos_kv_dequant_i8");
}

int launch_append_i8(cudaStream_t st, const void *src_k, const void *src_v, void *dst_k, void *dst_v, void *k_scales,
                     void *v_scales, int n_s, int nkv, int l_hd, int l_kvd, int cache_cap, int cache_hd, int base_pos) {
    append_i8_kernel<<<blocks_for((long)n_s * nkv, ROWS_PER_BLOCK), ROWS_PER_BLOCK * 32, 0, st>>>(
        static_cast<const float *>(src_k), static_cast<const float *>(src_v), static_cast<int8_t *>(dst_k),
        static_cast<int8_t *>(dst_v), static_cast<float *>(k_scales), static_cast<float *>(v_scales), n_s, nkv, l_hd, l_kvd,
        cache_cap, cache_hd, base_pos);
    return check_launch("nomos_kv_append_quant_i8");
}

int launch_append_paged_i8(cudaStream_t st, const void *src_k, const void *src_v, void *k_pool, void *v_pool, void *ks_pool,
                           void *vs_pool, const int *block_table, const int *positions, int batch, int nkv, int l_hd, int l_kvd,
                           int max_pages) {
    append_paged_i8_kernel<<<blocks_for((long)batch * nkv, ROWS_PER_BLOCK), ROWS_PER_BLOCK * 32, 0, st>>>(
        static_cast<const float *>(src_k), static_cast<const float *>(src_v), static_cast<int8_t *>(k_pool),
        static_cast<int8_t *>(v_pool), static_cast<float *>(ks_pool), static_cast<float *>(vs_pool), block_table, positions, batch,
        nkv, l_hd, l_kvd, max_pages);
    return check_launch("nomos_kv_paged_append_quant_i8");
}

int launch_append_i4(cudaStream_t st, const void *src_k, const void *src_v, void *dst_k, void *dst_v, void *k_scales,
                     void *v_scales, void *k_q8, void *v_q8, void *k_q8_scales, void *v_q8_scales, int n_s, int nkv,
                     int l_hd, int l_kvd, int cache_cap, int cache_hd, int base_pos, int q8_pitch, int scale_blocks) {
    AppendI4Args a;
    a.src_k = static_cast<const float *>(src_k); a.src_v = static_cast<const float *>(src_v);
    a.dst_k = static_cast<uint8_t *>(dst_k); a.dst_v = static_cast<uint8_t *>(dst_v);
    a.k_scales = k_scales; a.v_scales = v_scales;
    a.k_q8 = static_cast<int8_t *>(k_q8); a.v_q8 = static_cast<int8_t *>(v_q8);
    a.k_q8_scales = static_cast<float *>(k_q8_scales); a.v_q8_scales = static_cast<float *>(v_q8_scales);
    a.n_s = n_s; a.nkv = nkv; a.l_hd = l_hd; a.l_kvd = l_kvd; a.cache_cap = cache_cap; a.cache_hd = cache_hd;
    a.base_pos = base_pos; a.q8_pitch = q8_pitch; a.scale_blocks = scale_blocks;
    append_i4_kernel<<<blocks_for((long)n_s * nkv, ROWS_PER_BLOCK), ROWS_PER_BLOCK * 32, 0, st>>>(a);
    return check_launch("nomos_kv_append_quant_i4");
}

int launch_window_reader(cudaStream_t st, int mode, const void *src, const void *scales, void *dst, void *dst_scale, int nkv,
                         int klen, int cache_hd, int pitch, int cache_cap, int win_start, int scale_blocks) {
    const long n = (long)nkv * klen * (cache_hd / 8);
    const unsigned nb = blocks_for(n, 256);
    float *ds = static_cast<float *>(dst_scale);
#define NOMOS_RD(M) window_reader_kernel<M><<<nb, 256, 0, st>>>(src, scales, dst, ds, nkv, klen, cache_hd, pitch, cache_cap, win_start, scale_blocks)
    switch (mode) {
        case RD_I8_BF16: NOMOS_RD(RD_I8_BF16); break;
        case RD_I4_BF16: NOMOS_RD(RD_I4_BF16); break;
        case RD_I4B32_BF16: NOMOS_RD(RD_I4B32_BF16); break;
        case RD_I4_Q8: NOMOS_RD(RD_I4_Q8); break;
        case RD_I4B32_Q8: NOMOS_RD(RD_I4B32_Q8); break;
        default: set_error("window reader: bad mode %d", mode); return NOMOS_EBADARG;
    }
#undef NOMOS_RD
    return check_launch("nomos_kv_dequant_layer");
}

int launch_append_dense(cudaStream_t st, int dst_is_bf16, const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                        int n_s, int nkv, int l_hd, int l_kvd, int max_seq, int cache_hd, int base_pos) {
    const long n = (long)n_s * nkv * l_hd;
    if (dst_is_bf16)
        append_dense_kernel<__nv_bfloat16><<<blocks_for(n, 256), 256, 0, st>>>(
            static_cast<const float *>(src_k), static_cast<const float *>(src_v), static_cast<__nv_bfloat16 *>(dst_k),
            static_cast<__nv_bfloat16 *>(dst_v), n_s, nkv, l_hd, l_kvd, max_seq, cache_hd, base_pos);
    else
        append_dense_kernel<float><<<blocks_for(n, 256), 256, 0, st>>>(
            static_cast<const float *>(src_k), static_cast<const float *>(src_v), static_cast<float *>(dst_k),
            static_cast<float *>(dst_v), n_s, nkv, l_hd, l_kvd, max_seq, cache_hd, base_pos);
    return check_launch("nomos_kv_append_dense");
}

}  // namespace nomos
