// Attention over an UNQUANTISED (fp32 or bf16) KV cache: single-token GQA decode
// and the prefix-batched (verify / chunked-prefill) form, sm_100a.
//
// These are the legacy KV modes of the reference (two cuBLAS strided-batched GEMMs
// with a softmax kernel between them, scores materialised in HBM):
//   lib/attention_gpu.mojo:165-204 (fp32), :207-248 (bf16 operands)
//   lib/batched_attn_gpu.mojo:499-548 (fp32 prefix), :613-666 (bf16 prefix)
//   masks: lib/batched_attn_gpu.mojo:285-409
// Here they are one split-K streaming kernel (+ the shared merge): a warp takes
// whole key rows with 16-byte coalesced loads, keeps the GQA group's query rows in
// registers, and carries (m, l, o) online; nothing is written to HBM but the
// partials.  Arithmetic is fp32 on the stored values (bf16 widens exactly).
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"
#include "launch.h"

namespace nomos {
namespace {

constexpr int DW = 4;                 // warps per CTA
constexpr float LOG2E = 1.4426950408889634f;
constexpr float M_INIT = -1.0e30f;

struct DParams {
    const float *q;
    const uint8_t *k, *v;
    float *out, *partial;
    int write_partial;
    int S, nh, nkv, kvg, cache_hd, max_seq, key_len, window, query_base_pos, key_base_pos;
    int keys_per_split, grows;
};

template <typename T, int VEC>
__device__ __forceinline__ void load_row(const uint8_t *base, size_t elem_off, float (&x)[VEC]) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(base) + elem_off + i);
            x[i] = v.x; x[i + 1] = v.y; x[i + 2] = v.z; x[i + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const uint2 v = *reinterpret_cast<const uint2 *>(reinterpret_cast<const __nv_bfloat16 *>(base) + elem_off + i);
            x[i] = __uint_as_float(v.x << 16); x[i + 1] = __uint_as_float(v.x & 0xffff0000u);
            x[i + 2] = __uint_as_float(v.y << 16); x[i + 3] = __uint_as_float(v.y & 0xffff0000u);
        }
    }
}

// grid = (splits, nkv * subgroups, S); one CTA = one KV head, one query row and KVG of
// the group's query heads (a GQA group wider than KVG is covered by several CTAs).
template <typename T, int HD, int KVG>
__global__ void __launch_bounds__(DW * 32) attn_dense_kernel(const DParams p) {
    constexpr int VEC = HD / 32;
    __shared__ float mbuf[DW][KVG][HD + 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsub = p.kvg / KVG;
    const int split = blockIdx.x, kvh = blockIdx.y / nsub, sub = blockIdx.y % nsub, s = blockIdx.z;
    const int h0 = kvh * p.kvg + sub * KVG;

    // valid key range of row s (lib/batched_attn_gpu.mojo:314-326)
    const int q_abs = p.query_base_pos + s;
    int hi = min(q_abs - p.key_base_pos, p.key_len - 1);
    int lo = (p.window > 0 && q_abs - p.window + 1 > 0) ? q_abs - p.window + 1 : 0;
    lo = max(lo - p.key_base_pos, 0);

    float q[KVG][VEC];
#pragma unroll
    for (int j = 0; j < KVG; ++j)
#pragma unroll
        for (int i = 0; i < VEC; ++i)
            q[j][i] = p.q[((size_t)s * p.nh + h0 + j) * HD + lane * VEC + i] * LOG2E;

    float M[KVG], l[KVG], acc[KVG][VEC];
#pragma unroll
    for (int j = 0; j < KVG; ++j) {
        M[j] = M_INIT; l[j] = 0.0f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[j][i] = 0.0f;
    }

    const int k_begin = max(lo, split * p.keys_per_split);
    const int k_end = min(hi + 1, (split + 1) * p.keys_per_split);
    const size_t head_off = (size_t)kvh * p.max_seq * p.cache_hd;
    for (int key = k_begin + warp; key < k_end; key += DW) {
        float kx[VEC], vx[VEC];
        const size_t off = head_off + (size_t)key * p.cache_hd + lane * VEC;
        load_row<T, VEC>(p.k, off, kx);
        load_row<T, VEC>(p.v, off, vx);
        float sc[KVG];
#pragma unroll
        for (int j = 0; j < KVG; ++j) {
            float d = 0.0f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) d = fmaf(q[j][i], kx[i], d);
            sc[j] = d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int j = 0; j < KVG; ++j) sc[j] += __shfl_xor_sync(0xffffffffu, sc[j], o);
#pragma unroll
        for (int j = 0; j < KVG; ++j) {
            const float m_new = fmaxf(M[j], sc[j]);
            const float alpha = ex2f(M[j] - m_new);
            const float pe = ex2f(sc[j] - m_new);
            M[j] = m_new;
            l[j] = l[j] * alpha + pe;
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[j][i] = fmaf(pe, vx[i], acc[j][i] * alpha);
        }
    }

#pragma unroll
    for (int j = 0; j < KVG; ++j) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) mbuf[warp][j][lane * VEC + i] = acc[j][i];
        if (lane == 0) { mbuf[warp][j][HD] = M[j]; mbuf[warp][j][HD + 1] = l[j]; }
    }
    __syncthreads();
    for (int j = 0; j < KVG; ++j) {
        float mstar = M_INIT;
#pragma unroll
        for (int w = 0; w < DW; ++w) mstar = fmaxf(mstar, mbuf[w][j][HD]);
        float wgt[DW], lstar = 0.0f;
#pragma unroll
        for (int w = 0; w < DW; ++w) { wgt[w] = ex2f(mbuf[w][j][HD] - mstar); lstar += wgt[w] * mbuf[w][j][HD + 1]; }
        const long grow = (long)s * p.nh + h0 + j;
        for (int d = threadIdx.x; d < HD; d += DW * 32) {
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < DW; ++w) o += wgt[w] * mbuf[w][j][d];
            if (p.write_partial) p.partial[((size_t)split * p.grows + grow) * (HD + 2) + d] = o;
            else p.out[grow * HD + d] = lstar > 0.0f ? o / lstar : 0.0f;
        }
        if (p.write_partial && threadIdx.x == 0) {
            p.partial[((size_t)split * p.grows + grow) * (HD + 2) + HD] = mstar;
            p.partial[((size_t)split * p.grows + grow) * (HD + 2) + HD + 1] = lstar;
        }
    }
}

template <typename T, int HD, int KVG>
static int launch_dense_inst(cudaStream_t st, const DenseAttnArgs &a) {
    int sm = 148;
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
    const int grows = a.S * a.nh;
    const int units = a.nkv * (a.kvg / KVG) * a.S;
    int splits = std::max(1, (sm * 4) / std::max(1, units));
    splits = std::min(splits, std::max(1, a.key_len / (DW * 8)));
    const long per_split = (long)grows * (HD + 2) * 4;
    if (splits > 1 && per_split * splits > a.ws_bytes) splits = (int)std::max<long>(1, a.ws_bytes / per_split);
    const int kps = (a.key_len + splits - 1) / splits;
    splits = (a.key_len + kps - 1) / kps;
    DParams p;
    p.q = a.q; p.k = static_cast<const uint8_t *>(a.k_cache); p.v = static_cast<const uint8_t *>(a.v_cache);
    p.out = a.out; p.partial = static_cast<float *>(a.workspace); p.write_partial = splits > 1;
    p.S = a.S; p.nh = a.nh; p.nkv = a.nkv; p.kvg = a.kvg; p.cache_hd = a.cache_hd; p.max_seq = a.max_seq;
    p.key_len = a.key_len; p.window = a.window; p.query_base_pos = a.query_base_pos; p.key_base_pos = a.key_base_pos;
    p.keys_per_split = kps; p.grows = grows;
    attn_dense_kernel<T, HD, KVG><<<dim3(splits, a.nkv * (a.kvg / KVG), a.S), DW * 32, 0, st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("attn_dense launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    if (splits > 1) return launch_merge_partials_log2(st, static_cast<const float *>(a.workspace), splits, grows, HD, a.out);
    return NOMOS_OK;
}

template <typename T>
static int dispatch_dense(cudaStream_t st, const DenseAttnArgs &a) {
    // heads of one GQA group handled per CTA: 4 / 2 / 1, whichever divides kvg
#define NOMOS_DENSE(HD_)                                                              \
    if (a.l_hd == HD_) {                                                              \
        if (HD_ <= 256 && a.kvg % 4 == 0) return launch_dense_inst<T, HD_, 4>(st, a); \
        if (a.kvg % 2 == 0) return launch_dense_inst<T, HD_, 2>(st, a);               \
        return launch_dense_inst<T, HD_, 1>(st, a);                                   \
    }
    NOMOS_DENSE(128) NOMOS_DENSE(256) NOMOS_DENSE(512)
#undef NOMOS_DENSE
    set_error("dense attention: head_dim %d unsupported (128, 256, 512)", a.l_hd);
    return NOMOS_EUNSUPPORTED;
}

}  // namespace

int launch_attn_dense(cudaStream_t st, const DenseAttnArgs &a) {
    return a.kv_is_bf16 ? dispatch_dense<__nv_bfloat16>(st, a) : dispatch_dense<float>(st, a);
}

}  // namespace nomos
