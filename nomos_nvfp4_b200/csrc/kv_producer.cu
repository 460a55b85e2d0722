// K / V / Q producer epilogue fused with quantize-on-write (sm_100a).
//
// From the raw projection rows of the new tokens to cache bytes in ONE launch, where the
// reference runs five kernels and then the append (lib/gemma4_layer.mojo:326-340):
//   V: per-head RMSNorm without weight      lib/ops_gpu_mojo_reductions.mojo:353-417
//   K: per-head RMSNorm x shared weight     lib/ops_gpu_mojo_reductions.mojo:422-485
//      then RoPE                            lib/ops_gpu_mojo.mojo:310-368 (batched: 371 ff.)
//   Q: the same as K, written back in place (it stays fp32 for the attention call)
//   append: the row codecs of kv_rows.cuh, bit for bit those of the append kernels.
// One warp per (token, head) row: the row lives in registers (head_dim / 32 values per
// lane), is normalised and rotated there, staged in shared memory and handed to the
// row codec.  Latency-bound: a few KB per call.
#include "kv_rows.cuh"
#include "launch.h"

namespace nomos {

namespace {

constexpr int ROWS_PER_BLOCK = 4;
constexpr int MAX_HD = 512;
constexpr float EPS_RMSNORM = 1e-6f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(ROWS_PER_BLOCK * 32) kv_producer_kernel(ProducerArgs a) {
    __shared__ __align__(16) float rows[ROWS_PER_BLOCK][MAX_HD];
    // Programmatic dependent launch on both sides: wait for the stream predecessor (the projections that
    // wrote the source rows), then let the attention grid that follows be set up right away -- it blocks in
    // its own wait until this grid is done, but may already stream the cache rows declared settled.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w = blockIdx.x * ROWS_PER_BLOCK + wib;
    const int n_kv = a.n_s * a.nkv, n_q = a.q ? a.n_s * a.nh : 0;
    if (w >= 2 * n_kv + n_q) return;
    // row kind: 0 = K, 1 = V, 2 = Q
    const int kind = w < n_kv ? 0 : (w < 2 * n_kv ? 1 : 2);
    const int r = kind == 0 ? w : (kind == 1 ? w - n_kv : w - 2 * n_kv);
    const int heads = kind == 2 ? a.nh : a.nkv;
    const int s = r / heads, h = r - s * heads;
    const int hd = a.l_hd;
    float *q_row = kind == 2 ? a.q + ((size_t)s * a.nh + h) * hd : nullptr;
    const float *src = kind == 2 ? q_row : (kind == 0 ? a.src_k : a.src_v) + (size_t)s * a.l_kvd + (size_t)h * hd;
    const float *wv = kind == 0 ? a.k_norm_w : (kind == 2 ? a.q_norm_w : nullptr);
    float *row = rows[wib];

    // ---- RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) (* w[j])
    float sq = 0.0f;
    for (int j = lane; j < hd; j += 32) {
        const float x = src[j];
        row[j] = x;
        sq = fmaf(x, x, sq);
    }
    sq = warp_sum(sq);
    const float inv = 1.0f / sqrtf(sq / (float)hd + EPS_RMSNORM);
    __syncwarp();
    for (int j = lane; j < hd; j += 32) row[j] = wv ? row[j] * inv * wv[j] : row[j] * inv;
    __syncwarp();

    // ---- RoPE on K and Q rows: pairs (i, i + hd/2), i < rope_dim/2, frequency denominator hd.
    // The reference keys ln(theta) on equality with 1e6 and otherwise uses ln(10000).
    if (kind != 1 && a.rope_dim > 0) {
        const float ln_theta = a.theta == 1000000.0f ? 13.81551056f : 9.21034037f;
        const float pos = (float)(a.base_pos + s);
        const int half = hd / 2;
        for (int i = lane; i < a.rope_dim / 2; i += 32) {
            const float exponent = (2.0f * (float)i) / (float)hd;
            const float inv_freq = expf(-exponent * ln_theta);
            const float angle = pos * inv_freq;
            float sn, cs;
            sincosf(angle, &sn, &cs);
            const float x0 = row[i], x1 = row[i + half];
            row[i] = x0 * cs - x1 * sn;
            row[i + half] = x0 * sn + x1 * cs;
        }
        __syncwarp();
    }

    if (kind == 2) {
        for (int j = lane; j < hd; j += 32) q_row[j] = row[j];
        return;
    }
    // ---- optional copy of the values that get quantised, then the row codec
    float *vals = kind == 0 ? a.k_out : a.v_out;
    if (vals) {
        float *o = vals + ((size_t)s * a.nkv + h) * hd;
        for (int j = lane; j < hd; j += 32) o[j] = row[j];
    }
    if (a.kv_fmt < 0) return;
    const size_t crow = (size_t)h * a.cache_cap + (size_t)((a.base_pos + s) % a.cache_cap);
    uint8_t *dst = kind == 0 ? a.dst_k : a.dst_v;
    uint8_t *sc = kind == 0 ? a.k_scales : a.v_scales;
    if (a.kv_fmt == KV_I8) {
        quant_row_i8(row, hd, a.cache_hd, reinterpret_cast<int8_t *>(dst) + crow * a.cache_hd, reinterpret_cast<float *>(sc) + crow, lane);
    } else if (a.kv_fmt == KV_I4) {
        const float scale = quant_row_i4(row, hd, a.cache_hd, dst + crow * (a.cache_hd / 2), nullptr, lane);
        if (lane == 0) reinterpret_cast<float *>(sc)[crow] = scale;
    } else {
        const int nblocks = (hd + 31) / 32;
        const float q8s = quant_row_i4_block32(row, hd, dst + crow * (a.cache_hd / 2), reinterpret_cast<__half *>(sc) + crow * nblocks, lane);
        if (lane == 0) reinterpret_cast<float *>(sc + (size_t)a.nkv * a.cache_cap * nblocks * 2)[crow] = q8s;
    }
}

}  // namespace

int launch_kv_producer(cudaStream_t st, const ProducerArgs &a) {
    const long rows = 2L * a.n_s * a.nkv + (a.q ? (long)a.n_s * a.nh : 0);
    const unsigned blocks = (unsigned)((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(ROWS_PER_BLOCK * 32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cfg.attrs = pdl; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kv_producer_kernel, a);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("nomos_kv_norm_rope_append launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

}  // namespace nomos
