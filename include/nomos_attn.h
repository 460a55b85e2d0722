/*
 * nomos_attn.h -- C ABI of libnomos_attn.so: B200 (sm_100a) quantized-KV attention
 * for the Nomos kernel (lightofbaldr/nomos-nvfp4).
 *
 * The library is a drop-in for ONE path of the reference: the KV-cache
 * quantize-on-write codecs, the single-token GQA decode attention and the
 * multi-row speculative-verify attention.  Each "thin" entry point keeps the
 * argument order of the internal Mojo operator it replaces (cited per function,
 * paths relative to the reference root); the DeviceContext argument becomes a
 * `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *
 * Conventions (those of the reference's own C ABI, nomos_ffi.mojo:18-23):
 *   - every device pointer is a uint64_t address, every dimension an int32_t;
 *   - the return value is an int32_t status: 0 ok, negative = error;
 *   - calls are asynchronous on `stream`; the library never synchronises,
 *     never allocates device memory and never touches another stream;
 *   - the caller owns every buffer, including scratch/workspace;
 *   - early-return no-ops follow the reference (nh <= 0 or seq_len <= 0 -> 0).
 *
 * Status codes:
 *    0  NOMOS_ATTN_OK
 *   -1  bad argument (null pointer, non-positive dimension, misalignment,
 *       nh != nkv*kvg, window longer than the ring, ...)
 *   -2  unsupported configuration (head_dim other than 128/256/512, ...)
 *   -3  capacity (workspace too small, position beyond a linear cache)
 *   -4  output not produced
 *  -99  CUDA runtime error reported by the launch
 * nomos_attn_last_error() returns a thread-local message for the last failure.
 *
 * Alignment: cache rows, scale buffers and Q/out rows must be 16-byte aligned;
 * cache_hd must be a multiple of 16 (int8) or 32 (int4) elements.
 */
#ifndef NOMOS_ATTN_H
#define NOMOS_ATTN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NOMOS_ATTN_OK 0
#define NOMOS_ATTN_EBADARG (-1)
#define NOMOS_ATTN_EUNSUPPORTED (-2)
#define NOMOS_ATTN_ECAPACITY (-3)
#define NOMOS_ATTN_ENOTWRITTEN (-4)
#define NOMOS_ATTN_ECUDA (-99)

/* KV cache formats of the fused entry points */
#define NOMOS_KV_I8 0     /* int8 rows + one fp32 scale per (head, slot)              */
#define NOMOS_KV_I4 1     /* packed int4 rows + one fp32 scale per (head, slot)       */
#define NOMOS_KV_I4B32 2  /* packed int4 rows + one fp16 scale per 32 values, followed
                             by one cached fp32 "q8" scale per (head, slot)           */
/* element types of Q and of the output */
#define NOMOS_F32 0
#define NOMOS_BF16 1

/* Library version (cf. nomos_version, nomos_ffi.mojo:117-120). */
int32_t nomos_attn_version(void);
/* Message describing the last non-zero status returned on this thread. */
const char *nomos_attn_last_error(void);
/* Device-side fault bits of the current device, accumulated since the last clearing read.
 * The kernels never wait without a limit; a wait that ran out ORs a bit in here and the
 * launch carries on (its output is then undefined).  Bit 0: a tile requested from the cache
 * did not arrive within about two seconds (mma.sync kernel).  Bit 1: a hand-off between the
 * roles of the tcgen05 kernel (copy engine, tensor core, softmax warps) ran out of time.
 * Bit 2: a peer GPU's partial result did not arrive (nomos_attn_seq_sharded_*).  After a
 * fault the split workspace of the call may hold arrival counts of the unfinished launch:
 * zero it (cudaMemsetAsync) before using it again.  Synchronises the device; a health check
 * between steps, not a per-call status.  `clear` != 0 resets the word after reading.
 * No counterpart in the reference (its kernels have no waits). */
int32_t nomos_attn_device_faults(uint32_t *out_bits, int32_t clear);

/* ------------------------------------------------------------------------- *
 *  KV cache codecs (thin, call-for-call)                                     *
 * ------------------------------------------------------------------------- */

/* gpu_quant_kv_i8, lib/kv_cache_quant.mojo:100-113: bf16 [n_rows, dim] -> int8 +
 * fp32 row scale (amax/127, 0 -> 1). */
int32_t nomos_kv_quant_i8(void *stream, uint64_t in_bf16, uint64_t out_i8, uint64_t out_scales,
                          int32_t n_rows, int32_t dim);

/* gpu_dequant_kv_i8, lib/kv_cache_quant.mojo:116-131. */
int32_t nomos_kv_dequant_i8(void *stream, uint64_t in_i8, uint64_t in_scales, uint64_t out_bf16,
                            int32_t n_rows, int32_t dim);

/* gpu_append_quant_kv_i8, lib/kv_cache_quant.mojo:252-271: quantize n_s new
 * tokens' K/V (fp32 [n_s, nkv, l_hd], token stride l_kvd) into ring slots
 * (base_pos + s) % cache_cap of the int8 cache [nkv, cache_cap, cache_hd]. */
int32_t nomos_kv_append_quant_i8(void *stream, uint64_t src_k, uint64_t src_v,
                                 uint64_t dst_k_i8, uint64_t dst_v_i8, uint64_t k_scales, uint64_t v_scales,
                                 int32_t n_s, int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap,
                                 int32_t cache_hd, int32_t base_pos);

/* gpu_dequant_kv_i8_layer, lib/kv_cache_quant.mojo:274-290: ring window
 * [win_start, win_start+klen) -> linear bf16 scratch [nkv, max_seq, cache_hd]. */
int32_t nomos_kv_dequant_i8_layer(void *stream, uint64_t src_i8, uint64_t scales, uint64_t dst_bf16,
                                  int32_t nkv, int32_t klen, int32_t cache_hd, int32_t max_seq,
                                  int32_t cache_cap, int32_t win_start);

/* gpu_append_quant_kv_i4, lib/kv_cache_quant.mojo:803-836.  scale_blocks == 1:
 * one fp32 scale per row (amax/7); scale_blocks > 1: block-32 layout, the scale
 * buffer holds [nkv, cache_cap, nblocks] fp16 then [nkv, cache_cap] fp32. */
int32_t nomos_kv_append_quant_i4(void *stream, uint64_t src_k, uint64_t src_v,
                                 uint64_t dst_k_i4, uint64_t dst_v_i4, uint64_t k_scales, uint64_t v_scales,
                                 int32_t n_s, int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap,
                                 int32_t cache_hd, int32_t base_pos, int32_t scale_blocks);

/* gpu_append_quant_kv_i4_with_q8, lib/kv_cache_quant.mojo:839-882: as above and
 * publishes each row as int8 at ABSOLUTE row h*q8_pitch + base_pos + s of a linear
 * view [nkv, q8_pitch, cache_hd] with its fp32 scale [nkv, q8_pitch]. */
int32_t nomos_kv_append_quant_i4_with_q8(void *stream, uint64_t src_k, uint64_t src_v,
                                         uint64_t dst_k_i4, uint64_t dst_v_i4, uint64_t k_scales, uint64_t v_scales,
                                         uint64_t dst_k_q8, uint64_t dst_v_q8, uint64_t k_q8_scales, uint64_t v_q8_scales,
                                         int32_t n_s, int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap,
                                         int32_t cache_hd, int32_t base_pos, int32_t q8_pitch, int32_t scale_blocks);

/* gpu_dequant_kv_i4_layer, lib/kv_cache_quant.mojo:885-918: int4 ring window ->
 * linear bf16 scratch (row-scale or block-32). */
int32_t nomos_kv_dequant_i4_layer(void *stream, uint64_t src_i4, uint64_t scales, uint64_t dst_bf16,
                                  int32_t nkv, int32_t klen, int32_t cache_hd, int32_t max_seq,
                                  int32_t cache_cap, int32_t win_start, int32_t scale_blocks);

/* gpu_dequant_kv_i4_to_q8_layer, lib/kv_cache_quant.mojo:956-989: int4 ring window
 * -> linear int8 scratch + linear fp32 row scales. */
int32_t nomos_kv_dequant_i4_to_q8_layer(void *stream, uint64_t src_i4, uint64_t scales, uint64_t dst_i8,
                                        uint64_t dst_scale, int32_t nkv, int32_t klen, int32_t cache_hd,
                                        int32_t max_seq, int32_t cache_cap, int32_t win_start, int32_t scale_blocks);

/* append_kv_gpu_dev / append_kv_gpu_dev_async, lib/attention_gpu.mojo:87-133:
 * one token's fp32 K,V [nkv, l_hd] -> fp32 cache [nkv, max_seq, cache_hd] at cl. */
int32_t nomos_kv_append_fp32(void *stream, uint64_t k_cache, uint64_t v_cache, uint64_t k_new, uint64_t v_new,
                             int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t cl);

/* append_kv_gpu_bf16_dev, lib/attention_gpu.mojo:136-162: same into a bf16 cache
 * (the two bf16 scratch arguments of the reference are accepted and unused). */
int32_t nomos_kv_append_bf16(void *stream, uint64_t k_cache, uint64_t v_cache, uint64_t k_new, uint64_t v_new,
                             uint64_t k_bf16_scratch, uint64_t v_bf16_scratch,
                             int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t cl);

/* gpu_append_kv_batched_bf16, lib/batched_attn_gpu.mojo:87-102. */
int32_t nomos_kv_append_batched_bf16(void *stream, uint64_t src_k, uint64_t src_v, uint64_t dst_k, uint64_t dst_v,
                                     int32_t n_s, int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t max_seq,
                                     int32_t cache_hd, int32_t base_pos);

/* ------------------------------------------------------------------------- *
 *  Attention (thin, call-for-call)                                           *
 * ------------------------------------------------------------------------- *
 * In all of these `max_seq` is the row pitch per head of the K/V/scale arrays
 * handed in (the caller may pre-offset the base pointers), `seq_len` counts keys
 * from that base, and no softmax scale or softcap is applied
 * (lib/attention_gpu_int8.mojo:8-9).  Q and the output are fp32.  The scratch
 * arguments keep the reference's sizes and are used only as split-K workspace.
 */

/* attention_gpu_int8_dev, lib/attention_gpu_int8.mojo:598-631.
 * scores_scratch: >= nh*seq_len floats. */
int32_t nomos_attn_decode_i8(void *stream, uint64_t q, uint64_t k_i8, uint64_t v_i8, uint64_t k_scale,
                             uint64_t v_scale, uint64_t scores_scratch, uint64_t out,
                             int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                             int32_t seq_len, int32_t kvg);

/* attention_decode_order_multirow_int8, lib/attention_gpu_int8.mojo:634-708:
 * S query rows [S, nh, l_hd]; row r attends absolute keys
 * [max(0, apos-window+1) if window>0 else 0, apos], apos = query_base_pos + r.
 * scores: >= S*nh*score_stride floats. */
int32_t nomos_attn_decode_multirow_i8(void *stream, uint64_t q_b, uint64_t scores, uint64_t attn_b,
                                      uint64_t k_i8, uint64_t v_i8, uint64_t k_scale, uint64_t v_scale,
                                      int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                      int32_t S, int32_t score_stride, int32_t kvg, int32_t window,
                                      int32_t query_base_pos);

/* attention_prefill_prefix_batched_int8, lib/attention_gpu_int8.mojo:844-887.
 * q_t / attn_t are the reference's transpose scratches (accepted, unused).  K / V / scale
 * pointers may be pre-offset by key_base_pos rows, exactly as the engine passes them on
 * sliding layers (lib/engine_prefill.mojo:926-941): key t of the arrays is absolute position
 * key_base_pos + t, row s attends [max(0, q_abs-window+1) - key_base_pos, q_abs - key_base_pos]
 * clipped to [0, key_len), q_abs = query_base_pos + s. */
int32_t nomos_attn_prefix_batched_i8(void *stream, uint64_t q_b, uint64_t q_t, uint64_t scores, uint64_t attn_t,
                                     uint64_t attn_b, uint64_t k_i8, uint64_t v_i8, uint64_t k_scale, uint64_t v_scale,
                                     int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                     int32_t S, int32_t key_len, int32_t kvg, int32_t window,
                                     int32_t query_base_pos, int32_t key_base_pos);

/* attention_prefill_batched_int8, lib/attention_gpu_int8.mojo:804-841: the square causal
 * prefill (S query rows over the S keys at positions 0..S-1), without its [nkv, S*kvg, S]
 * score matrix. */
int32_t nomos_attn_prefill_batched_i8(void *stream, uint64_t q_b, uint64_t q_t, uint64_t scores, uint64_t attn_t,
                                      uint64_t attn_b, uint64_t k_i8, uint64_t v_i8, uint64_t k_scale, uint64_t v_scale,
                                      int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                      int32_t S, int32_t kvg, int32_t window);

/* attention_gpu_fp32_dev, lib/attention_gpu.mojo:165-204 (cuBLAS handle dropped). */
int32_t nomos_attn_decode_fp32(void *stream, uint64_t q, uint64_t k_cache, uint64_t v_cache, uint64_t scores_scratch,
                               uint64_t out, int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd,
                               int32_t max_seq, int32_t seq_len, int32_t kvg);

/* attention_gpu_bf16_dev, lib/attention_gpu.mojo:207-248 (q_bf16 / scores_bf16
 * scratches accepted, unused). */
int32_t nomos_attn_decode_bf16(void *stream, uint64_t q, uint64_t k_cache, uint64_t v_cache, uint64_t scores_scratch,
                               uint64_t q_bf16, uint64_t scores_bf16, uint64_t out,
                               int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                               int32_t seq_len, int32_t kvg);

/* attention_prefill_prefix_batched_fp32, lib/batched_attn_gpu.mojo:499-548 (cuBLAS handle
 * dropped; q_t / attn_t transpose scratches accepted, unused). */
int32_t nomos_attn_prefix_batched_fp32(void *stream, uint64_t q_b, uint64_t q_t, uint64_t scores, uint64_t attn_t,
                                       uint64_t attn_b, uint64_t k_cache, uint64_t v_cache,
                                       int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                       int32_t S, int32_t key_len, int32_t kvg, int32_t window,
                                       int32_t query_base_pos, int32_t key_base_pos);
/* attention_prefill_prefix_batched_bf16, lib/batched_attn_gpu.mojo:613-666 (bf16 caches; the
 * q_t, q_t_bf16, scores_bf16 and attn_t scratches are accepted, unused). */
int32_t nomos_attn_prefix_batched_bf16(void *stream, uint64_t q_b, uint64_t q_t, uint64_t q_t_bf16, uint64_t scores,
                                       uint64_t scores_bf16, uint64_t attn_t, uint64_t attn_b, uint64_t k_cache,
                                       uint64_t v_cache, int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd,
                                       int32_t max_seq, int32_t S, int32_t key_len, int32_t kvg, int32_t window,
                                       int32_t query_base_pos, int32_t key_base_pos);
/* attention_prefill_batched_fp32 / _bf16, lib/batched_attn_gpu.mojo:448-496, 558-610: the
 * square causal forms (key_len = S, both bases 0). */
int32_t nomos_attn_prefill_batched_fp32(void *stream, uint64_t q_b, uint64_t q_t, uint64_t scores, uint64_t attn_t,
                                        uint64_t attn_b, uint64_t k_cache, uint64_t v_cache,
                                        int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                        int32_t S, int32_t kvg, int32_t window);
int32_t nomos_attn_prefill_batched_bf16(void *stream, uint64_t q_b, uint64_t q_t, uint64_t q_t_bf16, uint64_t scores,
                                        uint64_t scores_bf16, uint64_t attn_t, uint64_t attn_b, uint64_t k_cache,
                                        uint64_t v_cache, int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd,
                                        int32_t max_seq, int32_t S, int32_t kvg, int32_t window);
/* The shared body of the four operators above; kv_is_bf16 selects the cache element type. */
int32_t nomos_attn_prefix_batched_dense(void *stream, uint64_t q_b, uint64_t scores, uint64_t attn_b,
                                        uint64_t k_cache, uint64_t v_cache,
                                        int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                        int32_t S, int32_t key_len, int32_t kvg, int32_t window,
                                        int32_t query_base_pos, int32_t key_base_pos, int32_t kv_is_bf16);

/* ------------------------------------------------------------------------- *
 *  Fused superset: attention straight off the packed ring cache              *
 * ------------------------------------------------------------------------- *
 * One call = (optional) quantize-on-write of the new rows + attention of S query
 * rows over the window, with no dequant scratch and no score matrix.  It stands
 * for the reference's per-layer sequence append -> window reader -> attention
 * (lib/engine_decode.mojo:356-389, 445-460, 527-554; verify:
 * lib/engine_prefill.mojo:547-726).
 *
 * All fields are 8 bytes wide so a caller without C structs can fill an int64
 * array.  Zero-initialise, then set what you need.
 */
typedef struct nomos_attn_args {
    uint64_t struct_bytes;      /* sizeof(nomos_attn_args_t), for versioning              */
    uint64_t q;                 /* [batch][S][nh][l_hd], q_type                           */
    uint64_t k_cache, v_cache;  /* [batch][nkv][cache_cap][cache_hd] int8, or /2 bytes int4*/
    uint64_t k_scales, v_scales;/* per kv_fmt, see NOMOS_KV_*                             */
    uint64_t out;               /* [batch][S][nh][l_hd], out_type (may be 0 if partial_out)*/
    uint64_t partial_out;       /* 0, or fp32 [batch][S][nh][l_hd+2] = un-normalised o,
                                   then m (natural log), then l: for cross-GPU merging;
                                   a call that sets it does not write `out`                */
    uint64_t workspace;         /* split-K scratch                                        */
    int64_t ws_bytes;           /* >= nomos_attn_workspace_bytes(args)                     */
    uint64_t new_k, new_v;      /* 0, or fp32 [batch][n_new][nkv][l_hd] rows to quantize+append */
    int64_t n_new, new_stride;  /* rows, and elements between consecutive rows            */
    int64_t new_base_pos;       /* absolute position of the first new row                 */
    int64_t kv_fmt, q_type, out_type;
    int64_t batch, S, nh, nkv, kvg, l_hd, cache_hd, cache_cap;
    int64_t win_start;          /* absolute position of the first attended key            */
    int64_t klen;               /* attended keys INCLUDING the new rows; the S query rows
                                   are the last S keys, causal among themselves           */
    int64_t window;             /* per-row sliding window (0 = none)                      */
    double softmax_scale;       /* multiplies QK before the softmax; 1.0 = the reference  */
    int64_t q_batch_stride, out_batch_stride;      /* elements; 0 = dense                 */
    int64_t kv_batch_stride, scale_batch_stride;   /* bytes;    0 = dense                 */
    int64_t force_splits;       /* 0 = library chooses the sequence split                 */
    int64_t flags;              /* NOMOS_ATTN_* bits below                                */
} nomos_attn_args_t;

/* flags bit: the caller guarantees that every cache row (and scale) older than the newest
 * 2 * max(S, n_new) keys of the window was written by work that completed before the kernel
 * immediately preceding this call in the stream was launched.  True for a decode / verify
 * loop: the preceding kernel is either the append of this call's own rows or the previous
 * step's attention call with its fused append, and both only touch rows inside that margin
 * (a verify step that kept a of its VB rows is followed by a step whose rows start a
 * positions later).  The library may then start streaming the older rows while that
 * preceding kernel is still finishing (the query, the newest rows and every output are still
 * ordered after it).  Do not set it when the preceding kernel may have written older rows of
 * this cache (a prefill chunk, a KV-reuse copy). */
#define NOMOS_ATTN_SETTLED_CACHE 1
/* flags bit: fetch every tile with 16-byte cp.async copies instead of TMA tensor copies.
 * Same results bit for bit; for comparing the two copy paths. */
#define NOMOS_ATTN_NO_TMA 2
/* flags bit: keep int8 / head_dim 128 calls on the mma.sync kernel instead of the tcgen05 one
 * (both pass the same accuracy gate; their roundings differ). */
#define NOMOS_ATTN_NO_TCGEN05 4
/* flags bit: take the tcgen05 kernel for every call it supports, also where the library's
 * own choice would be the mma.sync kernel (for comparing the two). */
#define NOMOS_ATTN_TCGEN05_ALWAYS 8
/* flags bit: never run the splits of a KV head as a thread-block cluster (the mma.sync kernel then merges
 * them through the workspace and an arrival counter, as it does whenever a cluster does not fit; same
 * results; for comparing the two). */
#define NOMOS_ATTN_NO_CLUSTER 16

/* K / V / Q producer epilogue fused with the quantising append: from the raw projection rows of
 * n_s new tokens to cache bytes in one launch.  Replaces the sequence of lib/gemma4_layer.mojo:326-340
 *   gpu_rmsnorm_no_weight_mojo(v)           lib/ops_gpu_mojo_reductions.mojo:353-417
 *   gpu_qk_norm_mojo(q), gpu_qk_norm_mojo(k)  lib/ops_gpu_mojo_reductions.mojo:422-485
 *   gpu_rope_mojo(q), gpu_rope_mojo(k)      lib/ops_gpu_mojo.mojo:310-368 (token s at base_pos + s as in
 *                                           the batched kernel, :371 ff.)
 * followed by gpu_append_quant_kv_i8 / _i4 (lib/kv_cache_quant.mojo:252, :803).
 *   q        [n_s, nh, l_hd] fp32, normalised and rotated IN PLACE (0 = no query rows)
 *   src_k/v  [n_s, nkv, l_hd] fp32 with token stride l_kvd, not modified
 *   *_norm_w [l_hd] fp32 weights of the Q / K norms (V has none)
 *   k_out/v_out optional [n_s, nkv, l_hd] fp32: the rows exactly as they were quantised (0 = none)
 *   theta, rope_dim: pairs (i, i + l_hd/2) for i < rope_dim/2 rotate by (base_pos + s) *
 *     exp(-(2 i / l_hd) * ln theta); like the reference, ln theta is ln(1e6) when theta == 1e6 and
 *     ln(1e4) for every other value.  rope_dim = l_hd on sliding layers, l_hd / 4 on full layers.
 *   kv_fmt: NOMOS_KV_I8 / _I4 / _I4B32 select the cache layout (block-32: one scale block per 32
 *     values and the cached q8 row scale, as nomos_kv_append_quant_i4 with scale_blocks > 1);
 *     negative = no cache write (norm + rope only).
 * The cache bytes and scales are those the append entry points produce from k_out / v_out, bit for
 * bit; the normalised values themselves agree with the reference's float32 kernels to rounding. */
int32_t nomos_kv_norm_rope_append(void *stream, uint64_t q, uint64_t q_norm_w, uint64_t src_k, uint64_t src_v,
                                   uint64_t k_norm_w, uint64_t dst_k, uint64_t dst_v, uint64_t k_scales,
                                   uint64_t v_scales, uint64_t k_out, uint64_t v_out, int32_t n_s, int32_t nh,
                                   int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap, int32_t cache_hd,
                                   int32_t base_pos, float theta, int32_t rope_dim, int32_t kv_fmt);

/* ------------------------------------------------------------------------- *
 *  Ring bookkeeping (host only, no device work)                              *
 * ------------------------------------------------------------------------- *
 * One layer's lengths and window arithmetic, which the reference keeps in its engine loops
 * (lib/engine_decode.mojo:420-444: win_start / klen / lo; lib/gemma4_engine.mojo:897-901:
 * set_cache_len for KV reuse and for the roll-back after a verify pass).  The reference refuses
 * verify, offset prefill and chunked appends on its sliding-window ring (lib/engine_prefill.mojo:87-88,
 * lib/engine_decode.mojo:158-176) because a ring of exactly W slots lets a batch overwrite keys its
 * own earlier rows still need.  A ring with max_rows - 1 slots of slack does not have that problem:
 * nomos_kv_ring_init insists on cache_cap >= window + max_rows - 1. */
typedef struct nomos_kv_ring {
    int64_t struct_bytes;       /* sizeof(nomos_kv_ring_t), set by nomos_kv_ring_init            */
    int64_t cache_cap;          /* slots per KV head                                             */
    int64_t window;             /* sliding window W; 0 = linear cache (full attention)           */
    int64_t max_rows;           /* most rows one call appends (1 = decode only, VB = verify)     */
    int64_t len;                /* committed positions [0, len)                                  */
    int64_t staged;             /* rows the last plan placed at len .. len+staged-1, uncommitted */
    int64_t high;               /* one past the highest position ever written                    */
} nomos_kv_ring_t;

typedef struct nomos_kv_step {
    int64_t base_pos;           /* position of the first new row = append base = query_base_pos  */
    int64_t n_new;              /* rows of this call (S of the attention call)                   */
    int64_t win_start;          /* absolute position of window index 0                           */
    int64_t klen;               /* keys in the window, the new rows included                     */
    int64_t window;             /* per-row sliding window to pass on (0 = none)                  */
} nomos_kv_step_t;

int32_t nomos_kv_ring_init(nomos_kv_ring_t *ring, int64_t cache_cap, int64_t window, int64_t max_rows);
/* Places n_new rows at positions len .. len+n_new-1 and works out the attention window of the call
 * that appends and reads them (decode: n_new = 1; verify: n_new = VB).  -3 when a linear cache would
 * overflow (the reference's capacity guard, lib/engine_decode.mojo:166-188) or n_new > max_rows. */
int32_t nomos_kv_ring_plan(nomos_kv_ring_t *ring, int64_t n_new, nomos_kv_step_t *step);
/* Keeps the first `accepted` of the staged rows (len += accepted); the rest is overwritten later. */
int32_t nomos_kv_ring_commit(nomos_kv_ring_t *ring, int64_t accepted);
/* set_cache_len: truncate to n <= len committed positions (KV reuse).  On a ring, -3 if the rows the
 * next step needs have already been overwritten. */
int32_t nomos_kv_ring_set_len(nomos_kv_ring_t *ring, int64_t n);
/* Copies cache_cap, S, win_start, klen, window, n_new, new_base_pos of the step into args. */
int32_t nomos_kv_ring_fill_args(const nomos_kv_ring_t *ring, const nomos_kv_step_t *step, nomos_attn_args_t *args);

/* Bytes of workspace the call needs (>= 0), or a negative status. */
int64_t nomos_attn_workspace_bytes(const nomos_attn_args_t *args);
/* Which kernel nomos_attn_fused would run for these arguments: 2 = the query-major prefill kernel (tcgen05, 128
 * query rows per CTA: int8 caches at head_dim 128 with more than 24 query rows per KV head), 1 = the tcgen05 /
 * tensor-memory decode and verify kernel, 0 = the mma.sync kernel, negative = status.  Kernels 1 and 0 both serve
 * int8 caches at head_dim 128 for up to 24 rows per KV head; the library picks by a measured cost model (the tcgen05
 * kernel for verify, paged caches and calls streaming more than about 240 MB; the other for shorter decode calls), and
 * the NOMOS_ATTN_NO_TCGEN05 / NOMOS_ATTN_TCGEN05_ALWAYS flag bits override it (NO_TCGEN05 also keeps prefill-sized calls
 * on the mma.sync kernel, as row groups).  No reference counterpart (lib/attention_gpu_int8.mojo has a single kernel
 * chain). */
int32_t nomos_attn_kernel_choice(const nomos_attn_args_t *args);
/* What the calling thread's last decode / verify launch did (for logs and tests; no counterpart in the
 * reference): kernel 0 = mma.sync, 1 = tcgen05; sequence splits per KV head; how the splits were merged --
 * 0 one split, 1 by the last CTA to arrive (workspace + arrival counter), 2 cooperatively by all CTAs of the
 * head, 3 inside a thread-block cluster through distributed shared memory.  Any pointer may be NULL. */
int32_t nomos_attn_last_launch(int32_t *kernel, int32_t *splits, int32_t *merge_route);
/* Run it. */
int32_t nomos_attn_fused(void *stream, const nomos_attn_args_t *args);

/* One decode / verify step for a caller whose step inputs and result live in HOST memory: copies
 * in_bytes from host_in (pinned) to dev_in on the stream, runs nomos_attn_fused(stream, args) -- args
 * point into dev_in for the query and the new K/V rows, and at dev_out for the output --, copies
 * out_bytes from dev_out back to host_out (pinned) and synchronises the stream.  The KV cache stays
 * resident on the device.  Either byte count may be 0.  When host_out is pinned and addressable by the GPU
 * (cudaHostAlloc / cudaHostRegister memory) and at most 64 KB, the copy back is skipped: the kernel writes
 * its output into host memory directly and dev_out is left untouched.  The inputs are always staged in dev_in
 * (every CTA of the launch reads the query): by a small copy kernel when host_in is pinned, GPU-addressable,
 * 16-byte aligned like dev_in and at most 64 KB, else by cudaMemcpyAsync.  No counterpart in the reference (its decode
 * loop keeps activations on the device; only tokens cross the bus): it exists so that a host-side
 * caller pays one library call per step instead of three runtime calls and a synchronise. */
int32_t nomos_attn_fused_host(void *stream, const nomos_attn_args_t *args, uint64_t host_in, uint64_t dev_in,
                              int64_t in_bytes, uint64_t host_out, uint64_t dev_out, int64_t out_bytes);

/* nomos_attn_fused for callers that cannot pass a workspace.  No counterpart in the
 * reference (its engine allocates every scratch buffer itself at start-up).  The Nomos
 * engine commits its whole device-memory budget when it starts and treats a failed
 * cudaMalloc as fatal, and a decode loop must not call the allocator (it synchronises the
 * device); such callers have no spare buffer to hand in.  Here the split scratch is a
 * fixed 4 MiB array inside the library image (held by every GPU that loads the library
 * until exit); the call allocates nothing.  args->workspace / ws_bytes / new_k / new_v
 * are not used (new_k, new_v must be 0).  Returns NOMOS_ATTN_ECAPACITY when the call would
 * need more than 4 MiB of split scratch.  All calls on a device share the array: keep them
 * ordered (one stream); calls that overlap on the GPU corrupt each other.  The first call
 * on each device resolves the array's address and should be made before any stream
 * capture begins. */
int32_t nomos_attn_fused_static_ws(void *stream, const nomos_attn_args_t *args);

/* ------------------------------------------------------------------------- *
 *  Paged caches (batch > 1 serving; no counterpart in the reference, whose cache is one          *
 *  contiguous [nkv, cache_cap, hd] block per layer for a single sequence)                        *
 * ------------------------------------------------------------------------- *
 * int8 row-scale KV, head_dim 128, decode (one query row per sequence).  The pools hold n_pages pages;
 * a page is [nkv][128 rows][128] int8 (k_pool, v_pool) and [nkv][128] fp32 (ks_pool, vs_pool).  Key t of
 * sequence b lives in row t % 128 of page block_table[b * max_pages + t / 128] (int32); seq_lens[b]
 * (int32) keys of sequence b are attended, the query being the last of them.  q and out are
 * [batch, nh, 128].  max_len >= every seq_lens[b] sizes the launch.  Pools must be 16-byte aligned. */
int64_t nomos_attn_paged_workspace_bytes(int32_t batch, int32_t nh, int32_t nkv, int32_t kvg, int32_t l_hd, int32_t max_len);
int32_t nomos_attn_paged_decode_i8(void *stream, uint64_t q, uint64_t k_pool, uint64_t v_pool, uint64_t ks_pool,
                                   uint64_t vs_pool, uint64_t block_table, uint64_t seq_lens, uint64_t out,
                                   uint64_t workspace, int64_t ws_bytes, int32_t batch, int32_t nh, int32_t nkv,
                                   int32_t kvg, int32_t l_hd, int32_t n_pages, int32_t max_pages, int32_t max_len,
                                   double softmax_scale, int32_t q_type, int32_t out_type);
/* Quantising append of one new row per sequence (src [batch, nkv, l_hd] fp32, sequence stride l_kvd) at
 * position positions[b] (int32) of sequence b, with the row codec of nomos_kv_append_quant_i8. */
int32_t nomos_kv_paged_append_quant_i8(void *stream, uint64_t src_k, uint64_t src_v, uint64_t k_pool, uint64_t v_pool,
                                       uint64_t ks_pool, uint64_t vs_pool, uint64_t block_table, uint64_t positions,
                                       int32_t batch, int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t max_pages);

/* ------------------------------------------------------------------------- *
 *  Sequence-sharded decode across the GPUs of one node (no counterpart in the reference, which runs on   *
 *  one GPU, lib/gemma4_engine.mojo:229)                                                                  *
 * ------------------------------------------------------------------------- *
 * A long context is cut into `world` contiguous chunks, one per GPU (one process per GPU).  Every rank
 * calls nomos_attn_seq_sharded with ITS chunk as the window (args->klen = keys of the chunk) and the same
 * query; each call is ONE kernel launch that streams the chunk, merges its splits, stores the chunk's
 * un-normalised (o, m, l) rows straight into every peer's mailbox over NVLink (plain stores to peer-mapped
 * memory, a release stamp per row), waits -- with a limit -- for the peers' rows in its own mailbox, and
 * writes the final normalised output of every query row into args->out on every rank.  No collective
 * library call, no second launch, nothing multicast.
 *
 * Set-up, once: every rank creates a mailbox (nomos_attn_peer_mailbox_create: the one call of this library
 * that allocates device memory; zero-filled), passes the 64-byte handle to the other ranks by any host-side
 * means, and opens theirs (nomos_attn_peer_mailbox_open).  mailbox[g] is rank g's mailbox as addressable
 * from THIS process (mailbox[rank] = the pointer create returned).
 * Per call: `step` must be the same on every rank and grow by one with every call (start at 1); every rank
 * must make every call, with the same batch, S, nh and l_hd.  A rank may be at most one call ahead of its
 * peers (the mailboxes hold two steps).  timeout_us (0 = one second) bounds the wait for a peer: when it
 * runs out the kernel raises bit 2 of the device fault word and returns without writing the output;
 * nomos_attn_seq_sharded_status (synchronises the stream) then answers NOMOS_ATTN_ENOTWRITTEN.  After such
 * a failure the ranks must agree on a new step number on the host before they go on. */
typedef struct nomos_attn_peer {
    uint64_t struct_bytes;      /* sizeof(nomos_attn_peer_t)                                              */
    int64_t rank, world;        /* this shard's index, number of shards (1..8; 1 = plain nomos_attn_fused) */
    uint64_t mailbox[8];        /* device addresses of every rank's mailbox in this process               */
    int64_t mailbox_bytes;      /* size of each, >= nomos_attn_peer_mailbox_bytes(world, batch*S*nh, l_hd) */
    uint64_t step;              /* call counter, identical on every rank, never 0                          */
    int64_t timeout_us;         /* wait limit for a peer's rows; 0 = 1 000 000                             */
} nomos_attn_peer_t;
int64_t nomos_attn_peer_mailbox_bytes(int32_t world, int32_t rows, int32_t l_hd);
int32_t nomos_attn_peer_mailbox_create(int64_t bytes, uint64_t *dev_ptr, void *handle64);
int32_t nomos_attn_peer_mailbox_open(const void *handle64, uint64_t *dev_ptr);
int32_t nomos_attn_peer_mailbox_close(uint64_t dev_ptr, int32_t own);
int32_t nomos_attn_seq_sharded(void *stream, const nomos_attn_args_t *args, const nomos_attn_peer_t *peer);
int32_t nomos_attn_seq_sharded_status(void *stream, int32_t clear);

/* Merge G partial triples (as written through partial_out, gathered from G
 * sequence shards) into a normalised output.  partials: fp32 [G][rows][l_hd+2];
 * out: [rows][l_hd] of out_type.  No counterpart in the reference (which is
 * single-GPU); it is the on-device tail of the sequence-sharded decode. */
int32_t nomos_attn_merge_partials(void *stream, uint64_t partials, int32_t G, int32_t rows, int32_t l_hd,
                                  uint64_t out, int32_t out_type);

#ifdef __cplusplus
}
#endif
#endif /* NOMOS_ATTN_H */
