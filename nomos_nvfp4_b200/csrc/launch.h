// Internal host-side launch interface between the C-ABI layer (abi.cu) and the
// kernel translation units.  Every function enqueues on `st`, never synchronises,
// never allocates, and returns a NOMOS_* status.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace nomos {

// ---- kv_quant.cu
int launch_quant_i8(cudaStream_t st, const void *in_bf16, void *out_i8, void *out_scales, int n_rows, int dim);
int launch_dequant_i8(cudaStream_t st, const void *in_i8, const void *in_scales, void *out_bf16, int n_rows, int dim);
int launch_append_i8(cudaStream_t st, const void *src_k, const void *src_v, void *dst_k, void *dst_v, void *k_scales,
                     void *v_scales, int n_s, int nkv, int l_hd, int l_kvd, int cache_cap, int cache_hd, int base_pos);
int launch_append_paged_i8(cudaStream_t st, const void *src_k, const void *src_v, void *k_pool, void *v_pool, void *ks_pool,
                           void *vs_pool, const int *block_table, const int *positions, int batch, int nkv, int l_hd, int l_kvd,
                           int max_pages);
int launch_append_i4(cudaStream_t st, const void *src_k, const void *src_v, void *dst_k, void *dst_v, void *k_scales,
                     void *v_scales, void *k_q8, void *v_q8, void *k_q8_scales, void *v_q8_scales, int n_s, int nkv,
                     int l_hd, int l_kvd, int cache_cap, int cache_hd, int base_pos, int q8_pitch, int scale_blocks);
// mode: 0 i8->bf16, 1 i4->bf16, 2 i4 block-32->bf16, 3 i4->q8, 4 i4 block-32->q8
int launch_window_reader(cudaStream_t st, int mode, const void *src, const void *scales, void *dst, void *dst_scale, int nkv,
                         int klen, int cache_hd, int pitch, int cache_cap, int win_start, int scale_blocks);
int launch_append_dense(cudaStream_t st, int dst_is_bf16, const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                        int n_s, int nkv, int l_hd, int l_kvd, int max_seq, int cache_hd, int base_pos);

// ---- attn_fused.cu : split-K attention over the packed (quantised) ring cache

enum KvFmt { KV_I8 = 0, KV_I4 = 1, KV_I4B32 = 2 };
enum ElemType { ET_F32 = 0, ET_BF16 = 1 };

struct AttnArgs {
    // tensors (device pointers)
    const void *q;          // [batch][S][nh][l_hd]  fp32 or bf16
    const void *k_cache;    // [batch][nkv][cache_cap][cache_hd (/2 for int4)]
    const void *v_cache;
    const void *k_scales;   // [batch][nkv][cache_cap] fp32, or the block-32 buffer
    const void *v_scales;
    void *out;              // [batch][S][nh][l_hd]  fp32 or bf16 (ignored when partial_out is set)
    float *partial_out;     // optional [batch][S][nh][l_hd+2] un-normalised (o.., m, l); m in natural-log units
    void *workspace;        // split-K scratch, ws_bytes long
    long ws_bytes;
    // optional fused quantize-on-write of n_new rows at positions new_base_pos.. (decode: n_new = 1)
    const float *new_k;     // [n_new][nkv][l_hd] fp32, row stride new_stride (elements); nullptr = none
    const float *new_v;
    int n_new, new_stride, new_base_pos;
    // geometry
    int kv_fmt, q_type, out_type;
    int batch, S, nh, nkv, kvg, l_hd, cache_hd, cache_cap;
    int win_start;          // absolute position of window index 0
    int klen;               // keys in the window; query row r sees window indices [lo_r, klen - (S-1-r))
    int window;             // sliding window per row (0 = none): lo_r = max(0, hi_r - window)
    float softmax_scale;
    long q_batch_stride, kv_batch_stride, scale_batch_stride, out_batch_stride;   // elements (q/out), bytes (kv, scales)
    // paged caches (int8, head_dim 128, tcgen05 kernel only): k_cache/v_cache/k_scales/v_scales are pools of
    // n_pages pages of [nkv][128 rows]; tile j of sequence b is page block_table[b * max_pages + j]; klen is
    // the longest sequence (for the plan), seq_lens[b] the keys of sequence b.  nullptr = contiguous caches.
    const int *block_table;
    const int *seq_lens;
    int max_pages, n_pages;
    // sequence-sharded decode across GPUs (peer_world > 1, see nomos_attn_seq_sharded): every rank's mailbox as mapped
    // in this process, this rank's index, the step number and the wait limit
    void *peer_box[8];
    int peer_rank, peer_world;
    unsigned long long peer_seq;
    long peer_timeout_us;
    // general prefix bounds (prefill kernel only): when d0_set, query row s may attend window indices <= d0 + s
    // (clipped to klen - 1; d0 may be negative, rows before the first key see nothing) instead of the default
    // d0 = klen - S ("the query rows are the last S keys")
    int d0_set, d0;
    int force_splits;       // 0 = choose; >0 = use exactly this many splits (tests)
    int no_tma;             // 1: keep every tile on the cp.async path
    int no_cluster;         // 1: never run a unit's splits as a thread-block cluster
    int no_tcgen05;         // 1: never take the tcgen05 kernel
    int tcgen05_always;     // 1: take the tcgen05 kernel whenever it supports the call
    int settled_cache;      // 1: rows older than the S query rows may be read before the stream predecessor completes
    int fit_splits_to_ws;   // 1: use fewer splits rather than fail when the workspace is small (thin entry points)
};

// Bytes of one rank's mailbox for `world` sequence shards of `grows` query rows (batch x S x nh) of head dim l_hd:
// [2 step slots][world][grows][l_hd + 2] fp32 rows, then [2][world][grows] 64-bit stamps.
long attn_peer_mailbox_rows_bytes(int world, long grows, int l_hd);
long attn_peer_mailbox_bytes(int world, long grows, int l_hd);
long attn_workspace_bytes(const AttnArgs &a);
// What the last attention launch of the calling thread did: sequence splits per unit and how they were merged
// (0: one split, nothing to merge; 1: by the last CTA to arrive; 2: cooperatively by the unit's CTAs; 3: in a
// thread-block cluster through distributed shared memory).
struct LaunchInfo { int kernel, splits, merge_route; };
LaunchInfo attn_last_launch_info();
int attn_kernel_choice(const AttnArgs &a);     // 2: the query-major prefill kernel, 1: the tcgen05 decode / verify kernel, 0: the mma.sync kernel
int launch_attn_fused(cudaStream_t st, const AttnArgs &a);
long attn_paged_workspace_bytes(const AttnArgs &a);
int launch_attn_paged(cudaStream_t st, const AttnArgs &a);
// Reads (and optionally clears) the device word the kernels OR into when a bounded wait runs out.
int read_attn_faults(unsigned int *out, bool clear);
int clear_attn_fault_bits(unsigned int bits);
// partials [G][rows][l_hd+2] = (o.., m, l) with m in natural-log units (the exported form)
int launch_merge_partials(cudaStream_t st, const float *partials, int G, int rows, int l_hd, void *out, int out_type);
// same, m in log2 units (in-library split partials), fp32 output
int launch_merge_partials_log2(cudaStream_t st, const float *partials, int G, int rows, int l_hd, float *out);

// ---- attn_dense.cu : fp32 / bf16 KV decode + prefix-batched attention
// K / V / Q producer epilogue (kv_producer.cu): RMSNorm (+ weight), RoPE, quantize-on-write.
struct ProducerArgs {
    float *q;                     // [n_s][nh][l_hd] fp32, normalised + rotated in place; nullptr = no query rows
    const float *q_norm_w;        // [l_hd]
    const float *src_k, *src_v;   // [n_s][nkv][l_hd] fp32 raw projection rows, token stride l_kvd (not modified)
    const float *k_norm_w;        // [l_hd]
    uint8_t *dst_k, *dst_v;       // cache planes (layout of kv_fmt)
    uint8_t *k_scales, *v_scales;
    float *k_out, *v_out;         // optional [n_s][nkv][l_hd] fp32: the rows exactly as they were quantised
    int n_s, nh, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, rope_dim, kv_fmt;   // kv_fmt < 0: no cache write
    float theta;
};
int launch_kv_producer(cudaStream_t st, const ProducerArgs &a);

struct DenseAttnArgs {
    const float *q;          // [S][nh][l_hd] fp32
    const void *k_cache;     // [nkv][max_seq][cache_hd] fp32 or bf16
    const void *v_cache;
    float *out;              // [S][nh][l_hd] fp32
    void *workspace; long ws_bytes;
    int kv_is_bf16;
    int S, nh, nkv, kvg, l_hd, cache_hd, max_seq, key_len, window, query_base_pos, key_base_pos;
};
int launch_attn_dense(cudaStream_t st, const DenseAttnArgs &a);

}  // namespace nomos
