// extern "C" surface of libnomos_attn.so: argument validation + forwarding.
// Declarations and per-function reference citations live in include/nomos_attn.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/nomos_attn.h"
#include "common.cuh"
#include "launch.h"

namespace nomos {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

}  // namespace nomos

using namespace nomos;

#define NOMOS_EXPORT extern "C" __attribute__((visibility("default")))

#define REQUIRE(cond, ...)                      \
    do {                                        \
        if (!(cond)) {                          \
            set_error(__VA_ARGS__);             \
            return NOMOS_EBADARG;               \
        }                                       \
    } while (0)

static inline bool aligned(uint64_t p, uint64_t a) { return (p & (a - 1)) == 0; }
static inline void *ptr(uint64_t a) { return reinterpret_cast<void *>(a); }
static inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }
static inline bool hd_ok(int hd) { return hd == 128 || hd == 256 || hd == 512; }

NOMOS_EXPORT int32_t nomos_attn_version(void) { return 100; }
NOMOS_EXPORT const char *nomos_attn_last_error(void) { return g_err; }
NOMOS_EXPORT int32_t nomos_attn_device_faults(uint32_t *out_bits, int32_t clear) {
    REQUIRE(out_bits, "nomos_attn_device_faults: null pointer");
    return nomos::read_attn_faults(out_bits, clear != 0);
}

// ------------------------------------------------------------------- codecs

NOMOS_EXPORT int32_t nomos_kv_quant_i8(void *stream, uint64_t in_bf16, uint64_t out_i8, uint64_t out_scales,
                                       int32_t n_rows, int32_t dim) {
    if (n_rows <= 0) return NOMOS_OK;
    REQUIRE(in_bf16 && out_i8 && out_scales, "nomos_kv_quant_i8: null pointer");
    REQUIRE(dim > 0, "nomos_kv_quant_i8: dim %d", dim);
    return launch_quant_i8(as_stream(stream), ptr(in_bf16), ptr(out_i8), ptr(out_scales), n_rows, dim);
}

NOMOS_EXPORT int32_t nomos_kv_dequant_i8(void *stream, uint64_t in_i8, uint64_t in_scales, uint64_t out_bf16,
                                         int32_t n_rows, int32_t dim) {
    if (n_rows <= 0) return NOMOS_OK;
    REQUIRE(in_i8 && in_scales && out_bf16, "nomos_kv_dequant_i8: null pointer");
    REQUIRE(dim > 0, "nomos_kv_dequant_i8: dim %d", dim);
    return launch_dequant_i8(as_stream(stream), ptr(in_i8), ptr(in_scales), ptr(out_bf16), n_rows, dim);
}

static int check_append(const char *who, uint64_t a, uint64_t b, uint64_t c, uint64_t d, uint64_t e, uint64_t f,
                        int n_s, int nkv, int l_hd, int l_kvd, int cache_cap, int cache_hd, int base_pos) {
    REQUIRE(a && b && c && d && e && f, "%s: null pointer", who);
    REQUIRE(nkv > 0 && l_hd > 0 && cache_cap > 0 && cache_hd >= l_hd, "%s: bad geometry nkv=%d l_hd=%d cache_cap=%d cache_hd=%d",
            who, nkv, l_hd, cache_cap, cache_hd);
    REQUIRE(l_kvd >= nkv * l_hd || n_s == 1, "%s: token stride l_kvd=%d < nkv*l_hd", who, l_kvd);
    REQUIRE(base_pos >= 0, "%s: base_pos %d", who, base_pos);
    REQUIRE(n_s <= cache_cap, "%s: n_s=%d rows would overwrite each other in a ring of %d", who, n_s, cache_cap);
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_append_quant_i8(void *stream, uint64_t src_k, uint64_t src_v, uint64_t dst_k_i8,
                                              uint64_t dst_v_i8, uint64_t k_scales, uint64_t v_scales, int32_t n_s,
                                              int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap,
                                              int32_t cache_hd, int32_t base_pos) {
    if (n_s <= 0) return NOMOS_OK;
    int rc = check_append("nomos_kv_append_quant_i8", src_k, src_v, dst_k_i8, dst_v_i8, k_scales, v_scales, n_s, nkv, l_hd,
                          l_kvd, cache_cap, cache_hd, base_pos);
    if (rc) return rc;
    return launch_append_i8(as_stream(stream), ptr(src_k), ptr(src_v), ptr(dst_k_i8), ptr(dst_v_i8), ptr(k_scales),
                            ptr(v_scales), n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos);
}

NOMOS_EXPORT int32_t nomos_kv_norm_rope_append(void *stream, uint64_t q, uint64_t q_norm_w, uint64_t src_k, uint64_t src_v,
                                                uint64_t k_norm_w, uint64_t dst_k, uint64_t dst_v, uint64_t k_scales,
                                                uint64_t v_scales, uint64_t k_out, uint64_t v_out, int32_t n_s, int32_t nh,
                                                int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap,
                                                int32_t cache_hd, int32_t base_pos, float theta, int32_t rope_dim,
                                                int32_t kv_fmt) {
    const char *who = "nomos_kv_norm_rope_append";
    if (n_s <= 0) return NOMOS_OK;
    REQUIRE(src_k && src_v && k_norm_w, "%s: null pointer", who);
    REQUIRE(!q || (q_norm_w && nh > 0), "%s: query rows need q_norm_w and nh", who);
    REQUIRE(nkv > 0 && l_hd > 0 && l_hd % 2 == 0, "%s: bad geometry nkv=%d l_hd=%d", who, nkv, l_hd);
    REQUIRE(l_kvd >= nkv * l_hd || n_s == 1, "%s: token stride l_kvd=%d < nkv*l_hd", who, l_kvd);
    REQUIRE(base_pos >= 0, "%s: base_pos %d", who, base_pos);
    REQUIRE(rope_dim >= 0 && rope_dim <= l_hd && rope_dim % 2 == 0, "%s: rope_dim %d for head_dim %d", who, rope_dim, l_hd);
    if (l_hd > 512) { set_error("%s: head_dim %d unsupported (at most 512)", who, l_hd); return NOMOS_EUNSUPPORTED; }
    if (kv_fmt >= 0) {
        if (kv_fmt != KV_I8 && kv_fmt != KV_I4 && kv_fmt != KV_I4B32) { set_error("%s: kv_fmt %d unknown", who, kv_fmt); return NOMOS_EBADARG; }
        REQUIRE(dst_k && dst_v && k_scales && v_scales, "%s: null cache pointer", who);
        REQUIRE(cache_cap > 0 && cache_hd >= l_hd, "%s: bad cache geometry cache_cap=%d cache_hd=%d", who, cache_cap, cache_hd);
        REQUIRE(kv_fmt == KV_I8 || cache_hd % 2 == 0, "%s: odd cache_hd %d", who, cache_hd);
        REQUIRE(n_s <= cache_cap, "%s: n_s=%d rows would overwrite each other in a ring of %d", who, n_s, cache_cap);
    }
    ProducerArgs a;
    a.q = static_cast<float *>(ptr(q)); a.q_norm_w = static_cast<const float *>(ptr(q_norm_w));
    a.src_k = static_cast<const float *>(ptr(src_k)); a.src_v = static_cast<const float *>(ptr(src_v));
    a.k_norm_w = static_cast<const float *>(ptr(k_norm_w));
    a.dst_k = static_cast<uint8_t *>(ptr(dst_k)); a.dst_v = static_cast<uint8_t *>(ptr(dst_v));
    a.k_scales = static_cast<uint8_t *>(ptr(k_scales)); a.v_scales = static_cast<uint8_t *>(ptr(v_scales));
    a.k_out = static_cast<float *>(ptr(k_out)); a.v_out = static_cast<float *>(ptr(v_out));
    a.n_s = n_s; a.nh = nh; a.nkv = nkv; a.l_hd = l_hd; a.l_kvd = l_kvd; a.cache_cap = cache_cap; a.cache_hd = cache_hd;
    a.base_pos = base_pos; a.rope_dim = rope_dim; a.kv_fmt = kv_fmt; a.theta = theta;
    return launch_kv_producer(as_stream(stream), a);
}

static int check_scale_blocks(const char *who, int l_hd, int scale_blocks) {
    REQUIRE(scale_blocks >= 1, "%s: scale_blocks %d", who, scale_blocks);
    if (scale_blocks > 1 && scale_blocks != (l_hd + 31) / 32) {
        set_error("%s: scale_blocks=%d but head_dim %d has %d blocks of 32", who, scale_blocks, l_hd, (l_hd + 31) / 32);
        return NOMOS_EUNSUPPORTED;
    }
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_append_quant_i4(void *stream, uint64_t src_k, uint64_t src_v, uint64_t dst_k_i4,
                                              uint64_t dst_v_i4, uint64_t k_scales, uint64_t v_scales, int32_t n_s,
                                              int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t cache_cap,
                                              int32_t cache_hd, int32_t base_pos, int32_t scale_blocks) {
    if (n_s <= 0) return NOMOS_OK;
    int rc = check_append("nomos_kv_append_quant_i4", src_k, src_v, dst_k_i4, dst_v_i4, k_scales, v_scales, n_s, nkv, l_hd,
                          l_kvd, cache_cap, cache_hd, base_pos);
    if (rc) return rc;
    REQUIRE(cache_hd % 2 == 0, "nomos_kv_append_quant_i4: odd cache_hd %d", cache_hd);
    if ((rc = check_scale_blocks("nomos_kv_append_quant_i4", l_hd, scale_blocks))) return rc;
    return launch_append_i4(as_stream(stream), ptr(src_k), ptr(src_v), ptr(dst_k_i4), ptr(dst_v_i4), ptr(k_scales),
                            ptr(v_scales), nullptr, nullptr, nullptr, nullptr, n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd,
                            base_pos, 0, scale_blocks);
}

NOMOS_EXPORT int32_t nomos_kv_append_quant_i4_with_q8(void *stream, uint64_t src_k, uint64_t src_v, uint64_t dst_k_i4,
                                                      uint64_t dst_v_i4, uint64_t k_scales, uint64_t v_scales,
                                                      uint64_t dst_k_q8, uint64_t dst_v_q8, uint64_t k_q8_scales,
                                                      uint64_t v_q8_scales, int32_t n_s, int32_t nkv, int32_t l_hd,
                                                      int32_t l_kvd, int32_t cache_cap, int32_t cache_hd, int32_t base_pos,
                                                      int32_t q8_pitch, int32_t scale_blocks) {
    if (n_s <= 0) return NOMOS_OK;
    int rc = check_append("nomos_kv_append_quant_i4_with_q8", src_k, src_v, dst_k_i4, dst_v_i4, k_scales, v_scales, n_s,
                          nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos);
    if (rc) return rc;
    REQUIRE(dst_k_q8 && dst_v_q8 && k_q8_scales && v_q8_scales, "nomos_kv_append_quant_i4_with_q8: null view pointer");
    REQUIRE(cache_hd % 2 == 0, "nomos_kv_append_quant_i4_with_q8: odd cache_hd %d", cache_hd);
    if (base_pos + n_s > q8_pitch) {
        set_error("nomos_kv_append_quant_i4_with_q8: rows [%d,%d) beyond the view pitch %d", base_pos, base_pos + n_s, q8_pitch);
        return NOMOS_ECAPACITY;
    }
    if ((rc = check_scale_blocks("nomos_kv_append_quant_i4_with_q8", l_hd, scale_blocks))) return rc;
    return launch_append_i4(as_stream(stream), ptr(src_k), ptr(src_v), ptr(dst_k_i4), ptr(dst_v_i4), ptr(k_scales),
                            ptr(v_scales), ptr(dst_k_q8), ptr(dst_v_q8), ptr(k_q8_scales), ptr(v_q8_scales), n_s, nkv, l_hd,
                            l_kvd, cache_cap, cache_hd, base_pos, q8_pitch, scale_blocks);
}

static int check_reader(const char *who, uint64_t src, uint64_t scales, uint64_t dst, int nkv, int klen, int cache_hd,
                        int max_seq, int cache_cap, int win_start) {
    REQUIRE(src && scales && dst, "%s: null pointer", who);
    REQUIRE(nkv > 0 && cache_hd > 0 && cache_cap > 0 && win_start >= 0, "%s: bad geometry", who);
    REQUIRE(cache_hd % 8 == 0, "%s: cache_hd %d must be a multiple of 8", who, cache_hd);
    REQUIRE(aligned(src, 8) && aligned(dst, 16), "%s: misaligned buffer", who);
    if (klen > max_seq) { set_error("%s: klen %d exceeds the scratch pitch %d", who, klen, max_seq); return NOMOS_ECAPACITY; }
    if (klen > cache_cap) { set_error("%s: klen %d exceeds the ring capacity %d", who, klen, cache_cap); return NOMOS_ECAPACITY; }
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_dequant_i8_layer(void *stream, uint64_t src_i8, uint64_t scales, uint64_t dst_bf16,
                                               int32_t nkv, int32_t klen, int32_t cache_hd, int32_t max_seq,
                                               int32_t cache_cap, int32_t win_start) {
    if (klen <= 0) return NOMOS_OK;
    int rc = check_reader("nomos_kv_dequant_i8_layer", src_i8, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start);
    if (rc) return rc;
    return launch_window_reader(as_stream(stream), 0, ptr(src_i8), ptr(scales), ptr(dst_bf16), nullptr, nkv, klen, cache_hd,
                                max_seq, cache_cap, win_start, 1);
}

NOMOS_EXPORT int32_t nomos_kv_dequant_i4_layer(void *stream, uint64_t src_i4, uint64_t scales, uint64_t dst_bf16,
                                               int32_t nkv, int32_t klen, int32_t cache_hd, int32_t max_seq,
                                               int32_t cache_cap, int32_t win_start, int32_t scale_blocks) {
    if (klen <= 0) return NOMOS_OK;
    int rc = check_reader("nomos_kv_dequant_i4_layer", src_i4, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start);
    if (rc) return rc;
    REQUIRE(scale_blocks >= 1, "nomos_kv_dequant_i4_layer: scale_blocks %d", scale_blocks);
    return launch_window_reader(as_stream(stream), scale_blocks > 1 ? 2 : 1, ptr(src_i4), ptr(scales), ptr(dst_bf16), nullptr,
                                nkv, klen, cache_hd, max_seq, cache_cap, win_start, scale_blocks);
}

NOMOS_EXPORT int32_t nomos_kv_dequant_i4_to_q8_layer(void *stream, uint64_t src_i4, uint64_t scales, uint64_t dst_i8,
                                                     uint64_t dst_scale, int32_t nkv, int32_t klen, int32_t cache_hd,
                                                     int32_t max_seq, int32_t cache_cap, int32_t win_start,
                                                     int32_t scale_blocks) {
    if (klen <= 0) return NOMOS_OK;
    int rc = check_reader("nomos_kv_dequant_i4_to_q8_layer", src_i4, scales, dst_i8, nkv, klen, cache_hd, max_seq, cache_cap, win_start);
    if (rc) return rc;
    REQUIRE(dst_scale, "nomos_kv_dequant_i4_to_q8_layer: null dst_scale");
    REQUIRE(scale_blocks >= 1, "nomos_kv_dequant_i4_to_q8_layer: scale_blocks %d", scale_blocks);
    return launch_window_reader(as_stream(stream), scale_blocks > 1 ? 4 : 3, ptr(src_i4), ptr(scales), ptr(dst_i8),
                                ptr(dst_scale), nkv, klen, cache_hd, max_seq, cache_cap, win_start, scale_blocks);
}

static int check_dense_append(const char *who, uint64_t a, uint64_t b, uint64_t c, uint64_t d, int nkv, int l_hd,
                              int cache_hd, int max_seq, int pos, int n_s) {
    REQUIRE(a && b && c && d, "%s: null pointer", who);
    REQUIRE(nkv > 0 && l_hd > 0 && cache_hd >= l_hd && max_seq > 0 && pos >= 0, "%s: bad geometry", who);
    if (pos + n_s > max_seq) { set_error("%s: rows [%d,%d) beyond max_seq %d", who, pos, pos + n_s, max_seq); return NOMOS_ECAPACITY; }
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_append_fp32(void *stream, uint64_t k_cache, uint64_t v_cache, uint64_t k_new, uint64_t v_new,
                                          int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t cl) {
    int rc = check_dense_append("nomos_kv_append_fp32", k_cache, v_cache, k_new, v_new, nkv, l_hd, cache_hd, max_seq, cl, 1);
    if (rc) return rc;
    return launch_append_dense(as_stream(stream), 0, ptr(k_new), ptr(v_new), ptr(k_cache), ptr(v_cache), 1, nkv, l_hd,
                               nkv * l_hd, max_seq, cache_hd, cl);
}

NOMOS_EXPORT int32_t nomos_kv_append_bf16(void *stream, uint64_t k_cache, uint64_t v_cache, uint64_t k_new, uint64_t v_new,
                                          uint64_t, uint64_t, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                          int32_t cl) {
    int rc = check_dense_append("nomos_kv_append_bf16", k_cache, v_cache, k_new, v_new, nkv, l_hd, cache_hd, max_seq, cl, 1);
    if (rc) return rc;
    return launch_append_dense(as_stream(stream), 1, ptr(k_new), ptr(v_new), ptr(k_cache), ptr(v_cache), 1, nkv, l_hd,
                               nkv * l_hd, max_seq, cache_hd, cl);
}

NOMOS_EXPORT int32_t nomos_kv_append_batched_bf16(void *stream, uint64_t src_k, uint64_t src_v, uint64_t dst_k,
                                                  uint64_t dst_v, int32_t n_s, int32_t nkv, int32_t l_hd, int32_t l_kvd,
                                                  int32_t max_seq, int32_t cache_hd, int32_t base_pos) {
    if (n_s <= 0) return NOMOS_OK;
    int rc = check_dense_append("nomos_kv_append_batched_bf16", dst_k, dst_v, src_k, src_v, nkv, l_hd, cache_hd, max_seq, base_pos, n_s);
    if (rc) return rc;
    return launch_append_dense(as_stream(stream), 1, ptr(src_k), ptr(src_v), ptr(dst_k), ptr(dst_v), n_s, nkv, l_hd, l_kvd,
                               max_seq, cache_hd, base_pos);
}

// ---------------------------------------------------------------- attention

static int check_attn_geometry(const char *who, int nh, int nkv, int l_hd, int cache_hd, int kvg) {
    REQUIRE(nkv > 0 && kvg > 0 && nh == nkv * kvg, "%s: nh=%d must equal nkv=%d * kvg=%d", who, nh, nkv, kvg);
    if (!hd_ok(l_hd)) { set_error("%s: head_dim %d unsupported (128, 256, 512)", who, l_hd); return NOMOS_EUNSUPPORTED; }
    REQUIRE(cache_hd >= l_hd, "%s: cache_hd %d < l_hd %d", who, cache_hd, l_hd);
    return NOMOS_OK;
}

static int run_fused(cudaStream_t st, AttnArgs &a, const char *who) {
    int rc = check_attn_geometry(who, a.nh, a.nkv, a.l_hd, a.cache_hd, a.kvg);
    if (rc) return rc;
    REQUIRE(a.q && a.k_cache && a.v_cache && a.k_scales && a.v_scales, "%s: null pointer", who);
    REQUIRE(a.out || a.partial_out, "%s: no output buffer", who);
    REQUIRE(a.batch > 0 && a.S > 0 && a.cache_cap > 0 && a.win_start >= 0, "%s: bad batch/S/cache_cap/win_start", who);
    REQUIRE(a.kv_fmt >= KV_I8 && a.kv_fmt <= KV_I4B32, "%s: kv_fmt %d", who, a.kv_fmt);
    REQUIRE((a.q_type == ET_F32 || a.q_type == ET_BF16) && (a.out_type == ET_F32 || a.out_type == ET_BF16), "%s: element type", who);
    const int row_bytes = a.kv_fmt == KV_I8 ? a.cache_hd : a.cache_hd / 2;
    REQUIRE(row_bytes % 16 == 0, "%s: cache rows must be a multiple of 16 bytes (cache_hd=%d)", who, a.cache_hd);
    REQUIRE(aligned((uint64_t)a.k_cache, 16) && aligned((uint64_t)a.v_cache, 16) && aligned((uint64_t)a.k_scales, 4) &&
                aligned((uint64_t)a.v_scales, 4) && aligned((uint64_t)a.q, 4),
            "%s: misaligned buffer", who);
    REQUIRE(a.kv_batch_stride % 16 == 0 && a.scale_batch_stride % 4 == 0, "%s: misaligned batch stride", who);
    REQUIRE(a.window >= 0, "%s: window %d", who, a.window);
    if (a.klen > a.cache_cap) { set_error("%s: klen %d exceeds the cache capacity %d", who, a.klen, a.cache_cap); return NOMOS_ECAPACITY; }
    REQUIRE(a.klen >= a.S, "%s: klen %d < S %d (the query rows are the last S keys)", who, a.klen, a.S);
    return launch_attn_fused(st, a);
}

static int run_prefill_general(cudaStream_t st, AttnArgs &a, const char *who, int S, int key_len, int window, int query_base_pos,
                               int key_base_pos);

static void fill_thin(AttnArgs &a, uint64_t q, uint64_t k, uint64_t v, uint64_t ks, uint64_t vs, uint64_t scratch,
                      long scratch_floats, uint64_t out, int nh, int nkv, int l_hd, int cache_hd, int max_seq, int kvg) {
    memset(&a, 0, sizeof(a));
    a.q = ptr(q); a.k_cache = ptr(k); a.v_cache = ptr(v); a.k_scales = ptr(ks); a.v_scales = ptr(vs);
    a.out = ptr(out); a.workspace = ptr(scratch); a.ws_bytes = scratch ? scratch_floats * 4 : 0;
    a.kv_fmt = KV_I8; a.q_type = ET_F32; a.out_type = ET_F32;
    a.batch = 1; a.S = 1; a.nh = nh; a.nkv = nkv; a.kvg = kvg; a.l_hd = l_hd; a.cache_hd = cache_hd; a.cache_cap = max_seq;
    a.softmax_scale = 1.0f;
    a.fit_splits_to_ws = 1;
}

NOMOS_EXPORT int32_t nomos_attn_decode_i8(void *stream, uint64_t q, uint64_t k_i8, uint64_t v_i8, uint64_t k_scale,
                                          uint64_t v_scale, uint64_t scores_scratch, uint64_t out, int32_t nh, int32_t nkv,
                                          int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t seq_len, int32_t kvg) {
    if (nh <= 0 || seq_len <= 0) return NOMOS_OK;
    AttnArgs a;
    fill_thin(a, q, k_i8, v_i8, k_scale, v_scale, scores_scratch, (long)nh * seq_len, out, nh, nkv, l_hd, cache_hd, max_seq, kvg);
    a.klen = seq_len;
    return run_fused(as_stream(stream), a, "nomos_attn_decode_i8");
}

NOMOS_EXPORT int32_t nomos_attn_decode_multirow_i8(void *stream, uint64_t q_b, uint64_t scores, uint64_t attn_b,
                                                   uint64_t k_i8, uint64_t v_i8, uint64_t k_scale, uint64_t v_scale,
                                                   int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq,
                                                   int32_t S, int32_t score_stride, int32_t kvg, int32_t window,
                                                   int32_t query_base_pos) {
    if (nh <= 0 || S <= 0 || score_stride <= 0) return NOMOS_OK;
    REQUIRE(query_base_pos >= 0, "nomos_attn_decode_multirow_i8: query_base_pos %d", query_base_pos);
    AttnArgs a;
    fill_thin(a, q_b, k_i8, v_i8, k_scale, v_scale, scores, (long)S * nh * score_stride, attn_b, nh, nkv, l_hd, cache_hd, max_seq, kvg);
    a.S = S; a.klen = query_base_pos + S; a.window = window;
    return run_fused(as_stream(stream), a, "nomos_attn_decode_multirow_i8");
}

// Key range of the prefix-batched operators expressed for the fused kernel.  The operators' row s sees keys
// [max(0, lo_abs - key_base_pos), min(q_abs - key_base_pos, key_len - 1)] of the array handed in, q_abs =
// query_base_pos + s (lib/batched_attn_gpu.mojo:314-326); the fused kernel's row s sees window indices up to
// klen - S + s.  The two agree when the array ends at the last query row: klen = query_base_pos - key_base_pos + S.
// Keys beyond that are never attended, so a longer key_len is cut down to it.  Returns klen, or a negative status
// for the ranges the fused kernel cannot express (a key array that ends before the last query row, queries
// before the first key): those take the general prefill kernel.
static int prefix_klen(int S, int key_len, int query_base_pos, int key_base_pos) {
    if (query_base_pos < key_base_pos) return -1;
    const long full = (long)query_base_pos - key_base_pos + S;
    return key_len >= full ? (int)full : -1;
}

NOMOS_EXPORT int32_t nomos_attn_prefix_batched_i8(void *stream, uint64_t q_b, uint64_t, uint64_t scores, uint64_t,
                                                  uint64_t attn_b, uint64_t k_i8, uint64_t v_i8, uint64_t k_scale,
                                                  uint64_t v_scale, int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd,
                                                  int32_t max_seq, int32_t S, int32_t key_len, int32_t kvg, int32_t window,
                                                  int32_t query_base_pos, int32_t key_base_pos) {
    const char *who = "nomos_attn_prefix_batched_i8";
    if (nh <= 0 || S <= 0 || key_len <= 0) return NOMOS_OK;
    REQUIRE(query_base_pos >= 0 && key_base_pos >= 0 && window >= 0, "%s: negative position or window", who);
    if (key_len > max_seq) { set_error("%s: key_len %d exceeds the row pitch %d", who, key_len, max_seq); return NOMOS_ECAPACITY; }
    AttnArgs a;
    fill_thin(a, q_b, k_i8, v_i8, k_scale, v_scale, scores, (long)S * nh * key_len, attn_b, nh, nkv, l_hd, cache_hd, max_seq, kvg);
    // The engine pre-offsets the K / V / scale pointers by key_base_pos rows (lib/engine_prefill.mojo:926-941), so
    // window index t of the array is absolute position key_base_pos + t and the sliding window needs no base.
    const int klen = prefix_klen(S, key_len, query_base_pos, key_base_pos);
    if (klen < 0) return run_prefill_general(as_stream(stream), a, who, S, key_len, window, query_base_pos, key_base_pos);
    a.S = S; a.klen = klen; a.window = window;
    return run_fused(as_stream(stream), a, who);
}

/* attention_prefill_batched_int8, lib/attention_gpu_int8.mojo:804-841: the square causal form. */
NOMOS_EXPORT int32_t nomos_attn_prefill_batched_i8(void *stream, uint64_t q_b, uint64_t q_t, uint64_t scores, uint64_t attn_t,
                                                   uint64_t attn_b, uint64_t k_i8, uint64_t v_i8, uint64_t k_scale,
                                                   uint64_t v_scale, int32_t nh, int32_t nkv, int32_t l_hd, int32_t cache_hd,
                                                   int32_t max_seq, int32_t S, int32_t kvg, int32_t window) {
    return nomos_attn_prefix_batched_i8(stream, q_b, q_t, scores, attn_t, attn_b, k_i8, v_i8, k_scale, v_scale, nh, nkv, l_hd,
                                        cache_hd, max_seq, S, S, kvg, window, 0, 0);
}

// Prefix ranges the decode-order kernels cannot express (see prefix_klen): the query-major prefill kernel takes
// the operator's bounds as they are (row s attends key indices up to min(d0 + s, key_len - 1), d0 = query_base_pos -
// key_base_pos, possibly negative; rows without a key get zeros).
static int run_prefill_general(cudaStream_t st, AttnArgs &a, const char *who, int S, int key_len, int window, int query_base_pos,
                               int key_base_pos) {
    a.S = S; a.klen = key_len; a.window = window;
    a.d0_set = 1; a.d0 = query_base_pos - key_base_pos;
    int rc = check_attn_geometry(who, a.nh, a.nkv, a.l_hd, a.cache_hd, a.kvg);
    if (rc) return rc;
    REQUIRE(a.q && a.k_cache && a.v_cache && a.k_scales && a.v_scales && a.out, "%s: null pointer", who);
    if (a.kv_fmt != KV_I8 || a.l_hd != 128) {
        set_error("%s: key range [%d, %d) must reach the last query row (position %d) and start at or before the first for this "
                  "cache format / head dim", who, key_base_pos, key_base_pos + key_len, query_base_pos + S - 1);
        return NOMOS_EUNSUPPORTED;
    }
    return launch_attn_fused(st, a);
}

static int run_dense(cudaStream_t st, const char *who, uint64_t q, uint64_t k, uint64_t v, uint64_t scratch, long scratch_floats,
                     uint64_t out, int nh, int nkv, int l_hd, int cache_hd, int max_seq, int S, int key_len, int kvg,
                     int window, int qbase, int kbase, int kv_is_bf16) {
    int rc = check_attn_geometry(who, nh, nkv, l_hd, cache_hd, kvg);
    if (rc) return rc;
    REQUIRE(q && k && v && out, "%s: null pointer", who);
    REQUIRE(aligned(k, 16) && aligned(v, 16) && aligned(q, 4) && (cache_hd * (kv_is_bf16 ? 2 : 4)) % 16 == 0, "%s: misaligned cache", who);
    if (key_len > max_seq) { set_error("%s: key_len %d exceeds max_seq %d", who, key_len, max_seq); return NOMOS_ECAPACITY; }
    DenseAttnArgs a;
    a.q = static_cast<const float *>(ptr(q)); a.k_cache = ptr(k); a.v_cache = ptr(v); a.out = static_cast<float *>(ptr(out));
    a.workspace = ptr(scratch); a.ws_bytes = scratch ? scratch_floats * 4 : 0;
    a.kv_is_bf16 = kv_is_bf16; a.S = S; a.nh = nh; a.nkv = nkv; a.kvg = kvg; a.l_hd = l_hd; a.cache_hd = cache_hd;
    a.max_seq = max_seq; a.key_len = key_len; a.window = window; a.query_base_pos = qbase; a.key_base_pos = kbase;
    return launch_attn_dense(st, a);
}

NOMOS_EXPORT int32_t nomos_attn_decode_fp32(void *stream, uint64_t q, uint64_t k_cache, uint64_t v_cache,
                                            uint64_t scores_scratch, uint64_t out, int32_t nh, int32_t nkv, int32_t l_hd,
                                            int32_t cache_hd, int32_t max_seq, int32_t seq_len, int32_t kvg) {
    if (nh <= 0 || seq_len <= 0) return NOMOS_OK;
    return run_dense(as_stream(stream), "nomos_attn_decode_fp32", q, k_cache, v_cache, scores_scratch, (long)nh * seq_len, out, nh,
                     nkv, l_hd, cache_hd, max_seq, 1, seq_len, kvg, 0, seq_len - 1, 0, 0);
}

NOMOS_EXPORT int32_t nomos_attn_decode_bf16(void *stream, uint64_t q, uint64_t k_cache, uint64_t v_cache,
                                            uint64_t scores_scratch, uint64_t, uint64_t, uint64_t out, int32_t nh,
                                            int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t seq_len,
                                            int32_t kvg) {
    if (nh <= 0 || seq_len <= 0) return NOMOS_OK;
    return run_dense(as_stream(stream), "nomos_attn_decode_bf16", q, k_cache, v_cache, scores_scratch, (long)nh * seq_len, out, nh,
                     nkv, l_hd, cache_hd, max_seq, 1, seq_len, kvg, 0, seq_len - 1, 0, 1);
}

NOMOS_EXPORT int32_t nomos_attn_prefix_batched_dense(void *stream, uint64_t q_b, uint64_t scores, uint64_t attn_b,
                                                     uint64_t k_cache, uint64_t v_cache, int32_t nh, int32_t nkv,
                                                     int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t S,
                                                     int32_t key_len, int32_t kvg, int32_t window, int32_t query_base_pos,
                                                     int32_t key_base_pos, int32_t kv_is_bf16) {
    if (nh <= 0 || S <= 0 || key_len <= 0) return NOMOS_OK;
    REQUIRE(query_base_pos >= 0 && key_base_pos >= 0 && window >= 0, "nomos_attn_prefix_batched_dense: negative position or window");
    return run_dense(as_stream(stream), "nomos_attn_prefix_batched_dense", q_b, k_cache, v_cache, scores, (long)S * nh * key_len,
                     attn_b, nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window, query_base_pos, key_base_pos,
                     kv_is_bf16 != 0);
}

// The four operators of lib/batched_attn_gpu.mojo with their own argument lists (the cuBLAS handle dropped, the
// transpose / cast scratches accepted and unused): one body, nomos_attn_prefix_batched_dense.
NOMOS_EXPORT int32_t nomos_attn_prefix_batched_fp32(void *stream, uint64_t q_b, uint64_t, uint64_t scores, uint64_t, uint64_t attn_b,
                                                    uint64_t k_cache, uint64_t v_cache, int32_t nh, int32_t nkv, int32_t l_hd,
                                                    int32_t cache_hd, int32_t max_seq, int32_t S, int32_t key_len, int32_t kvg,
                                                    int32_t window, int32_t query_base_pos, int32_t key_base_pos) {
    return nomos_attn_prefix_batched_dense(stream, q_b, scores, attn_b, k_cache, v_cache, nh, nkv, l_hd, cache_hd, max_seq, S,
                                           key_len, kvg, window, query_base_pos, key_base_pos, 0);
}
NOMOS_EXPORT int32_t nomos_attn_prefix_batched_bf16(void *stream, uint64_t q_b, uint64_t, uint64_t, uint64_t scores, uint64_t,
                                                    uint64_t, uint64_t attn_b, uint64_t k_cache, uint64_t v_cache, int32_t nh,
                                                    int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t S,
                                                    int32_t key_len, int32_t kvg, int32_t window, int32_t query_base_pos,
                                                    int32_t key_base_pos) {
    return nomos_attn_prefix_batched_dense(stream, q_b, scores, attn_b, k_cache, v_cache, nh, nkv, l_hd, cache_hd, max_seq, S,
                                           key_len, kvg, window, query_base_pos, key_base_pos, 1);
}
NOMOS_EXPORT int32_t nomos_attn_prefill_batched_fp32(void *stream, uint64_t q_b, uint64_t, uint64_t scores, uint64_t, uint64_t attn_b,
                                                     uint64_t k_cache, uint64_t v_cache, int32_t nh, int32_t nkv, int32_t l_hd,
                                                     int32_t cache_hd, int32_t max_seq, int32_t S, int32_t kvg, int32_t window) {
    return nomos_attn_prefix_batched_dense(stream, q_b, scores, attn_b, k_cache, v_cache, nh, nkv, l_hd, cache_hd, max_seq, S, S, kvg,
                                           window, 0, 0, 0);
}
NOMOS_EXPORT int32_t nomos_attn_prefill_batched_bf16(void *stream, uint64_t q_b, uint64_t, uint64_t, uint64_t scores, uint64_t,
                                                     uint64_t, uint64_t attn_b, uint64_t k_cache, uint64_t v_cache, int32_t nh,
                                                     int32_t nkv, int32_t l_hd, int32_t cache_hd, int32_t max_seq, int32_t S,
                                                     int32_t kvg, int32_t window) {
    return nomos_attn_prefix_batched_dense(stream, q_b, scores, attn_b, k_cache, v_cache, nh, nkv, l_hd, cache_hd, max_seq, S, S, kvg,
                                           window, 0, 0, 1);
}

// -------------------------------------------------------------------- fused

static int unpack_args(const nomos_attn_args_t *u, AttnArgs &a, const char *who) {
    REQUIRE(u != nullptr, "%s: null args", who);
    REQUIRE(u->struct_bytes == sizeof(nomos_attn_args_t), "%s: struct_bytes %llu != %zu", who,
            (unsigned long long)u->struct_bytes, sizeof(nomos_attn_args_t));
    memset(&a, 0, sizeof(a));
    a.q = ptr(u->q); a.k_cache = ptr(u->k_cache); a.v_cache = ptr(u->v_cache);
    a.k_scales = ptr(u->k_scales); a.v_scales = ptr(u->v_scales);
    a.out = ptr(u->out); a.partial_out = static_cast<float *>(ptr(u->partial_out));
    a.workspace = ptr(u->workspace); a.ws_bytes = u->ws_bytes;
    a.new_k = static_cast<const float *>(ptr(u->new_k)); a.new_v = static_cast<const float *>(ptr(u->new_v));
    a.n_new = (int)u->n_new; a.new_stride = (int)u->new_stride; a.new_base_pos = (int)u->new_base_pos;
    a.kv_fmt = (int)u->kv_fmt; a.q_type = (int)u->q_type; a.out_type = (int)u->out_type;
    a.batch = (int)u->batch; a.S = (int)u->S; a.nh = (int)u->nh; a.nkv = (int)u->nkv; a.kvg = (int)u->kvg;
    a.l_hd = (int)u->l_hd; a.cache_hd = (int)u->cache_hd; a.cache_cap = (int)u->cache_cap;
    a.win_start = (int)u->win_start; a.klen = (int)u->klen; a.window = (int)u->window;
    a.softmax_scale = (float)u->softmax_scale;
    const long row_bytes = a.kv_fmt == KV_I8 ? a.cache_hd : a.cache_hd / 2;
    const long rows = (long)a.nkv * a.cache_cap;
    long scale_bytes = rows * 4;
    if (a.kv_fmt == KV_I4B32) scale_bytes = rows * ((a.l_hd + 31) / 32) * 2 + rows * 4;
    a.q_batch_stride = u->q_batch_stride ? u->q_batch_stride : (long)a.S * a.nh * a.l_hd;
    a.out_batch_stride = u->out_batch_stride ? u->out_batch_stride : (long)a.S * a.nh * a.l_hd;
    a.kv_batch_stride = u->kv_batch_stride ? u->kv_batch_stride : rows * row_bytes;
    a.scale_batch_stride = u->scale_batch_stride ? u->scale_batch_stride : scale_bytes;
    a.force_splits = (int)u->force_splits;
    a.settled_cache = (u->flags & NOMOS_ATTN_SETTLED_CACHE) ? 1 : 0;
    a.no_tma = (u->flags & NOMOS_ATTN_NO_TMA) ? 1 : 0;
    a.no_tcgen05 = (u->flags & NOMOS_ATTN_NO_TCGEN05) ? 1 : 0;
    a.tcgen05_always = (u->flags & NOMOS_ATTN_TCGEN05_ALWAYS) ? 1 : 0;
    a.no_cluster = (u->flags & NOMOS_ATTN_NO_CLUSTER) ? 1 : 0;
    return NOMOS_OK;
}

NOMOS_EXPORT int64_t nomos_attn_workspace_bytes(const nomos_attn_args_t *args) {
    AttnArgs a;
    int rc = unpack_args(args, a, "nomos_attn_workspace_bytes");
    if (rc) return rc;
    if ((rc = check_attn_geometry("nomos_attn_workspace_bytes", a.nh, a.nkv, a.l_hd, a.cache_hd, a.kvg))) return rc;
    if (a.batch <= 0 || a.S <= 0 || a.klen <= 0 || a.cache_cap <= 0 || a.win_start < 0) { set_error("nomos_attn_workspace_bytes: bad batch/S/klen/cache_cap/win_start"); return NOMOS_EBADARG; }
    return attn_workspace_bytes(a);
}

NOMOS_EXPORT int32_t nomos_attn_kernel_choice(const nomos_attn_args_t *args) {
    AttnArgs a;
    int rc = unpack_args(args, a, "nomos_attn_kernel_choice");
    if (rc) return rc;
    if ((rc = check_attn_geometry("nomos_attn_kernel_choice", a.nh, a.nkv, a.l_hd, a.cache_hd, a.kvg))) return rc;
    if (a.batch <= 0 || a.S <= 0 || a.klen <= 0 || a.cache_cap <= 0 || a.win_start < 0) { set_error("nomos_attn_kernel_choice: bad batch/S/klen/cache_cap/win_start"); return NOMOS_EBADARG; }
    return attn_kernel_choice(a);
}

NOMOS_EXPORT int32_t nomos_attn_last_launch(int32_t *kernel, int32_t *splits, int32_t *merge_route) {
    const LaunchInfo li = attn_last_launch_info();
    if (kernel) *kernel = li.kernel;
    if (splits) *splits = li.splits;
    if (merge_route) *merge_route = li.merge_route;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_attn_fused(void *stream, const nomos_attn_args_t *args) {
    AttnArgs a;
    int rc = unpack_args(args, a, "nomos_attn_fused");
    if (rc) return rc;
    if (a.nh <= 0 || a.klen <= 0) return NOMOS_OK;
    if (a.new_k || a.new_v) {
        REQUIRE(a.new_k && a.new_v && a.n_new > 0, "nomos_attn_fused: new_k/new_v/n_new inconsistent");
        REQUIRE(a.new_base_pos + a.n_new == a.win_start + a.klen, "nomos_attn_fused: the new rows must be the last keys of the window");
        // Quantize-on-write happens inside the attention kernel: the warp that owns the newest tile
        // quantises the rows, uses them, and stores them into the ring.
        if (a.new_stride == 0) a.new_stride = a.nkv * a.l_hd;
        REQUIRE(a.n_new <= a.klen && a.n_new <= a.cache_cap, "nomos_attn_fused: n_new %d exceeds the window", a.n_new);
    }
    return run_fused(as_stream(stream), a, "nomos_attn_fused");
}

// Device-visible address of a pinned host buffer (0 if the GPU cannot address it).  Asked of the runtime on
// every call: a remembered answer would go stale when the caller frees or unregisters the buffer and the
// address comes back as pageable memory, and the question costs well under a microsecond next to the
// stream synchronise of the same call.
static uint64_t device_view_of_host(uint64_t host) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, ptr(host)) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer != nullptr)
        return (uint64_t)(uintptr_t)at.devicePointer;
    cudaGetLastError();                           // not an error of the call: just not mapped
    return 0;
}

// Copies a step's inputs from GPU-addressable host memory to the device staging buffer: a few CTAs, each thread
// moving 16 bytes at a time (the host lines are read uncached; the ragged tail goes byte by byte).  It lets the
// grid launched behind it be set up at once (programmatic dependent launch): the attention kernel runs its set-up
// and, with settled cache rows, its first tile requests while these bytes cross the bus, and waits for them in
// griddepcontrol.wait.
__global__ void __launch_bounds__(256) stage_in_kernel(const uint8_t *src, uint8_t *dst, long bytes) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const long n16 = bytes / 16;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long)gridDim.x * blockDim.x)
        reinterpret_cast<uint4 *>(dst)[i] = __ldcv(reinterpret_cast<const uint4 *>(src) + i);
    if (blockIdx.x == 0 && threadIdx.x < bytes - n16 * 16) dst[n16 * 16 + threadIdx.x] = __ldcv(src + n16 * 16 + threadIdx.x);
}

NOMOS_EXPORT int32_t nomos_attn_fused_host(void *stream, const nomos_attn_args_t *args, uint64_t host_in, uint64_t dev_in,
                                           int64_t in_bytes, uint64_t host_out, uint64_t dev_out, int64_t out_bytes) {
    const char *who = "nomos_attn_fused_host";
    REQUIRE(in_bytes >= 0 && out_bytes >= 0, "%s: negative byte count", who);
    REQUIRE(in_bytes == 0 || (host_in && dev_in), "%s: null input staging pointer", who);
    REQUIRE(out_bytes == 0 || (host_out && dev_out), "%s: null output staging pointer", who);
    cudaStream_t st = as_stream(stream);
    cudaError_t e = cudaSuccess;
    // Inputs: every CTA of the attention launch reads the query, and a hundred and more CTAs reading a few hundred
    // bytes each straight from host memory measured 20 us slower than one 24 KB transfer, so they are staged in
    // device memory first -- by a small copy kernel when the host buffer is pinned, GPU-addressable, 16-byte aligned
    // and at most 64 KB (the attention grid is set up behind it while the bytes cross the bus), else by the copy
    // engine.
    if (in_bytes) {
        const uint64_t hin = (in_bytes <= (64 << 10) && ((host_in | dev_in) & 15) == 0) ? device_view_of_host(host_in) : 0;
        if (hin) {
            const int ctas = (int)std::min<long>(8, (in_bytes / 16 + 255) / 256 + 1);
            stage_in_kernel<<<ctas, 256, 0, st>>>(reinterpret_cast<const uint8_t *>(ptr(hin)), static_cast<uint8_t *>(ptr(dev_in)), (long)in_bytes);
            e = cudaGetLastError();
        } else {
            e = cudaMemcpyAsync(ptr(dev_in), ptr(host_in), (size_t)in_bytes, cudaMemcpyHostToDevice, st);
        }
    }
    if (e != cudaSuccess) { set_error("%s: host-to-device copy: %s", who, cudaGetErrorString(e)); return NOMOS_ECUDA; }
    // A small output in pinned, GPU-addressable host memory is written there by the kernel itself (a few posted
    // stores per KV head across the bus) instead of by a third stream operation; dev_out is then left untouched.
    if (args != nullptr && args->struct_bytes == sizeof(nomos_attn_args_t) && out_bytes > 0 && out_bytes <= (64 << 10) &&
        args->out >= dev_out && args->out < dev_out + (uint64_t)out_bytes) {
        const uint64_t hout = device_view_of_host(host_out);
        if (hout) {
            nomos_attn_args_t z = *args;
            z.out = hout + (z.out - dev_out);
            const int rc = nomos_attn_fused(stream, &z);
            if (rc) return rc;
            e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) { set_error("%s: synchronise: %s", who, cudaGetErrorString(e)); return NOMOS_ECUDA; }
            return NOMOS_OK;
        }
    }
    const int rc = nomos_attn_fused(stream, args);
    if (rc) return rc;
    if (out_bytes) e = cudaMemcpyAsync(ptr(host_out), ptr(dev_out), (size_t)out_bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { set_error("%s: device-to-host copy / synchronise: %s", who, cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

// ------------------------------------------------------------------- paged caches

static int fill_paged(AttnArgs &a, const char *who, uint64_t q, uint64_t k_pool, uint64_t v_pool, uint64_t ks_pool, uint64_t vs_pool,
                      uint64_t block_table, uint64_t seq_lens, uint64_t out, uint64_t workspace, int64_t ws_bytes, int batch, int nh,
                      int nkv, int kvg, int l_hd, int n_pages, int max_pages, int max_len, double softmax_scale, int q_type,
                      int out_type) {
    int rc = check_attn_geometry(who, nh, nkv, l_hd, l_hd, kvg);
    if (rc) return rc;
    if (l_hd != 128 || kvg > 8) { set_error("%s: paged caches support head_dim 128 and at most 8 query heads per KV head", who); return NOMOS_EUNSUPPORTED; }
    REQUIRE(batch > 0 && n_pages > 0 && max_pages > 0 && max_len > 0, "%s: bad batch/n_pages/max_pages/max_len", who);
    REQUIRE((long)max_pages * 128 >= max_len, "%s: max_len %d exceeds max_pages %d x 128", who, max_len, max_pages);
    REQUIRE((long)n_pages * nkv * 128 < (1l << 31), "%s: pool of %d pages too large", who, n_pages);
    REQUIRE((q_type == ET_F32 || q_type == ET_BF16) && (out_type == ET_F32 || out_type == ET_BF16), "%s: element type", who);
    memset(&a, 0, sizeof(a));
    a.q = ptr(q); a.k_cache = ptr(k_pool); a.v_cache = ptr(v_pool); a.k_scales = ptr(ks_pool); a.v_scales = ptr(vs_pool);
    a.out = ptr(out); a.workspace = ptr(workspace); a.ws_bytes = ws_bytes;
    a.block_table = static_cast<const int *>(ptr(block_table)); a.seq_lens = static_cast<const int *>(ptr(seq_lens));
    a.max_pages = max_pages; a.n_pages = n_pages;
    a.kv_fmt = KV_I8; a.q_type = q_type; a.out_type = out_type;
    a.batch = batch; a.S = 1; a.nh = nh; a.nkv = nkv; a.kvg = kvg; a.l_hd = l_hd; a.cache_hd = l_hd;
    a.cache_cap = 128;                       // rows of one KV head inside a page
    a.klen = max_len; a.softmax_scale = (float)softmax_scale;
    a.q_batch_stride = (long)nh * l_hd; a.out_batch_stride = (long)nh * l_hd;
    a.kv_batch_stride = (long)n_pages * nkv * 128 * l_hd; a.scale_batch_stride = (long)n_pages * nkv * 128 * 4;
    a.tcgen05_always = 1;
    return NOMOS_OK;
}

NOMOS_EXPORT int64_t nomos_attn_paged_workspace_bytes(int32_t batch, int32_t nh, int32_t nkv, int32_t kvg, int32_t l_hd,
                                                      int32_t max_len) {
    AttnArgs a;
    static const int dummy = 0;
    int rc = fill_paged(a, "nomos_attn_paged_workspace_bytes", 0, 0, 0, 0, 0, (uint64_t)(uintptr_t)&dummy, (uint64_t)(uintptr_t)&dummy, 0, 0,
                        0, batch, nh, nkv, kvg, l_hd, 1, (max_len + 127) / 128, max_len, 1.0, ET_F32, ET_F32);
    if (rc) return rc;
    return attn_paged_workspace_bytes(a);
}

NOMOS_EXPORT int32_t nomos_attn_paged_decode_i8(void *stream, uint64_t q, uint64_t k_pool, uint64_t v_pool, uint64_t ks_pool,
                                                uint64_t vs_pool, uint64_t block_table, uint64_t seq_lens, uint64_t out,
                                                uint64_t workspace, int64_t ws_bytes, int32_t batch, int32_t nh, int32_t nkv,
                                                int32_t kvg, int32_t l_hd, int32_t n_pages, int32_t max_pages, int32_t max_len,
                                                double softmax_scale, int32_t q_type, int32_t out_type) {
    const char *who = "nomos_attn_paged_decode_i8";
    if (batch <= 0 || nh <= 0 || max_len <= 0) return NOMOS_OK;
    REQUIRE(q && k_pool && v_pool && ks_pool && vs_pool && block_table && seq_lens && out, "%s: null pointer", who);
    REQUIRE(aligned(k_pool, 16) && aligned(v_pool, 16) && aligned(ks_pool, 16) && aligned(vs_pool, 16) && aligned(q, 4), "%s: misaligned buffer", who);
    AttnArgs a;
    int rc = fill_paged(a, who, q, k_pool, v_pool, ks_pool, vs_pool, block_table, seq_lens, out, workspace, ws_bytes, batch, nh, nkv, kvg,
                        l_hd, n_pages, max_pages, max_len, softmax_scale, q_type, out_type);
    if (rc) return rc;
    return launch_attn_paged(as_stream(stream), a);
}

NOMOS_EXPORT int32_t nomos_kv_paged_append_quant_i8(void *stream, uint64_t src_k, uint64_t src_v, uint64_t k_pool, uint64_t v_pool,
                                                    uint64_t ks_pool, uint64_t vs_pool, uint64_t block_table, uint64_t positions,
                                                    int32_t batch, int32_t nkv, int32_t l_hd, int32_t l_kvd, int32_t max_pages) {
    const char *who = "nomos_kv_paged_append_quant_i8";
    if (batch <= 0) return NOMOS_OK;
    REQUIRE(src_k && src_v && k_pool && v_pool && ks_pool && vs_pool && block_table && positions, "%s: null pointer", who);
    REQUIRE(nkv > 0 && l_hd > 0 && max_pages > 0 && l_kvd >= nkv * l_hd, "%s: bad geometry", who);
    return launch_append_paged_i8(as_stream(stream), ptr(src_k), ptr(src_v), ptr(k_pool), ptr(v_pool), ptr(ks_pool), ptr(vs_pool),
                                  static_cast<const int *>(ptr(block_table)), static_cast<const int *>(ptr(positions)), batch, nkv,
                                  l_hd, l_kvd, max_pages);
}

NOMOS_EXPORT int32_t nomos_attn_merge_partials(void *stream, uint64_t partials, int32_t G, int32_t rows, int32_t l_hd,
                                               uint64_t out, int32_t out_type) {
    if (rows <= 0) return NOMOS_OK;
    REQUIRE(partials && out && G > 0 && l_hd > 0, "nomos_attn_merge_partials: bad argument");
    REQUIRE(out_type == ET_F32 || out_type == ET_BF16, "nomos_attn_merge_partials: out_type %d", out_type);
    return launch_merge_partials(as_stream(stream), static_cast<const float *>(ptr(partials)), G, rows, l_hd, ptr(out), out_type);
}

// ------------------------------------------------- sequence-sharded decode across the GPUs of one node

NOMOS_EXPORT int64_t nomos_attn_peer_mailbox_bytes(int32_t world, int32_t rows, int32_t l_hd) {
    if (world < 1 || world > 8 || rows <= 0 || l_hd <= 0) { set_error("nomos_attn_peer_mailbox_bytes: bad world/rows/l_hd"); return NOMOS_EBADARG; }
    return attn_peer_mailbox_bytes(world, rows, l_hd);
}

// Set-up, not the hot path: the one place the library allocates device memory, because the mailbox must be an
// allocation of its own (its interprocess handle names the whole allocation) and must start zeroed.
NOMOS_EXPORT int32_t nomos_attn_peer_mailbox_create(int64_t bytes, uint64_t *dev_ptr, void *handle64) {
    const char *who = "nomos_attn_peer_mailbox_create";
    REQUIRE(bytes > 0 && dev_ptr != nullptr, "%s: bad argument", who);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 opaque bytes");
    void *m = nullptr;
    cudaError_t e = cudaMalloc(&m, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(m, 0, (size_t)bytes);
    if (e == cudaSuccess && handle64 != nullptr) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t *>(handle64), m);
    if (e != cudaSuccess) {
        set_error("%s: %s", who, cudaGetErrorString(e));
        if (m) cudaFree(m);
        return NOMOS_ECUDA;
    }
    *dev_ptr = (uint64_t)(uintptr_t)m;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_attn_peer_mailbox_open(const void *handle64, uint64_t *dev_ptr) {
    const char *who = "nomos_attn_peer_mailbox_open";
    REQUIRE(handle64 != nullptr && dev_ptr != nullptr, "%s: null pointer", who);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void *m = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&m, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_error("%s: %s", who, cudaGetErrorString(e)); return NOMOS_ECUDA; }
    *dev_ptr = (uint64_t)(uintptr_t)m;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_attn_peer_mailbox_close(uint64_t dev_ptr, int32_t own) {
    if (dev_ptr == 0) return NOMOS_OK;
    cudaError_t e = own ? cudaFree(ptr(dev_ptr)) : cudaIpcCloseMemHandle(ptr(dev_ptr));
    if (e != cudaSuccess) { set_error("nomos_attn_peer_mailbox_close: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_attn_seq_sharded(void *stream, const nomos_attn_args_t *args, const nomos_attn_peer_t *peer) {
    const char *who = "nomos_attn_seq_sharded";
    AttnArgs a;
    int rc = unpack_args(args, a, who);
    if (rc) return rc;
    REQUIRE(peer != nullptr && peer->struct_bytes == sizeof(nomos_attn_peer_t), "%s: null peer block or struct_bytes mismatch", who);
    REQUIRE(peer->world >= 1 && peer->world <= 8 && peer->rank >= 0 && peer->rank < peer->world, "%s: rank %lld of %lld", who,
            (long long)peer->rank, (long long)peer->world);
    if (a.nh <= 0) return NOMOS_OK;
    REQUIRE(a.klen > 0, "%s: every shard must hold at least one key of the window", who);
    REQUIRE(a.out != nullptr && a.partial_out == nullptr, "%s: the call writes the final output (out) and exports no partials", who);
    if (a.new_k || a.new_v) {
        REQUIRE(a.new_k && a.new_v && a.n_new > 0, "%s: new_k/new_v/n_new inconsistent", who);
        REQUIRE(a.new_base_pos + a.n_new == a.win_start + a.klen, "%s: the new rows must be the last keys of the shard", who);
        if (a.new_stride == 0) a.new_stride = a.nkv * a.l_hd;
        REQUIRE(a.n_new <= a.klen && a.n_new <= a.cache_cap, "%s: n_new %d exceeds the window", who, a.n_new);
    }
    if (peer->world == 1) return run_fused(as_stream(stream), a, who);
    REQUIRE(peer->step != 0, "%s: step numbers start at 1 (a zeroed mailbox reads as step 0)", who);
    REQUIRE(a.batch > 0 && a.S > 0, "%s: bad batch/S", who);
    const long need = attn_peer_mailbox_bytes((int)peer->world, (long)a.batch * a.S * a.nh, a.l_hd);
    if (peer->mailbox_bytes < need) {
        set_error("%s: mailboxes hold %lld bytes, this call needs %ld", who, (long long)peer->mailbox_bytes, need);
        return NOMOS_ECAPACITY;
    }
    for (int g = 0; g < peer->world; ++g) {
        REQUIRE(peer->mailbox[g] != 0 && aligned(peer->mailbox[g], 16), "%s: mailbox %d null or misaligned", who, g);
        a.peer_box[g] = ptr(peer->mailbox[g]);
    }
    a.peer_rank = (int)peer->rank; a.peer_world = (int)peer->world; a.peer_seq = peer->step; a.peer_timeout_us = (long)peer->timeout_us;
    return run_fused(as_stream(stream), a, who);
}

NOMOS_EXPORT int32_t nomos_attn_seq_sharded_status(void *stream, int32_t clear) {
    cudaError_t e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) { set_error("nomos_attn_seq_sharded_status: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    uint32_t bits = 0;
    int rc = nomos::read_attn_faults(&bits, false);
    if (rc) return rc;
    if (bits & 4u) {
        if (clear) nomos::clear_attn_fault_bits(4u);
        set_error("nomos_attn_seq_sharded: a peer's partial result did not arrive within the time limit; no output was written");
        return NOMOS_ENOTWRITTEN;
    }
    return NOMOS_OK;
}

// ------------------------------------------------- fused call without a caller workspace
//
// Some callers of this library cannot give it a workspace: the Nomos engine hands its whole
// device-memory budget out once at start-up (the KV cache is sized to fill the card, and a
// failed cudaMalloc is fatal to the serving daemon), and a decode loop must not call the
// allocator at all because cudaMalloc/cudaFree synchronise the device.  For them the split
// scratch below is part of the library image: a fixed array in device memory, so this entry
// point never calls cudaMalloc, cudaFree or any allocating routine.
//
// Cost and limits, all deliberate:
//   * every GPU that loads the library holds NOMOS_STATIC_WS_BYTES (4 MiB) until the process exits;
//   * a call whose split scratch would be larger is refused with NOMOS_ECAPACITY;
//   * all calls on one device share the array, which keeps the previous call's contents.  Nothing in
//     it has to start at zero: the arrival counters carry a tag the library recognises (an untagged word reads
//     as "no arrivals yet"; the merging CTA leaves the word tagged with a zero count) and the partial results
//     are fully rewritten before they are read, so no clearing pass is needed.  Two calls that overlap
//     on the GPU (different streams) would overwrite each other's partial results: callers must
//     keep calls to this entry point ordered on a device, e.g. by using one stream.
//   * the first call on each device looks the array's device address up (cudaGetSymbolAddress);
//     make that first call before starting any stream capture.
#define NOMOS_STATIC_WS_BYTES (4 << 20)
static __device__ __align__(256) unsigned char g_static_ws[NOMOS_STATIC_WS_BYTES];

// In host code `g_static_ws` is only a handle for the runtime, not a device address; the address
// the kernels need is resolved here, once per device, with that device current.
static int static_ws_address(void **out) {
    static void *cached[64] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("nomos_attn_fused_static_ws: cannot identify the current device (%s)", cudaGetErrorString(e));
        return NOMOS_ECUDA;
    }
    if (cached[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_ws);
        if (e != cudaSuccess || p == nullptr) {
            set_error("nomos_attn_fused_static_ws: cudaGetSymbolAddress failed on device %d (%s)", dev, cudaGetErrorString(e));
            return NOMOS_ECUDA;
        }
        cached[dev] = p;
    }
    *out = cached[dev];
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_attn_fused_static_ws(void *stream, const nomos_attn_args_t *args) {
    AttnArgs a;
    int rc = unpack_args(args, a, "nomos_attn_fused_static_ws");
    if (rc) return rc;
    if (a.nh <= 0 || a.klen <= 0) return NOMOS_OK;
    REQUIRE(a.new_k == nullptr && a.new_v == nullptr, "nomos_attn_fused_static_ws: fused append is not offered here; append first");
    if ((rc = check_attn_geometry("nomos_attn_fused_static_ws", a.nh, a.nkv, a.l_hd, a.cache_hd, a.kvg))) return rc;
    REQUIRE(a.batch > 0 && a.S > 0 && a.cache_cap > 0 && a.win_start >= 0, "nomos_attn_fused_static_ws: bad batch/S/cache_cap/win_start");
    const long need = attn_workspace_bytes(a);
    if (need < 0) return (int32_t)need;
    if (need > NOMOS_STATIC_WS_BYTES) {
        set_error("nomos_attn_fused_static_ws: this call needs %ld bytes of split scratch, the built-in array holds %d; "
                  "use nomos_attn_fused with a caller workspace", need, NOMOS_STATIC_WS_BYTES);
        return NOMOS_ECAPACITY;
    }
    void *ws = nullptr;
    if ((rc = static_ws_address(&ws))) return rc;
    a.workspace = ws;                       // the resolved device address, never the host-side symbol
    a.ws_bytes = NOMOS_STATIC_WS_BYTES;
    return run_fused(as_stream(stream), a, "nomos_attn_fused_static_ws");
}
