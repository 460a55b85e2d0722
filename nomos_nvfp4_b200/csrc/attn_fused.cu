// Split-K flash-decoding attention over the PACKED quantised KV ring (sm_100a): host side of both
// kernels -- the mma.sync kernel described here (attn_fused_kernel.cuh) and the tcgen05 kernel for
// int8 / head_dim 128 (attn_tc5_kernel.cuh, described there; plan and launch further down).
//
// Replaces, in one launch, what the reference does per layer with 5-7 launches: window reader -> int8/bf16 scratch
// (lib/kv_cache_quant.mojo:221-249,708-800,925-953), QK (lib/attention_gpu_int8.mojo:48-91
// or cuBLAS, lib/attention_gpu.mojo:231-238), row softmax (lib/softmax_gpu_mojo.mojo:37-134)
// and PV (lib/attention_gpu_int8.mojo:94-137 / lib/attention_gpu.mojo:241-248), and for
// S>1 the multirow verify kernels (lib/attention_gpu_int8.mojo:322-584).
//
// Work decomposition
//   grid = (splits x head-dim slices, nkv, batch * row_groups); one CTA streams one KV head's
//   chunk of the window and serves every query row of the GQA group from the same bytes.
//   Each warp owns a private ring of 32-token tiles in an XOR-swizzled layout, with no CTA
//   barrier in the loop.  Whole tiles of 64- or 128-byte rows are fetched by TMA (one lane
//   issues two cp.async.bulk.tensor boxes + two bulk copies of scales against the stage's
//   mbarrier); ragged or ring-wrapping tiles and wider rows use 16-byte cp.async copies.
// Arithmetic per warp tile (all contractions on the tensor cores, no integer->float
// conversion of cache bytes anywhere)
//   QK:  int8 MMA m16n8k32.  A = the query rows as two int8 limbs of a 16-bit fixed
//        point (rows g / g+8 of the M tile = high / low limb of slot g), B = the K
//        bytes exactly as stored.  The int32 result is exact; one fp32 multiply per
//        (token, slot) applies q_scale * k_scale.
//   softmax: online, base-2, in the C-fragment registers (two xor-shuffles per tile).
//   PV:  u8 x s8 MMA m16n8k32 over the whole 32-token tile.  A = the softmax weights
//        times v_scale as two u8 limbs of a 16-bit fixed point relative to the tile
//        (the QK C fragment is already in A-fragment order), B = the V bytes as
//        stored, transposed by ldmatrix.trans + one byte permute.  Exact int32 sums
//        are folded into fp32 accumulators with the tile's weight.
// The un-normalised (m, l, o) of the warps are merged in shared memory, then across splits
// inside the same launch by the last CTA of the (batch, head, row group) to arrive
// (merge_splits_in_kernel), or exported for the multi-GPU all-gather (merge_kernel runs after it).
#include <algorithm>
#include <cstring>
#include <mutex>

#include <cudaTypedefs.h>     // PFN_cuTensorMapEncodeTiled

#include "attn_fused_kernel.cuh"
#include "attn_tc5_kernel.cuh"
#include "attn_prefill_kernel.cuh"

#ifndef NOMOS_DS512
#define NOMOS_DS512 4
#endif
namespace nomos {

using namespace fused;

namespace {

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

// ------------------------------------------------------------------ tensor maps
// cuTensorMapEncodeTiled is resolved through the runtime, so the library links against
// cudart only.  A null result (old driver) just keeps every tile on the cp.async path.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// kind 0: {row bytes, rows, batch} view of one byte plane of the cache, box = box_rows rows,
//         swizzled by the row length (64 or 128 bytes);
// kind 1: {rows, batch} view of an fp32 row-scale plane, box = box_rows scales.
struct MapKey {
    const void *base; int kind, row_bytes, row_stride, rows, batch, box_rows; long batch_stride;
    bool operator==(const MapKey &o) const {
        return base == o.base && kind == o.kind && row_bytes == o.row_bytes && row_stride == o.row_stride && rows == o.rows &&
               batch == o.batch && box_rows == o.box_rows && batch_stride == o.batch_stride;
    }
};
static bool encode_plane(const MapKey &k, CUtensorMap *out) {
    // small per-thread cache: a decode loop alternates between a few layer caches
    constexpr int NCACHE = 64;
    struct Entry { MapKey key; CUtensorMap map; bool used = false; };
    thread_local Entry cache[NCACHE];
    thread_local int next = 0;
    for (auto &e : cache)
        if (e.used && e.key == k) { *out = e.map; return true; }
    EncodeTiledFn enc = encode_tiled_fn();
    if (enc == nullptr) return false;
    const cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap m;
    CUresult rc;
    if (k.kind == 0) {
        const cuuint64_t dims[3] = {(cuuint64_t)k.row_bytes, (cuuint64_t)k.rows, (cuuint64_t)k.batch};
        const cuuint64_t strides[2] = {(cuuint64_t)k.row_stride,
                                       (cuuint64_t)(k.batch > 1 ? k.batch_stride : (long)k.rows * k.row_stride)};
        const cuuint32_t box[3] = {(cuuint32_t)k.row_bytes, (cuuint32_t)k.box_rows, 1};
        const CUtensorMapSwizzle swz = k.row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
        rc = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(k.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        const cuuint64_t dims[2] = {(cuuint64_t)k.rows, (cuuint64_t)k.batch};
        const cuuint64_t strides[1] = {(cuuint64_t)(k.batch > 1 ? k.batch_stride : (long)k.rows * 4)};
        const cuuint32_t box[2] = {(cuuint32_t)k.box_rows, 1};
        rc = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(k.base), dims, strides, box, estr,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (rc != CUDA_SUCCESS) return false;
    Entry &e = cache[next];
    next = (next + 1) % NCACHE;
    e.key = k; e.map = m; e.used = true;
    *out = m;
    return true;
}

// Sticky per-device fault word the kernels OR into when a bounded wait runs out.
__device__ unsigned int g_attn_fault;
static unsigned int *fault_word() {
    static unsigned int *cached[64];
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_attn_fault) == cudaSuccess) cached[dev] = static_cast<unsigned int *>(ptr);
    }
    return cached[dev];
}

#ifndef NOMOS_COOP_LAST_K
#define NOMOS_COOP_LAST_K 64
#endif
static constexpr int COOP_LAST_K = NOMOS_COOP_LAST_K;       // CTAs sharing a mid-sized unit merge

static thread_local LaunchInfo t_last_launch = {0, 0, 0};
static void note_launch(int kernel, const KParams &p) {
    t_last_launch.kernel = kernel;
    t_last_launch.splits = p.splits;
    t_last_launch.merge_route = p.splits <= 1 ? 0 : p.cluster_merge ? 3 : p.coop_merge ? 2 : 1;
}

struct Plan {
    int mt, row_groups, tile0, ntiles, splits, tiles_per_split, grows;
};

// How many CTAs of a unit share its merge (0: the last one to arrive merges all of it).  The last K to arrive each
// take 1/K of the rows once all have arrived; earlier arrivals leave at once.  Worth it when the partials of a unit
// are large (a verify call: 84 KB, 4 us through one SM; a 512-wide head: 600 KB), allowed when the whole grid is
// resident at once (a CTA then waits for CTAs that are running, not for ones that have no SM yet), the outputs take
// 8-byte stores and no peer exchange follows.  Measured on the 9-split verify call (one launch after another):
// K = 2: 27.6 us (as without), K = 4: 27.0, K = 9 (every CTA of the unit): 26.8 -- so K is the unit's CTA count.
static int use_coop_merge(const AttnArgs &a, int splits, int arrivals, long ctas, int occupancy, int rows_per_unit, int hd) {
    if (splits < 2 || splits > 64 || arrivals != splits || a.peer_world > 1) return 0;
    if (ctas > (long)device_info().sm_count * occupancy) return 0;
    const bool al8 = ((reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.partial_out)) & 7) == 0 && (a.out_batch_stride & 3) == 0;
    if (!al8) return 0;
    const long bytes = (long)splits * rows_per_unit * (hd + 2) * 4;
    if (bytes >= 256 * 1024) return arrivals;
    if (bytes >= 48 * 1024 && splits <= 12 && hd % 64 == 0) return std::min(arrivals, COOP_LAST_K);
    return 0;
}

// Peer fields of a sequence-sharded call; returns where this rank's own merged rows go.
static float *fill_peer_params(KParams &p, const AttnArgs &a, long grows) {
    p.peer_world = a.peer_world > 1 ? a.peer_world : 0;
    p.peer_rank = a.peer_rank; p.peer_seq = a.peer_seq;
    p.peer_timeout_ns = (unsigned long long)(a.peer_timeout_us > 0 ? a.peer_timeout_us : 1000000) * 1000ull;
    for (int g = 0; g < 8; ++g) { p.peer_rows[g] = nullptr; p.peer_flags[g] = nullptr; }
    if (p.peer_world == 0) return nullptr;
    const long rows_bytes = attn_peer_mailbox_rows_bytes(a.peer_world, grows, a.l_hd);
    for (int g = 0; g < a.peer_world; ++g) {
        p.peer_rows[g] = static_cast<float *>(a.peer_box[g]);
        p.peer_flags[g] = reinterpret_cast<unsigned long long *>(static_cast<char *>(a.peer_box[g]) + rows_bytes);
    }
    const size_t blk = (size_t)grows * (a.l_hd + 2);
    return p.peer_rows[a.peer_rank] + ((size_t)(a.peer_seq & 1ull) * a.peer_world + a.peer_rank) * blk;
}

// Window rows [0, settled_rows) may be requested before the stream-order wait when the caller set
// NOMOS_ATTN_SETTLED_CACHE.  The newest 2 x max(S, n_new) rows are left out: this call's own rows, and as many
// before them, which is where the preceding call of a decode / verify loop on the same cache (same batch size,
// any number of accepted rows) wrote the rows it appended -- whether through its own fused append or through an
// append kernel ordered before it.
static int settled_rows(const AttnArgs &a) {
    return a.settled_cache ? std::max(0, a.klen - 2 * std::max(a.S, a.n_new)) : 0;
}

template <int FMT, int HD, int MT, int DS, int QS>
static int kernel_occupancy() {
    static int occ[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (occ[dev] == 0) {
        using C = Cfg<FMT, HD, MT, DS, QS>;
        cudaFuncSetAttribute(attn_fused_kernel<FMT, HD, MT, DS, QS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        int n = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_fused_kernel<FMT, HD, MT, DS, QS>, C::NW * 32, C::SMEM_BYTES);
        occ[dev] = n > 0 ? n : 1;
    }
    return occ[dev];
}

// Query-row tiles per CTA.  Up to 24 rows (e.g. 9 verify tokens x 2 group heads) run as up to three
// 8-row groups of the 12-warp kernel: the groups stream the same cache bytes concurrently (one DRAM
// read, served to the other groups from L2), which measured faster than one 24-row CTA with 8 warps
// and 255 registers.  Beyond that the 24-row kernel keeps the number of L2 re-reads down.
static int pick_mt(int slots, int hd = 128) { return (slots <= 24 || hd > 128) ? 1 : 3; }

static Plan make_plan(const AttnArgs &a, int occupancy, int hd, int nwarp, int dsplit = 1) {
    Plan pl;
    const int slots = a.S * a.kvg;
    pl.mt = pick_mt(slots, hd);
    pl.row_groups = (slots + 8 * pl.mt - 1) / (8 * pl.mt);
    // first window index any row needs
    int j_begin = 0;
    if (a.window > 0) j_begin = std::max(0, (a.klen - (a.S - 1)) - a.window);
    pl.tile0 = j_begin / TILE;
    pl.ntiles = (a.klen + TILE - 1) / TILE - pl.tile0;
    pl.grows = a.batch * a.S * a.nh;
    const int units = a.nkv * a.batch * pl.row_groups * dsplit;      // CTAs per sequence split
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
            const long fixed = 16 + 16L * units;                    // alignment slack + arrival and departure counters
            max_splits = (int)std::max<long>(1, std::min<long>(max_splits, a.workspace ? (a.ws_bytes - fixed) / per_split : 0));
        }
        // The search costs about 3 us of host time at 1024 tiles; a decode loop asks the same question step after
        // step (the tile count moves every 32 tokens), so the last few answers are remembered per thread.
        struct Memo { int ntiles, units, slots_gpu, nwarp, max_splits, best; };
        static thread_local Memo memo[4] = {};
        static thread_local int memo_next = 0;
        bool hit = false;
        for (const Memo &m : memo)
            if (m.best > 0 && m.ntiles == pl.ntiles && m.units == units && m.slots_gpu == slots_gpu && m.nwarp == nwarp && m.max_splits == max_splits) {
                best = m.best; hit = true; break;
            }
        for (int n = 1; !hit && n <= max_splits; ++n) {
            const int tps = (pl.ntiles + n - 1) / n;
            const int n_eff = (pl.ntiles + tps - 1) / tps;
            if (n_eff != n) continue;
            const int per_warp = (tps + nwarp - 1) / nwarp;
            const long ctas = (long)units * n;
            const long waves = (ctas + slots_gpu - 1) / slots_gpu;
            // in units of one warp-tile (~1.7 us on B200): streaming rounds plus ~1.5 of CTA start-up per wave, and what a split costs at the
            // end (partial store, fence, arrival, merge by the last CTA) when there is more than one
            const double cost = (double)waves * (per_warp + 1.5) + (n > 1 ? 1.4 + 0.02 * n : 0.0);
            if (cost < best_cost) { best_cost = cost; best = n; }
        }
        if (!hit) { memo[memo_next] = Memo{pl.ntiles, units, slots_gpu, nwarp, max_splits, best}; memo_next = (memo_next + 1) % 4; }
    }
    pl.tiles_per_split = (pl.ntiles + best - 1) / best;
    pl.splits = (pl.ntiles + pl.tiles_per_split - 1) / pl.tiles_per_split;
    return pl;
}

// Whether a launch of this instance with `splits` CTAs per unit can run its units as thread-block clusters
// (cluster x = splits, at most 16; more than 8 needs the non-portable size) with every cluster of the grid
// resident at once.  Answered by the occupancy calculator once per (device, splits) and remembered; a launch
// that the driver refuses switches the route off for the instance.
template <int FMT, int HD, int MT, int DS, int QS>
static bool cluster_route(int splits, long clusters) {
    using C = Cfg<FMT, HD, MT, DS, QS>;
    static std::mutex mu;
    static int max_clusters[64][17];          // 0 = not asked yet, -1 = no
    static bool off = false;
    std::lock_guard<std::mutex> lock(mu);
    if (clusters < 0) { off = true; return false; }           // (called with -1 after a refused launch)
    if (off || !C::CLUSTER_OK || splits < 2 || splits > 16) return false;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    int &n = max_clusters[dev][splits];
    if (n == 0) {
        n = -1;
        if (splits <= 8 || cudaFuncSetAttribute(attn_fused_kernel<FMT, HD, MT, DS, QS>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(splits, 1, 1); cfg.blockDim = dim3(C::NW * 32); cfg.dynamicSmemBytes = C::SMEM_BYTES;
            cfg.attrs = at; cfg.numAttrs = 1;
            int got = 0;
            if (cudaOccupancyMaxActiveClusters(&got, attn_fused_kernel<FMT, HD, MT, DS, QS>, &cfg) == cudaSuccess && got > 0) n = got;
            else cudaGetLastError();
        } else {
            cudaGetLastError();
        }
    }
    return n > 0 && clusters <= n;
}

template <int FMT, int HD, int MT, int DS = 1, int QS = 1>
static int launch_inst(cudaStream_t st, const AttnArgs &a, bool query_ws, long *ws_needed) {
    using C = Cfg<FMT, HD, MT, DS, QS>;
    const int occ = kernel_occupancy<FMT, HD, MT, DS, QS>();
    const Plan pl = make_plan(a, occ, HD, C::NQ, DS);          // C::NQ tile streams per CTA (warps, or quads of QS warps)
    const long units = (long)a.nkv * a.batch * pl.row_groups;
    const long part_bytes = (((long)pl.splits * pl.grows * (HD + 2) * 4) + 15) / 16 * 16;
    // a sequence-sharded call always ends in the unit's merging CTA (it runs the exchange), also with one split
    const bool in_kernel_merge = pl.splits > 1 || a.peer_world > 1;
    // 16 bytes per unit: the arrival word (count, round bit and tag) and a spare
    const long need = in_kernel_merge ? part_bytes + units * 16 : 0;
    if (query_ws) { *ws_needed = part_bytes + units * 16; return NOMOS_OK; }   // also enough for a sequence-sharded call, which merges in the kernel even with one split
    if (need > a.ws_bytes || (need > 0 && a.workspace == nullptr)) {
        set_error("attention workspace too small: need %ld bytes, have %ld", need, a.ws_bytes);
        return NOMOS_ECAPACITY;
    }
    KParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = static_cast<const uint8_t *>(a.q);
    p.k_cache = static_cast<const uint8_t *>(a.k_cache);
    p.v_cache = static_cast<const uint8_t *>(a.v_cache);
    p.k_scales = static_cast<const uint8_t *>(a.k_scales);
    p.v_scales = static_cast<const uint8_t *>(a.v_scales);
    p.out = static_cast<uint8_t *>(a.out);
    const bool direct_export = (!in_kernel_merge && a.partial_out != nullptr);
    p.partial = direct_export ? a.partial_out : static_cast<float *>(a.workspace);
    p.write_partial = (in_kernel_merge || direct_export) ? 1 : 0;
    p.export_nat = direct_export ? 1 : 0;
    p.counters = in_kernel_merge ? reinterpret_cast<unsigned long long *>(static_cast<char *>(a.workspace) + part_bytes) : nullptr;
    p.splits = pl.splits;
    p.arrivals = pl.splits * DS;
    p.coop_merge = use_coop_merge(a, pl.splits, p.arrivals, (long)pl.splits * DS * units, occ, std::min(C::NSLOT, a.S * a.kvg), HD);
    p.partial_export = a.partial_out;
    if (float *own = fill_peer_params(p, a, pl.grows)) p.partial_export = own;
    // splits of a unit as one thread-block cluster merging through distributed shared memory: plain calls only
    // (final output, no export, no peer exchange), every cluster resident at once, and at least four query rows per
    // unit or at most four splits (small clusters start as easily as single CTAs: the 1024-key ring of a
    // sliding-window layer, 16 KV heads x 3 splits, replays at 8.0 against 8.4 us per call).  Measured against the arrival-counter merge, launches back to back: 8 KV heads x 4 group heads, 9
    // splits, 16384 keys 15.4 against 17.1 us; 4 x 8, 16 splits, 4096 keys 10.7 against 12.8 us; but 12 or 15 KV
    // heads x 2 group heads, 9 splits, 32768 keys 23.1 / 26.3 against 22.8 / 26.1 us (a two-row merge is one L2
    // round trip, and a cluster only starts when nine SMs of one GPC are free).  On B200 at most 15 clusters of 7 to
    // 9 CTAs of this kernel are resident (74 of 2, 33 of 4, 7 of 11 to 16), so 16 KV heads x 9 splits never qualify.
    p.cluster_merge = (!a.no_cluster && pl.splits > 1 && a.partial_out == nullptr && a.peer_world <= 1 && a.out != nullptr &&
                       (std::min(C::NSLOT, a.S * a.kvg) >= 4 || pl.splits <= 4) && cluster_route<FMT, HD, MT, DS, QS>(pl.splits, units)) ? 1 : 0;
    if (p.cluster_merge) p.coop_merge = 0;
    p.early_rows = settled_rows(a);
    // (row groups and head-dim slice CTAs share their bytes through L2; configuration 2: 27.4 -> 25.6 us per launch)
    p.kv_read_once = (pl.row_groups == 1 && DS == 1 && (long)a.batch * a.nkv * a.klen * 2 * a.cache_hd < (1024l << 20)) ? 1 : 0;
    p.new_k = a.new_k; p.new_v = a.new_v;
    p.n_new = a.new_k ? a.n_new : 0; p.new_stride = a.new_stride; p.new_base_pos = a.new_base_pos;
    p.k_cache_w = const_cast<uint8_t *>(p.k_cache); p.v_cache_w = const_cast<uint8_t *>(p.v_cache);
    p.k_scales_w = const_cast<uint8_t *>(p.k_scales); p.v_scales_w = const_cast<uint8_t *>(p.v_scales);
    if (pl.splits > MERGE_MAX_G) { set_error("too many splits (%d)", pl.splits); return NOMOS_EUNSUPPORTED; }
    p.q_type = a.q_type; p.out_type = a.out_type;
    p.S = a.S; p.nh = a.nh; p.nkv = a.nkv; p.kvg = a.kvg; p.cache_hd = a.cache_hd; p.cache_cap = a.cache_cap;
    p.win_start = a.win_start; p.klen = a.klen; p.window = a.window;
    p.tile0 = pl.tile0; p.ntiles = pl.ntiles; p.tiles_per_split = pl.tiles_per_split;
    p.row_groups = pl.row_groups; p.grows = pl.grows;
    p.qk_scale_log2 = a.softmax_scale * LOG2E;
    p.q_batch_stride = a.q_batch_stride; p.kv_batch_stride = a.kv_batch_stride;
    p.scale_batch_stride = a.scale_batch_stride; p.out_batch_stride = a.out_batch_stride;
    p.kvg_magic = a.kvg > 1 ? (unsigned int)(((1ull << 32) + a.kvg - 1) / a.kvg) : 0u;
    p.fault = fault_word();
    if (p.fault == nullptr) { set_error("attn_fused: device fault word unavailable"); return NOMOS_ECUDA; }
    // TMA for whole tiles when the row geometry matches a hardware swizzle pattern and the
    // planes satisfy the tensor-map rules (16-byte aligned base and strides).
    TmaMaps tm;
    std::memset(&tm, 0, sizeof(tm));
    p.use_tma = 0;
    if (C::TMA_OK && !a.no_tma) {
        const int row_stride = (FMT == KV_I8) ? a.cache_hd : a.cache_hd / 2;
        const auto al16 = [](const void *x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
        const long rows = (long)a.nkv * a.cache_cap;
        const bool ok = al16(a.k_cache) && al16(a.v_cache) && row_stride % 16 == 0 && (a.batch == 1 || a.kv_batch_stride % 16 == 0) &&
                        rows < (1l << 31);
        if (ok) {
            const MapKey kk{a.k_cache, 0, C::ROWB, row_stride, (int)rows, a.batch, TILE, a.kv_batch_stride};
            const MapKey kv{a.v_cache, 0, C::ROWB, row_stride, (int)rows, a.batch, TILE, a.kv_batch_stride};
            if (encode_plane(kk, &tm.k) && encode_plane(kv, &tm.v)) {
                p.use_tma = 1;
                if (al16(a.k_scales) && al16(a.v_scales) && ((long)a.cache_cap * C::SCB) % 16 == 0 &&
                    (a.batch == 1 || a.scale_batch_stride % 16 == 0))
                    p.use_tma |= 2;
            }
        }
    }
    dim3 grid(pl.splits * DS, a.nkv, a.batch * pl.row_groups);
    // The warming pass of the query preparation (run it once before the stream-order wait on whatever the buffers hold,
    // to have the code in the instruction caches) is off for this kernel: since every load it repeats goes through
    // L2 it no longer pays -- 27.9 against 28.2 us per launch back to back, 34.4 against 35.3 us for a launch on its
    // own, 29.4 against 31.3 us with a fused append, and 44 against 50 us for a synchronous step that appends a row
    // (its quantisation ran twice).  When the pass was introduced (loads through the read-only path) it took the
    // verify call's wait -> first tile from 6.0 to 1.6 us; the kernels keep the code, nothing switches it on.
    p.dry_pass = 0;
    // Launched with programmatic stream serialization allowed: after a grid that triggers early
    // (another attention call of this library) the grid is set up while the predecessor drains and
    // blocks in griddepcontrol.wait before its first global access; after any other kernel it
    // starts when that kernel has completed, as usual.
    cudaLaunchAttribute pdl[2];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    pdl[1].id = cudaLaunchAttributeClusterDimension;
    pdl[1].val.clusterDim.x = pl.splits; pdl[1].val.clusterDim.y = 1; pdl[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t mcfg = {};
    mcfg.gridDim = grid; mcfg.blockDim = dim3(C::NW * 32); mcfg.dynamicSmemBytes = C::SMEM_BYTES; mcfg.stream = st;
    mcfg.attrs = pdl; mcfg.numAttrs = p.cluster_merge ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&mcfg, attn_fused_kernel<FMT, HD, MT, DS, QS>, p, tm);
    if (e != cudaSuccess && p.cluster_merge) {
        // the driver refused the cluster shape: this instance goes back to the arrival-counter merge for good
        cudaGetLastError();
        cluster_route<FMT, HD, MT, DS, QS>(0, -1);
        p.cluster_merge = 0;
        p.coop_merge = use_coop_merge(a, pl.splits, p.arrivals, (long)pl.splits * DS * units, occ, std::min(C::NSLOT, a.S * a.kvg), HD);
        mcfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&mcfg, attn_fused_kernel<FMT, HD, MT, DS, QS>, p, tm);
    }
    if (e != cudaSuccess) { set_error("attn_fused launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    note_launch(0, p);
    return NOMOS_OK;
}

// ------------------------------------------------------------------ tcgen05 path
// int8 KV, head_dim 128, up to 24 query rows per KV head (decode and verify), with or without fused
// quantize-on-write: the contraction runs on tcgen05 with accumulators in tensor memory
// (attn_tc5_kernel.cuh).  Everything else stays on the kernel above.
static bool tc5_eligible(const AttnArgs &a);
static int launch_tc5(cudaStream_t st, const AttnArgs &a, bool q, long *ws);

static bool tc5_eligible(const AttnArgs &a) {
    if (a.kv_fmt != KV_I8 || a.l_hd != 128 || a.no_tma || a.no_tcgen05) return false;
    if (a.new_k != nullptr && (a.n_new > tc5::NEW_MAX || a.cache_hd != a.l_hd)) return false;
    // one CTA serves at most 24 query rows per KV head (9 verify tokens x 2 group heads = 18); more go to the
    // mma.sync kernel, which cuts them into row groups
    if (a.S * a.kvg > 24 && !a.tcgen05_always) return false;
    if (encode_tiled_fn() == nullptr) return false;
    const auto al16 = [](const void *x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    if (!al16(a.k_cache) || !al16(a.v_cache) || a.cache_hd % 16 != 0) return false;
    if (a.batch > 1 && a.kv_batch_stride % 16 != 0) return false;
    if ((long)a.nkv * a.cache_cap >= (1l << 31)) return false;
    return true;
}

struct Tc5Plan {
    int ns, row_groups, tbase, ntiles, splits, tiles_per_split, grows;
};

template <int NS>
static int tc5_occupancy() {
    static int occ[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (occ[dev] == 0) {
        cudaFuncSetAttribute(tc5::attn_tc5_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc5::Cfg<NS>::SMEM_BYTES);
        cudaFuncSetAttribute(tc5::attn_tc5_kernel<NS>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        int n = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, tc5::attn_tc5_kernel<NS>, tc5::Cfg<NS>::NTHREADS, tc5::Cfg<NS>::SMEM_BYTES);
        n = n > 0 ? n : 1;
        // The occupancy query has answered 1 for the decode instances although two of their CTAs (111 KB of
        // shared memory, 256 threads x <= 128 registers, 256 tensor-memory columns each) do run side by side
        // on an SM.  The plan uses the residency the launch bounds were written for only when this device's own
        // limits and this build's resource use say that it fits; otherwise the query's answer stands.
        if (n < tc5::Cfg<NS>::MIN_CTAS) {
            cudaFuncAttributes fa;
            int smem_sm = 0, smem_rsv = 0, regs_sm = 0, thr_sm = 0;
            const int want = tc5::Cfg<NS>::MIN_CTAS;
            const bool known = cudaFuncGetAttributes(&fa, tc5::attn_tc5_kernel<NS>) == cudaSuccess &&
                               cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess &&
                               cudaDeviceGetAttribute(&smem_rsv, cudaDevAttrReservedSharedMemoryPerBlock, dev) == cudaSuccess &&
                               cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev) == cudaSuccess &&
                               cudaDeviceGetAttribute(&thr_sm, cudaDevAttrMaxThreadsPerMultiProcessor, dev) == cudaSuccess;
            if (known) {
                const long smem_cta = (long)tc5::Cfg<NS>::SMEM_BYTES + (long)fa.sharedSizeBytes + smem_rsv;
                const long regs_cta = (long)((fa.numRegs + 7) / 8 * 8) * tc5::Cfg<NS>::NTHREADS;   // registers are granted in units of 8 per thread
                const bool fits = want * smem_cta <= smem_sm && want * regs_cta <= regs_sm && want * tc5::Cfg<NS>::NTHREADS <= thr_sm &&
                                  want * tc5::Cfg<NS>::TMEM_COLS <= 512;
                if (fits) n = want;
            }
        }
        occ[dev] = n;
    }
    return occ[dev];
}

static Tc5Plan tc5_plan(const AttnArgs &a, int ns, int occupancy) {
    Tc5Plan pl;
    const int slots = a.S * a.kvg;
    pl.ns = ns;
    pl.row_groups = (slots + ns - 1) / ns;
    pl.tbase = a.window > 0 ? std::max(0, (a.klen - (a.S - 1)) - a.window) : 0;
    const bool paged = a.block_table != nullptr;
    // the window's keys as up to two runs of ring slots, cut into 128-slot tiles (see WindowGeo)
    const int ring0 = (int)(((long)a.win_start + pl.tbase) % a.cache_cap);
    const int len = a.klen - pl.tbase;
    const int len_a = std::min(len, a.cache_cap - ring0);
    const int a0 = ring0 & ~3;
    const int n_a = (ring0 + len_a - a0 + tc5::KT - 1) / tc5::KT;
    const int n_b = (len - len_a + tc5::KT - 1) / tc5::KT;
    pl.ntiles = paged ? (a.klen + tc5::KT - 1) / tc5::KT : n_a + n_b;
    pl.grows = a.batch * a.S * a.nh;
    const int units = a.nkv * a.batch * pl.row_groups;
    const int slots_gpu = device_info().sm_count * occupancy;
    int best = 1;
    if (a.force_splits > 0) {
        best = std::min(a.force_splits, pl.ntiles);
    } else {
        double best_cost = 1e30;
        int max_splits = std::min(pl.ntiles, 512);
        if (a.fit_splits_to_ws) {
            const long per_split = (long)pl.grows * (a.l_hd + 2) * 4;
            const long fixed = 16 + 16L * units;
            max_splits = (int)std::max<long>(1, std::min<long>(max_splits, a.workspace ? (a.ws_bytes - fixed) / per_split : 0));
        }
        struct Memo { int ntiles, units, slots_gpu, max_splits, best; };          // (as in make_plan: the last few answers, per thread)
        static thread_local Memo memo[4] = {};
        static thread_local int memo_next = 0;
        bool hit = false;
        for (const Memo &m : memo)
            if (m.best > 0 && m.ntiles == pl.ntiles && m.units == units && m.slots_gpu == slots_gpu && m.max_splits == max_splits) { best = m.best; hit = true; break; }
        for (int n = 1; !hit && n <= max_splits; ++n) {
            const int tps = (pl.ntiles + n - 1) / n;
            if ((pl.ntiles + tps - 1) / tps != n) continue;
            const long ctas = (long)units * n;
            const long waves = (ctas + slots_gpu - 1) / slots_gpu;
            // in units of one tile's streaming time per CTA: a wave costs its tiles plus ~3 of start-up
            // and drain; more than one split adds the partial store, arrival and merge at the end
            const double cost = (double)waves * (tps + 3.0) + (n > 1 ? 3.0 + 0.03 * n : 0.0);
            if (cost < best_cost) { best_cost = cost; best = n; }
        }
        if (!hit) { memo[memo_next] = Memo{pl.ntiles, units, slots_gpu, max_splits, best}; memo_next = (memo_next + 1) % 4; }
    }
    if (paged && (pl.ntiles + best - 1) / best > tc5::MAX_PAGED_TILES) best = (pl.ntiles + tc5::MAX_PAGED_TILES - 1) / tc5::MAX_PAGED_TILES;
    pl.tiles_per_split = (pl.ntiles + best - 1) / best;
    pl.splits = (pl.ntiles + pl.tiles_per_split - 1) / pl.tiles_per_split;
    return pl;
}

template <int NS>
static int launch_tc5_inst(cudaStream_t st, const AttnArgs &a, bool query_ws, long *ws_needed) {
    using C = tc5::Cfg<NS>;
    const Tc5Plan pl = tc5_plan(a, NS, tc5_occupancy<NS>());
    const long units = (long)a.nkv * a.batch * pl.row_groups;
    const long part_bytes = (((long)pl.splits * pl.grows * (a.l_hd + 2) * 4) + 15) / 16 * 16;
    const bool in_kernel_merge = pl.splits > 1 || a.peer_world > 1;
    const long need = in_kernel_merge ? part_bytes + units * 16 : 0;
    if (query_ws) { *ws_needed = part_bytes + units * 16; return NOMOS_OK; }   // also enough for a sequence-sharded call, which merges in the kernel even with one split
    if (need > a.ws_bytes || (need > 0 && a.workspace == nullptr)) {
        set_error("attention workspace too small: need %ld bytes, have %ld", need, a.ws_bytes);
        return NOMOS_ECAPACITY;
    }
    if (pl.splits > MERGE_MAX_G) { set_error("too many splits (%d)", pl.splits); return NOMOS_EUNSUPPORTED; }
    tc5::TmaMaps4 tm;
    const bool paged = a.block_table != nullptr;
    const int rows = paged ? a.n_pages * a.nkv * tc5::KT : a.nkv * a.cache_cap;      // paged: the pools are one plane
    const int mb = paged ? 1 : a.batch;
    const MapKey mk{a.k_cache, 0, 128, a.cache_hd, rows, mb, tc5::KT, a.kv_batch_stride};
    const MapKey mv{a.v_cache, 0, 128, a.cache_hd, rows, mb, tc5::KT, a.kv_batch_stride};
    const MapKey mks{a.k_scales, 1, 4, 4, rows, mb, tc5::KT, a.scale_batch_stride};
    const MapKey mvs{a.v_scales, 1, 4, 4, rows, mb, tc5::KT, a.scale_batch_stride};
    if (!encode_plane(mk, &tm.k) || !encode_plane(mv, &tm.v)) return 1;
    const auto al16 = [](const void *x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    const bool scales_by_tma = al16(a.k_scales) && al16(a.v_scales) && (paged || a.cache_cap % 4 == 0) &&
                               (mb == 1 || a.scale_batch_stride % 16 == 0) && encode_plane(mks, &tm.ks) && encode_plane(mvs, &tm.vs);
    if (!scales_by_tma) { tm.ks = tm.k; tm.vs = tm.k; }       // never dereferenced
    if (paged && !scales_by_tma) { set_error("paged attention: scale pools must be 16-byte aligned"); return NOMOS_EBADARG; }
    KParams p;
    std::memset(&p, 0, sizeof(p));
    p.use_tma = scales_by_tma ? 3 : 1;
    p.k_scales = static_cast<const uint8_t *>(a.k_scales);
    p.v_scales = static_cast<const uint8_t *>(a.v_scales);
    p.q = static_cast<const uint8_t *>(a.q);
    p.out = static_cast<uint8_t *>(a.out);
    const bool direct_export = (!in_kernel_merge && a.partial_out != nullptr);
    p.partial = direct_export ? a.partial_out : static_cast<float *>(a.workspace);
    p.write_partial = (in_kernel_merge || direct_export) ? 1 : 0;
    p.export_nat = direct_export ? 1 : 0;
    p.counters = in_kernel_merge ? reinterpret_cast<unsigned long long *>(static_cast<char *>(a.workspace) + part_bytes) : nullptr;
    p.splits = pl.splits;
    p.arrivals = pl.splits;
    p.coop_merge = paged ? 0 : use_coop_merge(a, pl.splits, p.arrivals, (long)pl.splits * units, /* one CTA per SM, whatever the plan assumes */ 1, std::min(NS, a.S * a.kvg), a.l_hd);
    p.partial_export = a.partial_out;
    if (float *own = fill_peer_params(p, a, pl.grows)) p.partial_export = own;
    p.early_rows = paged ? 0 : settled_rows(a);
    // evict-first tile copies protect what the launch comes back to (code, query, partials) from its own stream:
    // verify at 16393 keys 26.5 -> 25.7 us; on streams of gigabytes, where that fixed part is noise, they measured
    // 3 % slower (C5a 612 -> 630 us, C5b 312 -> 323 us), hence the size limit (554 MB: 87.6 -> 86.8 us, 830 MB:
    // 125.7 -> 124.9, 1107 MB: 166.5 -> 167.0; the mma.sync kernel gains 3 to 4 % at all three)
    p.kv_read_once = (pl.row_groups == 1 && (long)a.batch * a.nkv * a.klen * 2 * a.cache_hd < (1024l << 20)) ? 1 : 0;
    p.block_table = a.block_table; p.seq_lens = a.seq_lens; p.max_pages = a.max_pages;
    p.q_type = a.q_type; p.out_type = a.out_type;
    p.S = a.S; p.nh = a.nh; p.nkv = a.nkv; p.kvg = a.kvg; p.cache_hd = a.cache_hd; p.cache_cap = a.cache_cap;
    p.win_start = a.win_start; p.klen = a.klen; p.window = a.window;
    p.tile0 = pl.tbase; p.ntiles = pl.ntiles; p.tiles_per_split = pl.tiles_per_split;
    p.row_groups = pl.row_groups; p.grows = pl.grows;
    p.qk_scale_log2 = a.softmax_scale * LOG2E;
    p.q_batch_stride = a.q_batch_stride; p.kv_batch_stride = a.kv_batch_stride;
    p.scale_batch_stride = a.scale_batch_stride; p.out_batch_stride = a.out_batch_stride;
    p.kvg_magic = a.kvg > 1 ? (unsigned int)(((1ull << 32) + a.kvg - 1) / a.kvg) : 0u;
    p.new_k = a.new_k; p.new_v = a.new_v;
    p.n_new = a.new_k ? a.n_new : 0; p.new_stride = a.new_stride; p.new_base_pos = a.new_base_pos;
    p.k_cache_w = static_cast<uint8_t *>(const_cast<void *>(a.k_cache)); p.v_cache_w = static_cast<uint8_t *>(const_cast<void *>(a.v_cache));
    p.k_scales_w = static_cast<uint8_t *>(const_cast<void *>(a.k_scales)); p.v_scales_w = static_cast<uint8_t *>(const_cast<void *>(a.v_scales));
    p.fault = fault_word();
    if (p.fault == nullptr) { set_error("attn_fused: device fault word unavailable"); return NOMOS_ECUDA; }
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.splits, a.nkv, a.batch * pl.row_groups);
    // (the warming pass of the query preparation is off here as well: verify 26.5 against 26.8 us without it)
    p.dry_pass = 0;
    cfg.blockDim = dim3(C::NTHREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = pdl; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, tc5::attn_tc5_kernel<NS>, p, tm);
    if (e != cudaSuccess) { set_error("attn_tc5 launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    note_launch(1, p);
    return NOMOS_OK;
}

// Returns 1 when the tensor maps could not be encoded (the caller then uses the other kernel).
static int launch_tc5(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    const int slots = a.S * a.kvg;
    if (slots <= 2) return launch_tc5_inst<2>(st, a, q, ws);
    if (slots <= 4) return launch_tc5_inst<4>(st, a, q, ws);
    if (slots <= 8) return launch_tc5_inst<8>(st, a, q, ws);
    if (slots <= 12) return launch_tc5_inst<12>(st, a, q, ws);
    if (slots <= 16) return launch_tc5_inst<16>(st, a, q, ws);
    if (slots <= 20) return launch_tc5_inst<20>(st, a, q, ws);
    return launch_tc5_inst<24>(st, a, q, ws);
}

template <int FMT, int HD>
static int dispatch_mt(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    return pick_mt(a.S * a.kvg) == 1 ? launch_inst<FMT, HD, 1>(st, a, q, ws) : launch_inst<FMT, HD, 3>(st, a, q, ws);
}

template <int FMT>
static int dispatch_hd(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    switch (a.l_hd) {
        case 128: return dispatch_mt<FMT, 128>(st, a, q, ws);
        // Wider heads: one 8-row tile per CTA (more query rows are covered by row groups), and quads of 2 / 4 warps
        // that take every tile together, each warp owning a 128-dim slice of K, V and the output (see Cfg).  Calls
        // that append rows in the same launch keep the unsliced kernel.  NOMOS_WIDE_BY_CTA selects the earlier
        // scheme (the PV product split over CTAs, the QK product repeated by each) for comparison builds.
#ifdef NOMOS_WIDE_BY_CTA
        case 256:
            if (a.new_k == nullptr && FMT == KV_I8) return launch_inst<FMT, 256, 1, 2>(st, a, q, ws);
            return launch_inst<FMT, 256, 1>(st, a, q, ws);
        case 512:
            if (a.new_k == nullptr) return launch_inst<FMT, 512, 1, NOMOS_DS512>(st, a, q, ws);
            return launch_inst<FMT, 512, 1>(st, a, q, ws);
#else
        case 256:
            if (a.new_k == nullptr) return launch_inst<FMT, 256, 1, 1, 2>(st, a, q, ws);
            return launch_inst<FMT, 256, 1>(st, a, q, ws);
        case 512:
            if (a.new_k == nullptr) return launch_inst<FMT, 512, 1, 1, 4>(st, a, q, ws);
            return launch_inst<FMT, 512, 1>(st, a, q, ws);
#endif
        default: set_error("head_dim %d unsupported (128, 256, 512)", a.l_hd); return NOMOS_EUNSUPPORTED;
    }
}

static int dispatch_mma(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    switch (a.kv_fmt) {
        case KV_I8: return dispatch_hd<KV_I8>(st, a, q, ws);
        case KV_I4: return dispatch_hd<KV_I4>(st, a, q, ws);
        case KV_I4B32: return dispatch_hd<KV_I4B32>(st, a, q, ws);
        default: set_error("kv_fmt %d unknown", a.kv_fmt); return NOMOS_EBADARG;
    }
}

// Calls both kernels can serve, decode shapes (up to 8 query rows per KV head).  Measured on B200 with both on
// one box: the tcgen05 kernel streams faster (batch 8 x 131072 keys 619 vs 641 us, 524288 keys 325 vs 346 us:
// about 7.0 against 6.6 TB/s), the mma.sync kernel has about 2 us less fixed cost per call (one CTA per SM, half
// as many partials to merge).  The crossing point moved from about 240 MB to about 330 MB of cache when the
// mma.sync kernel's tile copies became evict-first in L2; the table the threshold is read from is at prefers_mma().
// ------------------------------------------------------------------ query-major prefill (attn_prefill_kernel.cuh)
// int8 KV, head_dim 128, more query rows per KV head than the decode / verify kernels serve in one CTA (24), a
// window that does not wrap the ring, no fused append and no partial export.  Everything else -- int4 caches, wider
// heads, wrapped rings -- runs as row groups of the mma.sync kernel (also without any S x key_len scratch).
static bool prefill_eligible(const AttnArgs &a) {
    if (a.kv_fmt != KV_I8 || a.l_hd != 128 || a.no_tma || a.no_tcgen05 || a.block_table != nullptr) return false;
    if (a.new_k != nullptr || a.partial_out != nullptr || a.out == nullptr || a.peer_world > 1) return false;
    if (!a.d0_set && a.S * a.kvg <= 24) return false;
    if (a.kvg != 1 && a.kvg != 2 && a.kvg != 4 && a.kvg != 8) return false;
    if ((long)(a.win_start % a.cache_cap) + a.klen > a.cache_cap) return false;
    if (encode_tiled_fn() == nullptr) return false;
    const auto al16 = [](const void *x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    if (!al16(a.k_cache) || !al16(a.v_cache) || !al16(a.q) || !al16(a.out) || a.cache_hd % 16 != 0) return false;
    if (a.q_batch_stride % 8 != 0 || a.out_batch_stride % 8 != 0 || a.scale_batch_stride % 4 != 0) return false;
    if (a.batch > 1 && a.kv_batch_stride % 16 != 0) return false;
    if ((long)a.nkv * a.cache_cap >= (1l << 31)) return false;
    return true;
}

static int launch_prefill(cudaStream_t st, const AttnArgs &a) {
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_set[dev]) {
        cudaFuncSetAttribute(pf::attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pf::SMEM_BYTES);
        attr_set[dev] = true;
    }
    pf::PMaps tm;
    const int rows = a.nkv * a.cache_cap;
    const MapKey mk{a.k_cache, 0, 128, a.cache_hd, rows, a.batch, pf::KT, a.kv_batch_stride};
    const MapKey mv{a.v_cache, 0, 128, a.cache_hd, rows, a.batch, pf::KT, a.kv_batch_stride};
    if (!encode_plane(mk, &tm.k) || !encode_plane(mv, &tm.v)) return 1;
    pf::PParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = static_cast<const uint8_t *>(a.q);
    p.out = static_cast<uint8_t *>(a.out);
    p.k_scales = static_cast<const float *>(a.k_scales);
    p.v_scales = static_cast<const float *>(a.v_scales);
    p.q_type = a.q_type; p.out_type = a.out_type;
    p.S = a.S; p.nh = a.nh; p.nkv = a.nkv; p.kvg = a.kvg; p.cache_cap = a.cache_cap;
    p.row0 = a.win_start % a.cache_cap;
    p.key_len = a.klen;
    p.d0 = a.d0_set ? a.d0 : a.klen - a.S;
    p.window = a.window;
    p.pos_per_cta = pf::MR / a.kvg;
    p.q_blocks = (a.S + p.pos_per_cta - 1) / p.pos_per_cta;
    p.q_scale = a.softmax_scale * LOG2E;
    p.q_batch_stride = a.q_batch_stride; p.out_batch_stride = a.out_batch_stride; p.scale_batch_stride = a.scale_batch_stride;
    p.scales_vec = ((reinterpret_cast<uintptr_t>(a.k_scales) | reinterpret_cast<uintptr_t>(a.v_scales)) % 16 == 0 && a.cache_cap % 4 == 0 &&
                    p.row0 % 4 == 0 && a.scale_batch_stride % 16 == 0) ? 1 : 0;
    p.fault = fault_word();
    if (p.fault == nullptr) { set_error("attn_prefill: device fault word unavailable"); return NOMOS_ECUDA; }
    if (p.q_blocks > 65535 * 32 || a.batch > 65535) { set_error("attn_prefill: too many query blocks"); return NOMOS_EUNSUPPORTED; }
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.q_blocks, a.nkv, a.batch);
    cfg.blockDim = dim3(pf::NTHREADS);
    cfg.dynamicSmemBytes = pf::SMEM_BYTES;
    cfg.stream = st;
    cfg.attrs = pdl; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, pf::attn_prefill_kernel, p, tm);
    if (e != cudaSuccess) { set_error("attn_prefill launch: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

static bool prefers_mma(const AttnArgs &a) {
    if (a.tcgen05_always || a.block_table != nullptr || a.S * a.kvg > 8) return false;
    const int keys = a.window > 0 ? std::min(a.klen, a.window + a.S - 1) : a.klen;
    const double bytes = (double)a.batch * a.nkv * keys * (2.0 * a.cache_hd + 8.0);
    // same-box measurements, launches back to back, us (mma.sync / tcgen05): 69 MB 18.0 / 17.7, 138 MB 25.7 / 26.7,
    // 208 MB 35.7 / 35.8, 277 MB 46.1 / 46.6, 415 MB 66.5 / 64.6, 554 MB 93.4 / 88.3
    return bytes < 330e6;
}

static int dispatch(cudaStream_t st, const AttnArgs &a, bool q, long *ws) {
    if (!q && prefill_eligible(a)) {
        const int rc = launch_prefill(st, a);
        if (rc != 1) return rc;                    // 1: the tensor maps could not be encoded, use the other kernels
    }
    if (a.d0_set) { set_error("this key range needs the prefill kernel (int8 KV, head_dim 128, 16-byte aligned buffers)"); return NOMOS_EUNSUPPORTED; }
    if (!tc5_eligible(a)) return dispatch_mma(st, a, q, ws);
    if (q) {
        // a later call with the same geometry may carry new rows to append and take the other
        // kernel: report what either needs
        long w_tc = 0, w_mma = 0;
        const int rc1 = launch_tc5(st, a, true, &w_tc);
        const int rc2 = dispatch_mma(st, a, true, &w_mma);
        if (rc2 != NOMOS_OK) return rc2;
        *ws = rc1 == NOMOS_OK ? std::max(w_tc, w_mma) : w_mma;
        return NOMOS_OK;
    }
    if (prefers_mma(a)) return dispatch_mma(st, a, false, nullptr);
    const int rc = launch_tc5(st, a, false, nullptr);
    return rc == 1 ? dispatch_mma(st, a, false, nullptr) : rc;
}

}  // namespace

long attn_peer_mailbox_rows_bytes(int world, long grows, int l_hd) {
    return ((2L * world * grows * (l_hd + 2) * 4) + 15) / 16 * 16;
}
long attn_peer_mailbox_bytes(int world, long grows, int l_hd) {
    return attn_peer_mailbox_rows_bytes(world, grows, l_hd) + 2L * world * grows * 8;
}

LaunchInfo attn_last_launch_info() { return t_last_launch; }
int attn_kernel_choice(const AttnArgs &a) { return prefill_eligible(a) ? 2 : (tc5_eligible(a) && !prefers_mma(a) ? 1 : 0); }

long attn_workspace_bytes(const AttnArgs &a) {
    long ws = 0;
    const int rc = dispatch(nullptr, a, true, &ws);
    return rc == NOMOS_OK ? ws : (long)rc;
}

int launch_attn_fused(cudaStream_t st, const AttnArgs &a) { return dispatch(st, a, false, nullptr); }

// Paged caches exist in the tcgen05 kernel only.
long attn_paged_workspace_bytes(const AttnArgs &a) {
    long ws = 0;
    const int rc = launch_tc5(nullptr, a, true, &ws);
    return rc == NOMOS_OK ? ws : (long)(rc == 1 ? NOMOS_EUNSUPPORTED : rc);
}
int launch_attn_paged(cudaStream_t st, const AttnArgs &a) {
    if (encode_tiled_fn() == nullptr) { set_error("paged attention needs the driver's tensor-map encoder"); return NOMOS_EUNSUPPORTED; }
    const int rc = launch_tc5(st, a, false, nullptr);
    if (rc == 1) { set_error("paged attention: the pools do not satisfy the tensor-map rules (16-byte aligned)"); return NOMOS_EBADARG; }
    return rc;
}

int read_attn_faults(unsigned int *out, bool clear) {
    unsigned int *w = fault_word();
    if (w == nullptr) { set_error("device fault word unavailable"); return NOMOS_ECUDA; }
    cudaError_t e = cudaMemcpy(out, w, sizeof(unsigned int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && clear && *out != 0) e = cudaMemset(w, 0, sizeof(unsigned int));
    if (e != cudaSuccess) { set_error("fault word read: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}


__global__ void clear_fault_bits_kernel(unsigned int *w, unsigned int bits) { atomicAnd(w, ~bits); }
int clear_attn_fault_bits(unsigned int bits) {
    unsigned int *w = fault_word();
    if (w == nullptr) { set_error("device fault word unavailable"); return NOMOS_ECUDA; }
    clear_fault_bits_kernel<<<1, 1>>>(w, bits);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { set_error("fault word clear: %s", cudaGetErrorString(e)); return NOMOS_ECUDA; }
    return NOMOS_OK;
}

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
