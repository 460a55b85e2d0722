// Host-side bookkeeping of one layer's KV ring: lengths, window arithmetic, staged rows and
// roll-back.  No device work.
//
// The reference keeps this arithmetic in its engine loops (lib/engine_decode.mojo:420-444:
// win_start, klen, lo; lib/gemma4_engine.mojo:897-901: set_cache_len for KV reuse and for the
// roll-back after a verify pass) and refuses the combinations its ring cannot serve: verify or
// offset prefill with the sliding-window ring (lib/engine_prefill.mojo:87-88) and chunked appends
// (lib/engine_decode.mojo:158-176: with exactly W slots, the rows a batch appends overwrite slots
// that earlier rows of the same batch still need as keys).  Here the ring is given
// max_rows - 1 slots of slack: a batch of n <= max_rows rows at positions len .. len+n-1 then only
// overwrites positions older than len - W + 1, which no row of the batch (and no later one) reads,
// so verify over the ring is exact, and rejected rows are simply overwritten by the next append.
#include <cstring>

#include "../../include/nomos_attn.h"
#include "common.cuh"

using namespace nomos;

#define NOMOS_EXPORT extern "C" __attribute__((visibility("default")))

namespace {
bool ring_ok(const nomos_kv_ring_t *r) {
    return r && r->struct_bytes == (int64_t)sizeof(nomos_kv_ring_t) && r->cache_cap > 0 && r->max_rows > 0;
}
}  // namespace

NOMOS_EXPORT int32_t nomos_kv_ring_init(nomos_kv_ring_t *ring, int64_t cache_cap, int64_t window, int64_t max_rows) {
    if (!ring || cache_cap <= 0 || window < 0 || max_rows <= 0) { set_error("nomos_kv_ring_init: bad argument"); return NOMOS_EBADARG; }
    if (window > 0 && cache_cap < window + max_rows - 1) {
        set_error("nomos_kv_ring_init: a ring of %ld slots cannot serve batches of %ld rows over a window of %ld (needs %ld)",
                  (long)cache_cap, (long)max_rows, (long)window, (long)(window + max_rows - 1));
        return NOMOS_ECAPACITY;
    }
    std::memset(ring, 0, sizeof(*ring));
    ring->struct_bytes = sizeof(*ring);
    ring->cache_cap = cache_cap; ring->window = window; ring->max_rows = max_rows;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_ring_plan(nomos_kv_ring_t *ring, int64_t n_new, nomos_kv_step_t *step) {
    if (!ring_ok(ring) || !step || n_new <= 0) { set_error("nomos_kv_ring_plan: bad argument"); return NOMOS_EBADARG; }
    if (n_new > ring->max_rows) {
        set_error("nomos_kv_ring_plan: %ld rows exceed the max_rows %ld the ring was sized for", (long)n_new, (long)ring->max_rows);
        return NOMOS_ECAPACITY;
    }
    const int64_t end = ring->len + n_new;
    if (ring->window == 0 && end > ring->cache_cap) {      // a linear cache does not wrap: refuse, never overrun
        set_error("nomos_kv_ring_plan: positions [%ld,%ld) do not fit a linear cache of %ld rows", (long)ring->len, (long)end,
                  (long)ring->cache_cap);
        return NOMOS_ECAPACITY;
    }
    step->base_pos = ring->len;
    step->n_new = n_new;
    step->window = ring->window;
    // Row i (absolute position len + i) reads [max(0, len + i - W + 1), len + i]; the call's window is
    // the union over its rows, starting where row 0 starts.
    const int64_t span = ring->window > 0 ? ring->window + n_new - 1 : end;
    step->klen = end < span ? end : span;
    step->win_start = end - step->klen;
    ring->staged = n_new;
    if (end > ring->high) ring->high = end;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_ring_commit(nomos_kv_ring_t *ring, int64_t accepted) {
    if (!ring_ok(ring) || accepted < 0 || accepted > ring->staged) {
        set_error("nomos_kv_ring_commit: %ld rows accepted of %ld staged", (long)accepted, ring ? (long)ring->staged : 0L);
        return NOMOS_EBADARG;
    }
    ring->len += accepted;
    ring->staged = 0;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_ring_set_len(nomos_kv_ring_t *ring, int64_t n) {
    if (!ring_ok(ring) || n < 0 || n > ring->len) { set_error("nomos_kv_ring_set_len: bad length"); return NOMOS_EBADARG; }
    if (ring->window > 0) {
        // The ring still holds positions [high - cache_cap, high).  The next row (position n) reads from
        // n - W + 1 on: that must not have been overwritten.
        const int64_t oldest_kept = ring->high - ring->cache_cap;
        const int64_t oldest_needed = n - ring->window + 1 > 0 ? n - ring->window + 1 : 0;
        if (n > 0 && oldest_needed < oldest_kept) {
            set_error("nomos_kv_ring_set_len: position %ld is needed after a roll-back to %ld but the ring only keeps %ld and newer",
                      (long)oldest_needed, (long)n, (long)oldest_kept);
            return NOMOS_ECAPACITY;
        }
    }
    ring->len = n;
    ring->staged = 0;
    return NOMOS_OK;
}

NOMOS_EXPORT int32_t nomos_kv_ring_fill_args(const nomos_kv_ring_t *ring, const nomos_kv_step_t *step, nomos_attn_args_t *args) {
    if (!ring_ok(ring) || !step || !args) { set_error("nomos_kv_ring_fill_args: bad argument"); return NOMOS_EBADARG; }
    args->cache_cap = ring->cache_cap;
    args->S = step->n_new;
    args->win_start = step->win_start;
    args->klen = step->klen;
    args->window = step->window;
    args->n_new = step->n_new;
    args->new_base_pos = step->base_pos;
    return NOMOS_OK;
}
