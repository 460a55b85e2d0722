"""Host-side mirror of the reference's operator interface for the attention path.

Function names, argument order and argument meaning are those of the reference's
Mojo operators (cited per function, paths relative to the reference root); the
leading ``ctx`` becomes ``stream``: a raw ``cudaStream_t`` value, a
``torch.cuda.Stream``, or ``None`` for torch's current stream.  Buffer arguments
may be torch CUDA tensors or integer device addresses.  The reference's operators
``raise`` on failure; so do these (``NomosError`` carrying the library's status).

torch is used for nothing but device memory and streams; all compute is in
``libnomos_attn.so`` and there is no fallback if it is missing.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import AttnArgs, AttnPeer

KV_I8, KV_I4, KV_I4B32 = 0, 1, 2
F32, BF16 = 0, 1
SETTLED_CACHE = 1            # nomos_attn_args_t.flags bit, see include/nomos_attn.h
NO_TMA = 2                   # nomos_attn_args_t.flags bit: cp.async copies only
NO_TCGEN05 = 4               # nomos_attn_args_t.flags bit: stay on the mma.sync kernel
TCGEN05_ALWAYS = 8           # nomos_attn_args_t.flags bit: tcgen05 kernel wherever it supports the call
NO_CLUSTER = 16              # nomos_attn_args_t.flags bit: splits never merged through a thread-block cluster


class NomosError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"libnomos_attn status {status}: {message}")
        self.status = status


def _addr(x) -> int:
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    return x.data_ptr()            # torch tensor


def _stream(stream) -> C.c_void_p:
    if stream is None:
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return C.c_void_p(stream)
    return C.c_void_p(stream.cuda_stream)


def _check(status: int) -> None:
    if status != 0:
        raise NomosError(status, _lib.lib().nomos_attn_last_error().decode("utf-8", "replace"))


def version() -> int:
    return _lib.lib().nomos_attn_version()


def device_faults(clear: bool = False) -> int:
    """Fault bits the kernels of the current device have raised (0 = none); synchronises."""
    import ctypes

    bits = ctypes.c_uint32(0)
    _check(_lib.lib().nomos_attn_device_faults(ctypes.byref(bits), 1 if clear else 0))
    return int(bits.value)


# ---------------------------------------------------------------------- codecs

def gpu_quant_kv_i8(stream, in_bf16, out_i8, out_scales, n_rows, dim):
    """lib/kv_cache_quant.mojo:100"""
    _check(_lib.lib().nomos_kv_quant_i8(_stream(stream), _addr(in_bf16), _addr(out_i8), _addr(out_scales), n_rows, dim))


def gpu_dequant_kv_i8(stream, in_i8, in_scales, out_bf16, n_rows, dim):
    """lib/kv_cache_quant.mojo:116"""
    _check(_lib.lib().nomos_kv_dequant_i8(_stream(stream), _addr(in_i8), _addr(in_scales), _addr(out_bf16), n_rows, dim))


def gpu_append_quant_kv_i8(stream, src_k, src_v, dst_k_i8, dst_v_i8, k_scales, v_scales,
                           n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos):
    """lib/kv_cache_quant.mojo:252"""
    _check(_lib.lib().nomos_kv_append_quant_i8(
        _stream(stream), _addr(src_k), _addr(src_v), _addr(dst_k_i8), _addr(dst_v_i8), _addr(k_scales), _addr(v_scales),
        n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos))


def kv_norm_rope_append(stream, q, q_norm_w, src_k, src_v, k_norm_w, dst_k, dst_v, k_scales, v_scales, *,
                         n_s, nh, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, theta, rope_dim, kv_fmt,
                         k_out=None, v_out=None):
    """V-norm, QK-norm, RoPE (lib/gemma4_layer.mojo:326-340) and the quantising append in one launch.
    `q` (or None) is rewritten in place; `kv_fmt` < 0 skips the cache write."""
    def a(x):
        return 0 if x is None else _addr(x)
    _check(_lib.lib().nomos_kv_norm_rope_append(
        _stream(stream), a(q), a(q_norm_w), a(src_k), a(src_v), a(k_norm_w), a(dst_k), a(dst_v), a(k_scales), a(v_scales),
        a(k_out), a(v_out), n_s, nh, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, float(theta), rope_dim, kv_fmt))


def gpu_dequant_kv_i8_layer(stream, src_i8, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start):
    """lib/kv_cache_quant.mojo:274"""
    _check(_lib.lib().nomos_kv_dequant_i8_layer(
        _stream(stream), _addr(src_i8), _addr(scales), _addr(dst_bf16), nkv, klen, cache_hd, max_seq, cache_cap, win_start))


def gpu_append_quant_kv_i4(stream, src_k, src_v, dst_k_i4, dst_v_i4, k_scales, v_scales,
                           n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, scale_blocks=1):
    """lib/kv_cache_quant.mojo:803"""
    _check(_lib.lib().nomos_kv_append_quant_i4(
        _stream(stream), _addr(src_k), _addr(src_v), _addr(dst_k_i4), _addr(dst_v_i4), _addr(k_scales), _addr(v_scales),
        n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, scale_blocks))


def gpu_append_quant_kv_i4_with_q8(stream, src_k, src_v, dst_k_i4, dst_v_i4, k_scales, v_scales,
                                   dst_k_q8, dst_v_q8, k_q8_scales, v_q8_scales,
                                   n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, q8_pitch, scale_blocks=1):
    """lib/kv_cache_quant.mojo:839"""
    _check(_lib.lib().nomos_kv_append_quant_i4_with_q8(
        _stream(stream), _addr(src_k), _addr(src_v), _addr(dst_k_i4), _addr(dst_v_i4), _addr(k_scales), _addr(v_scales),
        _addr(dst_k_q8), _addr(dst_v_q8), _addr(k_q8_scales), _addr(v_q8_scales),
        n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, q8_pitch, scale_blocks))


def gpu_dequant_kv_i4_layer(stream, src_i4, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start,
                            scale_blocks=1):
    """lib/kv_cache_quant.mojo:885"""
    _check(_lib.lib().nomos_kv_dequant_i4_layer(
        _stream(stream), _addr(src_i4), _addr(scales), _addr(dst_bf16), nkv, klen, cache_hd, max_seq, cache_cap,
        win_start, scale_blocks))


def gpu_dequant_kv_i4_to_q8_layer(stream, src_i4, scales, dst_i8, dst_scale, nkv, klen, cache_hd, max_seq, cache_cap,
                                  win_start, scale_blocks=1):
    """lib/kv_cache_quant.mojo:956"""
    _check(_lib.lib().nomos_kv_dequant_i4_to_q8_layer(
        _stream(stream), _addr(src_i4), _addr(scales), _addr(dst_i8), _addr(dst_scale), nkv, klen, cache_hd, max_seq,
        cache_cap, win_start, scale_blocks))


def append_kv_gpu_dev_async(stream, d_k_cache_layer, d_v_cache_layer, d_k_new, d_v_new, nkv, l_hd, cache_hd, max_seq, cl):
    """lib/attention_gpu.mojo:109 (and the synchronous twin at :87)"""
    _check(_lib.lib().nomos_kv_append_fp32(
        _stream(stream), _addr(d_k_cache_layer), _addr(d_v_cache_layer), _addr(d_k_new), _addr(d_v_new),
        nkv, l_hd, cache_hd, max_seq, cl))


def append_kv_gpu_bf16_dev(stream, d_k_cache_layer, d_v_cache_layer, d_k_new, d_v_new, d_k_bf16, d_v_bf16,
                           nkv, l_hd, cache_hd, max_seq, cl):
    """lib/attention_gpu.mojo:136"""
    _check(_lib.lib().nomos_kv_append_bf16(
        _stream(stream), _addr(d_k_cache_layer), _addr(d_v_cache_layer), _addr(d_k_new), _addr(d_v_new),
        _addr(d_k_bf16), _addr(d_v_bf16), nkv, l_hd, cache_hd, max_seq, cl))


def gpu_append_kv_batched_bf16(stream, d_src_k, d_src_v, d_dst_k_cache, d_dst_v_cache,
                               n_s, nkv, l_hd, l_kvd, max_seq, cache_hd, base_pos=0):
    """lib/batched_attn_gpu.mojo:87"""
    _check(_lib.lib().nomos_kv_append_batched_bf16(
        _stream(stream), _addr(d_src_k), _addr(d_src_v), _addr(d_dst_k_cache), _addr(d_dst_v_cache),
        n_s, nkv, l_hd, l_kvd, max_seq, cache_hd, base_pos))


# ------------------------------------------------------------------- attention

def attention_gpu_int8_dev(stream, d_q_gpu, d_k_i8, d_v_i8, d_k_scale, d_v_scale, d_scores_scratch, d_attn_out_scratch,
                           nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg):
    """lib/attention_gpu_int8.mojo:598"""
    _check(_lib.lib().nomos_attn_decode_i8(
        _stream(stream), _addr(d_q_gpu), _addr(d_k_i8), _addr(d_v_i8), _addr(d_k_scale), _addr(d_v_scale),
        _addr(d_scores_scratch), _addr(d_attn_out_scratch), nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg))


def attention_decode_order_multirow_int8(stream, d_q_b, d_scores, d_attn_b, d_k_i8, d_v_i8, d_k_scale, d_v_scale,
                                         nh, nkv, l_hd, cache_hd, max_seq, S, score_stride, kvg, window, query_base_pos):
    """lib/attention_gpu_int8.mojo:634"""
    _check(_lib.lib().nomos_attn_decode_multirow_i8(
        _stream(stream), _addr(d_q_b), _addr(d_scores), _addr(d_attn_b), _addr(d_k_i8), _addr(d_v_i8),
        _addr(d_k_scale), _addr(d_v_scale), nh, nkv, l_hd, cache_hd, max_seq, S, score_stride, kvg, window, query_base_pos))


def attention_prefill_prefix_batched_int8(stream, d_q_b, d_q_t, d_scores, d_attn_t, d_attn_b, d_k_i8, d_v_i8,
                                          d_k_scale, d_v_scale, nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg,
                                          window, query_base_pos, key_base_pos):
    """lib/attention_gpu_int8.mojo:844"""
    _check(_lib.lib().nomos_attn_prefix_batched_i8(
        _stream(stream), _addr(d_q_b), _addr(d_q_t), _addr(d_scores), _addr(d_attn_t), _addr(d_attn_b),
        _addr(d_k_i8), _addr(d_v_i8), _addr(d_k_scale), _addr(d_v_scale),
        nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window, query_base_pos, key_base_pos))


def attention_gpu_fp32_dev(stream, handle, d_q_gpu, d_k_cache_layer, d_v_cache_layer, d_scores_scratch,
                           d_attn_out_scratch, nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg):
    """lib/attention_gpu.mojo:165 (the cuBLAS ``handle`` is accepted and ignored)"""
    _check(_lib.lib().nomos_attn_decode_fp32(
        _stream(stream), _addr(d_q_gpu), _addr(d_k_cache_layer), _addr(d_v_cache_layer), _addr(d_scores_scratch),
        _addr(d_attn_out_scratch), nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg))


def attention_gpu_bf16_dev(stream, handle, d_q_gpu, d_k_cache_layer, d_v_cache_layer, d_scores_scratch, d_q_bf16,
                           d_scores_bf16, d_attn_out_scratch, nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg):
    """lib/attention_gpu.mojo:207"""
    _check(_lib.lib().nomos_attn_decode_bf16(
        _stream(stream), _addr(d_q_gpu), _addr(d_k_cache_layer), _addr(d_v_cache_layer), _addr(d_scores_scratch),
        _addr(d_q_bf16), _addr(d_scores_bf16), _addr(d_attn_out_scratch), nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg))


def attention_prefill_batched_int8(stream, d_q_b, d_q_t, d_scores, d_attn_t, d_attn_b, d_k_i8, d_v_i8, d_k_scale,
                                   d_v_scale, nh, nkv, l_hd, cache_hd, max_seq, S, kvg, window):
    """lib/attention_gpu_int8.mojo:804"""
    _check(_lib.lib().nomos_attn_prefill_batched_i8(
        _stream(stream), _addr(d_q_b), _addr(d_q_t), _addr(d_scores), _addr(d_attn_t), _addr(d_attn_b),
        _addr(d_k_i8), _addr(d_v_i8), _addr(d_k_scale), _addr(d_v_scale), nh, nkv, l_hd, cache_hd, max_seq, S, kvg, window))


def attention_prefill_prefix_batched_fp32(stream, handle, d_q_b, d_q_t, d_scores, d_attn_t, d_attn_b,
                                          d_k_cache_layer, d_v_cache_layer, nh, nkv, l_hd, cache_hd, max_seq, S,
                                          key_len, kvg, window, query_base_pos, key_base_pos):
    """lib/batched_attn_gpu.mojo:499 (the cuBLAS ``handle`` is accepted and ignored)"""
    _check(_lib.lib().nomos_attn_prefix_batched_fp32(
        _stream(stream), _addr(d_q_b), _addr(d_q_t), _addr(d_scores), _addr(d_attn_t), _addr(d_attn_b),
        _addr(d_k_cache_layer), _addr(d_v_cache_layer),
        nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window, query_base_pos, key_base_pos))


def attention_prefill_prefix_batched_bf16(stream, handle, d_q_b, d_q_t, d_q_t_bf16, d_scores, d_scores_bf16, d_attn_t,
                                          d_attn_b, d_k_cache_layer, d_v_cache_layer, nh, nkv, l_hd, cache_hd, max_seq,
                                          S, key_len, kvg, window, query_base_pos, key_base_pos):
    """lib/batched_attn_gpu.mojo:613"""
    _check(_lib.lib().nomos_attn_prefix_batched_bf16(
        _stream(stream), _addr(d_q_b), _addr(d_q_t), _addr(d_q_t_bf16), _addr(d_scores), _addr(d_scores_bf16),
        _addr(d_attn_t), _addr(d_attn_b), _addr(d_k_cache_layer), _addr(d_v_cache_layer),
        nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window, query_base_pos, key_base_pos))


def attention_prefill_batched_fp32(stream, handle, d_q_b, d_q_t, d_scores, d_attn_t, d_attn_b, d_k_cache_layer,
                                   d_v_cache_layer, nh, nkv, l_hd, cache_hd, max_seq, S, kvg, window):
    """lib/batched_attn_gpu.mojo:448"""
    _check(_lib.lib().nomos_attn_prefill_batched_fp32(
        _stream(stream), _addr(d_q_b), _addr(d_q_t), _addr(d_scores), _addr(d_attn_t), _addr(d_attn_b),
        _addr(d_k_cache_layer), _addr(d_v_cache_layer), nh, nkv, l_hd, cache_hd, max_seq, S, kvg, window))


def attention_prefill_batched_bf16(stream, handle, d_q_b, d_q_t, d_q_t_bf16, d_scores, d_scores_bf16, d_attn_t, d_attn_b,
                                   d_k_cache_layer, d_v_cache_layer, nh, nkv, l_hd, cache_hd, max_seq, S, kvg, window):
    """lib/batched_attn_gpu.mojo:558"""
    _check(_lib.lib().nomos_attn_prefill_batched_bf16(
        _stream(stream), _addr(d_q_b), _addr(d_q_t), _addr(d_q_t_bf16), _addr(d_scores), _addr(d_scores_bf16),
        _addr(d_attn_t), _addr(d_attn_b), _addr(d_k_cache_layer), _addr(d_v_cache_layer),
        nh, nkv, l_hd, cache_hd, max_seq, S, kvg, window))


# ----------------------------------------------------------------------- fused

def make_args(**kw) -> AttnArgs:
    """Zero-initialised ``nomos_attn_args_t`` with the given fields set (tensors or addresses)."""
    a = AttnArgs()
    a.struct_bytes = C.sizeof(AttnArgs)
    a.batch, a.S, a.softmax_scale = 1, 1, 1.0
    ptr_fields = {"q", "k_cache", "v_cache", "k_scales", "v_scales", "out", "partial_out", "workspace", "new_k", "new_v"}
    for k, v in kw.items():
        if not hasattr(a, k):
            raise TypeError(f"nomos_attn_args_t has no field {k}")
        setattr(a, k, _addr(v) if k in ptr_fields else v)
    return a


def attn_workspace_bytes(args: AttnArgs) -> int:
    n = _lib.lib().nomos_attn_workspace_bytes(C.byref(args))
    if n < 0:
        _check(int(n))
    return int(n)


def attn_last_launch() -> tuple[int, int, int]:
    """(kernel, splits, merge route) of this thread's last decode / verify launch; routes: 0 one split, 1 last CTA,
    2 cooperative, 3 thread-block cluster."""
    k, n, r = C.c_int32(0), C.c_int32(0), C.c_int32(0)
    _check(_lib.lib().nomos_attn_last_launch(C.byref(k), C.byref(n), C.byref(r)))
    return k.value, n.value, r.value


def attn_kernel_choice(args: AttnArgs) -> int:
    """1 when `attn_fused` would run the tcgen05 kernel for these arguments, 0 for the mma.sync kernel."""
    n = _lib.lib().nomos_attn_kernel_choice(C.byref(args))
    if n < 0:
        _check(int(n))
    return int(n)


def attn_fused(stream, args: AttnArgs) -> None:
    """Append (optional) + attention over the packed ring in one call; replaces the
    reference's per-layer append -> window reader -> attention sequence
    (lib/engine_decode.mojo:356-389, 445-460, 527-554)."""
    _check(_lib.lib().nomos_attn_fused(_stream(stream), C.byref(args)))


def attn_paged_workspace_bytes(batch, nh, nkv, kvg, l_hd, max_len) -> int:
    n = _lib.lib().nomos_attn_paged_workspace_bytes(batch, nh, nkv, kvg, l_hd, max_len)
    if n < 0:
        _check(int(n))
    return int(n)


def attn_paged_decode_i8(stream, q, k_pool, v_pool, ks_pool, vs_pool, block_table, seq_lens, out, workspace, ws_bytes, *,
                         batch, nh, nkv, kvg, l_hd, n_pages, max_pages, max_len, softmax_scale=1.0, q_type=F32, out_type=F32):
    """Decode attention over paged int8 caches (pages of 128 keys); see include/nomos_attn.h."""
    _check(_lib.lib().nomos_attn_paged_decode_i8(
        _stream(stream), _addr(q), _addr(k_pool), _addr(v_pool), _addr(ks_pool), _addr(vs_pool), _addr(block_table),
        _addr(seq_lens), _addr(out), _addr(workspace), int(ws_bytes), batch, nh, nkv, kvg, l_hd, n_pages, max_pages, max_len,
        float(softmax_scale), q_type, out_type))


def kv_paged_append_quant_i8(stream, src_k, src_v, k_pool, v_pool, ks_pool, vs_pool, block_table, positions, *,
                             batch, nkv, l_hd, l_kvd, max_pages):
    _check(_lib.lib().nomos_kv_paged_append_quant_i8(
        _stream(stream), _addr(src_k), _addr(src_v), _addr(k_pool), _addr(v_pool), _addr(ks_pool), _addr(vs_pool),
        _addr(block_table), _addr(positions), batch, nkv, l_hd, l_kvd, max_pages))


class KvRing:
    """One layer's ring bookkeeping (``nomos_kv_ring_*``): lengths, window arithmetic, staged rows,
    roll-back.  ``window`` = 0 is a linear cache.  A ring that serves batches of ``max_rows`` rows needs
    ``cache_cap >= window + max_rows - 1``."""

    def __init__(self, cache_cap: int, window: int, max_rows: int = 1):
        self.c = _lib.KvRing()
        _check(_lib.lib().nomos_kv_ring_init(C.byref(self.c), cache_cap, window, max_rows))

    @property
    def len(self) -> int:
        return int(self.c.len)

    def plan(self, n_new: int) -> "_lib.KvStep":
        step = _lib.KvStep()
        _check(_lib.lib().nomos_kv_ring_plan(C.byref(self.c), n_new, C.byref(step)))
        return step

    def commit(self, accepted: int) -> None:
        _check(_lib.lib().nomos_kv_ring_commit(C.byref(self.c), accepted))

    def set_len(self, n: int) -> None:
        _check(_lib.lib().nomos_kv_ring_set_len(C.byref(self.c), n))

    def fill_args(self, step, args: AttnArgs) -> None:
        _check(_lib.lib().nomos_kv_ring_fill_args(C.byref(self.c), C.byref(step), C.byref(args)))


def attn_fused_host(stream, args: AttnArgs, host_in, dev_in, in_bytes: int, host_out, dev_out, out_bytes: int) -> None:
    """One step with host-resident inputs and result: pinned ``host_in`` -> ``dev_in``, ``attn_fused``,
    ``dev_out`` -> pinned ``host_out``, stream synchronised -- one library call instead of three runtime
    calls and a synchronise."""
    _check(_lib.lib().nomos_attn_fused_host(_stream(stream), C.byref(args), _addr(host_in), _addr(dev_in), int(in_bytes),
                                            _addr(host_out), _addr(dev_out), int(out_bytes)))


def attn_fused_static_ws(stream, args: AttnArgs) -> None:
    """``attn_fused`` for callers that cannot provide a workspace (an engine whose memory budget
    is fully committed at start-up, a decode loop that must never call the allocator): the split
    scratch is a fixed 4 MiB array inside the library, nothing is allocated, ``args.workspace`` is
    ignored.  Raises with status -3 if the call would need more scratch than that.  Calls on one
    device share the array, so issue them in order (one stream); make the first call on a device
    before any stream capture."""
    _check(_lib.lib().nomos_attn_fused_static_ws(_stream(stream), C.byref(args)))


def attn_merge_partials(stream, partials, G, rows, l_hd, out, out_type=F32) -> None:
    _check(_lib.lib().nomos_attn_merge_partials(_stream(stream), _addr(partials), G, rows, l_hd, _addr(out), out_type))


# ------------------------------------------------- sequence-sharded decode across GPUs

def attn_peer_mailbox_bytes(world: int, rows: int, l_hd: int) -> int:
    n = _lib.lib().nomos_attn_peer_mailbox_bytes(world, rows, l_hd)
    if n < 0:
        _check(int(n))
    return int(n)


def attn_peer_mailbox_create(nbytes: int) -> tuple[int, bytes]:
    """Allocates and zeroes one rank's mailbox; returns (device address, 64-byte interprocess handle)."""
    ptr = C.c_uint64(0)
    handle = C.create_string_buffer(64)
    _check(_lib.lib().nomos_attn_peer_mailbox_create(int(nbytes), C.byref(ptr), handle))
    return int(ptr.value), handle.raw


def attn_peer_mailbox_open(handle: bytes) -> int:
    ptr = C.c_uint64(0)
    buf = C.create_string_buffer(handle, 64)
    _check(_lib.lib().nomos_attn_peer_mailbox_open(buf, C.byref(ptr)))
    return int(ptr.value)


def attn_peer_mailbox_close(ptr: int, own: bool) -> None:
    _check(_lib.lib().nomos_attn_peer_mailbox_close(int(ptr), 1 if own else 0))


def make_peer(rank: int, world: int, mailboxes, mailbox_bytes: int, step: int, timeout_us: int = 0) -> AttnPeer:
    p = AttnPeer()
    p.struct_bytes = C.sizeof(AttnPeer)
    p.rank, p.world, p.mailbox_bytes, p.step, p.timeout_us = rank, world, mailbox_bytes, step, timeout_us
    for g, m in enumerate(mailboxes):
        p.mailbox[g] = _addr(m)
    return p


def attn_seq_sharded(stream, args: AttnArgs, peer: AttnPeer) -> None:
    """One rank's call of the sequence-sharded decode: attention over this rank's chunk, exchange of the (o, m, l)
    rows through the peers' mailboxes and the final merge, in one launch (include/nomos_attn.h)."""
    _check(_lib.lib().nomos_attn_seq_sharded(_stream(stream), C.byref(args), C.byref(peer)))


def attn_seq_sharded_status(stream, clear: bool = False) -> int:
    """Synchronises the stream; 0, or -4 when a peer's rows did not arrive in time (raises for other errors)."""
    rc = _lib.lib().nomos_attn_seq_sharded_status(_stream(stream), 1 if clear else 0)
    if rc not in (0, -4):
        _check(rc)
    return int(rc)
