"""Loads ``libnomos_attn.so`` through ctypes and declares every exported prototype.

There is no fallback: if the shared object is missing or a symbol cannot be
resolved the import raises, so a run can never silently use something else.
The idiom follows the reference's own Python binding (pyhost/host.py:108-144).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import os

PKG = Path(__file__).resolve().parent
# NOMOS_ATTN_LIB points at another build of the same library (e.g. one compiled with
# different tile parameters); the default is the in-tree build.
LIB_PATH = Path(os.environ.get("NOMOS_ATTN_LIB", PKG / "libnomos_attn.so"))

u64, i32, i64, vp = C.c_uint64, C.c_int32, C.c_int64, C.c_void_p


class AttnArgs(C.Structure):
    """Mirror of ``nomos_attn_args_t`` (include/nomos_attn.h); every field is 8 bytes."""
    _fields_ = [
        ("struct_bytes", u64),
        ("q", u64), ("k_cache", u64), ("v_cache", u64), ("k_scales", u64), ("v_scales", u64),
        ("out", u64), ("partial_out", u64), ("workspace", u64), ("ws_bytes", i64),
        ("new_k", u64), ("new_v", u64), ("n_new", i64), ("new_stride", i64), ("new_base_pos", i64),
        ("kv_fmt", i64), ("q_type", i64), ("out_type", i64),
        ("batch", i64), ("S", i64), ("nh", i64), ("nkv", i64), ("kvg", i64), ("l_hd", i64),
        ("cache_hd", i64), ("cache_cap", i64),
        ("win_start", i64), ("klen", i64), ("window", i64),
        ("softmax_scale", C.c_double),
        ("q_batch_stride", i64), ("out_batch_stride", i64), ("kv_batch_stride", i64), ("scale_batch_stride", i64),
        ("force_splits", i64), ("flags", i64),
    ]


class AttnPeer(C.Structure):
    """Mirror of ``nomos_attn_peer_t``."""
    _fields_ = [("struct_bytes", u64), ("rank", i64), ("world", i64), ("mailbox", u64 * 8), ("mailbox_bytes", i64),
                ("step", u64), ("timeout_us", i64)]


class KvRing(C.Structure):
    """Mirror of ``nomos_kv_ring_t``."""
    _fields_ = [("struct_bytes", i64), ("cache_cap", i64), ("window", i64), ("max_rows", i64), ("len", i64),
                ("staged", i64), ("high", i64)]


class KvStep(C.Structure):
    """Mirror of ``nomos_kv_step_t``."""
    _fields_ = [("base_pos", i64), ("n_new", i64), ("win_start", i64), ("klen", i64), ("window", i64)]


# name -> (restype, argtypes); must list every symbol include/nomos_attn.h declares.
PROTOTYPES = {
    "nomos_kv_ring_init": (i32, [C.POINTER(KvRing), i64, i64, i64]),
    "nomos_kv_ring_plan": (i32, [C.POINTER(KvRing), i64, C.POINTER(KvStep)]),
    "nomos_kv_ring_commit": (i32, [C.POINTER(KvRing), i64]),
    "nomos_kv_ring_set_len": (i32, [C.POINTER(KvRing), i64]),
    "nomos_kv_ring_fill_args": (i32, [C.POINTER(KvRing), C.POINTER(KvStep), C.POINTER(AttnArgs)]),
    "nomos_attn_version": (i32, []),
    "nomos_attn_last_error": (C.c_char_p, []),
    "nomos_attn_device_faults": (i32, [C.POINTER(C.c_uint32), i32]),
    "nomos_attn_paged_workspace_bytes": (i64, [i32] * 6),
    "nomos_attn_paged_decode_i8": (i32, [vp] + [u64] * 9 + [i64] + [i32] * 8 + [C.c_double, i32, i32]),
    "nomos_kv_paged_append_quant_i8": (i32, [vp] + [u64] * 8 + [i32] * 5),
    "nomos_attn_fused_host": (i32, [vp, C.POINTER(AttnArgs), u64, u64, C.c_int64, u64, u64, C.c_int64]),
    "nomos_kv_norm_rope_append": (i32, [vp] + [u64] * 11 + [i32] * 8 + [C.c_float, i32, i32]),
    "nomos_kv_quant_i8": (i32, [vp, u64, u64, u64, i32, i32]),
    "nomos_kv_dequant_i8": (i32, [vp, u64, u64, u64, i32, i32]),
    "nomos_kv_append_quant_i8": (i32, [vp] + [u64] * 6 + [i32] * 7),
    "nomos_kv_dequant_i8_layer": (i32, [vp] + [u64] * 3 + [i32] * 6),
    "nomos_kv_append_quant_i4": (i32, [vp] + [u64] * 6 + [i32] * 8),
    "nomos_kv_append_quant_i4_with_q8": (i32, [vp] + [u64] * 10 + [i32] * 9),
    "nomos_kv_dequant_i4_layer": (i32, [vp] + [u64] * 3 + [i32] * 7),
    "nomos_kv_dequant_i4_to_q8_layer": (i32, [vp] + [u64] * 4 + [i32] * 7),
    "nomos_kv_append_fp32": (i32, [vp] + [u64] * 4 + [i32] * 5),
    "nomos_kv_append_bf16": (i32, [vp] + [u64] * 6 + [i32] * 5),
    "nomos_kv_append_batched_bf16": (i32, [vp] + [u64] * 4 + [i32] * 7),
    "nomos_attn_decode_i8": (i32, [vp] + [u64] * 7 + [i32] * 7),
    "nomos_attn_decode_multirow_i8": (i32, [vp] + [u64] * 7 + [i32] * 10),
    "nomos_attn_prefix_batched_i8": (i32, [vp] + [u64] * 9 + [i32] * 11),
    "nomos_attn_decode_fp32": (i32, [vp] + [u64] * 5 + [i32] * 7),
    "nomos_attn_decode_bf16": (i32, [vp] + [u64] * 7 + [i32] * 7),
    "nomos_attn_prefix_batched_dense": (i32, [vp] + [u64] * 5 + [i32] * 12),
    "nomos_attn_prefill_batched_i8": (i32, [vp] + [u64] * 9 + [i32] * 8),
    "nomos_attn_prefix_batched_fp32": (i32, [vp] + [u64] * 7 + [i32] * 11),
    "nomos_attn_prefix_batched_bf16": (i32, [vp] + [u64] * 9 + [i32] * 11),
    "nomos_attn_prefill_batched_fp32": (i32, [vp] + [u64] * 7 + [i32] * 8),
    "nomos_attn_prefill_batched_bf16": (i32, [vp] + [u64] * 9 + [i32] * 8),
    "nomos_attn_workspace_bytes": (i64, [C.POINTER(AttnArgs)]),
    "nomos_attn_kernel_choice": (i32, [C.POINTER(AttnArgs)]),
    "nomos_attn_last_launch": (i32, [C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "nomos_attn_fused": (i32, [vp, C.POINTER(AttnArgs)]),
    "nomos_attn_fused_static_ws": (i32, [vp, C.POINTER(AttnArgs)]),
    "nomos_attn_merge_partials": (i32, [vp, u64, i32, i32, i32, u64, i32]),
    "nomos_attn_peer_mailbox_bytes": (i64, [i32, i32, i32]),
    "nomos_attn_peer_mailbox_create": (i32, [i64, C.POINTER(u64), vp]),
    "nomos_attn_peer_mailbox_open": (i32, [vp, C.POINTER(u64)]),
    "nomos_attn_peer_mailbox_close": (i32, [u64, i32]),
    "nomos_attn_seq_sharded": (i32, [vp, C.POINTER(AttnArgs), C.POINTER(AttnPeer)]),
    "nomos_attn_seq_sharded_status": (i32, [vp, i32]),
}


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nomos_nvfp4_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise ImportError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = res
        fn.argtypes = args
    return lib


_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB
