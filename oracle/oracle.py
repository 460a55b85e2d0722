"""ctypes front end of the CPU oracle (``nomos_oracle.c``).

TEST INFRASTRUCTURE ONLY.  The shipped library never imports this module; it is
used by the tests, by the smoke check and by the benchmark's CPU-baseline leg as
the *checker*.  Parity status: "parity unpinned" at the byte level (see the C
file's header): the reference publishes no golden KV bytes, so bit-exactness is
against this restatement of its arithmetic.

Every wrapper keeps the argument order of the reference operator it restates
(paths relative to the reference project root):

  quant_kv_i8 / dequant_kv_i8              lib/kv_cache_quant.mojo:100,116
  append_quant_kv_i8                       lib/kv_cache_quant.mojo:252
  dequant_kv_i8_layer                      lib/kv_cache_quant.mojo:274
  append_quant_kv_i4                       lib/kv_cache_quant.mojo:803
  append_quant_kv_i4_with_q8               lib/kv_cache_quant.mojo:839
  dequant_kv_i4_layer                      lib/kv_cache_quant.mojo:885
  dequant_kv_i4_to_q8_layer                lib/kv_cache_quant.mojo:956
  append_kv_fp32 / append_kv_batched_bf16  lib/attention_gpu.mojo:87, lib/batched_attn_gpu.mojo:87
  attn_decode_int8                         lib/attention_gpu_int8.mojo:598
  attn_multirow_int8                       lib/attention_gpu_int8.mojo:634
  attn_prefix_batched_int8                 lib/attention_gpu_int8.mojo:844
  attn_decode_dense                        lib/attention_gpu.mojo:165,207
  attn_prefix_batched_dense                lib/batched_attn_gpu.mojo:499,613
  attn_exact / merge_partials              the tolerance gate (exact dequant, fp64)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "_build" / "libnomos_oracle.so"

KV_I8, KV_I4, KV_I4B32 = 0, 1, 2


def build(force: bool = False) -> Path:
    """Compile the oracle with gcc (OpenMP if the compiler has it)."""
    src = _HERE / "nomos_oracle.c"
    if _SO.exists() and not force and _SO.stat().st_mtime >= src.stat().st_mtime:
        return _SO
    _SO.parent.mkdir(exist_ok=True)
    base = ["-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-fvisibility=hidden",
            "-shared", "-o", str(_SO), str(src), "-lm"]
    last = None
    for cc in ("/usr/bin/gcc", "gcc", "cc"):
        for omp in (["-fopenmp"], []):
            try:
                subprocess.run([cc, *omp, *base], check=True, capture_output=True)
                return _SO
            except (OSError, subprocess.CalledProcessError) as e:  # try the next spelling
                last = e
    raise RuntimeError(f"could not build the oracle: {last}")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            build()
        _lib = C.CDLL(str(_SO))
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle buffers must be C-contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _call(name: str, *args):
    fn = getattr(lib(), name)
    fn.restype = None
    conv = []
    for a in args:
        if isinstance(a, np.ndarray) or a is None:
            conv.append(_p(a))
        elif isinstance(a, float):
            conv.append(C.c_double(a))
        else:
            conv.append(C.c_int(int(a)))
    fn(*conv)


# ---------------------------------------------------------------- dtype helpers

def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    fn = lib().orc_f32_to_bf16
    fn.restype = None
    fn(_p(x), _p(out), C.c_long(x.size))
    return out


def bf16_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << 16).view(np.float32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 values rounded to the nearest bf16, returned as fp32."""
    return bf16_to_f32(f32_to_bf16(x))


# ----------------------------------------------------------------- cache buffers

def scale_buffer_bytes(nkv: int, cache_cap: int, l_hd: int, scale_blocks: int) -> int:
    """Bytes of one K (or V) scale buffer.  Row scale: fp32 per row.  Block-32:
    fp16 per block followed by an fp32 per row (lib/gemma4_engine.mojo:586-595,
    lib/kv_cache_quant.mojo:529-534)."""
    rows = nkv * cache_cap
    if scale_blocks > 1:
        return rows * scale_blocks * 2 + rows * 4
    return rows * 4


# ----------------------------------------------------------------------- codecs

def quant_kv_i8(in_bf16, out_i8, out_scales, n_rows, dim):
    _call("orc_quant_kv_i8", in_bf16, out_i8, out_scales, n_rows, dim)


def dequant_kv_i8(in_i8, in_scales, out_bf16, n_rows, dim):
    _call("orc_dequant_kv_i8", in_i8, in_scales, out_bf16, n_rows, dim)


def append_quant_kv_i8(src_k, src_v, dst_k, dst_v, k_scales, v_scales,
                       n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos):
    _call("orc_append_quant_kv_i8", src_k, src_v, dst_k, dst_v, k_scales, v_scales,
          n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos)


def dequant_kv_i8_layer(src, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start):
    _call("orc_dequant_kv_i8_layer", src, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start)


def append_quant_kv_i4(src_k, src_v, dst_k, dst_v, k_scales, v_scales,
                       n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, scale_blocks=1):
    _call("orc_append_quant_kv_i4", src_k, src_v, dst_k, dst_v, k_scales, v_scales,
          n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, scale_blocks)


def append_quant_kv_i4_with_q8(src_k, src_v, dst_k, dst_v, k_scales, v_scales,
                               k_q8, v_q8, k_q8_scales, v_q8_scales,
                               n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, q8_pitch, scale_blocks=1):
    _call("orc_append_quant_kv_i4_with_q8", src_k, src_v, dst_k, dst_v, k_scales, v_scales,
          k_q8, v_q8, k_q8_scales, v_q8_scales,
          n_s, nkv, l_hd, l_kvd, cache_cap, cache_hd, base_pos, q8_pitch, scale_blocks)


def dequant_kv_i4_layer(src, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap, win_start, scale_blocks=1):
    _call("orc_dequant_kv_i4_layer", src, scales, dst_bf16, nkv, klen, cache_hd, max_seq, cache_cap,
          win_start, scale_blocks)


def dequant_kv_i4_to_q8_layer(src, scales, dst_i8, dst_scale, nkv, klen, cache_hd, max_seq, cache_cap,
                              win_start, scale_blocks=1):
    _call("orc_dequant_kv_i4_to_q8_layer", src, scales, dst_i8, dst_scale, nkv, klen, cache_hd, max_seq,
          cache_cap, win_start, scale_blocks)


def block32_i4_q8_scales(scales16, dst_scale, nkv, klen, nblocks, max_seq, cache_cap, win_start):
    _call("orc_block32_i4_q8_scales", scales16, dst_scale, nkv, klen, nblocks, max_seq, cache_cap, win_start)


def append_kv_fp32(k_cache, v_cache, k_new, v_new, nkv, l_hd, cache_hd, max_seq, cl):
    _call("orc_append_kv_fp32", k_cache, v_cache, k_new, v_new, nkv, l_hd, cache_hd, max_seq, cl)


def append_kv_batched_bf16(src_k, src_v, dst_k, dst_v, n_s, nkv, l_hd, l_kvd, max_seq, cache_hd, base_pos=0):
    _call("orc_append_kv_batched_bf16", src_k, src_v, dst_k, dst_v, n_s, nkv, l_hd, l_kvd, max_seq,
          cache_hd, base_pos)


# -------------------------------------------------------------------- attention

def attn_decode_int8(q, k_i8, v_i8, k_scale, v_scale, scores, out, nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg):
    _call("orc_attn_decode_int8", q, k_i8, v_i8, k_scale, v_scale, scores, out,
          nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg)


def attn_multirow_int8(q_b, scores, out, k_i8, v_i8, k_scale, v_scale,
                       nh, nkv, l_hd, cache_hd, max_seq, S, score_stride, kvg, window, query_base_pos):
    _call("orc_attn_multirow_int8", q_b, scores, out, k_i8, v_i8, k_scale, v_scale,
          nh, nkv, l_hd, cache_hd, max_seq, S, score_stride, kvg, window, query_base_pos)


def attn_prefix_batched_int8(q_b, scores, out, k_i8, v_i8, k_scale, v_scale,
                             nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window,
                             query_base_pos, key_base_pos):
    _call("orc_attn_prefix_batched_int8", q_b, scores, out, k_i8, v_i8, k_scale, v_scale,
          nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window, query_base_pos, key_base_pos)


def attn_decode_dense(q, k_cache, v_cache, scores, out, nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg, kv_is_bf16):
    _call("orc_attn_decode_dense", q, k_cache, v_cache, scores, out,
          nh, nkv, l_hd, cache_hd, max_seq, seq_len, kvg, int(kv_is_bf16))


def attn_prefix_batched_dense(q_b, k_cache, v_cache, scores, out, nh, nkv, l_hd, cache_hd, max_seq, S, key_len,
                              kvg, window, query_base_pos, key_base_pos, kv_is_bf16):
    _call("orc_attn_prefix_batched_dense", q_b, k_cache, v_cache, scores, out,
          nh, nkv, l_hd, cache_hd, max_seq, S, key_len, kvg, window, query_base_pos, key_base_pos,
          int(kv_is_bf16))


def attn_exact(q, k_cache, v_cache, k_scales, v_scales, kv_fmt, nh, nkv, l_hd, cache_hd, cache_cap,
               S=1, kvg=None, window=0, query_base_pos=0, win_lo=0, softmax_scale=1.0, want_partial=False):
    """The tolerance gate: exact-dequant attention over the packed ring, fp64.

    q is [S, nh, l_hd] fp32; returns out [S, nh, l_hd] fp32 (and, if asked, the
    un-normalised partial triples [S*nh, l_hd+2] fp64 = o.., m, l)."""
    kvg = kvg if kvg is not None else nh // nkv
    q = np.ascontiguousarray(q, dtype=np.float32).reshape(S, nh, l_hd)
    out = np.full((S, nh, l_hd), np.nan, dtype=np.float32)
    part = np.zeros((S * nh, l_hd + 2), dtype=np.float64) if want_partial else None
    fn = lib().orc_attn_exact
    fn.restype = None
    fn(_p(q), _p(k_cache), _p(v_cache), _p(k_scales), _p(v_scales), _p(out), _p(part),
       C.c_int(kv_fmt), C.c_int(nh), C.c_int(nkv), C.c_int(l_hd), C.c_int(cache_hd), C.c_int(cache_cap),
       C.c_int(S), C.c_int(kvg), C.c_int(window), C.c_int(query_base_pos), C.c_int(win_lo),
       C.c_double(softmax_scale))
    return (out, part) if want_partial else out


def merge_partials(partials: np.ndarray, l_hd: int) -> np.ndarray:
    """partials [G, rows, l_hd+2] fp64 -> out [rows, l_hd] fp32."""
    partials = np.ascontiguousarray(partials, dtype=np.float64)
    G, rows, _ = partials.shape
    out = np.empty((rows, l_hd), dtype=np.float32)
    _call("orc_merge_partials", partials, out, G, rows, l_hd)
    return out


def set_threads(n: int) -> None:
    """Thread count of the OpenMP loops (CPU-baseline timing)."""
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        omp = C.CDLL("libgomp.so.1")
        omp.omp_set_num_threads(C.c_int(n))
    except OSError:
        pass
