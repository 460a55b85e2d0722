"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol
the public header declares, and rejects bad arguments with the documented status
before touching the device (no compute calls: this file needs no GPU)."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "nomos_attn.h"


@pytest.fixture(scope="module")
def lib():
    from nomos_nvfp4_b200 import _lib, build
    build.build()
    return _lib.load()


def declared_symbols():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nomos_(?:attn|kv)_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    from nomos_nvfp4_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.PROTOTYPES), "ctypes prototypes and header disagree"


def test_only_public_symbols_are_exported():
    import subprocess
    from nomos_nvfp4_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    exported = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert exported and all(s.startswith(("nomos_attn_", "nomos_kv_")) for s in exported), exported


def test_args_struct_matches_header(lib):
    from nomos_nvfp4_b200 import _lib
    text = HEADER.read_text()
    body = re.search(r"typedef struct nomos_attn_args \{(.*?)\} nomos_attn_args_t;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        _, names = decl.split(None, 1)
        fields += [n.strip() for n in names.split(",")]
    assert fields == [f[0] for f in _lib.AttnArgs._fields_]
    assert C.sizeof(_lib.AttnArgs) == 8 * len(fields)


def test_version_and_error_text(lib):
    assert lib.nomos_attn_version() >= 100
    assert isinstance(lib.nomos_attn_last_error(), bytes)


def test_bad_arguments_are_refused_before_launch(lib):
    from nomos_nvfp4_b200 import ops
    P = 0x1000   # never dereferenced: validation fails first
    with pytest.raises(ops.NomosError) as e:   # nh != nkv*kvg
        ops.attention_gpu_int8_dev(0, P, P, P, P, P, P, P, 8, 4, 128, 128, 64, 16, 3)
    assert e.value.status == -1 and b"nkv" in lib.nomos_attn_last_error()
    with pytest.raises(ops.NomosError) as e:   # unsupported head_dim
        ops.attention_gpu_int8_dev(0, P, P, P, P, P, P, P, 8, 4, 96, 96, 64, 16, 2)
    assert e.value.status == -2
    with pytest.raises(ops.NomosError) as e:   # null pointer
        ops.gpu_append_quant_kv_i8(0, P, 0, P, P, P, P, 1, 4, 128, 512, 64, 128, 0)
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:   # block-32 with the wrong block count
        ops.gpu_append_quant_kv_i4(0, P, P, P, P, P, P, 1, 4, 128, 512, 64, 128, 0, 3)
    assert e.value.status == -2
    with pytest.raises(ops.NomosError) as e:   # view rows beyond the pitch
        ops.gpu_append_quant_kv_i4_with_q8(0, P, P, P, P, P, P, P, P, P, P, 4, 4, 128, 512, 64, 128, 62, 64, 1)
    assert e.value.status == -3
    with pytest.raises(ops.NomosError) as e:   # window longer than the ring
        ops.gpu_dequant_kv_i8_layer(0, P, P, P, 4, 100, 128, 128, 64, 0)
    assert e.value.status == -3
    with pytest.raises(ops.NomosError) as e:   # misaligned cache
        ops.attention_gpu_int8_dev(0, P, P + 1, P, P, P, P, P, 8, 4, 128, 128, 64, 16, 2)
    assert e.value.status == -1
    # reference no-ops (lib/attention_gpu_int8.mojo:615-616) return ok without touching anything
    ops.attention_gpu_int8_dev(0, 0, 0, 0, 0, 0, 0, 0, 0, 4, 128, 128, 64, 16, 2)
    ops.attention_gpu_int8_dev(0, 0, 0, 0, 0, 0, 0, 0, 8, 4, 128, 128, 64, 0, 2)
    ops.gpu_append_quant_kv_i8(0, 0, 0, 0, 0, 0, 0, 0, 4, 128, 512, 64, 128, 0)


def test_paged_arguments_are_refused_before_launch(lib):
    from nomos_nvfp4_b200 import ops
    P = 0x1000   # never dereferenced: validation fails first
    kw = dict(batch=2, nh=8, nkv=4, kvg=2, l_hd=128, n_pages=8, max_pages=4, max_len=300)
    with pytest.raises(ops.NomosError) as e:                     # null block table
        ops.attn_paged_decode_i8(0, P, P, P, P, P, None, P, P, P, 64, **kw)
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:                     # head_dim 256 is not paged
        ops.attn_paged_decode_i8(0, P, P, P, P, P, P, P, P, P, 64, **{**kw, "l_hd": 256})
    assert e.value.status == -2
    with pytest.raises(ops.NomosError) as e:                     # max_len beyond the block table
        ops.attn_paged_decode_i8(0, P, P, P, P, P, P, P, P, P, 64, **{**kw, "max_len": 4 * 128 + 1})
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:                     # misaligned pool
        ops.attn_paged_decode_i8(0, P, P + 8, P, P, P, P, P, P, P, 64, **kw)
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:
        ops.kv_paged_append_quant_i8(0, P, P, P, P, P, P, P, None, batch=2, nkv=4, l_hd=128, l_kvd=512, max_pages=4)
    assert e.value.status == -1
    assert ops.attn_paged_workspace_bytes(2, 8, 4, 2, 128, 100) >= 0


def test_fused_args_validation(lib):
    from nomos_nvfp4_b200 import ops
    a = ops.make_args(q=0x1000, k_cache=0x1000, v_cache=0x1000, k_scales=0x1000, v_scales=0x1000, out=0x1000,
                      nh=32, nkv=16, kvg=2, l_hd=128, cache_hd=128, cache_cap=1024, klen=2048)
    with pytest.raises(ops.NomosError) as e:   # window longer than the ring
        ops.attn_fused(0, a)
    assert e.value.status == -3
    a.struct_bytes = 8
    with pytest.raises(ops.NomosError) as e:
        ops.attn_fused(0, a)
    assert e.value.status == -1


def test_planning_calls_refuse_a_zero_capacity(lib):
    """A zero-initialised argument block (cache_cap = 0) is a bad argument for the planning entry points and for
    the workspace-free call, not a division by zero inside the planner."""
    from nomos_nvfp4_b200 import ops
    a = ops.make_args(q=0x1000, k_cache=0x10000, v_cache=0x20000, k_scales=0x30000, v_scales=0x40000, out=0x50000,
                      nh=32, nkv=16, kvg=2, l_hd=128, cache_hd=128, cache_cap=0, klen=2048)
    for call in (ops.attn_workspace_bytes, ops.attn_kernel_choice, lambda x: ops.attn_fused_static_ws(0, x),
                 lambda x: ops.attn_fused(0, x)):
        with pytest.raises(ops.NomosError) as e:
            call(a)
        assert e.value.status == -1
    a.cache_cap, a.win_start = 4096, -1
    with pytest.raises(ops.NomosError) as e:
        ops.attn_workspace_bytes(a)
    assert e.value.status == -1


def test_prefix_operator_ranges(lib):
    """The prefix-batched int8 operator: ranges the decode-order kernel cannot express are refused with -2 rather
    than computed wrongly; negative positions are bad arguments."""
    from nomos_nvfp4_b200 import ops
    P = 0x1000
    with pytest.raises(ops.NomosError) as e:   # key array longer than the row pitch
        ops.attention_prefill_prefix_batched_int8(0, P, 0, P, 0, P, P, P, P, P, 8, 4, 128, 128, 64, 4, 65, 2, 0, 61, 0)
    assert e.value.status == -3
    with pytest.raises(ops.NomosError) as e:
        ops.attention_prefill_prefix_batched_int8(0, P, 0, P, 0, P, P, P, P, P, 8, 4, 128, 128, 64, 4, 20, 2, 0, -1, 0)
    assert e.value.status == -1
