"""The ring bookkeeping API (host only): window arithmetic against the reference's formulas
(lib/engine_decode.mojo:420-444), the capacity guards, staged rows and roll-back, and a
slot-level simulation showing that a ring with max_rows - 1 slots of slack never overwrites a
key a row of the current or a later batch still needs."""
import numpy as np
import pytest

from nomos_nvfp4_b200 import build, ops


@pytest.fixture(scope="module", autouse=True)
def _built():
    build.build()


def test_decode_steps_follow_the_reference_window_arithmetic():
    W = 16
    r = ops.KvRing(cache_cap=W, window=W, max_rows=1)
    for pos in range(50):
        st = r.plan(1)
        seq_len = pos + 1
        win_start = max(0, seq_len - W)                       # engine_decode.mojo:431-433
        assert (st.base_pos, st.n_new, st.win_start, st.klen, st.window) == (pos, 1, win_start, seq_len - win_start, W)
        r.commit(1)
    assert r.len == 50


def test_linear_cache_refuses_to_overflow():
    r = ops.KvRing(cache_cap=8, window=0, max_rows=4)
    r.plan(4); r.commit(4)
    r.plan(4); r.commit(4)
    with pytest.raises(ops.NomosError) as e:                  # "prompt does not fit": loud, never an overrun
        r.plan(1)
    assert e.value.status == -3
    st = ops.KvRing(cache_cap=8, window=0, max_rows=4).plan(3)
    assert (st.win_start, st.klen, st.window) == (0, 3, 0)


def test_ring_without_slack_cannot_be_sized_for_batches():
    with pytest.raises(ops.NomosError) as e:
        ops.KvRing(cache_cap=1024, window=1024, max_rows=9)   # the reference's ring: verify would alias
    assert e.value.status == -3
    ops.KvRing(cache_cap=1032, window=1024, max_rows=9)
    r = ops.KvRing(cache_cap=1032, window=1024, max_rows=9)
    with pytest.raises(ops.NomosError):
        r.plan(10)                                            # more rows than the ring was sized for


def test_verify_commit_and_rollback():
    W, VB = 8, 4
    r = ops.KvRing(cache_cap=W + VB - 1, window=W, max_rows=VB)
    r.plan(VB); r.commit(VB)                                  # "prefill" of 4 positions
    for _ in range(10):
        L = r.len
        st = r.plan(VB)
        assert st.base_pos == L and st.n_new == VB
        assert st.klen == min(L + VB, W + VB - 1) and st.win_start == L + VB - st.klen
        with pytest.raises(ops.NomosError):
            r.commit(VB + 1)
        r.commit(2)                                           # two drafts accepted, two rejected
        assert r.len == L + 2
    # KV reuse: truncate to a shorter prefix, as far back as the ring still holds what is needed
    L = r.len                                                 # 24 committed, 26 written, 11 slots: 15.. are kept
    r.set_len(L - 1)                                          # needs 16..22: still there
    with pytest.raises(ops.NomosError) as e:
        r.set_len(L - 5)                                      # would need 12..: overwritten
    assert e.value.status == -3
    with pytest.raises(ops.NomosError) as e:
        r.set_len(L + 5)                                      # cannot grow
    assert e.value.status == -1
    r.set_len(0)                                              # an empty cache needs nothing
    assert r.len == 0


def test_slack_rule_keeps_every_needed_key():
    """Simulate slot contents: after each batch of rows is written to slot pos % cap, every key
    position in a row's window [max(0, p - W + 1), p] must still be the one stored in its slot."""
    rng = np.random.default_rng(0)
    W, VB = 32, 5
    cap = W + VB - 1
    r = ops.KvRing(cache_cap=cap, window=W, max_rows=VB)
    slots = np.full(cap, -1, np.int64)
    for _ in range(300):
        n = int(rng.integers(1, VB + 1))
        st = r.plan(n)
        for i in range(n):
            slots[(st.base_pos + i) % cap] = st.base_pos + i              # the append
        for i in range(n):                                                # the attention of row i
            p = st.base_pos + i
            for key in range(max(0, p - W + 1), p + 1):
                assert slots[key % cap] == key, f"row at {p} lost key {key}"
            assert st.win_start <= max(0, p - W + 1) and p < st.win_start + st.klen
        r.commit(int(rng.integers(0, n + 1)))                             # rejected rows get overwritten later


def test_fill_args_copies_the_step():
    r = ops.KvRing(cache_cap=40, window=32, max_rows=9)
    r.plan(9); r.commit(9)
    st = r.plan(9)
    a = ops.make_args(nh=8, nkv=4, kvg=2, l_hd=128, cache_hd=128, cache_cap=1, klen=1)
    r.fill_args(st, a)
    assert (a.cache_cap, a.S, a.win_start, a.klen, a.window, a.n_new, a.new_base_pos) == (40, 9, 0, 18, 32, 9, 9)
