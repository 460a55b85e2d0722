"""CPU checks of the producer-epilogue oracle (V-norm, QK-norm, RoPE) and of the argument
validation of nomos_kv_norm_rope_append (no GPU work: every call is refused before a launch)."""
import numpy as np
import pytest

from oracle import np_producer as npp


def test_rms_norms_have_unit_mean_square():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 4, 128)) * 7.0
    v = npp.rmsnorm_no_weight(x)
    assert np.allclose(np.mean(v * v, axis=-1), 1.0, atol=1e-6)
    w = rng.standard_normal(128)
    k = npp.qk_norm(x, w)
    assert np.allclose(k, v * w)
    # an all-zero head stays zero (eps keeps the reciprocal finite), ops_gpu_mojo_reductions.mojo:396
    z = npp.rmsnorm_no_weight(np.zeros((1, 1, 128)))
    assert np.all(z == 0.0)


@pytest.mark.parametrize("hd,rope_dim,theta", [(128, 128, 10000.0), (256, 256, 10000.0), (512, 128, 1000000.0)])
def test_rope_is_a_rotation_of_half_split_pairs(hd, rope_dim, theta):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 3, hd))
    y = npp.rope(x, base_pos=17, theta=theta, rope_dim=rope_dim)
    n, half = rope_dim // 2, hd // 2
    # pair norms are preserved, untouched dims are untouched
    assert np.allclose(np.hypot(y[..., :n], y[..., half:half + n]), np.hypot(x[..., :n], x[..., half:half + n]))
    assert np.array_equal(y[..., n:half], x[..., n:half]) and np.array_equal(y[..., half + n:], x[..., half + n:])
    # position 0 is the identity; a rotation by pos then by -pos returns the input
    assert np.allclose(npp.rope(x[:1], 0, theta, rope_dim), x[:1])
    # pair 0 has frequency 1: token s rotates by exactly base_pos + s radians
    a, b = x[2, 0, 0], x[2, 0, half]
    ang = 17 + 2
    assert np.allclose([y[2, 0, 0], y[2, 0, half]], [a * np.cos(ang) - b * np.sin(ang), a * np.sin(ang) + b * np.cos(ang)])


def test_ln_theta_follows_the_reference_switch():
    assert npp.ln_theta(1000000.0) == npp.LN_THETA_1E6
    assert npp.ln_theta(10000.0) == npp.LN_THETA_DEFAULT
    assert npp.ln_theta(500000.0) == npp.LN_THETA_DEFAULT      # any other value: ln(10000), ops_gpu_mojo.mojo:335-337
    assert abs(npp.LN_THETA_1E6 - np.log(1e6)) < 1e-7 and abs(npp.LN_THETA_DEFAULT - np.log(1e4)) < 1e-7


def test_producer_arguments_are_refused_before_launch():
    from nomos_nvfp4_b200 import build, ops
    build.build()
    P = 0x1000   # never dereferenced: validation fails first
    kw = dict(n_s=1, nh=8, nkv=4, l_hd=128, l_kvd=512, cache_cap=64, cache_hd=128, base_pos=0, theta=1e4, rope_dim=128,
              kv_fmt=ops.KV_I8)
    with pytest.raises(ops.NomosError) as e:                     # null source
        ops.kv_norm_rope_append(0, None, None, P, None, P, P, P, P, P, **kw)
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:                     # query rows without their norm weight
        ops.kv_norm_rope_append(0, P, None, P, P, P, P, P, P, P, **kw)
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:                     # odd rope_dim
        ops.kv_norm_rope_append(0, None, None, P, P, P, P, P, P, P, **{**kw, "rope_dim": 63})
    assert e.value.status == -1
    with pytest.raises(ops.NomosError) as e:                     # head_dim beyond the staging row
        ops.kv_norm_rope_append(0, None, None, P, P, P, P, P, P, P, **{**kw, "l_hd": 1024, "cache_hd": 1024, "l_kvd": 4096, "rope_dim": 256})
    assert e.value.status == -2
    with pytest.raises(ops.NomosError) as e:                     # cache pointers missing although a format is given
        ops.kv_norm_rope_append(0, None, None, P, P, P, None, P, P, P, **kw)
    assert e.value.status == -1
    ops.kv_norm_rope_append(0, None, None, P, P, P, P, P, P, P, **{**kw, "n_s": 0})   # nothing to do: ok
