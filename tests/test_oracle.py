"""The CPU oracle against the reference: golden vectors generated from the
reference's own build, bit-for-bit agreement with that build where it is
present, and the behavioural pins of the reference's CPU tests
(tests/test_attention.py:71-149, tests/test_attention_paged.py:62-151)."""

import hashlib
import math

import numpy as np
import pytest

import cases
import oracle


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest()[:8], dtype=np.uint64)[0]


def ref64(q, k, v, lens=None):
    """float64 eager reference (tests/test_attention.py:26-45)."""
    b, hq, d = q.shape
    _, hkv, t, _ = k.shape
    group = hq // hkv
    out = np.zeros((b, hq, d), dtype=np.float64)
    for bi in range(b):
        length = t if lens is None else int(lens[bi])
        if length == 0:
            continue
        for h in range(hq):
            kv = h // group
            s = k[bi, kv, :length].astype(np.float64) @ q[bi, h].astype(np.float64)
            s /= math.sqrt(d)
            p = np.exp(s - s.max())
            p /= p.sum()
            out[bi, h] = p @ v[bi, kv, :length].astype(np.float64)
    return out


@pytest.mark.parametrize("b,hq,hkv,t,d,wl", cases.SHAPES)
def test_oracle_matches_golden_bit_exact(golden, b, hq, hkv, t, d, wl):
    rng = np.random.default_rng(cases.shape_seed(b, hq, hkv, t, d))
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, wl)
    name = "shape_%d_%d_%d_%d_%d" % (b, hq, hkv, t, d)
    assert digest(q, k, v, lens) == golden[name + "_sum"], "input generator drifted"
    y = oracle.decode(q, k, v, lens)
    np.testing.assert_array_equal(y, golden[name])
    np.testing.assert_allclose(y, ref64(q, k, v, lens), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", sorted(cases.PAGED_CASES))
def test_oracle_paged_matches_golden_bit_exact(golden, name):
    seed, b, hq, hkv, d, nb, lens = cases.PAGED_CASES[name]
    rng = np.random.default_rng(seed)
    q, kp, vp, tbl, kc, vc, la = cases.make_paged_case(rng, b, hq, hkv, d, nb, lens)
    assert digest(q, kp, vp, tbl, la) == golden[name + "_sum"]
    y = oracle.decode_paged(q, kp, vp, tbl, la)
    np.testing.assert_array_equal(y, golden[name])
    # the paged walk must equal the contiguous walk on the materialised cache
    np.testing.assert_array_equal(y, oracle.decode(q, kc, vc, la))


def test_oracle_benchmark_configs_golden(golden):
    import torch
    q, k, v = cases.config1()
    assert digest(q, k, v) == golden["config1_sum"]
    np.testing.assert_array_equal(oracle.decode(q, k, v), golden["config1"])
    q, k, v = cases.config2(batch=1, t=1024)
    qr, kr, vr = (cases.round_to(x, torch.bfloat16) for x in (q, k, v))
    assert digest(qr, kr, vr) == golden["config2_b1_t1024_bf16_sum"]
    np.testing.assert_array_equal(oracle.decode(qr, kr, vr),
                                  golden["config2_b1_t1024_bf16"])


@pytest.mark.skipif(not oracle.ref_available(), reason="reference build absent")
@pytest.mark.parametrize("seed", range(6))
def test_oracle_equals_reference_build(seed):
    rng = np.random.default_rng(900 + seed)
    b = int(rng.integers(1, 4))
    hkv = int(rng.choice([1, 2, 3, 8]))
    g = int(rng.choice([1, 2, 4, 5, 8]))
    d = int(rng.choice([4, 8, 64, 128]))
    t = int(rng.integers(1, 300))
    q, k, v, lens = cases.make_case(rng, b, hkv * g, hkv, t, d, True)
    np.testing.assert_array_equal(oracle.decode(q, k, v, lens),
                                  oracle.ref_decode(q, k, v, lens))
    lens_l = [int(x) for x in rng.integers(0, 80, b)]
    qp, kp, vp, tbl, kc, vc, la = cases.make_paged_case(rng, b, hkv * g, hkv, d, 9, lens_l)
    np.testing.assert_array_equal(oracle.decode_paged(qp, kp, vp, tbl, la),
                                  oracle.ref_decode_paged(qp, kp, vp, tbl, la))


def test_gqa_mapping_constant_v():
    # tests/test_attention.py:82-95
    rng = np.random.default_rng(5)
    b, hq, hkv, t, d = 1, 6, 3, 4, 8
    q = np.ones((b, hq, d), np.float32)
    k = np.zeros((b, hkv, t, d), np.float32)
    v = rng.standard_normal((b, hkv, d)).astype(np.float32)
    v = np.broadcast_to(v[:, :, None, :], (b, hkv, t, d)).copy()
    y = oracle.decode(q, k, v)
    for h in range(hq):
        np.testing.assert_allclose(y[0, h], v[0, h // 2].mean(axis=0), rtol=1e-5, atol=1e-6)


def test_padding_ignored_and_zero_len():
    # tests/test_attention.py:98-115
    rng = np.random.default_rng(6)
    q, k, v, _ = cases.make_case(rng, 2, 8, 4, 16, 32, False)
    lens = np.array([16, 5], np.int32)
    y = oracle.decode(q, k, v, lens)
    k2, v2 = k.copy(), v.copy()
    k2[1, :, 5:] = 1e6
    v2[1, :, 5:] = 1e6
    np.testing.assert_array_equal(oracle.decode(q, k2, v2, lens)[1], y[1])
    y0 = oracle.decode(q, k, v, np.array([0, 5], np.int32))
    assert np.all(y0[0] == 0)


def test_error_contract():
    # tests/test_attention.py:118-149, tests/test_attention_paged.py:127-138
    q = np.zeros((1, 6, 32), np.float32)
    k = np.zeros((1, 2, 8, 32), np.float32)
    with pytest.raises(ValueError):
        oracle.decode(np.zeros((1, 5, 32), np.float32), k, k)
    with pytest.raises(ValueError):
        oracle.decode(np.zeros((1, 6, 30), np.float32),
                      np.zeros((1, 2, 8, 30), np.float32),
                      np.zeros((1, 2, 8, 30), np.float32))
    with pytest.raises(ValueError):
        oracle.decode(np.zeros((1, 2, 516), np.float32),
                      np.zeros((1, 1, 4, 516), np.float32),
                      np.zeros((1, 1, 4, 516), np.float32))
    with pytest.raises(ValueError):
        oracle.decode(q, k, k, np.array([9], np.int32))
    with pytest.raises(ValueError):
        oracle.decode(q, k, k, np.array([-1], np.int32))
    rng = np.random.default_rng(46)
    qp, kp, vp, tbl, kc, vc, lens = cases.make_paged_case(rng, 2, 4, 2, 32, 8, [16, 32])
    bad = tbl.copy()
    bad[0, 0] = 999
    with pytest.raises(ValueError):
        oracle.decode_paged(qp, kp, vp, bad, lens)
    with pytest.raises(ValueError):
        oracle.decode_paged(qp, kp, vp, tbl, np.array([2 * cases.PAGE + 1, 3], np.int32))


def test_partial_merge_algebra():
    """Splitting the cache rows of one (b, h) into shards, taking (m, l, acc)
    of each and merging equals the unsharded result - including empty shards
    (short sequences on a KV-length split)."""
    rng = np.random.default_rng(77)
    d, t = 64, 333
    q = rng.standard_normal(d).astype(np.float32)
    k = rng.standard_normal((t, d)).astype(np.float32)
    v = rng.standard_normal((t, d)).astype(np.float32)
    full = oracle.decode(q[None, None], k[None, None], v[None, None])[0, 0]
    for bounds in ([0, 100, 200, 333], [0, 333, 333, 333], [0, 0, 1, 333], [0, 64, 64, 128, 333]):
        ml, acc = [], []
        for t0, t1 in zip(bounds[:-1], bounds[1:]):
            m, l, a = oracle.partial(q, k, v, t0, t1)
            ml.append([m, l])
            acc.append(a)
        y = oracle.merge(np.array(ml, np.float32), np.array(acc, np.float32))
        np.testing.assert_allclose(y, full, rtol=2e-5, atol=2e-6)
    # every shard empty -> zero row
    y = oracle.merge(np.array([[-np.inf, 0.0]] * 3, np.float32), np.zeros((3, d), np.float32))
    assert np.all(y == 0)
