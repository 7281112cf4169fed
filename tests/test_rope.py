"""RoPE: the oracle against the reference's pins on CPU, the CUDA kernel against the oracle on a GPU.
Shapes, seeds and tolerances follow the reference's tests/test_rope.py."""

import math

import numpy as np
import pytest

import oracle


def ref64(x, theta, pos_offset, neox):
    """The eager statement in the reference's tests (test_rope.py:17-44)."""
    seq, dim = x.shape
    y = np.zeros_like(x)
    for r in range(seq):
        for j in range(dim // 2):
            a = (r + pos_offset) * theta ** (-2.0 * j / dim)
            c, s = math.cos(a), math.sin(a)
            ia, ib = (j, dim // 2 + j) if neox else (2 * j, 2 * j + 1)
            y[r, ia] = x[r, ia] * c - x[r, ib] * s
            y[r, ib] = x[r, ia] * s + x[r, ib] * c
    return y


def make_qk(seq, dim, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((seq, dim)).astype(np.float32), rng.standard_normal((seq, dim)).astype(np.float32))


@pytest.mark.parametrize("neox", [False, True])
def test_oracle_matches_eager_statement(neox):
    q, k = make_qk(4, 16, seed=1)
    np.testing.assert_allclose(oracle.rope(q, 10000.0, 0, neox), ref64(q, 10000.0, 0, neox), atol=1e-4)
    np.testing.assert_allclose(oracle.rope(k, 10000.0, 7, neox), ref64(k, 10000.0, 7, neox), atol=1e-4)
    np.testing.assert_allclose(oracle.rope(q, 500000.0, 0, neox), ref64(q, 500000.0, 0, neox), atol=1e-4)


@pytest.mark.skipif(not oracle.ref_available(), reason="reference build not present")
@pytest.mark.parametrize("neox", [False, True])
def test_oracle_equals_reference_build(neox):
    for seed, (seq, dim, off) in enumerate([(3, 8, 0), (9, 64, 5), (33, 128, 4000), (2, 6, 1)]):
        q, _ = make_qk(seq, dim, seed)
        np.testing.assert_array_equal(oracle.rope(q, 10000.0, off, neox), oracle.ref_rope(q, 10000.0, off, neox))


def test_oracle_properties():
    q, _ = make_qk(8, 16, seed=3)
    np.testing.assert_allclose(oracle.rope(q)[0], q[0], atol=1e-6)                  # position 0 is the identity
    np.testing.assert_allclose(oracle.rope(q[5:7].copy(), pos_offset=5), oracle.rope(q)[5:7], atol=1e-6)
    q2 = oracle.rope(q)
    np.testing.assert_allclose(np.hypot(q2[:, 0::2], q2[:, 1::2]), np.hypot(q[:, 0::2], q[:, 1::2]), atol=1e-5)
    with pytest.raises(ValueError):
        oracle.rope(np.zeros((2, 7), np.float32))
    with pytest.raises(ValueError):
        oracle.rope(np.zeros((2, 8), np.float32), pos_offset=-1)


# ---------------------------------------------------------------------------- GPU

@pytest.mark.gpu
@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("seq,dim,off", [(4, 64, 3), (1, 128, 4095), (257, 128, 0), (5, 6, 2), (3, 2, 0), (64, 256, 100000)])
def test_gpu_staged_and_zero_copy_match_oracle(neox, seq, dim, off):
    import torch
    import fusedtok_b200 as ft
    q, k = make_qk(seq, dim, seed=seq + dim)
    want_q, want_k = oracle.rope(q, 10000.0, off, neox), oracle.rope(k, 10000.0, off, neox)
    atol = 1e-4
    gq, gk = ft.rope(q, k, neox=neox, pos_offset=off, cuda=True)
    np.testing.assert_allclose(gq, want_q, atol=atol)
    np.testing.assert_allclose(gk, want_k, atol=atol)
    tq, tk = ft.rope(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), neox=neox, pos_offset=off)
    np.testing.assert_array_equal(tq.cpu().numpy(), gq)
    np.testing.assert_array_equal(tk.cpu().numpy(), gk)
    oq, none = ft.rope(torch.from_numpy(q).cuda(), None, neox=neox, pos_offset=off)
    assert none is None and torch.equal(oq, tq)
    bq, _ = ft.rope(torch.from_numpy(q).cuda().bfloat16(), None, neox=neox, pos_offset=off)
    assert bq.dtype is torch.bfloat16
    qr = torch.from_numpy(q).bfloat16().float().numpy()
    np.testing.assert_allclose(bq.float().cpu().numpy(), oracle.rope(qr, 10000.0, off, neox), atol=3e-2, rtol=1e-2)


@pytest.mark.gpu
def test_gpu_theta_errors_and_empty():
    import torch
    import fusedtok_b200 as ft
    q, _ = make_qk(2, 8, seed=5)
    g, _ = ft.rope(torch.from_numpy(q).cuda(), None, theta=500000.0)
    np.testing.assert_allclose(g.cpu().numpy(), oracle.rope(q, 500000.0), atol=1e-4)
    with pytest.raises(ValueError):
        ft.rope(torch.zeros(2, 7, device="cuda"), None)
    with pytest.raises(ValueError):
        ft.rope(torch.zeros(2, 8, device="cuda"), None, pos_offset=-1)
    with pytest.raises(ValueError):
        ft.rope(torch.zeros(2, 2, 8, device="cuda"), None)
    with pytest.raises(TypeError):
        ft.rope(torch.zeros(2, 8, device="cuda"), torch.zeros(2, 8, device="cuda").bfloat16())
    with pytest.raises(RuntimeError):
        ft.rope(q, None)
    e, _ = ft.rope(torch.zeros(0, 8, device="cuda"), None)
    assert e.shape == (0, 8)
