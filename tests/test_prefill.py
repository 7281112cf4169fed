"""Prefill (fresh-sequence) attention: the oracle against the reference's pins on CPU, the CUDA
kernels against the oracle on a GPU. Shapes, seeds and tolerances follow the reference's own
tests (tests/test_attention.py:157-240 for the CPU pins, :319-330 and :631-730 for the GPU ones)."""

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


def ref64(q, k, v, causal=True):
    """float64 eager statement of the operator (the reference's ref_prefill, test_attention.py:157-173)."""
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = np.zeros((b, hq, s, d), dtype=np.float64)
    for bi in range(b):
        for h in range(hq):
            kv = h // group
            scores = q[bi, h].astype(np.float64) @ k[bi, kv].astype(np.float64).T / math.sqrt(d)
            if causal:
                scores = np.where(np.tril(np.ones((s, s), bool)), scores, -np.inf)
            p = np.exp(scores - scores.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            out[bi, h] = p @ v[bi, kv].astype(np.float64)
    return out


@pytest.mark.parametrize("b,hq,hkv,s,d", cases.PREFILL_SHAPES)
@pytest.mark.parametrize("causal", [True, False])
def test_oracle_matches_golden_bit_exact(prefill_golden, b, hq, hkv, s, d, causal):
    q, k, v = cases.make_prefill_case(b, hq, hkv, s, d, causal)
    name = "prefill_%d_%d_%d_%d_%d_%d" % (b, hq, hkv, s, d, int(causal))
    assert digest(q, k, v) == prefill_golden[name + "_sum"], "input generator drifted"
    y = oracle.prefill(q, k, v, causal)
    assert digest(y) == prefill_golden[name + "_out_sum"]
    if name in prefill_golden:
        np.testing.assert_array_equal(y, prefill_golden[name])
    np.testing.assert_allclose(y, ref64(q, k, v, causal), rtol=1e-4, atol=1e-5)


@pytest.mark.skipif(not oracle.ref_available(), reason="reference build not present")
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_equals_reference_build(seed):
    rng = np.random.default_rng(900 + seed)
    b, hq, hkv = int(rng.integers(1, 3)), 8, int(rng.choice([1, 2, 8]))
    s, d = int(rng.integers(1, 70)), int(rng.choice([4, 36, 64, 128]))
    q = rng.standard_normal((b, hq, s, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, s, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, s, d)).astype(np.float32)
    for causal in (True, False):
        np.testing.assert_array_equal(oracle.prefill(q, k, v, causal), oracle.ref_prefill(q, k, v, causal))


def test_first_row_attends_only_to_itself():
    rng = np.random.default_rng(50)
    q = rng.standard_normal((1, 4, 9, 32)).astype(np.float32)
    k = rng.standard_normal((1, 2, 9, 32)).astype(np.float32)
    v = rng.standard_normal((1, 2, 9, 32)).astype(np.float32)
    y = oracle.prefill(q, k, v, True)
    for h in range(4):
        np.testing.assert_allclose(y[0, h, 0], v[0, h // 2, 0], rtol=1e-5, atol=1e-6)


def test_s1_equals_decode():
    rng = np.random.default_rng(51)
    q = rng.standard_normal((2, 8, 1, 64)).astype(np.float32)
    k = rng.standard_normal((2, 2, 1, 64)).astype(np.float32)
    v = rng.standard_normal((2, 2, 1, 64)).astype(np.float32)
    pre = oracle.prefill(q, k, v, True)
    dec = oracle.decode(q.reshape(2, 8, 64), k, v)
    np.testing.assert_array_equal(pre.reshape(2, 8, 64), dec)


def test_oracle_error_contract():
    z = np.zeros
    with pytest.raises(ValueError):
        oracle.prefill(z((1, 5, 8, 32), np.float32), z((1, 2, 8, 32), np.float32), z((1, 2, 8, 32), np.float32))
    with pytest.raises(ValueError):
        oracle.prefill(z((1, 4, 8, 30), np.float32), z((1, 2, 8, 30), np.float32), z((1, 2, 8, 30), np.float32))


# ---------------------------------------------------------------------------- GPU: kernels against the oracle

HALF = [("bfloat16", 2e-2, 2e-2), ("float16", 2e-3, 2e-3)]     # reference: HALF_DTYPES, test_attention.py:566


def _torch():
    import torch
    return torch


@pytest.mark.gpu
@pytest.mark.parametrize("b,hq,hkv,s,d", cases.PREFILL_SHAPES)
@pytest.mark.parametrize("causal", [True, False])
def test_gpu_staged_matches_oracle(b, hq, hkv, s, d, causal):
    import fusedtok_b200 as ft
    q, k, v = cases.make_prefill_case(b, hq, hkv, s, d, causal)
    y = ft.attention_prefill(q, k, v, causal=causal, cuda=True)
    assert y.shape == (b, hq, s, d) and y.dtype == np.float32
    np.testing.assert_allclose(y, oracle.prefill(q, k, v, causal), rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("s,d", [(1, 128), (63, 64), (64, 64), (65, 128), (200, 128), (130, 36), (70, 256), (40, 512),
                                 (257, 4)])
def test_gpu_fp32_tile_edges(s, d):
    torch = _torch()
    import fusedtok_b200 as ft
    rng = np.random.default_rng(s * 7 + d)
    b, hq, hkv = 2, 4, 2
    q = rng.standard_normal((b, hq, s, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, s, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, s, d)).astype(np.float32)
    for causal in (True, False):
        out = ft.attention_prefill(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                                   causal=causal)
        assert out.dtype is torch.float32
        np.testing.assert_allclose(out.cpu().numpy(), oracle.prefill(q, k, v, causal), rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtname,rtol,atol", HALF)
@pytest.mark.parametrize("d", [32, 64, 128])
@pytest.mark.parametrize("s", [65, 96, 200])
def test_gpu_half_dim_matrix(dtname, rtol, atol, s, d):
    """reference: test_prefill_wmma_dim_matrix, tests/test_attention.py:665-695 (every row checked here)."""
    torch = _torch()
    import fusedtok_b200 as ft
    dt = getattr(torch, dtname)
    b, hq, hkv = 2, 4, 2
    g = torch.Generator().manual_seed(s * 131 + d)
    q = torch.randn(b, hq, s, d, generator=g).to(dt)
    k = torch.randn(b, hkv, s, d, generator=g).to(dt)
    v = torch.randn(b, hkv, s, d, generator=g).to(dt)
    for causal in (True, False):
        out = ft.attention_prefill(q.cuda(), k.cuda(), v.cuda(), causal=causal)
        assert out.dtype is dt
        want = oracle.prefill(q.float().numpy(), k.float().numpy(), v.float().numpy(), causal)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=rtol, atol=atol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtname,rtol,atol", HALF)
@pytest.mark.parametrize("s", [64, 129, 300])
def test_gpu_half_head_dim_256(dtname, rtol, atol, s):
    """Head dim 256 on the tensor-core kernel (512 tensor-memory columns, one CTA per SM)."""
    torch = _torch()
    import fusedtok_b200 as ft
    dt = getattr(torch, dtname)
    b, hq, hkv, d = 2, 4, 2, 256
    g = torch.Generator().manual_seed(s)
    q = torch.randn(b, hq, s, d, generator=g).to(dt)
    k = torch.randn(b, hkv, s, d, generator=g).to(dt)
    v = torch.randn(b, hkv, s, d, generator=g).to(dt)
    for causal in (True, False):
        out = ft.attention_prefill(q.cuda(), k.cuda(), v.cuda(), causal=causal)
        want = oracle.prefill(q.float().numpy(), k.float().numpy(), v.float().numpy(), causal)
        np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=rtol, atol=atol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtname,rtol,atol", HALF)
@pytest.mark.parametrize("d", [36, 48, 80, 96, 112, 256])
def test_gpu_half_other_dims(dtname, rtol, atol, d):
    """reference: test_prefill_non_instantiated_wmma_dims / _wmma_and_fallback_agree, test_attention.py:697-730."""
    torch = _torch()
    import fusedtok_b200 as ft
    dt = getattr(torch, dtname)
    b, hq, hkv, s = 1, 4, 2, 70
    g = torch.Generator().manual_seed(d)
    q = torch.randn(b, hq, s, d, generator=g).to(dt)
    k = torch.randn(b, hkv, s, d, generator=g).to(dt)
    v = torch.randn(b, hkv, s, d, generator=g).to(dt)
    out = ft.attention_prefill(q.cuda(), k.cuda(), v.cuda(), causal=True)
    want = oracle.prefill(q.float().numpy(), k.float().numpy(), v.float().numpy(), True)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=rtol, atol=atol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtname,rtol,atol", [("float32", 1e-4, 1e-5)] + HALF)
def test_gpu_llama_shape_long(dtname, rtol, atol):
    """The reference's benchmark shape (benchmarks/bench.py:518-541) shortened to what the oracle does in
    seconds, plus properties at full length: row 0 equals v[0]; S=1 equals the decode step."""
    torch = _torch()
    import fusedtok_b200 as ft
    dt = getattr(torch, dtname)
    b, hq, hkv, d = 1, 32, 8, 128
    g = torch.Generator().manual_seed(7)
    s = 320
    q = torch.randn(b, hq, s, d, generator=g).to(dt)
    k = torch.randn(b, hkv, s, d, generator=g).to(dt)
    v = torch.randn(b, hkv, s, d, generator=g).to(dt)
    out = ft.attention_prefill(q.cuda(), k.cuda(), v.cuda(), causal=True)
    want = oracle.prefill(q.float().numpy(), k.float().numpy(), v.float().numpy(), True)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, rtol=rtol, atol=atol)
    s = 1024
    q = torch.randn(b, hq, s, d, generator=g).to(dt).cuda()
    k = torch.randn(b, hkv, s, d, generator=g).to(dt).cuda()
    v = torch.randn(b, hkv, s, d, generator=g).to(dt).cuda()
    out = ft.attention_prefill(q, k, v, causal=True)
    for h in range(hq):
        np.testing.assert_allclose(out[0, h, 0].float().cpu().numpy(), v[0, h // 4, 0].float().cpu().numpy(),
                                   rtol=1e-5, atol=1e-6)
    # the last causal row is a decode step over the whole sequence
    dec = ft.attention_decode(q[:, :, -1, :].contiguous(), k, v)
    np.testing.assert_allclose(out[:, :, -1, :].float().cpu().numpy(), dec.float().cpu().numpy(), rtol=rtol, atol=atol)
    # bit-exact repeatability
    assert torch.equal(out, ft.attention_prefill(q, k, v, causal=True))


@pytest.mark.gpu
def test_gpu_errors_and_empty():
    torch = _torch()
    import fusedtok_b200 as ft
    z = lambda *s: torch.zeros(*s, device="cuda")
    with pytest.raises(ValueError):
        ft.attention_prefill(z(1, 5, 8, 32), z(1, 2, 8, 32), z(1, 2, 8, 32))
    with pytest.raises(ValueError):
        ft.attention_prefill(z(1, 4, 8, 32), z(1, 2, 8, 32), z(1, 2, 7, 32))
    with pytest.raises(ValueError):
        ft.attention_prefill(z(1, 4, 8, 30), z(1, 2, 8, 30), z(1, 2, 8, 30))
    with pytest.raises(TypeError):
        ft.attention_prefill(z(1, 4, 8, 32), z(1, 2, 8, 32).half(), z(1, 2, 8, 32))
    assert ft.attention_prefill(z(0, 4, 8, 32), z(0, 2, 8, 32), z(0, 2, 8, 32)).shape == (0, 4, 8, 32)
    assert ft.attention_prefill(z(2, 4, 0, 32), z(2, 2, 0, 32), z(2, 2, 0, 32)).shape == (2, 4, 0, 32)
    with pytest.raises(RuntimeError):
        ft.attention_prefill(np.zeros((1, 4, 8, 32), np.float32), np.zeros((1, 2, 8, 32), np.float32),
                             np.zeros((1, 2, 8, 32), np.float32))


@pytest.mark.gpu
def test_gpu_graph_capture():
    torch = _torch()
    import fusedtok_b200 as ft
    g0 = torch.Generator().manual_seed(3)
    q = torch.randn(1, 8, 100, 64, generator=g0).bfloat16().cuda()
    k = torch.randn(1, 2, 100, 64, generator=g0).bfloat16().cuda()
    v = torch.randn(1, 2, 100, 64, generator=g0).bfloat16().cuda()
    eager = ft.attention_prefill(q, k, v)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = ft.attention_prefill(q, k, v)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
