"""The fused decode-step front end (RoPE of q and k_new + kv-cache append in one launch).

Expectation = the reference's operators composed: its rope on every head as a one-row matrix at
position lens[b] + pos_offset (src/rope.cu:95-146 through the oracle), then its kv_append /
kv_append_paged (src/attention.cu:1753-1782 through the oracle). The fused kernel must also equal
this library's own rope followed by kv_append bit for bit, and leave every other cache row untouched.
"""

import numpy as np
import pytest
import torch

import oracle

import fusedtok_b200 as ft
from fusedtok_b200 import _fusedtok

gpu = pytest.mark.gpu


def _case(seed, b, hq, hkv, t, d):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    kn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    vn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    kc = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    vc = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    lens = rng.integers(0, t, size=b).astype(np.int32)
    lens[0] = t - 1
    if b > 1:
        lens[1] = 0
    return q, kn, vn, kc, vc, lens


def _rot_rows(x, lens, theta, off, neox):
    """The reference's rope on each [heads, D] block with every head at position lens[b] + off."""
    y = np.empty_like(x)
    for b in range(x.shape[0]):
        for h in range(x.shape[1]):
            y[b, h] = oracle.rope(x[b, h][None, :].copy(), theta, int(lens[b]) + off, neox)[0]
    return y


def test_oracle_composition_is_positionwise():
    # one-row rope at pos_offset = p equals row p of a longer matrix: the composition used below is the
    # reference's own rope semantics, not a new definition
    rng = np.random.default_rng(0)
    x = rng.standard_normal((9, 16)).astype(np.float32)
    full = oracle.rope(x, 10000.0, 3, True)
    for r in range(9):
        np.testing.assert_array_equal(oracle.rope(x[r][None, :].copy(), 10000.0, 3 + r, True)[0], full[r])


@gpu
@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("dt,atol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2), (torch.float16, 4e-3)])
@pytest.mark.parametrize("shape", [(3, 8, 2, 40, 32), (2, 32, 8, 4100, 128), (1, 4, 4, 7, 4), (5, 40, 8, 64, 256)])
def test_contiguous_matches_reference_composition(shape, dt, atol, neox):
    b, hq, hkv, t, d = shape
    q, kn, vn, kc, vc, lens = _case(sum(shape), *shape)
    off = 5
    dev = lambda x: torch.from_numpy(x).cuda().to(dt)
    tq, tkn, tvn, tkc, tvc = map(dev, (q, kn, vn, kc, vc))
    tl = torch.from_numpy(lens).cuda()
    # expectations from the storage-rounded inputs
    rq, rkn, rvn, rkc, rvc = (x.float().cpu().numpy() for x in (tq, tkn, tvn, tkc, tvc))
    want_q = _rot_rows(rq, lens, 10000.0, off, neox)
    want_k, want_v = oracle.kv_append(rkc, rvc, _rot_rows(rkn, lens, 10000.0, off, neox), rvn, lens)

    # this library's separate operators, for the bit-exact comparison
    sep_k, sep_v = tkc.clone(), tvc.clone()
    if dt is not torch.float16:                                   # the stand-alone rope has no float16 form
        sep_q = torch.empty_like(tq)
        sep_kn = torch.empty_like(tkn)
        for i in range(b):
            sep_q[i] = torch.cat([ft.rope(tq[i, h:h + 1], None, pos_offset=int(lens[i]) + off, neox=neox)[0]
                                  for h in range(hq)])
            sep_kn[i] = torch.cat([ft.rope(tkn[i, h:h + 1], None, pos_offset=int(lens[i]) + off, neox=neox)[0]
                                   for h in range(hkv)])
        ft.kv_append(sep_k, sep_v, sep_kn, tvn, tl)

    got_q = ft.rope_kv_append(tq, tkc, tvc, tkn, tvn, tl, pos_offset=off, neox=neox)
    torch.cuda.synchronize()
    np.testing.assert_allclose(got_q.float().cpu().numpy(), want_q, atol=atol, rtol=1e-2)
    np.testing.assert_allclose(tkc.float().cpu().numpy(), want_k, atol=atol, rtol=1e-2)
    np.testing.assert_array_equal(tvc.float().cpu().numpy(), want_v)          # V is a copy: exact
    # rows other than lens[b] are untouched, exactly
    keep = np.ones((b, t), bool)
    keep[np.arange(b), lens] = False
    keep = np.broadcast_to(keep[:, None, :], (b, hkv, t))
    np.testing.assert_array_equal(tkc.float().cpu().numpy()[keep], rkc[keep])
    if dt is not torch.float16:
        assert torch.equal(got_q, sep_q)
        assert torch.equal(tkc, sep_k) and torch.equal(tvc, sep_v)


@gpu
@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("dt,atol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2), (torch.float16, 4e-3)])
def test_paged_matches_reference_composition_and_in_place_q(dt, atol, neox):
    rng = np.random.default_rng(7)
    b, hq, hkv, d, page, nb, width = 4, 16, 4, 64, 16, 40, 6
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    kn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    vn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    kp = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
    vp = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
    table = rng.permutation(nb)[:b * width].reshape(b, width).astype(np.int32)
    lens = np.array([0, 15, 16, width * page - 1], np.int32)                  # page boundaries and the last slot
    dev = lambda x: torch.from_numpy(x).cuda().to(dt)
    tq, tkn, tvn, tkp, tvp = map(dev, (q, kn, vn, kp, vp))
    tt, tl = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    rq, rkn, rvn, rkp, rvp = (x.float().cpu().numpy() for x in (tq, tkn, tvn, tkp, tvp))
    want_q = _rot_rows(rq, lens, 500000.0, 0, neox)
    want_k, want_v = oracle.kv_append_paged(rkp, rvp, table, _rot_rows(rkn, lens, 500000.0, 0, neox), rvn, lens)
    res = ft.rope_kv_append_paged(tq, tkp, tvp, tt, tkn, tvn, tl, theta=500000.0, neox=neox, out=tq)
    torch.cuda.synchronize()
    assert res is tq                                                          # rotated in place
    np.testing.assert_allclose(tq.float().cpu().numpy(), want_q, atol=atol, rtol=1e-2)
    np.testing.assert_allclose(tkp.float().cpu().numpy(), want_k, atol=atol, rtol=1e-2)
    np.testing.assert_array_equal(tvp.float().cpu().numpy(), want_v)
    untouched = np.ones(nb, bool)
    untouched[[table[i, lens[i] // page] for i in range(b)]] = False
    np.testing.assert_array_equal(tkp.float().cpu().numpy()[untouched], rkp[untouched])


@gpu
def test_fused_step_then_decode_in_one_graph_equals_separate_operators():
    # rope_kv_append + attention_decode captured as one CUDA graph and replayed over three steps
    # against the separate operators run eagerly on a second copy of the cache
    b, hq, hkv, t, d = 4, 32, 8, 600, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    mk = lambda *s: torch.randn(*s, generator=g, device="cuda").bfloat16()
    kc, vc = mk(b, hkv, t, d), mk(b, hkv, t, d)
    kc2, vc2 = kc.clone(), vc.clone()
    lens = torch.tensor([17, 300, 596, 0], dtype=torch.int32, device="cuda")
    lens1 = lens + 1
    q, kn, vn = mk(b, hq, d), mk(b, hkv, d), mk(b, hkv, d)
    qr = torch.empty_like(q)
    out = torch.empty_like(q)

    def step():
        st = torch.cuda.current_stream().cuda_stream
        _fusedtok.rope_kv_append_launch(1, True, q.data_ptr(), qr.data_ptr(), kn.data_ptr(), vn.data_ptr(),
                                        lens.data_ptr(), kc.data_ptr(), vc.data_ptr(), b, hq, hkv, d, t, 10000.0, 0,
                                        st)
        _fusedtok.attention_decode_launch_bf16(qr.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens1.data_ptr(),
                                               out.data_ptr(), b, hq, hkv, t, d, st)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                                                # warm-up outside capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    kc.copy_(kc2)
    vc.copy_(vc2)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(3):
        q.copy_(mk(b, hq, d))
        kn.copy_(mk(b, hkv, d))
        vn.copy_(mk(b, hkv, d))
        graph.replay()
        torch.cuda.synchronize()
        sq = torch.stack([torch.cat([ft.rope(q[i, h:h + 1], None, pos_offset=int(lens[i]), neox=True)[0]
                                     for h in range(hq)]) for i in range(b)])
        sk = torch.stack([torch.cat([ft.rope(kn[i, h:h + 1], None, pos_offset=int(lens[i]), neox=True)[0]
                                     for h in range(hkv)]) for i in range(b)])
        ft.kv_append(kc2, vc2, sk, vn, lens)
        want = ft.attention_decode(sq, kc2, vc2, lens + 1)
        assert torch.equal(out, want)
        assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
        lens += 1
        lens1 += 1


@gpu
def test_error_contract():
    z = lambda *s, dt=torch.float32: torch.zeros(*s, device="cuda", dtype=dt)
    q, kc, vc, kn, vn = z(2, 8, 16), z(2, 2, 10, 16), z(2, 2, 10, 16), z(2, 2, 16), z(2, 2, 16)
    lens = torch.zeros(2, dtype=torch.int32, device="cuda")
    with pytest.raises(TypeError):
        ft.rope_kv_append(q.cpu(), kc, vc, kn, vn, lens)
    with pytest.raises(TypeError):
        ft.rope_kv_append(q.bfloat16(), kc, vc, kn, vn, lens)
    with pytest.raises(TypeError):
        ft.rope_kv_append(q, kc.cpu(), vc, kn, vn, lens)
    with pytest.raises(ValueError):
        ft.rope_kv_append(z(2, 7, 16), kc, vc, kn, vn, lens)                 # heads not a multiple
    with pytest.raises(ValueError):
        ft.rope_kv_append(q, kc, vc, z(2, 2, 12), vn, lens)
    with pytest.raises(ValueError):
        ft.rope_kv_append(q, kc, vc, kn, vn, lens, pos_offset=-1)
    with pytest.raises(ValueError):
        ft.rope_kv_append(q, kc, vc, kn, vn, lens, theta=0.0)
    with pytest.raises(ValueError):
        ft.rope_kv_append(q, kc, vc, kn, vn, np.array([0, 10], np.int32))    # host lens validated: row 10 of 10
    with pytest.raises(ValueError):
        ft.rope_kv_append(z(2, 8, 6), z(2, 2, 10, 6), z(2, 2, 10, 6), z(2, 2, 6), z(2, 2, 6), lens)  # D % 4
    with pytest.raises(ValueError):
        ft.rope_kv_append_paged(q, z(5, 2, 4, 16), z(5, 2, 4, 16), np.array([[0, 9], [1, 2]], np.int32), kn, vn,
                                lens)                                        # table entry out of range
    # a device position outside the cache skips the write and still rotates q
    far = torch.tensor([3, 99], dtype=torch.int32, device="cuda")
    kn.fill_(1.0)
    before = kc.clone()
    ft.rope_kv_append(q + 1.0, kc, vc, kn, vn, far)
    torch.cuda.synchronize()
    assert torch.equal(kc[1], before[1]) and not torch.equal(kc[0], before[0])
    assert ft.rope_kv_append(z(0, 8, 16), z(0, 2, 10, 16), z(0, 2, 10, 16), z(0, 2, 16), z(0, 2, 16),
                             z(0, dt=torch.int32)).shape == (0, 8, 16)
