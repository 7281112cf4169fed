"""kv-cache append (the step before decode in the serving loop): oracle pinned
to the reference's CPU code, GPU parity for both cache layouts and every
storage type, append-then-decode loops, graph capture, error contract.
Mirrors the reference's tests/test_kv_append.py and tests/test_kv_append_paged.py."""

import numpy as np
import pytest
import torch

import cases
import oracle

import fusedtok_b200 as ft
from fusedtok_b200 import _fusedtok

PAGE = 16
gpu = pytest.mark.gpu


def _contig(rng, b=3, hkv=2, t=40, d=32):
    kc = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    vc = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    kn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    vn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    return kc, vc, kn, vn


def _paged(rng, b=3, hkv=2, d=32, nb=12, width=3):
    kp = rng.standard_normal((nb, hkv, PAGE, d)).astype(np.float32)
    vp = rng.standard_normal((nb, hkv, PAGE, d)).astype(np.float32)
    tbl = rng.permutation(nb)[: b * width].reshape(b, width).astype(np.int32)   # distinct blocks
    kn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    vn = rng.standard_normal((b, hkv, d)).astype(np.float32)
    return kp, vp, tbl, kn, vn


# ---- oracle (CPU) -----------------------------------------------------------

def test_oracle_append_positions_and_reference_pin():
    rng = np.random.default_rng(1)
    kc, vc, kn, vn = _contig(rng)
    lens = np.array([0, 39, 17], np.int32)           # first row, last row, middle
    k2, v2 = oracle.kv_append(kc, vc, kn, vn, lens)
    for b in range(3):
        np.testing.assert_array_equal(k2[b, :, lens[b]], kn[b])
        np.testing.assert_array_equal(v2[b, :, lens[b]], vn[b])
    mask = np.ones_like(kc, bool)
    for b in range(3):
        mask[b, :, lens[b]] = False
    np.testing.assert_array_equal(k2[mask], kc[mask])  # nothing else touched
    if oracle.ref_available():
        rk, rv = oracle.ref_kv_append(kc, vc, kn, vn, lens)
        np.testing.assert_array_equal(k2, rk)
        np.testing.assert_array_equal(v2, rv)
    for bad in ([40, 0, 0], [-1, 0, 0]):
        with pytest.raises(ValueError):
            oracle.kv_append(kc, vc, kn, vn, np.array(bad, np.int32))


def test_oracle_paged_append_page_boundaries_and_reference_pin():
    rng = np.random.default_rng(2)
    kp, vp, tbl, kn, vn = _paged(rng)
    lens = np.array([0, PAGE - 1, 2 * PAGE], np.int32)   # page start, page end, first row of page 2
    k2, v2 = oracle.kv_append_paged(kp, vp, tbl, kn, vn, lens)
    for b in range(3):
        blk, off = tbl[b, lens[b] // PAGE], lens[b] % PAGE
        np.testing.assert_array_equal(k2[blk, :, off], kn[b])
        np.testing.assert_array_equal(v2[blk, :, off], vn[b])
    assert (k2 != kp).sum() <= 3 * 2 * 32
    if oracle.ref_available():
        rk, rv = oracle.ref_kv_append_paged(kp, vp, tbl, kn, vn, lens)
        np.testing.assert_array_equal(k2, rk)
        np.testing.assert_array_equal(v2, rv)
    with pytest.raises(ValueError):
        oracle.kv_append_paged(kp, vp, tbl, kn, vn, np.array([3 * PAGE, 0, 0], np.int32))
    bad = tbl.copy()
    bad[0, 0] = 99
    with pytest.raises(ValueError):
        oracle.kv_append_paged(kp, vp, bad, kn, vn, lens)


def test_host_error_contract_before_any_launch():
    rng = np.random.default_rng(3)
    kc, vc, kn, vn = _contig(rng)
    with pytest.raises(RuntimeError):                  # no CPU path
        ft.kv_append(kc, vc, kn, vn, [0, 1, 2])
    with pytest.raises(ValueError):
        ft.kv_append(kc, vc, kn, vn, [40, 0, 0], cuda=True)
    with pytest.raises(ValueError):
        ft.kv_append(kc, vc, kn, vn, [-1, 0, 0], cuda=True)
    with pytest.raises(ValueError):
        ft.kv_append(kc, vc, kn[:, :1], vn[:, :1], [0, 0, 0], cuda=True)
    with pytest.raises(TypeError):                     # in-place op: no silent conversion of the cache
        ft.kv_append(kc.astype(np.float64), vc, kn, vn, [0, 0, 0], cuda=True)
    kp, vp, tbl, kn2, vn2 = _paged(rng)
    with pytest.raises(ValueError):
        ft.kv_append_paged(kp, vp, tbl, kn2, vn2, [3 * PAGE, 0, 0], cuda=True)
    bad = tbl.copy()
    bad[0, 0] = 99
    with pytest.raises(ValueError):
        ft.kv_append_paged(kp, vp, bad, kn2, vn2, [0, 0, 0], cuda=True)
    with pytest.raises(TypeError):
        ft.kv_append_paged(kp, vp, tbl, kn2, vn2, [0.5, 0, 0], cuda=True)
    # C ABI: validation precedes any CUDA call
    lib = _fusedtok._lib
    assert lib.fusedtok_kv_append_launch(256, 256, 256, 256, 256, 2, 2, 30, 8, 0) == 1
    assert lib.fusedtok_kv_append_paged_launch_bf16(256, 256, 256, 256, 256, 256, 2, 2, 32, 0, 4, 0) == 1
    assert lib.fusedtok_kv_append_launch_fp16(256, 256, 256, 256, 256, 0, 2, 32, 8, 0) == 0   # batch 0: no-op


# ---- GPU --------------------------------------------------------------------

@gpu
def test_staged_matches_oracle():
    rng = np.random.default_rng(4)
    kc, vc, kn, vn = _contig(rng)
    lens = np.array([5, 0, 39], np.int32)
    want_k, want_v = oracle.kv_append(kc, vc, kn, vn, lens)
    ft.kv_append(kc, vc, kn, vn, lens, cuda=True)      # in place on the host arrays
    np.testing.assert_array_equal(kc, want_k)
    np.testing.assert_array_equal(vc, want_v)
    kp, vp, tbl, kn2, vn2 = _paged(rng)
    lens = np.array([PAGE, 7, 2 * PAGE + 15], np.int32)
    want_k, want_v = oracle.kv_append_paged(kp, vp, tbl, kn2, vn2, lens)
    ft.kv_append_paged(kp, vp, tbl, kn2, vn2, lens, cuda=True)
    np.testing.assert_array_equal(kp, want_k)
    np.testing.assert_array_equal(vp, want_v)


@gpu
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [4, 32, 128])
def test_zero_copy_dtype_matrix(dt, d):
    rng = np.random.default_rng(5 + d)
    kc, vc, kn, vn = _contig(rng, b=4, hkv=3, t=50, d=d)
    lens = np.array([0, 49, 20, 7], np.int32)
    t = lambda x: torch.from_numpy(x).cuda().to(dt)
    kct, vct, knt, vnt = t(kc), t(vc), t(kn), t(vn)
    want_k, want_v = oracle.kv_append(kct.float().cpu().numpy(), vct.float().cpu().numpy(),
                                      knt.float().cpu().numpy(), vnt.float().cpu().numpy(), lens)
    assert ft.kv_append(kct, vct, knt, vnt, torch.from_numpy(lens).cuda()) is None
    torch.cuda.synchronize()
    np.testing.assert_array_equal(kct.float().cpu().numpy(), want_k)     # byte copy: exact in every dtype
    np.testing.assert_array_equal(vct.float().cpu().numpy(), want_v)
    kp, vp, tbl, kn2, vn2 = _paged(rng, b=4, hkv=3, d=d, nb=20, width=4)
    lens = np.array([0, PAGE - 1, PAGE, 4 * PAGE - 1], np.int32)
    kpt, vpt, kn2t, vn2t = t(kp), t(vp), t(kn2), t(vn2)
    want_k, want_v = oracle.kv_append_paged(kpt.float().cpu().numpy(), vpt.float().cpu().numpy(), tbl,
                                            kn2t.float().cpu().numpy(), vn2t.float().cpu().numpy(), lens)
    ft.kv_append_paged(kpt, vpt, torch.from_numpy(tbl).cuda(), kn2t, vn2t, lens.tolist())
    torch.cuda.synchronize()
    np.testing.assert_array_equal(kpt.float().cpu().numpy(), want_k)
    np.testing.assert_array_equal(vpt.float().cpu().numpy(), want_v)


@gpu
def test_append_then_decode_loop_contiguous_and_paged():
    """The serving loop: append at lens, decode over lens + 1, several steps;
    contiguous and paged caches must agree with each other and with the oracle."""
    rng = np.random.default_rng(9)
    b, hq, hkv, d, steps = 2, 8, 2, 64, 5
    t_rows = 3 * PAGE
    dt = torch.bfloat16
    kc = torch.zeros(b, hkv, t_rows, d, device="cuda", dtype=dt)
    vc = torch.zeros_like(kc)
    nb = 8
    kp = torch.zeros(nb, hkv, PAGE, d, device="cuda", dtype=dt)
    vp = torch.zeros_like(kp)
    tbl = torch.tensor([[5, 1, 6], [2, 7, 0]], dtype=torch.int32, device="cuda")
    lens = torch.tensor([14, 0], dtype=torch.int32, device="cuda")     # sequence 0 crosses a page boundary
    kc[0, :, :14] = torch.randn(hkv, 14, d, device="cuda").to(dt)
    vc[0, :, :14] = torch.randn(hkv, 14, d, device="cuda").to(dt)
    kp[5, :, :14] = kc[0, :, :14]
    vp[5, :, :14] = vc[0, :, :14]
    for _ in range(steps):
        kn = torch.from_numpy(rng.standard_normal((b, hkv, d)).astype(np.float32)).cuda().to(dt)
        vn = torch.from_numpy(rng.standard_normal((b, hkv, d)).astype(np.float32)).cuda().to(dt)
        q = torch.from_numpy(rng.standard_normal((b, hq, d)).astype(np.float32)).cuda().to(dt)
        ft.kv_append(kc, vc, kn, vn, lens)
        ft.kv_append_paged(kp, vp, tbl, kn, vn, lens)
        lens += 1
        y_c = ft.attention_decode(q, kc, vc, lens)
        y_p = ft.attention_decode_paged(q, kp, vp, tbl, lens)
        torch.cuda.synchronize()
        ref = oracle.decode(q.float().cpu().numpy(), kc.float().cpu().numpy(), vc.float().cpu().numpy(),
                            lens.cpu().numpy())
        assert np.abs(y_c.float().cpu().numpy() - ref).max() <= 2e-2
        assert (y_c.float() - y_p.float()).abs().max().item() <= 4e-3


@gpu
def test_graph_capture_append_and_decode_step():
    """One decode step = append + attention, captured as one CUDA graph and
    replayed with device-side lens advancing (reference: tests/test_kv_append.py:162-186)."""
    b, hq, hkv, d, t_rows = 2, 8, 2, 64, 64
    kc = torch.zeros(b, hkv, t_rows, d, device="cuda")
    vc = torch.zeros_like(kc)
    kn = torch.randn(b, hkv, d, device="cuda")
    vn = torch.randn(b, hkv, d, device="cuda")
    q = torch.randn(b, hq, d, device="cuda")
    lens_w = torch.tensor([0, 3], dtype=torch.int32, device="cuda")    # write position
    lens_r = lens_w + 1                                                # rows to attend over
    out = torch.empty(b, hq, d, device="cuda")

    def run():
        st = torch.cuda.current_stream().cuda_stream
        _fusedtok.kv_append_launch(kn.data_ptr(), vn.data_ptr(), lens_w.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                   b, hkv, d, t_rows, st)
        _fusedtok.attention_decode_launch(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens_r.data_ptr(),
                                          out.data_ptr(), b, hq, hkv, t_rows, d, st)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            run()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    kc.zero_(); vc.zero_()
    ref_k, ref_v = kc.cpu().numpy().copy(), vc.cpu().numpy().copy()
    for step in range(3):
        kn.copy_(torch.randn_like(kn)); vn.copy_(torch.randn_like(vn))
        g.replay()
        torch.cuda.synchronize()
        ref_k, ref_v = oracle.kv_append(ref_k, ref_v, kn.cpu().numpy(), vn.cpu().numpy(), lens_w.cpu().numpy())
        ref = oracle.decode(q.cpu().numpy(), ref_k, ref_v, lens_r.cpu().numpy())
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5
        lens_w += 1; lens_r += 1


@gpu
def test_zero_copy_error_contract():
    kc = torch.zeros(2, 2, 8, 32, device="cuda")
    kn = torch.zeros(2, 2, 32, device="cuda")
    with pytest.raises(ValueError):
        ft.kv_append(kc, kc.clone(), kn, kn, [8, 0])
    with pytest.raises(TypeError):
        ft.kv_append(kc, kc.clone(), kn.half(), kn.half(), [0, 0])
    with pytest.raises(TypeError):
        ft.kv_append(kc, kc.clone().cpu(), kn, kn, [0, 0])
    with pytest.raises(ValueError):
        ft.kv_append(kc, kc.clone(), kn[:1], kn[:1], [0])
    # a device lens outside the cache is skipped, not written (trusted values never fault)
    bad = torch.tensor([100, -5], dtype=torch.int32, device="cuda")
    before = kc.clone()
    ft.kv_append(kc, kc.clone(), torch.ones_like(kn), torch.ones_like(kn), bad)
    torch.cuda.synchronize()
    assert torch.equal(kc, before)
