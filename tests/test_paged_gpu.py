"""GPU parity tests for the paged-cache decode path. Mirrors the reference's
tests/test_attention_paged.py:154-276 (paged vs contiguous, half precision,
staged vs zero-copy, determinism, graph capture, error contract) and adds the
ragged benchmark configurations at oracle size."""

import numpy as np
import pytest
import torch

import cases
import oracle

import fusedtok_b200 as ft
from fusedtok_b200 import _fusedtok

pytestmark = pytest.mark.gpu

HALF = [pytest.param(torch.bfloat16, 2e-2, id="bf16"), pytest.param(torch.float16, 5e-3, id="fp16")]


def _case(seed, dt=torch.float32, lens=(511, 100, 1024), b=3, hq=8, hkv=2, d=64, nb=20, page=16):
    rng = np.random.default_rng(seed)
    q, kp, vp, tbl, kc, vc, la = cases.make_paged_case(rng, b, hq, hkv, d, nb, list(lens), page)
    t = lambda x: torch.from_numpy(x).cuda()
    return (t(q).to(dt), t(kp).to(dt), t(vp).to(dt), t(tbl), t(la), t(kc).to(dt), t(vc).to(dt), tbl, la)


def _oracle(qt, kpt, vpt, tbl, la):
    return oracle.decode_paged(qt.float().cpu().numpy(), kpt.float().cpu().numpy(),
                               vpt.float().cpu().numpy(), tbl, la)


@pytest.mark.parametrize("name", sorted(cases.PAGED_CASES))
def test_staged_paged_matches_golden(golden, name):
    seed, b, hq, hkv, d, nb, lens = cases.PAGED_CASES[name]
    rng = np.random.default_rng(seed)
    q, kp, vp, tbl, kc, vc, la = cases.make_paged_case(rng, b, hq, hkv, d, nb, lens)
    y = ft.attention_decode_paged(q, kp, vp, tbl, la, cuda=True)
    np.testing.assert_allclose(y, golden[name], rtol=0, atol=1e-5)
    y_none = ft.attention_decode_paged(q, kp, vp, tbl, cuda=True)      # lens=None: full table width
    full = np.full(b, tbl.shape[1] * cases.PAGE, np.int32)
    np.testing.assert_allclose(y_none, oracle.decode_paged(q, kp, vp, tbl, full), rtol=0, atol=1e-5)


def test_paged_vs_contiguous_f32():
    qt, kpt, vpt, tblt, lenst, kct, vct, tbl, la = _case(47)
    out = ft.attention_decode_paged(qt, kpt, vpt, tblt, lenst)
    ref = ft.attention_decode(qt, kct, vct, lenst)
    torch.cuda.synchronize()
    assert out.dtype is torch.float32
    torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
    assert np.abs(out.cpu().numpy() - _oracle(qt, kpt, vpt, tbl, la)).max() <= 1e-5


@pytest.mark.parametrize("dt,tol", HALF)
@pytest.mark.parametrize("d,hq,hkv", [(64, 8, 2), (128, 32, 8), (128, 40, 8), (128, 16, 1)])
def test_paged_half_precision_parity(dt, tol, d, hq, hkv):
    qt, kpt, vpt, tblt, lenst, kct, vct, tbl, la = _case(48, dt, lens=(511, 100, 1024, 17), b=4,
                                                         hq=hq, hkv=hkv, d=d, nb=150)
    st = torch.cuda.current_stream().cuda_stream
    out = torch.empty_like(qt)
    b, nb = qt.shape[0], kpt.shape[0]
    fn = _fusedtok.attention_decode_paged_launch_bf16 if dt is torch.bfloat16 \
        else _fusedtok.attention_decode_paged_launch_fp16
    # direct launcher: accepts any GQA group (40/8 = 5 is benchmark configuration 5's group)
    fn(qt.data_ptr(), kpt.data_ptr(), vpt.data_ptr(), tblt.data_ptr(), lenst.data_ptr(), out.data_ptr(),
       b, hq, hkv, 16, tblt.shape[1], d, st)
    torch.cuda.synchronize()
    assert np.abs(out.float().cpu().numpy() - _oracle(qt, kpt, vpt, tbl, la)).max() <= tol
    assert _fusedtok.attention_device_status() == 0


@pytest.mark.parametrize("page", [1, 3, 8, 16, 32, 64, 128, 48])
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_page_sizes(page, dt, tol):
    qt, kpt, vpt, tblt, lenst, kct, vct, tbl, la = _case(60 + page, dt, lens=(300, 129, 64, 1), b=4,
                                                         hq=8, hkv=2, d=128, nb=40, page=page)
    out = ft.attention_decode_paged(qt, kpt, vpt, tblt, lenst)
    torch.cuda.synchronize()
    assert np.abs(out.float().cpu().numpy() - _oracle(qt, kpt, vpt, tbl, la)).max() <= tol


def test_paged_staged_matches_zero_copy():
    rng = np.random.default_rng(49)
    q, kp, vp, tbl, kc, vc, lens = cases.make_paged_case(rng, 2, 8, 2, 64, 12, [100, 512])
    out_gpu = ft.attention_decode_paged(q, kp, vp, tbl, lens, cuda=True)
    t = lambda x: torch.from_numpy(x).cuda()
    out_t = ft.attention_decode_paged(t(q), t(kp), t(vp), t(tbl), t(lens))
    torch.cuda.synchronize()
    np.testing.assert_allclose(out_gpu, out_t.cpu().numpy(), atol=1e-5)


def test_paged_deterministic_repeat():
    qt, kpt, vpt, tblt, lenst, *_ = _case(50)
    a = ft.attention_decode_paged(qt, kpt, vpt, tblt, lenst)
    b = ft.attention_decode_paged(qt, kpt, vpt, tblt, lenst)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_paged_graph_capture_replay(dt):
    qt, kpt, vpt, tblt, lenst, kct, vct, tbl, la = _case(51, dt)
    for _ in range(2):
        ft.attention_decode_paged(qt, kpt, vpt, tblt, lenst)
    out = torch.empty_like(qt)
    fn = _fusedtok.attention_decode_paged_launch if dt is torch.float32 \
        else _fusedtok.attention_decode_paged_launch_bf16

    def run():
        b, hq, d = qt.shape
        nb, hkv, page, _ = kpt.shape
        fn(qt.data_ptr(), kpt.data_ptr(), vpt.data_ptr(), tblt.data_ptr(), lenst.data_ptr(),
           out.data_ptr(), b, hq, hkv, page, tblt.shape[1], d, torch.cuda.current_stream().cuda_stream)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            run()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    tol = 1e-5 if dt is torch.float32 else 2e-2
    g.replay()
    torch.cuda.synchronize()
    assert np.abs(out.float().cpu().numpy() - _oracle(qt, kpt, vpt, tbl, la)).max() <= tol
    kpt.mul_(2.0)
    g.replay()
    torch.cuda.synchronize()
    assert np.abs(out.float().cpu().numpy() - _oracle(qt, kpt, vpt, tbl, la)).max() <= tol


def test_paged_torch_errors():
    qt, kpt, vpt, tblt, lenst, *_ = _case(52)
    with pytest.raises(TypeError):
        ft.attention_decode_paged(qt.double(), kpt, vpt, tblt)
    with pytest.raises(TypeError):
        ft.attention_decode_paged(qt, kpt.bfloat16(), vpt, tblt)
    with pytest.raises(ValueError):
        ft.attention_decode_paged(qt, kpt, vpt, tblt[:1])
    with pytest.raises(TypeError):
        ft.attention_decode_paged(qt, kpt.cpu(), vpt, tblt)
    bad = tblt.cpu().clone()
    bad[0, 0] = 999
    with pytest.raises(ValueError):        # host-origin table values are validated
        ft.attention_decode_paged(qt, kpt, vpt, bad)


def test_config3_reduced_fp16():
    """Benchmark configuration 3 (ragged lengths uniform in [128, 8192], page
    16, permuted block table with 10% slack, fp16, 32/8 heads, D=128) on the
    first 6 sequences of the seeded draw plus the shortest and the longest."""
    lens_all = cases.config3_lens()
    pick = list(range(6)) + [int(np.argmin(lens_all)), int(np.argmax(lens_all))]
    lens = lens_all[pick]
    table, nb, width = cases.paged_layout(lens)
    g = torch.Generator(device="cuda").manual_seed(0)
    kp = torch.randn(nb, 8, 16, 128, device="cuda", generator=g).half()
    vp = torch.randn(nb, 8, 16, 128, device="cuda", generator=g).half()
    q = torch.randn(len(lens), 32, 128, device="cuda", generator=g).half()
    out = ft.attention_decode_paged(q, kp, vp, torch.from_numpy(table).cuda(),
                                    torch.from_numpy(lens).cuda())
    ref = _oracle(q, kp, vp, table, lens)
    y = out.float().cpu().numpy()
    assert np.abs(y - ref).max() <= 2e-2
    assert np.abs(y - ref).mean() / np.abs(ref).mean() <= 1e-2
    assert _fusedtok.attention_device_status() == 0


def test_config5_reduced_bf16_group5():
    """Benchmark configuration 5 (40/8 heads = group 5, log-uniform lengths in
    [1024, 32768], page 16, bf16) on 4 sequences incl. the shortest, through
    the direct launcher (the Python wrapper keeps the reference's 1/2/4/8/16
    group rule)."""
    lens_all = cases.config5_lens()
    order = np.argsort(lens_all)
    lens = lens_all[[order[0], order[40], order[100], order[130]]]
    table, nb, width = cases.paged_layout(lens)
    g = torch.Generator(device="cuda").manual_seed(0)
    kp = torch.randn(nb, 8, 16, 128, device="cuda", generator=g).bfloat16()
    vp = torch.randn(nb, 8, 16, 128, device="cuda", generator=g).bfloat16()
    q = torch.randn(len(lens), 40, 128, device="cuda", generator=g).bfloat16()
    tbl = torch.from_numpy(table).cuda()
    ln = torch.from_numpy(lens).cuda()
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q, kp, vp, tbl, ln)
    out = torch.empty_like(q)
    _fusedtok.attention_decode_paged_launch_bf16(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), tbl.data_ptr(),
                                                 ln.data_ptr(), out.data_ptr(), len(lens), 40, 8, 16, width,
                                                 128, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ref = _oracle(q, kp, vp, table, lens)
    y = out.float().cpu().numpy()
    assert np.abs(y - ref).max() <= 2e-2
    assert np.abs(y - ref).mean() / np.abs(ref).mean() <= 1e-2
