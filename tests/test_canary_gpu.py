"""Canary-padded buffers: the stand-in for a memory checker on a pool where compute-sanitizer is closed
(the reference's own checklist asks for a sanitizer run, CONTRIBUTING.md:61-64).

Every operand of a decode call sits inside a larger allocation whose slack is filled with NaN (inputs) or a
bit pattern (output). A read of a row that does not belong to the call would poison the result, which must
stay finite and equal to the oracle's; a write outside the output view would disturb the pattern, which must
come back bit for bit. Covers the tensor-core kernel (contiguous and paged, ragged lengths, head dims with
per-column-block copies), the CUDA-core kernel (float32, 16-bit odd head dims) and the cache appends."""

import numpy as np
import pytest
import torch

import cases
import oracle

import fusedtok_b200 as ft
from fusedtok_b200 import _fusedtok

pytestmark = pytest.mark.gpu

GUARD = 4096            # elements of slack on either side


def guarded(x, fill):
    """x inside a larger allocation: [GUARD slack | x | GUARD slack], slack filled with `fill`. The view
    keeps x's alignment class (the slack is a multiple of 16 bytes)."""
    raw = torch.full((x.numel() + 2 * GUARD,), fill, dtype=x.dtype, device="cuda")
    view = raw[GUARD:GUARD + x.numel()].view(x.shape)
    view.copy_(x)
    return raw, view


def slack_intact(raw, n, fill):
    lo, hi = raw[:GUARD], raw[GUARD + n:]
    if fill != fill:                                   # NaN
        return bool(torch.isnan(lo).all() and torch.isnan(hi).all())
    return bool((lo == fill).all() and (hi == fill).all())


@pytest.mark.parametrize("dt,tol,shape", [
    (torch.bfloat16, 2e-2, (3, 32, 8, 1000, 128)),     # tensor-core kernel, units split over CTAs
    (torch.float16, 2e-3, (2, 16, 2, 700, 96)),        # per-column-block copies (head dim not a multiple of 64)
    (torch.float16, 2e-3, (2, 8, 2, 300, 256)),        # two-stage ring
    (torch.float32, 1e-5, (2, 8, 2, 900, 128)),        # CUDA-core kernel
    (torch.bfloat16, 2e-2, (2, 10, 2, 500, 48)),       # CUDA-core kernel, 16-bit storage, group 5
])
def test_contiguous_decode_stays_inside_its_operands(dt, tol, shape):
    b, hq, hkv, t, d = shape
    rng = np.random.default_rng(t + d)
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[0] = t
    lens[-1] = max(1, t // 3)
    nan = float("nan")
    rq, qt = guarded(torch.from_numpy(q).cuda().to(dt), nan)
    rk, kt = guarded(torch.from_numpy(k).cuda().to(dt), nan)
    rv, vt = guarded(torch.from_numpy(v).cuda().to(dt), nan)
    # rows past lens[b] inside the cache are poisoned too: they must never be used
    for bi in range(b):
        kt[bi, :, int(lens[bi]):] = nan
        vt[bi, :, int(lens[bi]):] = nan
    ro, out = guarded(torch.zeros(b, hq, d, device="cuda", dtype=dt), 123.0)
    name = {torch.float32: "", torch.bfloat16: "_bf16", torch.float16: "_fp16"}[dt]
    lt = torch.from_numpy(lens).cuda()
    getattr(_fusedtok, "attention_decode_launch" + name)(
        qt.data_ptr(), kt.data_ptr(), vt.data_ptr(), lt.data_ptr(), out.data_ptr(), b, hq, hkv, t, d,
        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    y = out.float().cpu().numpy()
    assert np.isfinite(y).all()
    kr = np.nan_to_num(kt.float().cpu().numpy())
    vr = np.nan_to_num(vt.float().cpu().numpy())
    ref = oracle.decode(qt.float().cpu().numpy(), kr, vr, lens)
    assert np.abs(y - ref).max() <= tol
    assert slack_intact(ro, out.numel(), 123.0)
    for raw, view in ((rq, qt), (rk, kt), (rv, vt)):
        assert slack_intact(raw, view.numel(), nan)     # inputs are never written
    assert _fusedtok.attention_device_status() == 0


@pytest.mark.parametrize("dt,tol", [(torch.float16, 5e-3), (torch.float32, 1e-5)])
def test_paged_decode_stays_inside_its_pools(dt, tol):
    rng = np.random.default_rng(17)
    b, hq, hkv, d = 3, 16, 4, 128
    lens_list = [300, 17, 129]
    qp, kp, vp, tbl, kc, vc, lens = cases.make_paged_case(rng, b, hq, hkv, d, 40, lens_list)
    nan = float("nan")
    rq, qt = guarded(torch.from_numpy(qp).cuda().to(dt), nan)
    rk, kt = guarded(torch.from_numpy(kp).cuda().to(dt), nan)
    rv, vt = guarded(torch.from_numpy(vp).cuda().to(dt), nan)
    # pool blocks no sequence maps are poisoned: the table must be the only way into the pool
    used = set(int(x) for bi in range(b) for x in tbl[bi, :(lens_list[bi] + cases.PAGE - 1) // cases.PAGE])
    for blk in range(kt.shape[0]):
        if blk not in used:
            kt[blk] = nan
            vt[blk] = nan
    ro, out = guarded(torch.zeros(b, hq, d, device="cuda", dtype=dt), 123.0)
    y = ft.attention_decode_paged(qt, kt, vt, torch.from_numpy(tbl).cuda(), torch.from_numpy(lens).cuda())
    out.copy_(y)
    torch.cuda.synchronize()
    yn = y.float().cpu().numpy()
    assert np.isfinite(yn).all()
    ref = oracle.decode_paged(qt.float().cpu().numpy(), np.nan_to_num(kt.float().cpu().numpy()),
                              np.nan_to_num(vt.float().cpu().numpy()), tbl, lens)
    assert np.abs(yn - ref).max() <= tol
    for raw, view in ((rq, qt), (rk, kt), (rv, vt)):
        assert slack_intact(raw, view.numel(), nan)
    assert _fusedtok.attention_device_status() == 0


def test_appends_write_exactly_one_row_per_sequence():
    b, hkv, t, d = 3, 4, 64, 128
    g = torch.Generator().manual_seed(3)
    kc = torch.randn(b, hkv, t, d, generator=g).bfloat16()
    rk, kt = guarded(kc.cuda(), 7.0)
    rv, vt = guarded(kc.cuda() * 2, 7.0)
    before_k, before_v = kt.clone(), vt.clone()
    kn = torch.randn(b, hkv, d, generator=g).bfloat16().cuda()
    vn = torch.randn(b, hkv, d, generator=g).bfloat16().cuda()
    lens = torch.tensor([0, 63, 17], dtype=torch.int32, device="cuda")
    ft.kv_append(kt, vt, kn, vn, lens)
    torch.cuda.synchronize()
    for bi, pos in enumerate([0, 63, 17]):
        assert torch.equal(kt[bi, :, pos], kn[bi]) and torch.equal(vt[bi, :, pos], vn[bi])
        before_k[bi, :, pos] = kn[bi]
        before_v[bi, :, pos] = vn[bi]
    assert torch.equal(kt, before_k) and torch.equal(vt, before_v)      # nothing else moved
    assert slack_intact(rk, kt.numel(), 7.0) and slack_intact(rv, vt.numel(), 7.0)
