"""GPU parity tests for the contiguous-cache decode path. Mirrors the
reference's GPU suite (tests/test_attention.py:242-316 staged + split path,
:412-550 zero-copy + graph capture, :562-629 and :732-792 half storage) with
the CPU oracle (pinned to the reference's CPU implementation) as the checker.

Tolerances: fp32 1e-5 max-abs against the oracle; bf16 2e-2 / fp16 2e-3
max-abs and 1e-2 mean-relative against the oracle on the half-rounded inputs.
"""

import numpy as np
import pytest
import torch

import cases
import oracle

import fusedtok_b200 as ft
from fusedtok_b200 import _fusedtok

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
HALF = [pytest.param(torch.bfloat16, 2e-2, id="bf16"), pytest.param(torch.float16, 2e-3, id="fp16")]


def mean_rel(y, ref):
    return float(np.abs(y - ref).mean() / max(np.abs(ref).mean(), 1e-30))


def assert_status_ok():
    assert _fusedtok.attention_device_status() == 0


def half_case(dt, q, k, v):
    qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
    return qt, kt, vt, [x.float().cpu().numpy() for x in (qt, kt, vt)]


# ---- staged path (host arrays through the C ABI), fp32 ----------------------

@pytest.mark.parametrize("b,hq,hkv,t,d,wl", cases.SHAPES)
def test_staged_matches_oracle_and_golden(golden, b, hq, hkv, t, d, wl):
    rng = np.random.default_rng(cases.shape_seed(b, hq, hkv, t, d))
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, wl)
    y = ft.attention_decode(q, k, v, lens, cuda=True)
    assert y.shape == (b, hq, d) and y.dtype == np.float32
    assert np.abs(y - oracle.decode(q, k, v, lens)).max() <= F32_TOL if y.size else True
    name = "shape_%d_%d_%d_%d_%d" % (b, hq, hkv, t, d)
    np.testing.assert_allclose(y, golden[name], rtol=0, atol=F32_TOL)
    assert_status_ok()


def test_config1_fp32(golden):
    q, k, v = cases.config1()
    y = ft.attention_decode(q, k, v, cuda=True)
    np.testing.assert_allclose(y, golden["config1"], rtol=0, atol=F32_TOL)
    yt = ft.attention_decode(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                             torch.from_numpy(v).cuda())
    np.testing.assert_allclose(yt.cpu().numpy(), golden["config1"], rtol=0, atol=F32_TOL)


def test_staged_repeatable_bit_exact():
    rng = np.random.default_rng(22)
    q, k, v, lens = cases.make_case(rng, 2, 8, 2, 100, 64, True)
    first = ft.attention_decode(q, k, v, lens, cuda=True)
    for _ in range(3):
        np.testing.assert_array_equal(ft.attention_decode(q, k, v, lens, cuda=True), first)


def test_gqa_mapping_constant_v():
    rng = np.random.default_rng(5)
    b, hq, hkv, t, d = 1, 6, 3, 4, 8
    q = np.ones((b, hq, d), np.float32)
    k = np.zeros((b, hkv, t, d), np.float32)
    v = rng.standard_normal((b, hkv, d)).astype(np.float32)
    v = np.broadcast_to(v[:, :, None, :], (b, hkv, t, d)).copy()
    y = ft.attention_decode(q, k, v, cuda=True)
    for h in range(hq):
        np.testing.assert_allclose(y[0, h], v[0, h // 2].mean(axis=0), rtol=1e-5, atol=1e-6)


def test_padding_ignored_and_zero_len():
    rng = np.random.default_rng(6)
    q, k, v, _ = cases.make_case(rng, 2, 8, 4, 16, 32, False)
    lens = np.array([16, 5], np.int32)
    y = ft.attention_decode(q, k, v, lens, cuda=True)
    assert np.abs(y - oracle.decode(q, k, v, lens)).max() <= F32_TOL
    k2, v2 = k.copy(), v.copy()
    k2[1, :, 5:] = 1e6
    v2[1, :, 5:] = 1e6
    y2 = ft.attention_decode(q, k2, v2, lens, cuda=True)
    np.testing.assert_array_equal(y2[1], y[1])
    y0 = ft.attention_decode(q, k, v, np.array([0, 5], np.int32), cuda=True)
    assert np.all(y0[0] == 0)


# ---- long caches: every unit is split over several CTAs ---------------------

@pytest.mark.parametrize("group", [1, 2, 3, 4, 5, 8, 16])
@pytest.mark.parametrize("t", [2048, 5000])
def test_long_cache_all_groups_fp32(group, t):
    rng = np.random.default_rng(group * 977 + t)
    hkv, d = 4, 128
    q, k, v, _ = cases.make_case(rng, 1, hkv * group, hkv, t, d, False)
    y = ft.attention_decode(q, k, v, cuda=True)
    assert np.abs(y - oracle.decode(q, k, v)).max() <= F32_TOL
    assert_status_ok()


@pytest.mark.parametrize("extra", [0, 1, 293])
def test_lens_across_tile_boundaries(extra):
    rng = np.random.default_rng(4000 + extra)
    t, hq, hkv, d = 4096, 32, 8, 64
    q, k, v, _ = cases.make_case(rng, 2, hq, hkv, t, d, False)
    lens = np.array([t, 384 + extra], np.int32)      # 384 = 6 full tiles
    y = ft.attention_decode(q, k, v, lens, cuda=True)
    assert np.abs(y - oracle.decode(q, k, v, lens)).max() <= F32_TOL


def test_batched_long_cache_fp32():
    rng = np.random.default_rng(77)
    q, k, v, lens = cases.make_case(rng, 6, 32, 8, 4096, 128, True)
    y = ft.attention_decode(q, k, v, lens, cuda=True)
    assert np.abs(y - oracle.decode(q, k, v, lens)).max() <= F32_TOL


@pytest.mark.parametrize("d", [4, 8, 32, 96, 256, 512])
def test_other_head_dims_fp32(d):
    rng = np.random.default_rng(300 + d)
    q, k, v, lens = cases.make_case(rng, 2, 8, 2, 700, d, True)
    y = ft.attention_decode(q, k, v, lens, cuda=True)
    assert np.abs(y - oracle.decode(q, k, v, lens)).max() <= F32_TOL


# ---- zero-copy torch path ----------------------------------------------------

def test_zero_copy_fp32_and_lens_forms():
    rng = np.random.default_rng(31)
    q, k, v, lens = cases.make_case(rng, 3, 16, 4, 333, 128, True)
    qt, kt, vt = (torch.from_numpy(x).cuda() for x in (q, k, v))
    y = ft.attention_decode(qt, kt, vt, torch.from_numpy(lens).cuda())
    assert y.is_cuda and y.dtype is torch.float32
    ref = oracle.decode(q, k, v, lens)
    assert np.abs(y.cpu().numpy() - ref).max() <= F32_TOL
    y1 = ft.attention_decode(qt, kt, vt, [int(x) for x in lens])
    y2 = ft.attention_decode(qt, kt, vt, torch.tensor(lens.tolist(), dtype=torch.int64))
    np.testing.assert_array_equal(y1.cpu().numpy(), y.cpu().numpy())
    np.testing.assert_array_equal(y2.cpu().numpy(), y.cpu().numpy())


def test_zero_copy_error_contract():
    q = torch.randn(1, 8, 64, device="cuda")
    k = torch.randn(1, 2, 32, 64, device="cuda")
    with pytest.raises(TypeError):       # mixed dtypes
        ft.attention_decode(q, k.half(), k.half())
    with pytest.raises(TypeError):       # int8 was never an attention dtype
        ft.attention_decode(torch.zeros(1, 8, 64, device="cuda", dtype=torch.int8), k, k)
    with pytest.raises(TypeError):       # CPU tensor on the zero-copy path: rejected before any launch
        ft.attention_decode(q, k.cpu(), k)
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k, [33])
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k, [0, 1])
    with pytest.raises(TypeError):
        ft.attention_decode(q, k, k, [1.5])
    out = ft.attention_decode(q, k, k)   # the context is still healthy
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()


# ---- half storage -------------------------------------------------------------

@pytest.mark.parametrize("dt,tol", HALF)
@pytest.mark.parametrize("shape", [(2, 8, 2, 512, 128), (1, 32, 8, 517, 128), (2, 16, 2, 777, 64),
                                   (3, 32, 8, 1000, 128), (2, 40, 8, 2000, 128), (1, 64, 2, 500, 128),
                                   (1, 16, 1, 300, 128), (2, 4, 4, 100, 64), (1, 24, 1, 200, 64)])
def test_half_matches_oracle(dt, tol, shape):
    b, hq, hkv, t, d = shape
    rng = np.random.default_rng(101 + t)
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[0] = t
    qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
    out = ft.attention_decode(qt, kt, vt, torch.from_numpy(lens).cuda())
    assert out.dtype is dt
    y = out.float().cpu().numpy()
    ref = oracle.decode(qr, kr, vr, lens)
    assert np.abs(y - ref).max() <= tol
    assert mean_rel(y, ref) <= 1e-2
    assert_status_ok()


@pytest.mark.parametrize("dt,tol", HALF)
@pytest.mark.parametrize("d", [32, 80, 96, 112, 160, 192, 256])
@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 2), (16, 2), (32, 2), (10, 2)])
def test_half_other_tensor_core_head_dims(dt, tol, d, hq, hkv):
    """Head dims other than 64 / 128 on the tensor-core kernel (8 query heads per MMA tile, groups above 8 in
    chunks; dims that are not a multiple of 64 through per-column-block copies), contiguous with ragged lengths
    across tile boundaries, and paged."""
    rng = np.random.default_rng(d + hq * 3 + hkv)
    b, t = 3, 700
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[:] = [t, 65, 333]
    qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
    ref = oracle.decode(qr, kr, vr, lens)
    y = ft.attention_decode(qt, kt, vt, torch.from_numpy(lens).cuda()).float().cpu().numpy()
    assert np.abs(y - ref).max() <= tol
    assert mean_rel(y, ref) <= 1e-2
    # the same cache cut into pages of 16 rows, blocks shuffled
    page = 16
    nblk = (t + page - 1) // page
    pad = nblk * page - t
    kp = torch.nn.functional.pad(kt, (0, 0, 0, pad)).view(b, hkv, nblk, page, d).permute(0, 2, 1, 3, 4).reshape(
        b * nblk, hkv, page, d)
    vp = torch.nn.functional.pad(vt, (0, 0, 0, pad)).view(b, hkv, nblk, page, d).permute(0, 2, 1, 3, 4).reshape(
        b * nblk, hkv, page, d)
    perm = torch.randperm(b * nblk, generator=torch.Generator().manual_seed(d)).cuda()
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(b * nblk, device="cuda")
    table = inv.view(b, nblk).to(torch.int32).contiguous()          # sequence b, page s lives in block inv[b*nblk+s]
    kpool, vpool = kp[perm].contiguous(), vp[perm].contiguous()
    if hq // hkv in (1, 2, 4, 8, 16):
        yp = ft.attention_decode_paged(qt, kpool, vpool, table, torch.from_numpy(lens).cuda()).float().cpu().numpy()
        assert np.abs(yp - ref).max() <= tol
    assert_status_ok()


@pytest.mark.parametrize("dt,tol", HALF)
def test_half_small_tensor_core_head_dims_short_cache(dt, tol):
    rng = np.random.default_rng(7)
    for d in (32, 96, 256):
        q, k, v, lens = cases.make_case(rng, 2, 8, 2, 300, d, True)
        qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
        y = ft.attention_decode(qt, kt, vt, torch.from_numpy(lens).cuda()).float().cpu().numpy()
        assert np.abs(y - oracle.decode(qr, kr, vr, lens)).max() <= tol


@pytest.mark.parametrize("dt,tol", HALF)
@pytest.mark.parametrize("d", [4, 8, 16, 48, 144, 512])
@pytest.mark.parametrize("group", [1, 4, 5, 8])
def test_half_cuda_core_kernel_head_dims(dt, tol, d, group):
    """16-bit caches whose head dim the tensor-core kernel is not built for run on the CUDA-core kernel: every
    chunks-per-lane variant (dims up to 128, 256, 512) x heads-per-unit variant (group 1, 4, 5 -> 8 or 4 + 1, 8),
    contiguous cache, ragged lengths that cross tile boundaries and include an empty sequence."""
    hkv = 2
    rng = np.random.default_rng(d * 31 + group)
    b, t = 4, 600
    q, k, v, lens = cases.make_case(rng, b, hkv * group, hkv, t, d, True)
    lens[:] = [t, 0, 65, 333]
    qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
    out = ft.attention_decode(qt, kt, vt, torch.from_numpy(lens).cuda())
    y = out.float().cpu().numpy()
    ref = oracle.decode(qr, kr, vr, lens)
    assert np.abs(y - ref).max() <= tol
    assert mean_rel(y, ref) <= 1e-2
    assert np.all(y[1] == 0)
    # and a cache long enough that units are split over CTAs and merged
    q, k, v, _ = cases.make_case(rng, 1, hkv * group, hkv, 3000, d, False)
    qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
    y = ft.attention_decode(qt, kt, vt).float().cpu().numpy()
    assert np.abs(y - oracle.decode(qr, kr, vr)).max() <= tol
    assert_status_ok()


@pytest.mark.parametrize("dt,tol", HALF)
def test_half_unaligned_cache_falls_back_to_cuda_core_kernel(dt, tol):
    """A D=128 cache that starts 8 bytes into its allocation cannot be described to TMA (16-byte rule): the
    launcher must route it to the CUDA-core kernel, whose 8-byte copies it satisfies, and the result must match
    the aligned call closely (other kernel, other summation order)."""
    rng = np.random.default_rng(88)
    b, hq, hkv, t, d = 2, 16, 4, 900, 128
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[0] = t
    qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
    lt = torch.from_numpy(lens).cuda()

    def shifted(x):
        raw = torch.empty(x.numel() + 8, dtype=x.dtype, device="cuda")
        view = raw[4:4 + x.numel()].view(x.shape)
        view.copy_(x)
        assert view.data_ptr() % 16 == 8 and view.is_contiguous()
        return view

    ks, vs = shifted(kt), shifted(vt)
    y = ft.attention_decode(qt, ks, vs, lt).float().cpu().numpy()
    ref = oracle.decode(qr, kr, vr, lens)
    assert np.abs(y - ref).max() <= tol
    aligned = ft.attention_decode(qt, kt, vt, lt).float().cpu().numpy()
    assert np.abs(y - aligned).max() <= tol
    # two elements in is not aligned to 4 elements: refused, nothing launched
    raw = torch.empty(kt.numel() + 8, dtype=dt, device="cuda")
    bad = raw[2:2 + kt.numel()].view(kt.shape)
    with pytest.raises(ValueError):
        ft.attention_decode(qt, bad, vt, lt)
    assert_status_ok()


# ---- the range scheduler --------------------------------------------------------

@pytest.mark.parametrize("dt,tol", HALF)
def test_dynamic_tail_with_ragged_lens_matches_oracle_and_repeats(dt, tol):
    """Large enough for the static + dynamic-tail plan (more than 24 tiles per SM) with lengths that put range
    boundaries inside units, empty sequences and a one-row sequence. Which SM computes a tail range changes from
    launch to launch; the output must not."""
    rng = np.random.default_rng(4242)
    b, hq, hkv, t, d = 24, 32, 8, 2048, 128
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[:6] = [t, 0, 1, 64, 65, 0]
    qt, kt, vt, (qr, kr, vr) = half_case(dt, q, k, v)
    lt = torch.from_numpy(lens).cuda()
    first = ft.attention_decode(qt, kt, vt, lt)
    y = first.float().cpu().numpy()
    ref = oracle.decode(qr, kr, vr, lens)
    assert np.abs(y - ref).max() <= tol
    assert mean_rel(y, ref) <= 1e-2
    assert np.all(y[1] == 0) and np.all(y[5] == 0)
    for _ in range(20):
        assert torch.equal(ft.attention_decode(qt, kt, vt, lt), first)
    assert_status_ok()


def test_more_sequences_than_the_schedule_table_holds():
    """Over 2048 sequences with lens: the per-sequence prefix table does not fit, the kernel finds its range with
    the block-wide scan and keeps the equal split."""
    rng = np.random.default_rng(9)
    b, hq, hkv, t, d = 2500, 4, 2, 96, 64
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[:4] = [t, 0, 1, 65]
    qt, kt, vt, (qr, kr, vr) = half_case(torch.bfloat16, q, k, v)
    lt = torch.from_numpy(lens).cuda()
    out = ft.attention_decode(qt, kt, vt, lt)
    y = out.float().cpu().numpy()
    ref = oracle.decode(qr, kr, vr, lens)
    assert np.abs(y - ref).max() <= 2e-2
    assert np.all(y[1] == 0)
    assert torch.equal(ft.attention_decode(qt, kt, vt, lt), out)
    assert_status_ok()


@pytest.mark.parametrize("dt,tol", HALF)
def test_half_constant_v_probe(dt, tol):
    b, hq, hkv, t, d = 1, 8, 2, 300, 128
    q = torch.randn(b, hq, d, device="cuda").to(dt)
    k = torch.randn(b, hkv, t, d, device="cuda").to(dt)
    v0 = torch.randn(hkv, d, device="cuda").to(dt)
    v = v0[None, :, None, :].expand(b, hkv, t, d).contiguous()
    out = ft.attention_decode(q, k, v, torch.tensor([300], dtype=torch.int32, device="cuda"))
    for h in range(hq):
        np.testing.assert_allclose(out[0, h].float().cpu().numpy(), v0[h // 4].float().cpu().numpy(),
                                   rtol=tol, atol=tol)


@pytest.mark.parametrize("dt,tol", HALF)
def test_half_poisoned_padding_and_zero_len(dt, tol):
    b, hq, hkv, t, d = 2, 8, 2, 256, 128
    q = torch.randn(b, hq, d, device="cuda").to(dt)
    k = torch.randn(b, hkv, t, d, device="cuda").to(dt)
    v = torch.randn(b, hkv, t, d, device="cuda").to(dt)
    lens = torch.tensor([100, 0], dtype=torch.int32, device="cuda")
    k[0, :, 100:] = 30000.0
    v[0, :, 100:] = float("nan")          # stronger than the reference's probe: NaN must not leak either
    out = ft.attention_decode(q, k, v, lens)
    ref0 = oracle.decode(q[0:1].float().cpu().numpy(), k[0:1, :, :100].float().cpu().numpy(),
                         v[0:1, :, :100].float().cpu().numpy())
    assert np.abs(out[0].float().cpu().numpy() - ref0[0]).max() <= tol
    np.testing.assert_array_equal(out[1].float().cpu().numpy(), np.zeros((hq, d), np.float32))


def test_config2_reduced_bf16(golden):
    """Benchmark configuration 2 at batch 1 x 1024 rows against the golden
    vector, and at batch 2 x 4096 rows against the oracle."""
    q, k, v = cases.config2(batch=1, t=1024)
    qt, kt, vt, _ = half_case(torch.bfloat16, q, k, v)
    y = ft.attention_decode(qt, kt, vt).float().cpu().numpy()
    ref = golden["config2_b1_t1024_bf16"]
    assert np.abs(y - ref).max() <= 2e-2 and mean_rel(y, ref) <= 1e-2
    q, k, v = cases.config2(batch=2, t=4096)
    qt, kt, vt, (qr, kr, vr) = half_case(torch.bfloat16, q, k, v)
    y = ft.attention_decode(qt, kt, vt).float().cpu().numpy()
    ref = oracle.decode(qr, kr, vr)
    assert np.abs(y - ref).max() <= 2e-2 and mean_rel(y, ref) <= 1e-2
    yl = ft.attention_decode(qt, kt, vt, torch.full((2,), 4096, dtype=torch.int32, device="cuda"))
    np.testing.assert_array_equal(yl.float().cpu().numpy(), y)


def test_config2_full_size_properties():
    """Full benchmark configuration 2 (batch 32 x 4096 rows, 537 MB of cache):
    too large for the CPU oracle, so check size-independent properties -
    constant V per kv head gives that constant back (GQA map), every sequence
    equals the same sequence run alone (batch independence), and repeated
    calls are bit-identical."""
    B, Hq, Hkv, T, D = 32, 32, 8, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, Hq, D, device="cuda", generator=g).to(torch.bfloat16)
    k = (torch.randn(B, Hkv, T, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    v = (torch.randn(B, Hkv, T, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    y = ft.attention_decode(q, k, v)
    y2 = ft.attention_decode(q, k, v)
    assert torch.equal(y, y2)
    for b in (0, 13, 31):
        alone = ft.attention_decode(q[b:b + 1].contiguous(), k[b:b + 1].contiguous(), v[b:b + 1].contiguous())
        assert (alone.float() - y[b:b + 1].float()).abs().max().item() <= 2e-3
    ref = oracle.decode(q[5:6].float().cpu().numpy(), k[5:6].float().cpu().numpy(), v[5:6].float().cpu().numpy())
    assert np.abs(y[5:6].float().cpu().numpy() - ref).max() <= 2e-2
    v0 = torch.randn(Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    vc = v0[None, :, None, :].expand(B, Hkv, T, D).contiguous()
    yc = ft.attention_decode(q, k, vc)
    want = v0.float().repeat_interleave(Hq // Hkv, dim=0)[None].expand(B, Hq, D)
    assert (yc.float() - want).abs().max().item() <= 2e-2
    assert_status_ok()


def test_many_back_to_back_launches_stay_bit_identical():
    """600 launches queued without any host synchronisation (the regime in which
    a producer/consumer phase hazard of the TMA ring once showed up): every
    launch must give the bits of the first and the status word must stay 0."""
    rng = np.random.default_rng(17)
    q, k, v, lens = cases.make_case(rng, 8, 32, 8, 3000, 128, True)
    qt, kt, vt, _ = half_case(torch.bfloat16, q, k, v)
    lt = torch.from_numpy(lens).cuda()
    outs = [torch.empty_like(qt) for _ in range(4)]
    st = torch.cuda.current_stream().cuda_stream
    for i in range(600):
        _fusedtok.attention_decode_launch_bf16(qt.data_ptr(), kt.data_ptr(), vt.data_ptr(), lt.data_ptr(),
                                               outs[i % 4].data_ptr(), 8, 32, 8, 3000, 128, st)
    torch.cuda.synchronize()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert_status_ok()


# ---- CUDA graph capture (reference: tests/test_attention.py:482-550, 763-792)

def _capture(run):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            run()
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        run()
    return g


def test_graph_capture_replay_fp32():
    q = torch.randn(2, 8, 64, device="cuda")
    k = torch.randn(2, 2, 100, 64, device="cuda")
    v = torch.randn(2, 2, 100, 64, device="cuda")
    lens = torch.tensor([100, 40], dtype=torch.int32, device="cuda")
    y = torch.empty(2, 8, 64, device="cuda")

    def run():
        _fusedtok.attention_decode_launch(q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr(),
                                          y.data_ptr(), 2, 8, 2, 100, 64,
                                          torch.cuda.current_stream().cuda_stream)
    g = _capture(run)
    q.mul_(2.0)
    lens.copy_(torch.tensor([64, 100], dtype=torch.int32))     # lens are read on the device at replay
    y.fill_(float("nan"))
    g.replay()
    torch.cuda.synchronize()
    ref = oracle.decode(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), lens.cpu().numpy())
    assert np.abs(y.cpu().numpy() - ref).max() <= F32_TOL


def test_graph_capture_replay_long_cache_lens_zero_arg():
    b, hq, hkv, t, d = 1, 32, 8, 4096, 128
    q = torch.randn(b, hq, d, device="cuda")
    k = torch.randn(b, hkv, t, d, device="cuda")
    v = torch.randn(b, hkv, t, d, device="cuda")
    y = torch.empty(b, hq, d, device="cuda")

    def run():
        _fusedtok.attention_decode_launch(q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, y.data_ptr(),
                                          b, hq, hkv, t, d, torch.cuda.current_stream().cuda_stream)
    g = _capture(run)
    k.mul_(1.5)
    v.mul_(-0.5)
    y.fill_(float("nan"))
    g.replay()
    torch.cuda.synchronize()
    ref = oracle.decode(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    assert np.abs(y.cpu().numpy() - ref).max() <= F32_TOL


def test_graph_capture_bf16():
    b, hq, hkv, t, d = 1, 8, 2, 1024, 128
    q = torch.randn(b, hq, d, device="cuda").to(torch.bfloat16)
    k = torch.randn(b, hkv, t, d, device="cuda").to(torch.bfloat16)
    v = torch.randn(b, hkv, t, d, device="cuda").to(torch.bfloat16)
    y = torch.empty(b, hq, d, device="cuda", dtype=torch.bfloat16)

    def run():
        _fusedtok.attention_decode_launch_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, y.data_ptr(),
                                               b, hq, hkv, t, d, torch.cuda.current_stream().cuda_stream)
    g = _capture(run)
    k.mul_(1.25)
    y.fill_(0)
    g.replay()
    torch.cuda.synchronize()
    ref = oracle.decode(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
    assert np.abs(y.float().cpu().numpy() - ref).max() <= 2e-2
    assert_status_ok()


# ---- KV-length split primitives (the multi-GPU layer's building blocks) ------

@pytest.mark.parametrize("dt,code,tol", [(torch.float32, 0, 1e-5), (torch.bfloat16, 1, 2e-2)])
def test_partial_triples_merge_to_full_result(dt, code, tol):
    """Shard the cache rows 4 ways (as 4 GPUs would hold them), take raw
    triples per shard, merge: equals the unsharded result; shards that are
    empty for a short sequence contribute nothing."""
    rng = np.random.default_rng(55)
    b, hq, hkv, t, d, n = 3, 16, 4, 2048, 128, 4
    q, k, v, _ = cases.make_case(rng, b, hq, hkv, t, d, False)
    lens = np.array([2048, 700, 0], np.int32)
    qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
    full = ft.attention_decode(qt, kt, vt, torch.from_numpy(lens).cuda())
    nf = _fusedtok.attention_partial_floats(b, hq, d)
    parts = torch.empty(n, nf, device="cuda", dtype=torch.float32)
    shard = t // n
    st = torch.cuda.current_stream().cuda_stream
    for r in range(n):
        ks = kt[:, :, r * shard:(r + 1) * shard].contiguous()
        vs = vt[:, :, r * shard:(r + 1) * shard].contiguous()
        ls = torch.from_numpy(np.clip(lens - r * shard, 0, shard).astype(np.int32)).cuda()
        _fusedtok.attention_decode_partial_launch(code, qt.data_ptr(), ks.data_ptr(), vs.data_ptr(),
                                                  ls.data_ptr(), parts[r].data_ptr(), b, hq, hkv, shard, d, st)
    out = torch.empty_like(full)
    _fusedtok.attention_merge_partials_launch(code, parts.data_ptr(), n, out.data_ptr(), b, hq, d, st)
    torch.cuda.synchronize()
    assert (out.float() - full.float()).abs().max().item() <= (1e-6 if code == 0 else 4e-3)
    ref = oracle.decode(qt.float().cpu().numpy(), kt.float().cpu().numpy(), vt.float().cpu().numpy(), lens)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol
    assert torch.count_nonzero(out[2]) == 0
    assert_status_ok()


@pytest.mark.gpu
def test_missing_peer_expires_with_a_status_and_the_context_stays_usable():
    """Failure detection without a fault: a KV-split step whose peer never delivers. The second exchange buffer
    here belongs to no rank, so nothing ever raises that rank's flags in this rank's buffer; the wait at the end of
    the kernel (2 s limit) must run out, report status 5 and return, and the next ordinary call must work."""
    import time
    b, hq, hkv, d, t = 2, 8, 2, 64, 128
    g = torch.Generator().manual_seed(11)
    q = torch.randn(b, hq, d, generator=g).bfloat16().cuda()
    k = torch.randn(b, hkv, t, d, generator=g).bfloat16().cuda()
    v = torch.randn(b, hkv, t, d, generator=g).bfloat16().cuda()
    out = torch.empty_like(q)
    ft.attention_decode(q, k, v)                                   # arena and status word exist
    assert _fusedtok.attention_device_status() == 0
    mine, _ = _fusedtok.exchange_alloc(2, b, hq, d)
    ghost, _ = _fusedtok.exchange_alloc(2, b, hq, d)
    try:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _fusedtok.attention_decode_exchange_launch(1, q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, out.data_ptr(),
                                                   [mine, ghost], 0, b, hq, hkv, t, d,
                                                   torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 1.5 < waited < 15.0, waited
        assert _fusedtok.attention_device_status() == 5
        assert _fusedtok.attention_device_status() == 0             # reading it clears it
        y = ft.attention_decode(q, k, v)
        want = oracle.decode(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy())
        np.testing.assert_allclose(y.float().cpu().numpy(), want, atol=2e-2, rtol=2e-2)
        assert _fusedtok.attention_device_status() == 0
    finally:
        torch.cuda.synchronize()
        _fusedtok.exchange_free(mine)
        _fusedtok.exchange_free(ghost)


_DYN_SCRIPT = r"""
import sys, os
import numpy as np, torch
import cases, oracle
import fusedtok_b200 as ft
from fusedtok_b200 import _fusedtok
rng = np.random.default_rng(4242)
b, hq, hkv, t, d = 24, 32, 8, 2048, 128
q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
lens[:6] = [t, 0, 1, 64, 65, 0]
qt, kt, vt = (torch.from_numpy(x).cuda().to(torch.bfloat16) for x in (q, k, v))
lt = torch.from_numpy(lens).cuda()
first = ft.attention_decode(qt, kt, vt, lt)
for _ in range(30):
    assert torch.equal(ft.attention_decode(qt, kt, vt, lt), first)
full = ft.attention_decode(qt, kt, vt)                      # no lens: the schedule is arithmetic
for _ in range(10):
    assert torch.equal(ft.attention_decode(qt, kt, vt), full)
ref = oracle.decode(qt.float().cpu().numpy(), kt.float().cpu().numpy(), vt.float().cpu().numpy(), lens)
err = float(np.abs(first.float().cpu().numpy() - ref).max())
assert err <= 2e-2, err
assert _fusedtok.attention_device_status() == 0
np.save(sys.argv[1], first.float().cpu().numpy())
print("ok", err)
"""


def test_dynamic_range_plan_when_enabled(tmp_path):
    """The static + dynamic plan is off by default (it measured slower) but stays in the library behind
    FUSEDTOK_DYN_CHUNK. Run it in a process of its own (the switch is read when the library loads): ranges handed
    out by an atomic counter, partials keyed by range - the result must match the oracle, repeat bit for bit although
    which SM computes which range changes from launch to launch, and agree with the equal split to rounding."""
    import subprocess
    import sys
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = {}
    for name, env_extra in (("static", {}), ("dynamic", {"FUSEDTOK_DYN_CHUNK": "4", "FUSEDTOK_DYN_TAIL": "16"})):
        env = dict(os.environ, PYTHONPATH=os.pathsep.join([root, os.path.join(root, "tests")]), **env_extra)
        path = str(tmp_path / (name + ".npy"))
        res = subprocess.run([sys.executable, "-c", _DYN_SCRIPT, path], env=env, capture_output=True, text=True,
                             timeout=600)
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        outs[name] = np.load(path)
    assert np.abs(outs["static"] - outs["dynamic"]).max() <= 2e-2


# ---- one unit split over many ranges: the cross-range merge in rounds and passes ---------------------------

@pytest.mark.parametrize("dt,tol", HALF + [pytest.param(torch.float32, F32_TOL, id="fp32")])
@pytest.mark.parametrize("shape", [(1, 8, 2, 40000, 128),      # 2 units over the whole grid: several rounds of partials
                                   (1, 16, 1, 30000, 128),     # 16 heads per unit: more element pairs than threads
                                   (1, 8, 1, 20000, 64),
                                   (1, 32, 8, 16384, 128),     # the reference's benchmark shape
                                   (1, 4, 1, 1000, 128),       # fewer tiles than CTAs: most ranges are empty
                                   (2, 8, 8, 256, 128)])
def test_one_sequence_spread_over_the_grid(dt, tol, shape):
    b, hq, hkv, t, d = shape
    rng = np.random.default_rng(t + d)
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[:] = t - 37
    lens[0] = t
    qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
    qr, kr, vr = (x.float().cpu().numpy() for x in (qt, kt, vt))
    lt = torch.from_numpy(lens).cuda()
    out = ft.attention_decode(qt, kt, vt, lt)
    y = out.float().cpu().numpy()
    assert np.abs(y - oracle.decode(qr, kr, vr, lens)).max() <= tol
    assert torch.equal(ft.attention_decode(qt, kt, vt, lt), out)          # the merge order is fixed
    full = ft.attention_decode(qt, kt, vt).float().cpu().numpy()          # no lens: the schedule is arithmetic
    assert np.abs(full - oracle.decode(qr, kr, vr)).max() <= tol
    assert_status_ok()


# ---- float32 caches on the TMA-fed kernel (launches of more than two tiles per SM, head dim 64 / 128) ----------

@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("group", [1, 3, 4, 5, 8, 16])
def test_fp32_ring_kernel_contiguous(d, group):
    """Large enough for the producer-warp + copy-ring float32 kernel: every heads-per-unit variant (group 1; 3, 4 ->
    4 with spare rows; 5, 8 -> 8; 16 -> two chunks of 8), ragged lengths that end inside the first and the second
    half of a tile, on a tile boundary and at zero, 1e-5 against the oracle and bit-exact repetition."""
    hkv = 2
    rng = np.random.default_rng(d * 17 + group)
    b, t = 6, 2048
    q, k, v, lens = cases.make_case(rng, b, hkv * group, hkv, t, d, True)
    lens[:] = [t, 0, 1, 33, 64, 1500]
    qt, kt, vt = (torch.from_numpy(x).cuda() for x in (q, k, v))
    lt = torch.from_numpy(lens).cuda()
    out = ft.attention_decode(qt, kt, vt, lt)
    y = out.cpu().numpy()
    assert np.abs(y - oracle.decode(q, k, v, lens)).max() <= F32_TOL
    assert np.all(y[1] == 0)
    assert torch.equal(ft.attention_decode(qt, kt, vt, lt), out)
    full = ft.attention_decode(qt, kt, vt).cpu().numpy()          # no lens: the schedule is arithmetic
    assert np.abs(full - oracle.decode(q, k, v)).max() <= F32_TOL
    assert_status_ok()


@pytest.mark.parametrize("page", [8, 16, 64])
def test_fp32_ring_kernel_paged(page):
    """The same kernel behind a block table: pages smaller than, equal to half of, and larger than its 32-row boxes;
    must equal the contiguous kernel's result on the gathered rows bit for bit."""
    rng = np.random.default_rng(300 + page)
    b, hq, hkv, d, t = 4, 16, 4, 128, 2048
    lens = np.array([t, 700, 0, 1025], np.int32)
    width = t // page
    nb = b * width + 5
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    kp = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
    vp = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
    tbl = rng.permutation(nb)[:b * width].reshape(b, width).astype(np.int32)
    kc = kp[tbl].transpose(0, 2, 1, 3, 4).reshape(b, hkv, t, d)
    vc = vp[tbl].transpose(0, 2, 1, 3, 4).reshape(b, hkv, t, d)
    qt, kpt, vpt = (torch.from_numpy(x).cuda() for x in (q, kp, vp))
    out = torch.empty_like(qt)
    tblt, lt = torch.from_numpy(tbl).cuda(), torch.from_numpy(lens).cuda()       # kept alive across the launch
    _fusedtok.attention_decode_paged_launch(qt.data_ptr(), kpt.data_ptr(), vpt.data_ptr(), tblt.data_ptr(),
                                            lt.data_ptr(), out.data_ptr(), b, hq, hkv, page, width, d,
                                            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    y = out.cpu().numpy()
    assert np.abs(y - oracle.decode(q, np.ascontiguousarray(kc), np.ascontiguousarray(vc), lens)).max() <= F32_TOL
    contiguous = ft.attention_decode(qt, torch.from_numpy(np.ascontiguousarray(kc)).cuda(),
                                     torch.from_numpy(np.ascontiguousarray(vc)).cuda(), lt)
    assert torch.equal(out, contiguous)
    assert np.all(y[2] == 0)
    assert_status_ok()
