"""The allocation-free launcher against the ordinary one.

Some hosts cannot allocate device memory once they are running - a serving
process that pre-budgets all of HBM into its own pool, a host under an
allocator-policing shim, a latency-critical loop that cannot absorb
cudaMalloc's device synchronisation. ``fusedtok_attention_decode_launch_noalloc``
gives them the contiguous-cache decode with its split-KV scratch in a fixed
4 MiB array inside the library. These tests call it through the C ABI and
require the SAME output, bit for bit, as ``fusedtok_attention_decode_launch*``
on the same inputs (both launch the same kernel on the same split), on two
calls in a row (the scratch keeps the previous call's contents, so the second
call, on different inputs, would show anything stale); that device memory in
use does not move across the calls; that a shape beyond the fixed scratch is
refused with a clear error; and that the status word this path keeps in its
static scratch comes back through ``fusedtok_attention_device_status``.

Collected last on purpose, so a run that stops at the first failure has already
run every other test.
"""

import numpy as np
import pytest
import torch

import cases
import oracle

from fusedtok_b200 import _fusedtok

pytestmark = pytest.mark.gpu

lib = _fusedtok._lib
NAMES = {0: "fusedtok_attention_decode_launch", 1: "fusedtok_attention_decode_launch_bf16",
         2: "fusedtok_attention_decode_launch_fp16"}


def _launch_pair(dt, code, b, hq, hkv, t, d, seed, with_lens=True):
    rng = np.random.default_rng(seed)
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[0] = t
    qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
    lt = torch.from_numpy(lens).cuda()
    lp = lt.data_ptr() if with_lens else None
    st = torch.cuda.current_stream().cuda_stream
    want = torch.empty_like(qt)
    got = torch.full_like(qt, float("nan"))
    rc = getattr(lib, NAMES[code])(qt.data_ptr(), kt.data_ptr(), vt.data_ptr(), lp, want.data_ptr(),
                                   b, hq, hkv, t, d, st)
    assert rc == 0, lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_launch_noalloc(code, qt.data_ptr(), kt.data_ptr(), vt.data_ptr(),
                                                      lp, got.data_ptr(), b, hq, hkv, t, d, st)
    assert rc == 0, lib.fusedtok_last_error()
    torch.cuda.synchronize()
    ref = oracle.decode(qt.float().cpu().numpy(), kt.float().cpu().numpy(), vt.float().cpu().numpy(),
                        lens if with_lens else None)
    return got, want, ref


@pytest.mark.parametrize("dt,code,tol", [(torch.bfloat16, 1, 2e-2), (torch.float16, 2, 2e-3),
                                         (torch.float32, 0, 1e-5)])
def test_noalloc_matches_allocating_launcher_twice_in_a_row(dt, code, tol):
    # first call: many units split over CTAs; second call: other inputs and a
    # different split, reusing the same static scratch
    for seed, shape in ((11, (3, 32, 8, 2000, 128)), (12, (2, 16, 4, 3000, 128))):
        got, want, ref = _launch_pair(dt, code, *shape, seed)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)                   # same kernel, same split: identical bits
        assert np.abs(got.float().cpu().numpy() - ref).max() <= tol
    assert _fusedtok.attention_device_status() == 0


def test_noalloc_other_kernel_variants_and_no_allocation():
    """Head chunking and kernel variants change from call to call (CUDA-core kernel with two and four chunks
    per lane, one head per unit, no lens, then the 16-head tensor-core tile), all through the one static array;
    device memory in use must not move while only the allocation-free entry point is called."""
    cases_ = [(torch.float32, 0, (2, 4, 4, 700, 256), True, 1e-5),      # G = 1, two chunks per lane
              (torch.float32, 0, (1, 4, 2, 300, 512), True, 1e-5),      # four chunks per lane
              (torch.bfloat16, 1, (2, 8, 8, 900, 64), False, 2e-2),     # no lens
              (torch.bfloat16, 1, (2, 32, 2, 1500, 128), True, 2e-2),   # 16 heads per unit
              (torch.float16, 2, (8, 32, 8, 4096, 128), False, 2e-3)]   # large enough for the dynamic tail
    # warm every path up (first calls may set attributes and, for the allocating twin, allocate)
    for dt, code, shape, wl, tol in cases_:
        _launch_pair(dt, code, *shape, 5, wl)
    torch.cuda.synchronize()
    inputs = []
    for dt, code, (b, hq, hkv, t, d), wl, tol in cases_:
        g = torch.Generator(device="cuda").manual_seed(b * 7 + d)
        q = torch.randn(b, hq, d, device="cuda", generator=g).to(dt)
        k = torch.randn(b, hkv, t, d, device="cuda", generator=g).to(dt)
        v = torch.randn(b, hkv, t, d, device="cuda", generator=g).to(dt)
        inputs.append((code, q, k, v, torch.empty_like(q), (b, hq, hkv, t, d)))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(3):
        for code, q, k, v, out, (b, hq, hkv, t, d) in inputs:
            rc = lib.fusedtok_attention_decode_launch_noalloc(code, q.data_ptr(), k.data_ptr(), v.data_ptr(), None,
                                                              out.data_ptr(), b, hq, hkv, t, d, st)
            assert rc == 0, lib.fusedtok_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    for dt, code, shape, wl, tol in cases_:
        got, want, ref = _launch_pair(dt, code, *shape, 21, wl)
        assert torch.equal(got, want)
        assert np.abs(got.float().cpu().numpy() - ref).max() <= tol
    assert _fusedtok.attention_device_status() == 0


def test_noalloc_rejects_shapes_beyond_the_fixed_scratch():
    # 64 x 8 units x 16 heads x 130 floats is far more than 4 MiB; validation
    # happens before anything is launched, so dummy pointers are never touched
    rc = lib.fusedtok_attention_decode_launch_noalloc(1, 256, 256, 256, None, 256, 64, 128, 8, 4096, 128, 0)
    assert rc == 1
    msg = lib.fusedtok_last_error().decode()
    assert "allocation-free" in msg and "4194304" in msg
    # more (sequence, kv head) units than the counter region tracks
    rc = lib.fusedtok_attention_decode_launch_noalloc(1, 256, 256, 256, None, 256, 4096, 8, 8, 64, 64, 0)
    assert rc == 1
    assert "units" in lib.fusedtok_last_error().decode()
    rc = lib.fusedtok_attention_decode_launch_noalloc(7, 256, 256, 256, None, 256, 1, 8, 8, 64, 64, 0)
    assert rc == 1
    # operands that are not aligned to 4 elements are refused, not launched
    rc = lib.fusedtok_attention_decode_launch_noalloc(1, 258, 256, 256, None, 256, 1, 8, 8, 64, 64, 0)
    assert rc == 1


def test_noalloc_status_word_is_reported_and_recovers():
    """What an expired bounded wait would leave behind on this path - a status code in the header of the static
    scratch and a half-counted arrival counter - written from the host (no wait is made to expire, no fault):
    fusedtok_attention_device_status must report the code, clear it together with the counters, and the next
    call must be correct."""
    got, want, _ = _launch_pair(torch.bfloat16, 1, 3, 32, 8, 2000, 128, 31)     # the path has run: set-up done
    assert torch.equal(got, want)
    assert _fusedtok.attention_device_status() == 0
    assert lib.fusedtok_debug_poke_status(1, 2, 3) == 0         # code 2, arrival counter of unit 3 left at 1
    assert lib.fusedtok_debug_poke_status(1, -1, 3) == 101      # the counter really is 1
    assert _fusedtok.attention_device_status() == 2             # reported through the public call ...
    assert _fusedtok.attention_device_status() == 0             # ... and cleared
    assert lib.fusedtok_debug_poke_status(1, -1, 3) == 100      # the counters were cleared with it
    got, want, ref = _launch_pair(torch.bfloat16, 1, 3, 32, 8, 2000, 128, 32)
    assert torch.equal(got, want)
    assert np.abs(got.float().cpu().numpy() - ref).max() <= 2e-2
    # the allocating path's word goes through the same call
    assert lib.fusedtok_debug_poke_status(0, 4, -1) == 0
    assert _fusedtok.attention_device_status() == 4
    assert _fusedtok.attention_device_status() == 0
