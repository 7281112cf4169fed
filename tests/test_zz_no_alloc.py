"""The allocation-free launcher against the ordinary one.

Some hosts cannot allocate device memory once they are running - a serving
process that pre-budgets all of HBM into its own pool, a host under an
allocator-policing shim, a latency-critical loop that cannot absorb
cudaMalloc's device synchronisation. ``fusedtok_attention_decode_launch_noalloc``
gives them the contiguous-cache decode with its split-KV scratch in a fixed
4 MiB array inside the library. These tests call it through the C ABI and
require the same output as ``fusedtok_attention_decode_launch*`` on the same
inputs, on two calls in a row (the scratch keeps the previous call's contents,
so the second call, on different inputs, would show anything stale), and check
that a shape beyond the fixed scratch is refused with a clear error.

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


def _launch_pair(dt, code, b, hq, hkv, t, d, seed):
    rng = np.random.default_rng(seed)
    q, k, v, lens = cases.make_case(rng, b, hq, hkv, t, d, True)
    lens[0] = t
    qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
    lt = torch.from_numpy(lens).cuda()
    st = torch.cuda.current_stream().cuda_stream
    want = torch.empty_like(qt)
    got = torch.full_like(qt, float("nan"))
    name = {0: "fusedtok_attention_decode_launch", 1: "fusedtok_attention_decode_launch_bf16",
            2: "fusedtok_attention_decode_launch_fp16"}[code]
    rc = getattr(lib, name)(qt.data_ptr(), kt.data_ptr(), vt.data_ptr(), lt.data_ptr(), want.data_ptr(),
                            b, hq, hkv, t, d, st)
    assert rc == 0, lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_launch_noalloc(code, qt.data_ptr(), kt.data_ptr(), vt.data_ptr(),
                                                      lt.data_ptr(), got.data_ptr(), b, hq, hkv, t, d, st)
    assert rc == 0, lib.fusedtok_last_error()
    torch.cuda.synchronize()
    ref = oracle.decode(qt.float().cpu().numpy(), kt.float().cpu().numpy(), vt.float().cpu().numpy(), lens)
    return got.float().cpu().numpy(), want.float().cpu().numpy(), ref


@pytest.mark.parametrize("dt,code,tol", [(torch.bfloat16, 1, 2e-2), (torch.float16, 2, 2e-3),
                                         (torch.float32, 0, 1e-5)])
def test_noalloc_matches_allocating_launcher_twice_in_a_row(dt, code, tol):
    # first call: many units split over CTAs; second call: other inputs and a
    # different split, reusing the same static scratch
    for seed, shape in ((11, (3, 32, 8, 2000, 128)), (12, (2, 16, 4, 3000, 128))):
        got, want, ref = _launch_pair(dt, code, *shape, seed)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= tol          # same kernels, same split: in practice identical
        assert np.abs(got - ref).max() <= tol


def test_noalloc_rejects_shapes_beyond_the_fixed_scratch():
    # 64 x 8 units x 16 heads x 130 floats is far more than 4 MiB; validation
    # happens before anything is launched, so dummy pointers are never touched
    rc = lib.fusedtok_attention_decode_launch_noalloc(1, 256, 256, 256, None, 256, 64, 128, 8, 4096, 128, 0)
    assert rc == 1
    msg = lib.fusedtok_last_error().decode()
    assert "allocation-free" in msg and "4194304" in msg
    rc = lib.fusedtok_attention_decode_launch_noalloc(7, 256, 256, 256, None, 256, 1, 8, 8, 64, 64, 0)
    assert rc == 1
