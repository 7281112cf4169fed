"""The self-checking build of the library (compiled with -DFTK_BOUNDS, beside the product:
``python fusedtok_b200/_build.py -DFTK_BOUNDS --out fusedtok_b200/libfusedtok_b200_bounds.so``) stands in for a
memory checker: every cache row, partial slot and arrival counter the decode kernels compute is compared with what
the launch owns. Across the kernels and front ends the status word must stay 0 and the results must match the
oracle; a block table that points outside the pool must be reported as status 8 - and is not followed, so nothing
faults. Skipped where the variant has not been built. Each case runs in a fresh process that loads the variant
through FUSEDTOK_B200_LIB."""

import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
VARIANT = os.path.join(ROOT, "fusedtok_b200", "libfusedtok_b200_bounds.so")

CHILD = textwrap.dedent("""
    import sys
    import numpy as np
    import torch
    sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
    import oracle
    import fusedtok_b200 as ft
    from fusedtok_b200 import _fusedtok

    mode = sys.argv[1]
    rng = np.random.default_rng(5)

    def paged_case(dt, b, hq, hkv, t, d, page, bad=False):
        lens = rng.integers(1, t + 1, b).astype(np.int32)
        lens[0] = t
        width = (t + page - 1) // page
        nb = b * width + 4
        q = rng.standard_normal((b, hq, d)).astype(np.float32)
        kp = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
        vp = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
        tbl = rng.permutation(nb)[:b * width].reshape(b, width).astype(np.int32)
        if bad:
            tbl[1, 0] = nb + 3                      # outside the pool: the product build would read foreign memory
        qt, kpt, vpt = (torch.from_numpy(x).cuda().to(dt) for x in (q, kp, vp))
        tblt, lt = torch.from_numpy(tbl).cuda(), torch.from_numpy(lens).cuda()
        _fusedtok._lib.fusedtok_debug_set_pool_blocks(nb)
        out = torch.empty_like(qt)
        sfx = {{torch.float32: "", torch.bfloat16: "_bf16", torch.float16: "_fp16"}}[dt]
        getattr(_fusedtok, "attention_decode_paged_launch" + sfx)(
            qt.data_ptr(), kpt.data_ptr(), vpt.data_ptr(), tblt.data_ptr(), lt.data_ptr(), out.data_ptr(),
            b, hq, hkv, page, width, d, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        _fusedtok._lib.fusedtok_debug_set_pool_blocks(0)
        if bad:
            return None
        safe = np.minimum(tbl, nb - 1)
        kc = kpt.float().cpu().numpy()[safe].transpose(0, 2, 1, 3, 4).reshape(b, hkv, width * page, d)
        vc = vpt.float().cpu().numpy()[safe].transpose(0, 2, 1, 3, 4).reshape(b, hkv, width * page, d)
        ref = oracle.decode(qt.float().cpu().numpy(), np.ascontiguousarray(kc), np.ascontiguousarray(vc), lens)
        return float(np.abs(out.float().cpu().numpy() - ref).max())

    def contiguous_case(dt, b, hq, hkv, t, d):
        lens = rng.integers(0, t + 1, b).astype(np.int32)
        lens[0] = t
        q = rng.standard_normal((b, hq, d)).astype(np.float32)
        k = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
        v = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
        qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
        lt = torch.from_numpy(lens).cuda()
        errs = []
        for lens_arg, lens_np in ((lt, lens), (None, None)):
            out = ft.attention_decode(qt, kt, vt, lens_arg)
            ref = oracle.decode(*(x.float().cpu().numpy() for x in (qt, kt, vt)), lens_np)
            errs.append(float(np.abs(out.float().cpu().numpy() - ref).max()))
        return max(errs)

    tol = {{torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-3}}
    if mode == "clean":
        for dt in (torch.bfloat16, torch.float16, torch.float32):
            # tensor-core / float32 ring kernels (split units, many ranges per unit), generic kernel (odd head dim)
            for shape in ((3, 16, 4, 3000, 128), (1, 8, 2, 20000, 128), (2, 8, 8, 700, 64), (2, 6, 2, 900, 48)):
                e = contiguous_case(dt, *shape)
                assert e <= tol[dt], (dt, shape, e)
            for page in (8, 16, 64, 5):                       # page 5: generic kernel
                e = paged_case(dt, 3, 16, 4, 2000, 128, page)
                assert e <= tol[dt], (dt, page, e)
            assert _fusedtok.attention_device_status() == 0, dt
    else:
        for dt, page in ((torch.bfloat16, 16), (torch.float32, 16), (torch.float16, 5)):
            paged_case(dt, 3, 16, 4, 2000, 128, page, bad=True)
            assert _fusedtok.attention_device_status() == 8, (dt, page)
            assert _fusedtok.attention_device_status() == 0          # reading cleared it
        e = paged_case(torch.bfloat16, 3, 16, 4, 2000, 128, 16)      # and the library is fine afterwards
        assert e <= 2e-2
        assert _fusedtok.attention_device_status() == 0
    print("ok")
""")


@pytest.mark.skipif(not os.path.exists(VARIANT), reason="self-checking variant of the library not built")
@pytest.mark.parametrize("mode", ["clean", "table_entry_outside_the_pool"])
def test_self_checking_build(mode, tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT, tests=os.path.join(ROOT, "tests")))
    env = dict(os.environ, FUSEDTOK_B200_LIB=VARIANT)
    r = subprocess.run([sys.executable, str(script), mode], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-4000:]
