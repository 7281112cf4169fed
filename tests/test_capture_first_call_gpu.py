"""A decode call whose workspace does not exist yet, made while the stream is being captured: the library
allocates nothing and launches the workspace-free form (generic kernel, one CTA per unit), as the reference
does (src/attention.cu:1498-1509). Runs in a fresh process so that the call really is the first one."""

import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import sys
    import numpy as np
    import torch
    sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
    import oracle
    import fusedtok_b200 as ft
    from fusedtok_b200 import _fusedtok

    kind = sys.argv[1]
    dt = dict(f32=torch.float32, bf16=torch.bfloat16, fp16=torch.float16)[sys.argv[2]]
    tol = dict(f32=1e-5, bf16=2e-2, fp16=2e-3)[sys.argv[2]]
    rng = np.random.default_rng(11)
    b, hq, hkv, t, d = 5, 16, 4, 1500, 128
    lens = np.array([t, 0, 1, 700, 64], np.int32)
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    qt, kt, vt = (torch.from_numpy(x).cuda().to(dt) for x in (q, k, v))
    qr, kr, vr = (x.float().cpu().numpy() for x in (qt, kt, vt))
    lt = torch.from_numpy(lens).cuda()
    free0 = torch.cuda.mem_get_info()[0]
    if kind == "paged":
        page = 16
        width = (t + page - 1) // page
        nb = b * width + 3
        perm = rng.permutation(nb)[:b * width].reshape(b, width).astype(np.int32)
        kp = torch.zeros(nb, hkv, page, d, device="cuda", dtype=dt)
        vp = torch.zeros(nb, hkv, page, d, device="cuda", dtype=dt)
        pad = width * page - t
        kpad = torch.nn.functional.pad(kt, (0, 0, 0, pad)).view(b, hkv, width, page, d)
        vpad = torch.nn.functional.pad(vt, (0, 0, 0, pad)).view(b, hkv, width, page, d)
        tbl = torch.from_numpy(perm).cuda()
        kp[tbl.long()] = kpad.permute(0, 2, 1, 3, 4)
        vp[tbl.long()] = vpad.permute(0, 2, 1, 3, 4)
        call = lambda: ft.attention_decode_paged(qt, kp, vp, tbl, lt)
    else:
        call = lambda: ft.attention_decode(qt, kt, vt, lt)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            out = call()                                   # the library's first call of this process
    graph.replay()
    torch.cuda.synchronize()
    ref = oracle.decode(qr, kr, vr, lens)
    y = out.float().cpu().numpy()
    assert np.abs(y - ref).max() <= tol, np.abs(y - ref).max()
    assert np.all(y[1] == 0)
    first = out.clone()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, first)
    # afterwards, outside a capture, the ordinary path sets its workspace up and agrees within the tolerance
    y2 = call().float().cpu().numpy()
    assert np.abs(y2 - ref).max() <= tol
    assert np.abs(y2 - y).max() <= 2 * tol
    assert _fusedtok.attention_device_status() == 0
    print("ok")
""")


@pytest.mark.parametrize("kind", ["contiguous", "paged"])
@pytest.mark.parametrize("dtype", ["f32", "bf16", "fp16"])
def test_first_call_inside_a_capture_needs_no_workspace(kind, dtype, tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT, tests=os.path.join(ROOT, "tests")))
    r = subprocess.run([sys.executable, str(script), kind, dtype], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-4000:]
