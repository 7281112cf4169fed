"""Benchmark configurations 3, 4 and 5 at their FULL sizes.

The CPU oracle cannot finish these in seconds, so each configuration is checked through properties that do
not depend on the size, plus the oracle on a stated subset of whole sequences (sequences are independent, so
a subset check is exact for the sequences it covers):
  * every checked sequence of the full-size launch against the oracle fed with that sequence's own cache rows;
  * the paged result against the contiguous kernel on the same rows gathered into a contiguous cache;
  * invariance under a permutation of the batch (another split of the work over the CTAs);
  * bit-identical repetition, and a clean device status word.
Tolerances: 2e-2 max-abs / 1e-2 mean-relative for bf16 and fp16 against the fp32-accumulated oracle on the
storage-rounded inputs (configuration 2 at full size is covered in test_decode_gpu.py).
"""

import numpy as np
import pytest
import torch

import cases
import oracle

from fusedtok_b200 import _fusedtok

pytestmark = pytest.mark.gpu

PAGE = 16


def _fill(shape, dt, gen):
    """Seeded N(0,1) in the storage type, generated in slabs to bound the fp32 temporaries."""
    t = torch.empty(shape, device="cuda", dtype=dt)
    flat = t.view(-1)
    step = 1 << 26
    for o in range(0, flat.numel(), step):
        n = min(step, flat.numel() - o)
        flat[o:o + n] = torch.randn(n, device="cuda", generator=gen).to(dt)
    return t


def _paged_launch(dt, q, kp, vp, tbl, lens, out, width):
    fn = _fusedtok.attention_decode_paged_launch_bf16 if dt is torch.bfloat16 else \
        _fusedtok.attention_decode_paged_launch_fp16
    b, hq, d = q.shape
    fn(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), tbl.data_ptr(), lens.data_ptr(), out.data_ptr(), b, hq,
       kp.shape[1], PAGE, width, d, torch.cuda.current_stream().cuda_stream)


def _seq_rows(pool, table_row, n):
    """Rows [0, n) of one sequence gathered from the pool: [Hkv, n, D] float32 on the host."""
    pages = (n + PAGE - 1) // PAGE
    blocks = pool[torch.from_numpy(table_row[:pages].astype(np.int64)).cuda()]      # [pages, Hkv, P, D]
    rows = blocks.permute(1, 0, 2, 3).reshape(pool.shape[1], pages * PAGE, pool.shape[3])[:, :n]
    return rows.float().cpu().numpy()


def _check_against_oracle(y, q, kp, vp, table, lens, picks):
    worst = 0.0
    for i in picks:
        n = int(lens[i])
        ref = oracle.decode(q[i:i + 1].float().cpu().numpy(), _seq_rows(kp, table[i], n)[None],
                            _seq_rows(vp, table[i], n)[None])
        got = y[i:i + 1].float().cpu().numpy()
        assert np.abs(got - ref).max() <= 2e-2, (i, n)
        assert np.abs(got - ref).mean() / np.abs(ref).mean() <= 1e-2, (i, n)
        worst = max(worst, float(np.abs(got - ref).max()))
    return worst


def _paged_config(lens, hq, dt, picks, seed=0):
    b = len(lens)
    table, nb, width = cases.paged_layout(lens)
    g = torch.Generator(device="cuda").manual_seed(seed)
    kp = _fill((nb, 8, PAGE, 128), dt, g)
    vp = _fill((nb, 8, PAGE, 128), dt, g)
    q = torch.randn(b, hq, 128, device="cuda", generator=g).to(dt)
    tbl, ln = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    out = torch.full_like(q, float("nan"))
    _paged_launch(dt, q, kp, vp, tbl, ln, out, width)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    _check_against_oracle(out, q, kp, vp, table, lens, picks)
    # repetition is bit-identical
    again = torch.empty_like(out)
    _paged_launch(dt, q, kp, vp, tbl, ln, again, width)
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    # a permuted batch is another split of the same work: same rows, same result within rounding of the
    # partial merges (fp32 partials, one rounding to the storage type at the end)
    perm = np.random.default_rng(5).permutation(b)
    pt = torch.from_numpy(perm).cuda()
    out_p = torch.empty_like(out)
    _paged_launch(dt, q[pt].contiguous(), kp, vp, tbl[pt].contiguous(), ln[pt].contiguous(), out_p, width)
    torch.cuda.synchronize()
    assert (out_p.float() - out[pt].float()).abs().max().item() <= 4e-3
    assert _fusedtok.attention_device_status() == 0
    return q, kp, vp, table, out


def test_config3_full_size_fp16_paged():
    """Batch 64, 32/8 heads, D=128, page 16, lengths uniform in [128, 8192] (271,311 rows), fp16: the shortest,
    the longest and six more sequences against the oracle; paged equals contiguous on the gathered rows."""
    lens = cases.config3_lens()
    assert lens.shape == (64,) and int(lens.sum()) == 271311
    picks = sorted({int(np.argmin(lens)), int(np.argmax(lens)), 0, 1, 17, 31, 45, 63})
    q, kp, vp, table, out = _paged_config(lens, 32, torch.float16, picks)
    # the same rows in a contiguous cache through the contiguous launcher
    t_max = int(lens.max())
    kc = torch.zeros(64, 8, t_max, 128, device="cuda", dtype=torch.float16)
    vc = torch.zeros_like(kc)
    for i in range(64):
        n = int(lens[i])
        pages = (n + PAGE - 1) // PAGE
        idx = torch.from_numpy(table[i, :pages].astype(np.int64)).cuda()
        kc[i, :, :n] = kp[idx].permute(1, 0, 2, 3).reshape(8, pages * PAGE, 128)[:, :n]
        vc[i, :, :n] = vp[idx].permute(1, 0, 2, 3).reshape(8, pages * PAGE, 128)[:, :n]
    out_c = torch.empty_like(out)
    ln = torch.from_numpy(lens).cuda()
    _fusedtok.attention_decode_launch_fp16(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ln.data_ptr(), out_c.data_ptr(),
                                           64, 32, 8, t_max, 128, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(out_c, out)               # same tiles, same split, same arithmetic: identical


def test_config5_full_size_bf16_paged_group5():
    """Batch 256, 40/8 heads (group 5), D=128, page 16, lengths log-uniform in [1024, 32768] (2,680,292 rows,
    10.98 GB of K/V), bf16: 16 sequences incl. the shortest and the longest against the oracle."""
    lens = cases.config5_lens()
    assert lens.shape == (256,) and int(lens.sum()) == 2680292
    order = np.argsort(lens)
    picks = sorted({int(order[0]), int(order[-1])} | {int(order[i]) for i in range(9, 256, 18)})[:16]
    _paged_config(lens, 40, torch.bfloat16, picks)


def test_config4_full_size_bf16_long_context():
    """Batch 4, 64/8 heads, D=128, 131,072 rows per sequence, bf16 (2.1 GB of K/V): one whole sequence against
    the oracle; the two halves of the KV length as raw (m, l, acc) partials merge to the full result (the
    multi-GPU split on one GPU); bit-identical repetition."""
    b, hq, hkv, t, d = 4, 64, 8, 131072, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(b, hq, d, device="cuda", generator=g).bfloat16()
    k = _fill((b, hkv, t, d), torch.bfloat16, g)
    v = _fill((b, hkv, t, d), torch.bfloat16, g)
    st = torch.cuda.current_stream().cuda_stream
    out = torch.full_like(q, float("nan"))
    _fusedtok.attention_decode_launch_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, out.data_ptr(), b, hq, hkv, t,
                                           d, st)
    again = torch.empty_like(out)
    _fusedtok.attention_decode_launch_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, again.data_ptr(), b, hq, hkv,
                                           t, d, st)
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    i = 2
    ref = oracle.decode(q[i:i + 1].float().cpu().numpy(), k[i:i + 1].float().cpu().numpy(),
                        v[i:i + 1].float().cpu().numpy())
    got = out[i:i + 1].float().cpu().numpy()
    assert np.abs(got - ref).max() <= 2e-2
    assert np.abs(got - ref).mean() / np.abs(ref).mean() <= 1e-2
    # KV-length split: rows [0, T/2) and [T/2, T) as two "ranks" on this GPU
    n = int(_fusedtok.attention_partial_floats(b, hq, d))
    parts = torch.empty(2, n, device="cuda", dtype=torch.float32)
    half = t // 2
    for r in range(2):
        kr = k[:, :, r * half:(r + 1) * half].contiguous()
        vr = v[:, :, r * half:(r + 1) * half].contiguous()
        _fusedtok.attention_decode_partial_launch(1, q.data_ptr(), kr.data_ptr(), vr.data_ptr(), 0,
                                                  parts[r].data_ptr(), b, hq, hkv, half, d, st)
        torch.cuda.synchronize()
        del kr, vr
    merged = torch.empty_like(out)
    _fusedtok.attention_merge_partials_launch(1, parts.data_ptr(), 2, merged.data_ptr(), b, hq, d, st)
    torch.cuda.synchronize()
    assert (merged.float() - out.float()).abs().max().item() <= 4e-3
    assert _fusedtok.attention_device_status() == 0
