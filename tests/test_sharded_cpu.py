"""Host-side logic of the multi-GPU layer, on CPU: partition functions cover
every unit exactly once, and the KV-length split algebra survives a real
collective - two gloo ranks each produce the raw (m, l, acc) triples of their
slice of the cache rows (computed by the CPU oracle, standing in for the CUDA
partial kernel, which needs a GPU), all-gather them in the library's block
layout and merge: the result equals the unsharded decode, including a short
sequence whose rows all live on rank 0 (rank 1's shard is empty) and an empty
sequence."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
import oracle
from fusedtok_b200 import sharded
from fusedtok_b200 import _fusedtok


def test_batch_slices_partition_the_batch():
    for batch in (0, 1, 7, 32, 257):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                lo, hi = sharded.batch_slice(batch, world, r)
                assert 0 <= lo <= hi <= batch
                seen.extend(range(lo, hi))
            assert seen == list(range(batch))
            sizes = [b - a for a, b in (sharded.batch_slice(batch, world, r) for r in range(world))]
            assert max(sizes) - min(sizes) <= 1


def test_kv_head_slices_keep_gqa_groups_together():
    hq, hkv = 40, 8
    group = hq // hkv
    for world in (1, 2, 4, 8):
        q_seen = []
        for r in range(world):
            kv_lo, kv_hi, q_lo, q_hi = sharded.kv_head_slice(hq, hkv, world, r)
            for h in range(q_lo, q_hi):
                assert kv_lo <= h // group < kv_hi       # every query head finds its kv head locally
            q_seen.extend(range(q_lo, q_hi))
        assert q_seen == list(range(hq))
    with pytest.raises(ValueError):
        sharded.kv_head_slice(40, 8, 3, 0)


def test_local_lens_cover_every_row_once():
    lens = np.array([0, 1, 511, 512, 513, 2048, 1300], np.int64)
    world, rows = 4, 2048
    per = rows // world
    total = np.zeros_like(lens)
    for r in range(world):
        lo, hi = sharded.kv_row_slice(rows, world, r)
        assert (lo, hi) == (r * per, (r + 1) * per)
        ll = sharded.local_lens(lens, per, r)
        assert ll.min() >= 0 and ll.max() <= per
        total += ll
        lt = sharded.local_lens(torch.from_numpy(lens), per, r)
        np.testing.assert_array_equal(lt.numpy(), ll)
    np.testing.assert_array_equal(total, lens)
    with pytest.raises(ValueError):
        sharded.kv_row_slice(10, 3, 0)


def _rank_main(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)                 # same inputs on every rank
        b, hq, hkv, t, d = 3, 8, 2, 256, 32
        q, k, v, _ = cases.make_case(rng, b, hq, hkv, t, d, False)
        lens = np.array([256, 100, 0], np.int64)       # 100 rows: rank 1's shard is empty; 0: empty sequence
        per = t // world
        lo, hi = sharded.kv_row_slice(t, world, rank)
        ll = sharded.local_lens(lens, per, rank)
        rows = b * hq
        nf = _fusedtok.attention_partial_floats(b, hq, d)
        acc_off = nf - rows * d
        mine = np.zeros(nf, np.float32)
        group = hq // hkv
        for bi in range(b):
            for h in range(hq):
                kv = h // group
                m, l, a = oracle.partial(q[bi, h], k[bi, kv, lo:hi], v[bi, kv, lo:hi], 0, int(ll[bi]))
                r = bi * hq + h
                mine[2 * r], mine[2 * r + 1] = m, l
                mine[acc_off + r * d: acc_off + (r + 1) * d] = a
        gathered = torch.empty(world * nf, dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, torch.from_numpy(mine))
        g = gathered.numpy().reshape(world, nf)
        out = np.zeros((b, hq, d), np.float32)
        for r in range(rows):
            ml = np.stack([g[s, 2 * r: 2 * r + 2] for s in range(world)])
            acc = np.stack([g[s, acc_off + r * d: acc_off + (r + 1) * d] for s in range(world)])
            out[r // hq, r % hq] = oracle.merge(ml, acc)
        ref = oracle.decode(q, k, v, lens.astype(np.int32))
        np.testing.assert_allclose(out, ref, rtol=2e-5, atol=2e-6)
        assert np.all(out[2] == 0)
        if rank == 0:
            np.save(out_path, out)
    finally:
        dist.destroy_process_group()


def test_kv_length_split_over_two_gloo_ranks(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "merged.npy")
    mp.spawn(_rank_main, args=(2, port, out_path), nprocs=2, join=True)
    assert os.path.exists(out_path)


# ---- host-side failure handling of the split decoders: every mistake is caught before any launch ----------

def _disagreeing_rank(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        notes = []
        # ranks that were given different shapes: both learn of it, as a ValueError, in the constructor
        try:
            sharded._SplitBase(3 + rank, 8, 2, 32, torch.float32, "cpu", None, None)
            notes.append("no error")
        except ValueError as exc:
            notes.append("shape:" + ("disagree" in str(exc) and "ok" or str(exc)))
        # ... and ranks that were given different dtypes
        try:
            sharded._SplitBase(3, 8, 2, 32, torch.float32 if rank == 0 else torch.float16, "cpu", None, None)
            notes.append("no error")
        except ValueError as exc:
            notes.append("dtype:" + ("disagree" in str(exc) and "ok" or str(exc)))
        # a decoder built for another number of ranks than the group has
        try:
            sharded._SplitBase(3, 8, 2, 32, torch.float32, "cpu", None, world + 1)
            notes.append("no error")
        except ValueError as exc:
            notes.append("world:" + ("process group has" in str(exc) and "ok" or str(exc)))
        # agreement passes when the ranks do agree; per-call checks are local
        base = sharded._SplitBase(3, 8, 2, 32, torch.float32, "cpu", None, world)
        q = torch.zeros(3, 8, 32)
        k = torch.zeros(3, 2, 64, 32)
        assert base._check_call(q, k, k.clone(), None, torch.empty_like(q)) == 64
        assert base._check_call(q, k, k.clone(), torch.zeros(3, dtype=torch.int32), torch.empty_like(q)) == 64
        bad_calls = [
            (TypeError, (q.half(), k, k.clone(), None, torch.empty_like(q))),                  # dtype
            (ValueError, (q[:2], k, k.clone(), None, torch.empty_like(q[:2]))),                # batch
            (ValueError, (q, k[:, :1], k[:, :1].clone(), None, torch.empty_like(q))),          # kv heads
            (ValueError, (q, k, k[:, :, :32].clone(), None, torch.empty_like(q))),             # v rows
            (ValueError, (q, k.transpose(1, 2), k.clone(), None, torch.empty_like(q))),        # not contiguous
            (ValueError, (q, k, k.clone(), torch.zeros(3, dtype=torch.int64), torch.empty_like(q))),   # lens type
            (ValueError, (q, k, k.clone(), torch.zeros(2, dtype=torch.int32), torch.empty_like(q))),   # lens size
            (TypeError, (q.numpy(), k, k.clone(), None, torch.empty_like(q))),                 # not a tensor
        ]
        for kind, args in bad_calls:
            with pytest.raises(kind):
                base._check_call(*args)
        notes.append("calls:ok")
        # ranks that would run different numbers of cache rows
        try:
            sharded.agree_across_ranks(dist, None, "cache rows per rank", 64 + rank)
            notes.append("no error")
        except ValueError as exc:
            notes.append("rows:" + ("cache rows" in str(exc) and "ok" or str(exc)))
        open(os.path.join(out_dir, "notes%d" % rank), "w").write(",".join(notes))
    finally:
        dist.destroy_process_group()


def test_split_decoders_refuse_inconsistent_ranks_before_any_launch(tmp_path):
    """Two gloo ranks on CPU: shape, dtype and rank-count disagreement and every per-call mistake raise on the
    host (no GPU, no fault, nothing launched)."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_disagreeing_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        notes = open(str(tmp_path / ("notes%d" % r))).read()
        assert notes == "shape:ok,dtype:ok,world:ok,calls:ok,rows:ok", notes
