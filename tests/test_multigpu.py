"""Multi-GPU layer on real GPUs (needs >= 2 devices, skipped otherwise): the
KV-length split must give the single-GPU result, including a short sequence
whose rows all live on rank 0 and an empty sequence, both through NCCL (partial
kernel -> all-gather of raw triples -> merge kernel) and through the library's
own exchange (one kernel per rank: rows stored into every peer's buffer, flagged
per unit, folded at the end of the same kernel), which must match the NCCL path
bit for bit - on the tensor-core kernel (bf16), on the CUDA-core kernel (fp32),
over many steps and when replayed as a CUDA graph; batch sharding is a pure
concatenation. One process per GPU, NCCL without NVLS (plain ring/tree), as
child processes."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worker(rank, world, port, out_dir):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import cases
    import fusedtok_b200 as ft
    from fusedtok_b200 import sharded
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        rng = np.random.default_rng(11)                       # same inputs on every rank
        b, hq, hkv, t, d = 3, 16, 4, 4096, 128
        q, k, v, _ = cases.make_case(rng, b, hq, hkv, t, d, False)
        lens = np.array([4096, 900, 0], np.int32)
        qt, kt, vt = (torch.from_numpy(x).to(dev).to(torch.bfloat16) for x in (q, k, v))
        lens_t = torch.from_numpy(lens).to(dev)
        full = ft.attention_decode(qt, kt, vt, lens_t)        # single-GPU reference on this rank
        per = t // world
        lo, hi = sharded.kv_row_slice(t, world, rank)
        k_loc = kt[:, :, lo:hi].contiguous()
        v_loc = vt[:, :, lo:hi].contiguous()
        dec = sharded.SplitKVDecoder(b, hq, hkv, d, torch.bfloat16, dev, dist.group.WORLD)
        out = torch.empty_like(qt)
        for _ in range(2):                                    # twice: buffers are reused
            dec.decode(qt, k_loc, v_loc, sharded.local_lens(lens_t, per, rank), out)
        torch.cuda.synchronize()
        err = (out.float() - full.float()).abs().max().item()
        assert err <= 4e-3, err
        assert torch.count_nonzero(out[2]) == 0
        # the same split with the library's own peer exchange: same result as the NCCL path
        from fusedtok_b200 import _fusedtok
        peer = sharded.PeerSplitKVDecoder(b, hq, hkv, d, torch.bfloat16, dev, dist.group.WORLD)
        out2 = torch.full_like(qt, float("nan"))
        for step in range(5):                                 # several steps: both buffer parities, flags reused
            qs = (qt.float() * (1.0 + 0.1 * step)).to(torch.bfloat16)
            dec.decode(qs, k_loc, v_loc, sharded.local_lens(lens_t, per, rank), out)
            peer.decode(qs, k_loc, v_loc, sharded.local_lens(lens_t, per, rank), out2)
            torch.cuda.synchronize()
            assert torch.equal(out, out2), (out.float() - out2.float()).abs().max().item()
        assert _fusedtok.attention_device_status() == 0
        # the same step captured once and replayed: the step number lives in the exchange buffer
        graph = torch.cuda.CUDAGraph()
        ll = sharded.local_lens(lens_t, per, rank)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            peer.decode(qt, k_loc, v_loc, ll, out2)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.graph(graph):
            peer.decode(qt, k_loc, v_loc, ll, out2)
        dec.decode(qt, k_loc, v_loc, ll, out)
        for _ in range(4):
            out2.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, out2)
        assert _fusedtok.attention_device_status() == 0
        dist.barrier()
        peer.close()
        # float32 on the CUDA-core kernel (two CTAs per SM), group 5 (chunks of 4 + 1 heads), ragged
        b3, hq3, hkv3, t3, d3 = 4, 10, 2, 2048, 64
        q3, k3, v3, _ = cases.make_case(np.random.default_rng(12), b3, hq3, hkv3, t3, d3, False)
        lens3 = torch.tensor([2048, 0, 1025, 7], dtype=torch.int32, device=dev)
        q3t, k3t, v3t = (torch.from_numpy(x).to(dev) for x in (q3, k3, v3))
        full3 = ft.attention_decode(q3t, k3t, v3t, lens3)
        per3 = t3 // world
        lo3, hi3 = sharded.kv_row_slice(t3, world, rank)
        k3l, v3l = k3t[:, :, lo3:hi3].contiguous(), v3t[:, :, lo3:hi3].contiguous()
        dec3 = sharded.SplitKVDecoder(b3, hq3, hkv3, d3, torch.float32, dev, dist.group.WORLD)
        peer3 = sharded.PeerSplitKVDecoder(b3, hq3, hkv3, d3, torch.float32, dev, dist.group.WORLD)
        o3a, o3b = torch.empty_like(q3t), torch.full_like(q3t, float("nan"))
        for _ in range(3):
            dec3.decode(q3t, k3l, v3l, sharded.local_lens(lens3, per3, rank), o3a)
            peer3.decode(q3t, k3l, v3l, sharded.local_lens(lens3, per3, rank), o3b)
            torch.cuda.synchronize()
            assert torch.equal(o3a, o3b)
        assert (o3a - full3).abs().max().item() <= 1e-5
        assert torch.count_nonzero(o3a[1]) == 0
        assert _fusedtok.attention_device_status() == 0
        dist.barrier()
        peer3.close()
        # batch sharding: each rank decodes its rows; concatenation equals the full result
        blo, bhi = sharded.batch_slice(b, world, rank)
        mine = ft.attention_decode(qt[blo:bhi].contiguous(), kt[blo:bhi].contiguous(), vt[blo:bhi].contiguous(),
                                   lens_t[blo:bhi].contiguous()) if bhi > blo else qt[:0]
        assert (mine.float() - full[blo:bhi].float()).abs().max().item() <= 4e-3 if bhi > blo else True
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("%g" % err)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(NGPU < 2, reason="needs at least 2 GPUs")
def test_kv_length_split_matches_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert os.path.exists(str(tmp_path / ("ok%d" % r)))
