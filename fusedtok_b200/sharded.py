"""Multi-GPU layer for one NVLink-connected box: one process per GPU,
``torch.distributed`` (NCCL) for the plumbing. The reference is single-GPU
(no counterpart); correctness is pinned by equality with the single-GPU
result.

Two ways to use several GPUs:

* **Batch x kv-head sharding, no communication.** Every (sequence, kv head)
  pair is an independent unit, so a rank just owns a slice of the batch
  (``batch_slice``) and/or a contiguous block of kv heads together with the
  query heads of their groups (``kv_head_slice``) and runs the ordinary
  operator on its slice. Outputs are disjoint; nothing is exchanged.

* **KV-length split for very long sequences** (``SplitKVDecoder``). Rank r
  holds cache rows ``[r*T/n, (r+1)*T/n)`` of every sequence. Each rank runs the
  split-KV kernel over its rows and emits one raw triple (m, l, acc[D]) per
  (sequence, query head) straight into its block of a gather buffer; one
  ``all_gather_into_tensor`` over NVLink (133 KB per rank at 4 x 64 heads x 128)
  puts the n blocks in every rank's HBM; the merge kernel folds them with the
  reference's log-sum-exp rule. All three steps are stream-ordered and can be
  captured in one CUDA graph.
  ``PeerSplitKVDecoder`` does the same exchange without a collective library:
  the split-KV kernel stores each rank's triple block straight into every
  peer's buffer (CUDA IPC mapping, plain stores over NVLink) and the merge
  kernel synchronises on per-step flags - two launches per step instead of
  three, and no collective latency.
"""

import torch

from . import _fusedtok

_DT_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def batch_slice(batch, world, rank):
    """Rows [lo, hi) of the batch owned by `rank`: sizes differ by at most one."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def kv_head_slice(q_heads, kv_heads, world, rank):
    """(kv_lo, kv_hi, q_lo, q_hi): a contiguous block of kv heads and the
    query heads of their GQA groups (heads of a group are contiguous:
    h -> h // (Hq // Hkv))."""
    if kv_heads % world:
        raise ValueError("kv heads must divide evenly over the ranks")
    group = q_heads // kv_heads
    per = kv_heads // world
    return rank * per, (rank + 1) * per, rank * per * group, (rank + 1) * per * group


def kv_row_slice(rows, world, rank):
    """Cache rows [lo, hi) held by `rank` under the KV-length split."""
    if rows % world:
        raise ValueError("cache rows must divide evenly over the ranks")
    per = rows // world
    return rank * per, (rank + 1) * per


def local_lens(lens, rows_per_rank, rank):
    """Valid rows of each sequence inside this rank's slice:
    clamp(len - rank * rows_per_rank, 0, rows_per_rank). Works on torch
    tensors (stays on the device, no readback) and numpy arrays."""
    shifted = lens - rank * rows_per_rank
    if torch.is_tensor(shifted):
        return shifted.clamp(0, rows_per_rank).to(torch.int32)
    return shifted.clip(0, rows_per_rank).astype("int32")


class SplitKVDecoder:
    """Decode attention with the cache rows of every sequence split across the
    ranks of `group`. Buffers are allocated once (fixed addresses, so a step
    can be captured and replayed as a CUDA graph)."""

    def __init__(self, batch, q_heads, kv_heads, dim, dtype, device, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.shape = (batch, q_heads, kv_heads, dim)
        self.dtype = dtype
        self.code = _DT_CODE[dtype]
        nf = _fusedtok.attention_partial_floats(batch, q_heads, dim)
        self.gathered = torch.empty(self.world, nf, device=device, dtype=torch.float32)
        self.mine = self.gathered[self.rank]

    def decode(self, q, k_local, v_local, lens_local, out):
        """q [B, Hq, D] (replicated), k_local / v_local [B, Hkv, T/n, D] (this
        rank's rows), lens_local [B] int32 device tensor from ``local_lens`` or
        None; writes out [B, Hq, D] on every rank."""
        b, hq, hkv, d = self.shape
        rows = k_local.shape[2]
        st = torch.cuda.current_stream().cuda_stream
        _fusedtok.attention_decode_partial_launch(
            self.code, q.data_ptr(), k_local.data_ptr(), v_local.data_ptr(),
            lens_local.data_ptr() if lens_local is not None else 0, self.mine.data_ptr(),
            b, hq, hkv, rows, d, st)
        self.dist.all_gather_into_tensor(self.gathered.view(-1), self.mine, group=self.group)
        _fusedtok.attention_merge_partials_launch(self.code, self.gathered.data_ptr(), self.world,
                                                  out.data_ptr(), b, hq, d, st)
        return out


class PeerSplitKVDecoder:
    """KV-length split with the exchange done by the library's own kernels over
    peer memory. Construction is collective (it swaps IPC handles through
    ``torch.distributed``); every rank must then call ``decode`` the same number
    of times with the same shapes."""

    def __init__(self, batch, q_heads, kv_heads, dim, dtype, device, group=None):
        import torch.distributed as dist
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.shape = (batch, q_heads, kv_heads, dim)
        self.code = _DT_CODE[dtype]
        with torch.cuda.device(device):
            self.mine, self.bytes = _fusedtok.exchange_alloc(self.world, batch, q_heads, dim)
            handle = _fusedtok.exchange_export(self.mine)
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            self.buffers = [self.mine if r == self.rank else _fusedtok.exchange_open(handles[r])
                            for r in range(self.world)]
        dist.barrier(group)           # every rank has mapped every buffer before anyone writes

    def decode(self, q, k_local, v_local, lens_local, out):
        b, hq, hkv, d = self.shape
        _fusedtok.attention_decode_exchange_launch(
            self.code, q.data_ptr(), k_local.data_ptr(), v_local.data_ptr(),
            lens_local.data_ptr() if lens_local is not None else 0, out.data_ptr(), self.buffers,
            self.rank, b, hq, hkv, k_local.shape[2], d, torch.cuda.current_stream().cuda_stream)
        return out

    def close(self):
        """Unmap the peers' buffers and free this rank's (after a device sync on every rank)."""
        for r, ptr in enumerate(self.buffers):
            if r != self.rank:
                _fusedtok.exchange_close(ptr)
        _fusedtok.exchange_free(self.mine)
        self.buffers = []
