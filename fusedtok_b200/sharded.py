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
  ``PeerSplitKVDecoder`` does the same exchange without a collective library and
  in ONE launch per step: the split-KV kernel stores the rows of every unit it
  finishes straight into every peer's buffer (CUDA IPC mapping, plain stores over
  NVLink), raises a per-unit flag there, and at its end folds its share of the
  rows over the n ranks - no second kernel, no collective latency.

Both decoders check on construction that every rank of the group was given the
same shapes (a collective of a few bytes), and on every call that the tensors
match what the decoder was built for - mistakes surface as ``ValueError`` /
``TypeError`` on the host before anything is launched. ``FUSEDTOK_NVTX=1`` in
the environment wraps the partial / exchange / merge steps in NVTX ranges.
"""

import contextlib
import os

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


_NVTX = os.environ.get("FUSEDTOK_NVTX") == "1"


@contextlib.contextmanager
def _range(name):
    """NVTX range around one step of the split (only with FUSEDTOK_NVTX=1)."""
    if _NVTX:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if _NVTX:
            torch.cuda.nvtx.range_pop()


def agree_across_ranks(dist, group, label, value):
    """Collective: every rank contributes `value`; raises ValueError on EVERY rank if they differ. Used for
    the things a KV-length split silently depends on (shapes, dtype, number of ranks expected)."""
    seen = [None] * dist.get_world_size(group)
    dist.all_gather_object(seen, value, group=group)
    if any(v != seen[0] for v in seen):
        raise ValueError(f"the ranks of the group disagree on {label}: {seen}")
    return seen[0]


class _SplitBase:
    """What the two KV-length-split decoders share: the shape contract and its checks."""

    def __init__(self, batch, q_heads, kv_heads, dim, dtype, device, group, world):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if world is not None and world != self.world:
            raise ValueError(f"built for {world} ranks but the process group has {self.world}")
        if dtype not in _DT_CODE:
            raise TypeError(f"dtype {dtype} is not float32, bfloat16 or float16")
        if batch < 0 or q_heads < 1 or kv_heads < 1 or q_heads % kv_heads or dim < 4 or dim % 4 or dim > 512:
            raise ValueError(f"bad attention shape: batch {batch}, heads {q_heads}/{kv_heads}, dim {dim}")
        self.shape = (batch, q_heads, kv_heads, dim)
        self.dtype = dtype
        self.device = torch.device(device)
        self.code = _DT_CODE[dtype]
        agree_across_ranks(dist, group, "batch, heads, dim and dtype", (self.shape, str(dtype)))

    def _check_call(self, q, k_local, v_local, lens_local, out):
        """Everything a rank can check about its own tensors before launching."""
        b, hq, hkv, d = self.shape
        for name, t in (("q", q), ("k_local", k_local), ("v_local", v_local), ("out", out)):
            if not torch.is_tensor(t) or t.device != self.device:
                raise TypeError(f"{name} must be a tensor on {self.device}")
            if t.dtype != self.dtype:
                raise TypeError(f"{name} has dtype {t.dtype}, the decoder was built for {self.dtype}")
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        if tuple(q.shape) != (b, hq, d) or out.shape != q.shape:
            raise ValueError(f"q / out must be {(b, hq, d)}, got {tuple(q.shape)} / {tuple(out.shape)}")
        if k_local.ndim != 4 or tuple(k_local.shape[:2]) != (b, hkv) or k_local.shape[3] != d \
                or v_local.shape != k_local.shape:
            raise ValueError(f"k_local / v_local must be [{b}, {hkv}, rows, {d}], got {tuple(k_local.shape)} / "
                             f"{tuple(v_local.shape)}")
        if lens_local is not None:
            if not torch.is_tensor(lens_local) or lens_local.device != self.device \
                    or lens_local.dtype != torch.int32 or tuple(lens_local.shape) != (b,):
                raise ValueError(f"lens_local must be an int32 tensor of {b} entries on {self.device} "
                                 "(see local_lens)")
        return k_local.shape[2]


class SplitKVDecoder(_SplitBase):
    """Decode attention with the cache rows of every sequence split across the
    ranks of `group`, exchanged with an NCCL all-gather. Buffers are allocated
    once (fixed addresses, so a step can be captured and replayed as a CUDA
    graph). Construction is collective."""

    def __init__(self, batch, q_heads, kv_heads, dim, dtype, device, group=None, world=None):
        super().__init__(batch, q_heads, kv_heads, dim, dtype, device, group, world)
        nf = _fusedtok.attention_partial_floats(batch, q_heads, dim)
        self.gathered = torch.empty(self.world, nf, device=device, dtype=torch.float32)
        self.mine = self.gathered[self.rank]

    def decode(self, q, k_local, v_local, lens_local, out):
        """q [B, Hq, D] (replicated), k_local / v_local [B, Hkv, T/n, D] (this
        rank's rows), lens_local [B] int32 device tensor from ``local_lens`` or
        None; writes out [B, Hq, D] on every rank."""
        b, hq, hkv, d = self.shape
        rows = self._check_call(q, k_local, v_local, lens_local, out)
        st = torch.cuda.current_stream().cuda_stream
        with _range("fusedtok.kv_split.partial"):
            _fusedtok.attention_decode_partial_launch(
                self.code, q.data_ptr(), k_local.data_ptr(), v_local.data_ptr(),
                lens_local.data_ptr() if lens_local is not None else 0, self.mine.data_ptr(),
                b, hq, hkv, rows, d, st)
        with _range("fusedtok.kv_split.all_gather"):
            self.dist.all_gather_into_tensor(self.gathered.view(-1), self.mine, group=self.group)
        with _range("fusedtok.kv_split.merge"):
            _fusedtok.attention_merge_partials_launch(self.code, self.gathered.data_ptr(), self.world,
                                                      out.data_ptr(), b, hq, d, st)
        return out


class PeerSplitKVDecoder(_SplitBase):
    """KV-length split with the exchange done by the library's own kernel over
    peer memory, one launch per step. Construction is collective (it swaps IPC
    handles through ``torch.distributed``); every rank must then call ``decode``
    the same number of times with the same shapes (the number of cache rows per
    rank is checked across the ranks on the first call and whenever it changes)."""

    def __init__(self, batch, q_heads, kv_heads, dim, dtype, device, group=None, world=None):
        super().__init__(batch, q_heads, kv_heads, dim, dtype, device, group, world)
        if self.world > 16:
            raise ValueError("the peer exchange serves at most 16 ranks")
        self._rows_agreed = None
        with torch.cuda.device(device):
            self.mine, self.bytes = _fusedtok.exchange_alloc(self.world, batch, q_heads, dim)
            handle = _fusedtok.exchange_export(self.mine)
            handles = [None] * self.world
            self.dist.all_gather_object(handles, handle, group=group)
            self.buffers = [self.mine if r == self.rank else _fusedtok.exchange_open(handles[r])
                            for r in range(self.world)]
        self.dist.barrier(group)      # every rank has mapped every buffer before anyone writes

    def decode(self, q, k_local, v_local, lens_local, out):
        b, hq, hkv, d = self.shape
        rows = self._check_call(q, k_local, v_local, lens_local, out)
        if rows < 1:
            raise ValueError("the peer exchange needs at least one cache row per rank")
        if rows != self._rows_agreed and not torch.cuda.is_current_stream_capturing():
            # a rank that ran a different number of rows would still exchange valid triples, but a rank
            # that skipped the call would leave the others waiting: agree before the first launch
            agree_across_ranks(self.dist, self.group, "cache rows per rank", rows)
            self._rows_agreed = rows
        with _range("fusedtok.kv_split.partial+exchange+merge"):
            _fusedtok.attention_decode_exchange_launch(
                self.code, q.data_ptr(), k_local.data_ptr(), v_local.data_ptr(),
                lens_local.data_ptr() if lens_local is not None else 0, out.data_ptr(), self.buffers,
                self.rank, b, hq, hkv, rows, d, torch.cuda.current_stream().cuda_stream)
        return out

    def close(self):
        """Unmap the peers' buffers and free this rank's (after a device sync on every rank)."""
        for r, ptr in enumerate(self.buffers):
            if r != self.rank:
                _fusedtok.exchange_close(ptr)
        _fusedtok.exchange_free(self.mine)
        self.buffers = []
