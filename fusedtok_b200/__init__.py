"""fusedtok_b200 - fusedtok's decode-attention operators on B200 (sm_100a).

The operators keep the call contract of fusedtok's Python surface for this
path (reference: python/fusedtok/__init__.py:710-788 ``attention_decode``,
:849-940 ``attention_decode_paged``, :791-846 ``attention_prefill``,
:943-1112 ``kv_append*``, :645-702 ``rope``): argument order, accepted types,
which mistake raises ``TypeError`` and which ``ValueError``, host index values
validated while device index tensors are trusted, zero-copy and stream-ordered
on CUDA tensors, capturable in a CUDA graph. The code behind the contract is
this package's own: a CUDA library (``csrc/``) reached through a C ABI
(``include/fusedtok_b200.h``).

Every operator has two routes:

* **device route** - the first operand is a CUDA tensor: all operands are
  gathered in a :class:`_DeviceCall`, checked, and the matching launcher runs on
  the current stream of the operands' device;
* **staged route** - host arrays with ``cuda=True``: values are converted to
  float32, copied to the GPU, computed there and copied back.

There is no CPU implementation. Host arrays without ``cuda=True`` (which the
reference computes on the CPU) are validated like any other call and then
raise :class:`NoHostPathError`, a ``RuntimeError``.
"""

import numpy as np

from . import _fusedtok

try:
    import torch
except ImportError:  # pragma: no cover - torch is optional for the staged route
    torch = None

__version__ = "0.2.0"
__all__ = ["attention_decode", "attention_decode_paged", "attention_prefill", "kv_append", "kv_append_paged",
           "rope", "rope_kv_append", "rope_kv_append_paged", "cuda_available", "NoHostPathError"]


class NoHostPathError(RuntimeError):
    """Host inputs were given without ``cuda=True``: this library computes on the GPU only."""


def cuda_available():
    """True if a usable CUDA device is present."""
    return _fusedtok.cuda_available()


# ---------------------------------------------------------------------------
# storage types and launcher lookup
# ---------------------------------------------------------------------------

# storage dtype -> (suffix of the launcher name, dtype code of the C ABI)
_STORAGE = {} if torch is None else {
    torch.float32: ("", 0),
    torch.bfloat16: ("_bf16", 1),
    torch.float16: ("_fp16", 2),
}
_launchers = {}          # (family name, dtype) -> bound launcher, filled on first use


def _launcher(family, dtype):
    fn = _launchers.get((family, dtype))
    if fn is None:
        fn = _launchers[(family, dtype)] = getattr(_fusedtok, family + _STORAGE[dtype][0])
    return fn


_raw_stream = getattr(getattr(torch, "_C", None), "_cuda_getCurrentRawStream", None)


_Tensor = torch.Tensor if torch is not None else ()


def _on_gpu(x):
    return isinstance(x, _Tensor) and x.is_cuda


def _gqa_heads(hq, hkv, paged=False):
    """The head-count rules every attention operator shares."""
    if hq < 1 or hkv < 1:
        raise ValueError(f"head counts must be positive (got {hq} query / {hkv} kv heads)")
    if hq % hkv:
        raise ValueError(f"{hq} query heads do not divide into {hkv} kv-head groups")
    if paged and hq // hkv not in (1, 2, 4, 8, 16):
        raise ValueError(f"the paged operator takes GQA groups of 1, 2, 4, 8 or 16 query heads, not {hq // hkv}; "
                         "attention_decode has no such limit")


# ---------------------------------------------------------------------------
# index operands (lens, block tables)
# ---------------------------------------------------------------------------

def _host_index(label, values, shape, stop, closed):
    """Validate index values that live on the host and return them as a C-contiguous int32 array.

    ``shape`` is the expected shape with ``None`` for a free dimension; valid values are ``0 <= v < stop``
    (``<= stop`` when ``closed``). Returns ``None`` for a CUDA tensor: device values are trusted and never
    read back, which is what keeps a call capturable. Wrong element type -> TypeError; wrong shape or an
    out-of-range value -> ValueError."""
    if _on_gpu(values):
        return None
    raw = values.detach().numpy() if (torch is not None and torch.is_tensor(values)) else np.asarray(values)
    if raw.size and raw.dtype.kind not in "iu":
        raise TypeError(f"{label}: integer values expected, found {raw.dtype}")
    _index_shape(label, raw.shape, shape)
    if raw.size:
        lo, hi = int(raw.min()), int(raw.max())
        if lo < 0 or hi > stop or (hi == stop and not closed):
            raise ValueError(f"{label}: values must lie in [0, {stop}{']' if closed else ')'} "
                             f"(found {lo if lo < 0 else hi})")
    return np.ascontiguousarray(raw, dtype=np.int32)


def _index_shape(label, got, want):
    if len(got) != len(want) or any(w is not None and g != w for g, w in zip(got, want)):
        dims = " x ".join("any" if w is None else str(w) for w in want)
        raise ValueError(f"{label}: shape {tuple(got)} where {dims} is expected")


# ---------------------------------------------------------------------------
# device route
# ---------------------------------------------------------------------------

class _DeviceCall:
    """The CUDA operands of one operator call.

    The first operand fixes the storage dtype and the device; every other one must be a CUDA tensor of that
    dtype on that device, and all must be contiguous. A host tensor is refused here, before anything is
    launched: a host pointer reaching a kernel would fault and take the CUDA context with it."""

    def __init__(self, dtypes=None, **operands):
        items = list(operands.items())
        lead_name, lead = items[0]
        allowed = _STORAGE if dtypes is None else dtypes
        for name, t in items:
            if not _on_gpu(t):
                raise TypeError(f"{name}: a CUDA tensor is required because {lead_name} is one")
            if t.dtype not in allowed:
                names = ", ".join(str(d).replace("torch.", "") for d in allowed)
                raise TypeError(f"{name}: dtype {t.dtype} is not supported here (one of {names})")
            if t.dtype != lead.dtype:
                raise TypeError(f"{name}: dtype {t.dtype} differs from {lead_name}'s {lead.dtype}")
            if t.device != lead.device:
                raise TypeError(f"{name}: on {t.device} while {lead_name} is on {lead.device}")
            if not t.is_contiguous():
                raise ValueError(f"{name}: a contiguous tensor is required")
        self.tensors = operands
        self.dtype = lead.dtype
        self.device = lead.device
        self.code = _STORAGE[lead.dtype][1] if lead.dtype in _STORAGE else None

    def dims(self, name, layout):
        """Shape of operand `name`, which must have as many dimensions as `layout` names (e.g. "B Hq D")."""
        t = self.tensors[name]
        if t.ndim != layout.count(" ") + 1:
            raise ValueError(f"{name}: {t.ndim}-D tensor where [{', '.join(layout.split())}] is expected")
        return tuple(t.shape)

    def same_shape(self, name, other):
        if self.tensors[name].shape != self.tensors[other].shape:
            raise ValueError(f"{name}: shape {tuple(self.tensors[name].shape)} differs from {other}'s "
                             f"{tuple(self.tensors[other].shape)}")

    def index(self, label, values, shape, stop, closed):
        """`values` as an int32 tensor on this call's device. Host values are validated and uploaded; a CUDA
        tensor is only cast / compacted if needed and checked for shape."""
        host = _host_index(label, values, shape, stop, closed)
        if host is not None:
            return torch.from_numpy(host).to(self.device)
        dev = values if values.dtype is torch.int32 else values.to(torch.int32)
        _index_shape(label, dev.shape, shape)
        return dev if dev.is_contiguous() else dev.contiguous()

    def new(self, shape):
        return torch.empty(shape, dtype=self.dtype, device=self.device)

    def launch(self, fn, *args):
        """Run launcher `fn(*args, stream)` on the current stream of this call's device."""
        idx = self.device.index
        cur = torch.cuda.current_device()
        if idx is None or idx == cur:
            return fn(*args, self._stream(cur))
        with torch.cuda.device(idx):
            return fn(*args, self._stream(idx))

    @staticmethod
    def _stream(idx):
        # the raw accessor skips building a Stream object on every call
        return _raw_stream(idx) if _raw_stream is not None else torch.cuda.current_stream(idx).cuda_stream


# ---------------------------------------------------------------------------
# staged route
# ---------------------------------------------------------------------------

class _HostCall:
    """Host operands of one call as float32 C-contiguous arrays (values are converted, never aliased)."""

    def __init__(self, **operands):
        self.arrays = {}
        self.torch_in = False
        for name, x in operands.items():
            if torch is not None and torch.is_tensor(x):
                if x.is_cuda:
                    raise TypeError(f"{name}: a CUDA tensor among host operands; keep all operands on one side")
                self.torch_in = True
                x = x.detach().to(torch.float32).numpy()
            self.arrays[name] = np.ascontiguousarray(x, dtype=np.float32)

    def dims(self, name, layout):
        a = self.arrays[name]
        want = layout.split()
        if a.ndim != len(want):
            raise ValueError(f"{name}: {a.ndim}-D array where [{', '.join(want)}] is expected")
        return a.shape

    def same_shape(self, name, other):
        if self.arrays[name].shape != self.arrays[other].shape:
            raise ValueError(f"{name}: shape {self.arrays[name].shape} differs from {other}'s "
                             f"{self.arrays[other].shape}")

    @staticmethod
    def index(label, values, shape, stop, closed):
        host = _host_index(label, values, shape, stop, closed)
        if host is None:
            raise TypeError(f"{label}: a CUDA tensor among host operands; keep all operands on one side")
        return host

    def result(self, arr):
        return torch.from_numpy(arr) if self.torch_in else arr


def _need_gpu_route(cuda):
    if not cuda:
        raise NoHostPathError(
            "fusedtok_b200 computes on the GPU only: give CUDA tensors, or host arrays with cuda=True "
            "to have them staged through the device")


def _writable_f32(arr, name):
    """A host cache that an append updates in place: it has to be float32 and C-contiguous already, since
    converting would write into a temporary."""
    raw = arr.numpy() if (torch is not None and torch.is_tensor(arr)) else arr
    if not (isinstance(raw, np.ndarray) and raw.dtype == np.float32 and raw.flags["C_CONTIGUOUS"]):
        raise TypeError(f"{name}: the in-place append needs a float32 C-contiguous array (a converted copy "
                        "would swallow the write)")
    return raw


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------

def _decode_shapes(call, cache_names, cache_layout, paged):
    """Shape rules shared by the device and staged routes of both decode operators."""
    kname, vname = cache_names
    b, hq, d = call.dims("q", "B Hq D")
    c0, hkv, c2, dk = call.dims(kname, cache_layout)
    call.dims(vname, cache_layout)
    call.same_shape(vname, kname)
    if dk != d:
        raise ValueError(f"{kname}: head dim {dk} differs from q's {d}")
    if not paged and c0 != b:
        raise ValueError(f"{kname}: batch {c0} differs from q's {b}")
    _gqa_heads(hq, hkv, paged)
    return b, hq, hkv, d, c0, c2


def attention_decode(q, k_cache, v_cache, lens=None, *, cuda=False):
    """One decode step of attention with grouped query heads over a contiguous cache:

    ``out[b, h] = softmax(q[b, h] . K[b, h // G]^T / sqrt(D)) . V[b, h // G]``,  ``G = Hq // Hkv``

    q ``[B, Hq, D]``; k_cache / v_cache ``[B, Hkv, T, D]``; lens optional ``[B]`` counts of valid rows
    (``<= T``; 0 gives a zero row; default: all T). CUDA tensors may be float32, bfloat16 or float16 and the
    result has their dtype (accumulation is float32). Host lens values are checked; a CUDA lens tensor is
    trusted and never read back. Reference: python/fusedtok/__init__.py:710-788.
    """
    names = ("k_cache", "v_cache")
    if _on_gpu(q):
        call = _DeviceCall(q=q, k_cache=k_cache, v_cache=v_cache)
        b, hq, hkv, d, _, rows = _decode_shapes(call, names, "B Hkv T D", False)
        lens_dev = None if lens is None else call.index("lens", lens, (b,), rows, True)
        out = call.new((b, hq, d))
        if b:
            call.launch(_launcher("attention_decode_launch", call.dtype), q.data_ptr(), k_cache.data_ptr(),
                        v_cache.data_ptr(), None if lens_dev is None else lens_dev.data_ptr(), out.data_ptr(),
                        b, hq, hkv, rows, d)
        return out
    call = _HostCall(q=q, k_cache=k_cache, v_cache=v_cache)
    b, hq, hkv, d, _, rows = _decode_shapes(call, names, "B Hkv T D", False)
    lens_host = None if lens is None else call.index("lens", lens, (b,), rows, True)
    _need_gpu_route(cuda)
    a = call.arrays
    return call.result(_fusedtok.attention_decode(a["q"], a["k_cache"], a["v_cache"], lens_host, b, hq, hkv, rows, d))


def attention_decode_paged(q, k_pool, v_pool, block_table, lens=None, *, cuda=False):
    """``attention_decode`` over a paged cache. Pools ``[Nb, Hkv, P, D]``; ``block_table`` ``[B, S]``: row t of
    sequence b is row ``t % P`` of pool block ``block_table[b, t // P]``; lens optional (default ``S * P``).
    GQA groups of 1/2/4/8/16 heads (the reference's rule; the launchers underneath take any group). Host
    table and lens values are checked, CUDA tensors trusted. Reference: python/fusedtok/__init__.py:849-940.
    """
    names = ("k_pool", "v_pool")
    if _on_gpu(q):
        call = _DeviceCall(q=q, k_pool=k_pool, v_pool=v_pool)
        b, hq, hkv, d, blocks, page = _decode_shapes(call, names, "Nb Hkv P D", True)
        table = call.index("block_table", block_table, (b, None), blocks, False)
        width = table.shape[1]
        lens_dev = None if lens is None else call.index("lens", lens, (b,), width * page, True)
        out = call.new((b, hq, d))
        if b:
            call.launch(_launcher("attention_decode_paged_launch", call.dtype), q.data_ptr(), k_pool.data_ptr(),
                        v_pool.data_ptr(), table.data_ptr(), None if lens_dev is None else lens_dev.data_ptr(),
                        out.data_ptr(), b, hq, hkv, page, width, d)
        return out
    call = _HostCall(q=q, k_pool=k_pool, v_pool=v_pool)
    b, hq, hkv, d, blocks, page = _decode_shapes(call, names, "Nb Hkv P D", True)
    table = call.index("block_table", block_table, (b, None), blocks, False)
    width = table.shape[1]
    lens_host = None if lens is None else call.index("lens", lens, (b,), width * page, True)
    _need_gpu_route(cuda)
    a = call.arrays
    return call.result(_fusedtok.attention_decode_paged(a["q"], a["k_pool"], a["v_pool"], table, lens_host,
                                                        b, hq, hkv, page, width, blocks, d))


def _prefill_shapes(call):
    b, hq, s, d = call.dims("q", "B Hq S D")
    kb, hkv, ks, kd = call.dims("k", "B Hkv S D")
    call.dims("v", "B Hkv S D")
    call.same_shape("v", "k")
    if (kb, ks, kd) != (b, s, d):
        raise ValueError(f"k: [B, S, D] = {(kb, ks, kd)} differs from q's {(b, s, d)}")
    _gqa_heads(hq, hkv)
    return b, hq, hkv, s, d


def attention_prefill(q, k, v, causal=True, *, cuda=False):
    """Attention of S fresh query rows over their own S key rows:

    ``out[b, h, i] = softmax(q[b, h, i] . K[b, h // G]^T / sqrt(D)) . V[b, h // G]`` over key rows ``0..i``
    (``causal=True``) or all of them. q ``[B, Hq, S, D]``; k / v ``[B, Hkv, S, D]``; the result has q's
    shape and dtype. Same head and dim rules as :func:`attention_decode`.
    Reference: python/fusedtok/__init__.py:791-846.
    """
    if _on_gpu(q):
        call = _DeviceCall(q=q, k=k, v=v)
        b, hq, hkv, s, d = _prefill_shapes(call)
        out = call.new((b, hq, s, d))
        if b and s:
            call.launch(_launcher("attention_prefill_launch", call.dtype), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                        out.data_ptr(), b, hq, hkv, s, d, bool(causal))
        return out
    call = _HostCall(q=q, k=k, v=v)
    b, hq, hkv, s, d = _prefill_shapes(call)
    _need_gpu_route(cuda)
    a = call.arrays
    return call.result(_fusedtok.attention_prefill(a["q"], a["k"], a["v"], b, hq, hkv, s, d, bool(causal)))


# ---------------------------------------------------------------------------
# cache append
# ---------------------------------------------------------------------------

def _append_shapes(call, cache_names, cache_layout, paged):
    kname, vname = cache_names
    c0, hkv, c2, d = call.dims(kname, cache_layout)
    call.dims(vname, cache_layout)
    call.same_shape(vname, kname)
    b, nh, nd = call.dims("k_new", "B Hkv D")
    call.dims("v_new", "B Hkv D")
    call.same_shape("v_new", "k_new")
    if (nh, nd) != (hkv, d):
        raise ValueError(f"k_new: [Hkv, D] = {(nh, nd)} differs from the cache's {(hkv, d)}")
    if not paged and b != c0:
        raise ValueError(f"k_new: batch {b} differs from the cache's {c0}")
    return b, hkv, d, c0, c2


def kv_append(k_cache, v_cache, k_new, v_new, lens, *, cuda=False):
    """Write one new token per sequence into the contiguous cache, in place: ``k_new[b]`` / ``v_new[b]``
    (``[Hkv, D]``) become row ``lens[b]`` of ``k_cache[b]`` / ``v_cache[b]`` (``[B, Hkv, T, D]``). lens is
    the write position and therefore required; host values must lie in ``[0, T)``, a CUDA tensor is trusted.
    Returns None. Reference: python/fusedtok/__init__.py:1029-1112."""
    names = ("k_cache", "v_cache")
    if _on_gpu(k_cache):
        call = _DeviceCall(k_cache=k_cache, v_cache=v_cache, k_new=k_new, v_new=v_new)
        b, hkv, d, _, rows = _append_shapes(call, names, "B Hkv T D", False)
        if b == 0:
            return None
        pos = call.index("lens", lens, (b,), rows, False)
        call.launch(_launcher("kv_append_launch", call.dtype), k_new.data_ptr(), v_new.data_ptr(), pos.data_ptr(),
                    k_cache.data_ptr(), v_cache.data_ptr(), b, hkv, d, rows)
        return None
    kc, vc = _writable_f32(k_cache, "k_cache"), _writable_f32(v_cache, "v_cache")
    call = _HostCall(k_new=k_new, v_new=v_new)
    call.arrays.update(k_cache=kc, v_cache=vc)
    b, hkv, d, _, rows = _append_shapes(call, names, "B Hkv T D", False)
    pos = call.index("lens", lens, (b,), rows, False)
    if b == 0:
        return None
    _need_gpu_route(cuda)
    _fusedtok.kv_append(call.arrays["k_new"], call.arrays["v_new"], pos, kc, vc, b, hkv, d, rows)
    return None


def kv_append_paged(k_pool, v_pool, block_table, k_new, v_new, lens, *, cuda=False):
    """``kv_append`` for a paged cache: the rows go to pool block ``block_table[b, lens[b] // P]`` at offset
    ``lens[b] % P`` (pools ``[Nb, Hkv, P, D]``, k_new / v_new ``[B, Hkv, D]``). The table is read only. Host
    table and lens values are checked (lens in ``[0, S * P)``), CUDA tensors trusted. Returns None.
    Reference: python/fusedtok/__init__.py:943-1026."""
    names = ("k_pool", "v_pool")
    if _on_gpu(k_pool):
        call = _DeviceCall(k_pool=k_pool, v_pool=v_pool, k_new=k_new, v_new=v_new)
        b, hkv, d, blocks, page = _append_shapes(call, names, "Nb Hkv P D", True)
        if b == 0:
            return None
        table = call.index("block_table", block_table, (b, None), blocks, False)
        pos = call.index("lens", lens, (b,), table.shape[1] * page, False)
        call.launch(_launcher("kv_append_paged_launch", call.dtype), k_new.data_ptr(), v_new.data_ptr(),
                    table.data_ptr(), pos.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), b, hkv, d, page,
                    table.shape[1])
        return None
    kp, vp = _writable_f32(k_pool, "k_pool"), _writable_f32(v_pool, "v_pool")
    call = _HostCall(k_new=k_new, v_new=v_new)
    call.arrays.update(k_pool=kp, v_pool=vp)
    b, hkv, d, blocks, page = _append_shapes(call, names, "Nb Hkv P D", True)
    table = call.index("block_table", block_table, (b, None), blocks, False)
    pos = call.index("lens", lens, (b,), table.shape[1] * page, False)
    if b == 0:
        return None
    _need_gpu_route(cuda)
    _fusedtok.kv_append_paged(call.arrays["k_new"], call.arrays["v_new"], table, pos, kp, vp, b, hkv, d, page,
                              table.shape[1], blocks)
    return None


# ---------------------------------------------------------------------------
# rotary embedding
# ---------------------------------------------------------------------------

def _rope_scalars(dim, theta, pos_offset):
    if dim % 2:
        raise ValueError(f"rotary embedding pairs elements, so the last dimension must be even (got {dim})")
    if pos_offset < 0:
        raise ValueError(f"pos_offset {pos_offset} is negative")
    if not theta > 0:
        raise ValueError(f"theta must be positive (got {theta})")


def rope(q, k=None, *, theta=10000.0, pos_offset=0, neox=False, cuda=False):
    """Rotary position embedding of ``q`` (and ``k``), each ``[seq, dim]`` with even dim; row r is rotated for
    position ``pos_offset + r``. ``neox=False`` pairs neighbours ``(2j, 2j+1)``, ``neox=True`` pairs
    ``(j, j + dim/2)``. CUDA tensors: float32 or bfloat16. Returns ``(q_rotated, k_rotated)``, the second
    None when k is. Reference: python/fusedtok/__init__.py:645-702."""
    given = {"q": q} if k is None else {"q": q, "k": k}
    if _on_gpu(q):
        call = _DeviceCall(dtypes=(torch.float32, torch.bfloat16), **given)
        seq, dim = call.dims("q", "seq dim")
        if k is not None:
            call.same_shape("k", "q")
        _rope_scalars(dim, theta, pos_offset)
        if call.dtype is torch.bfloat16:
            fn = _fusedtok.rope_neox_launch_bf16 if neox else _fusedtok.rope_launch_bf16
            head = ()
        else:
            fn, head = _fusedtok.rope_launch, (bool(neox),)
        rotated = []
        for src in given.values():
            dst = torch.empty_like(src)
            call.launch(fn, *head, src.data_ptr(), dst.data_ptr(), seq, dim, theta, pos_offset)
            rotated.append(dst)
        return rotated[0], (rotated[1] if k is not None else None)
    call = _HostCall(**given)
    seq, dim = call.dims("q", "seq dim")
    if k is not None:
        call.same_shape("k", "q")
    _rope_scalars(dim, theta, pos_offset)
    _need_gpu_route(cuda)
    q_rot, k_rot = _fusedtok.rope(bool(neox), call.arrays["q"], call.arrays.get("k"), theta, pos_offset)
    return call.result(q_rot), (None if k_rot is None else call.result(k_rot))


def _rope_append_call(q, k_new, v_new, k_store, v_store, store_layout, paged, theta, pos_offset, out):
    """Checks common to the two fused rope + append operators; returns (call, B, Hq, Hkv, D, c0, c2, q_out)."""
    if not _on_gpu(k_store):
        raise TypeError("the fused rope + append operators work on CUDA tensors only")
    operands = dict(q=q, k_new=k_new, v_new=v_new, k_store=k_store, v_store=v_store)
    if out is not None:
        operands["out"] = out
    call = _DeviceCall(**operands)
    b, hq, d = call.dims("q", "B Hq D")
    c0, hkv, c2, ds = call.dims("k_store", store_layout)
    call.same_shape("v_store", "k_store")
    if tuple(k_new.shape) != (b, hkv, d) or ds != d:
        raise ValueError(f"k_new: shape {tuple(k_new.shape)} where {(b, hkv, ds)} follows from q and the cache")
    call.same_shape("v_new", "k_new")
    if not paged and c0 != b:
        raise ValueError(f"q: batch {b} differs from the cache's {c0}")
    _gqa_heads(hq, hkv)
    if d % 4:
        raise ValueError(f"head dim {d} is not a multiple of 4")
    _rope_scalars(d, theta, pos_offset)
    if out is not None:
        call.same_shape("out", "q")
    return call, b, hq, hkv, d, c0, c2, (call.new((b, hq, d)) if out is None else out)


def rope_kv_append(q, k_cache, v_cache, k_new, v_new, lens, *, theta=10000.0, pos_offset=0, neox=False, out=None):
    """The elementwise front end of a decode step in ONE launch: rotate ``q`` (``[B, Hq, D]``) and ``k_new``
    (``[B, Hkv, D]``) for position ``lens[b] + pos_offset`` and store the rotated key and ``v_new`` as row
    ``lens[b]`` of the contiguous caches (``[B, Hkv, T, D]``), in place. Returns the rotated q (``out`` when
    given; ``out=q`` rotates q in place). CUDA float32 / bfloat16 / float16.

    Bit-identical to ``rope`` applied to each head as a one-row matrix at that position followed by
    ``kv_append`` (reference: python/fusedtok/__init__.py:645-702 and :1029-1112 - three to four launches)."""
    call, b, hq, hkv, d, _, rows, q_out = _rope_append_call(q, k_new, v_new, k_cache, v_cache, "B Hkv T D", False,
                                                            theta, pos_offset, out)
    if b == 0:
        return q_out
    pos = call.index("lens", lens, (b,), rows, False)
    call.launch(_fusedtok.rope_kv_append_launch, call.code, bool(neox), q.data_ptr(), q_out.data_ptr(),
                k_new.data_ptr(), v_new.data_ptr(), pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                b, hq, hkv, d, rows, theta, pos_offset)
    return q_out


def rope_kv_append_paged(q, k_pool, v_pool, block_table, k_new, v_new, lens, *, theta=10000.0, pos_offset=0,
                         neox=False, out=None):
    """``rope_kv_append`` for a paged cache: the rotated key and ``v_new`` go to pool block
    ``block_table[b, lens[b] // P]`` at offset ``lens[b] % P`` (pools ``[Nb, Hkv, P, D]``). Composes ``rope``
    with ``kv_append_paged`` (reference: python/fusedtok/__init__.py:645-702, :943-1026)."""
    call, b, hq, hkv, d, blocks, page, q_out = _rope_append_call(q, k_new, v_new, k_pool, v_pool, "Nb Hkv P D", True,
                                                                 theta, pos_offset, out)
    if b == 0:
        return q_out
    table = call.index("block_table", block_table, (b, None), blocks, False)
    pos = call.index("lens", lens, (b,), table.shape[1] * page, False)
    call.launch(_fusedtok.rope_kv_append_paged_launch, call.code, bool(neox), q.data_ptr(), q_out.data_ptr(),
                k_new.data_ptr(), v_new.data_ptr(), table.data_ptr(), pos.data_ptr(), k_pool.data_ptr(),
                v_pool.data_ptr(), b, hq, hkv, d, page, table.shape[1], theta, pos_offset)
    return q_out
