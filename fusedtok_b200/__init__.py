"""fusedtok_b200 - fusedtok's decode-attention operators on B200 (sm_100a).

Drop-in for the decode-attention path of fusedtok's Python surface
(reference: python/fusedtok/__init__.py:710-788 ``attention_decode``,
:849-940 ``attention_decode_paged``): same signatures, same validation and
error types, zero-copy on CUDA torch tensors, stream-ordered and CUDA-graph
capturable. Underneath is a from-scratch CUDA library (``csrc/``) reached
through a C ABI (``include/fusedtok_b200.h``).

One deliberate difference: there is no CPU implementation. The reference runs
host inputs without ``cuda=True`` through its float32 CPU reference; here that
combination raises ``RuntimeError`` - pass CUDA tensors (zero-copy path) or
``cuda=True`` (staged path: host arrays are copied to the GPU and back).
"""

import numpy as np

from . import _fusedtok

try:
    import torch
    _HAS_TORCH = True
except ImportError:  # pragma: no cover - torch is optional, as in the reference
    torch = None
    _HAS_TORCH = False

__version__ = "0.1.0"
__all__ = ["attention_decode", "attention_decode_paged", "attention_prefill", "kv_append", "kv_append_paged",
           "rope", "rope_kv_append", "rope_kv_append_paged", "cuda_available"]

_PAGED_GROUPS = (1, 2, 4, 8, 16)


def cuda_available():
    """True if a usable CUDA device is present."""
    return _fusedtok.cuda_available()


# ---------------------------------------------------------------------------
# helpers (reference: python/fusedtok/__init__.py:108-367)
# ---------------------------------------------------------------------------

def _is_torch(x):
    return _HAS_TORCH and torch.is_tensor(x)


def _check_torch_att(t, name):
    """CUDA tensor, float32 / bfloat16 / float16, contiguous
    (reference: _check_torch_att, :172-182). A host pointer must never reach a
    kernel, so CPU tensors are rejected before any launch."""
    if not (_is_torch(t) and t.is_cuda):
        raise TypeError(f"{name} must be a CUDA tensor (got a CPU tensor on the zero-copy path)")
    if t.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError(f"{name} must be float32, bfloat16 or float16, got {t.dtype} "
                        "(convert with .to(torch.float32))")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _att_launch_fn(t, base):
    if t.dtype is torch.bfloat16:
        return getattr(_fusedtok, base + "_bf16")
    if t.dtype is torch.float16:
        return getattr(_fusedtok, base + "_fp16")
    return getattr(_fusedtok, base)


_raw_stream = getattr(getattr(torch, "_C", None), "_cuda_getCurrentRawStream", None) if _HAS_TORCH else None


def _cuda_stream():
    """The current stream of the current device as a raw handle (the launch runs inside _on_device, so the
    current device is the tensors' device). The direct accessor avoids building a Stream object per call."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _on_device:
    """Make `device` current for the launch (the library works on the current
    device); free when it already is."""

    def __init__(self, device):
        self.ctx = None if device.index is None or device.index == torch.cuda.current_device() \
            else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


def _host_int_array(t, name="values"):
    """Host-origin value -> int numpy array; None for a device tensor (whose
    values are never read back). Non-integral host input is rejected
    (reference: _host_int_array, :220-235)."""
    if _is_torch(t):
        if t.is_cuda:
            return None
        host = t.detach().cpu().numpy()
    else:
        host = np.asarray(t)
    if host.size and not np.issubdtype(host.dtype, np.integer):
        raise TypeError(f"{name} must hold integer values (got dtype {host.dtype})")
    return host


def _host_lens_checked(lens, batch, limit, upper_inclusive=True):
    """Host lens values in [0, limit] - or [0, limit) for kv_append, which
    writes AT lens[b] (reference: _host_lens_checked, :258-275)."""
    host = _host_int_array(lens, "lens")
    if host is None:
        return None
    host = np.ascontiguousarray(host, dtype=np.int32)
    if host.ndim != 1 or host.shape[0] != batch:
        raise ValueError("lens must be 1-D with batch entries")
    bracket = "]" if upper_inclusive else ")"
    if host.size and (host.min() < 0 or host.max() > limit
                      or (not upper_inclusive and host.max() == limit)):
        raise ValueError(f"lens entries must be in [0, {limit}{bracket}")
    return host


def _i32_cuda(t):
    if t.dtype is not torch.int32:
        t = t.to(torch.int32)
    if not t.is_contiguous():
        t = t.contiguous()
    return t


def _lens_arg(lens, batch, limit, device, upper_inclusive=True):
    """Host values are validated then uploaded; a device tensor is trusted
    (reference: _lens_arg, :278-290)."""
    host = _host_lens_checked(lens, batch, limit, upper_inclusive)
    if host is not None:
        return torch.from_numpy(host).to(device)
    lt = _i32_cuda(lens)
    if lt.ndim != 1 or lt.numel() != batch:
        raise ValueError("lens must be 1-D with batch entries")
    return lt


def _host_table_checked(table, batch, nblocks):
    host = _host_int_array(table, "block_table")
    if host is None:
        return None
    host = np.ascontiguousarray(host, dtype=np.int32)
    if host.ndim != 2 or host.shape[0] != batch:
        raise ValueError("block_table must be [B, S] with batch rows")
    if host.size and (host.min() < 0 or host.max() >= nblocks):
        raise ValueError(f"block_table entries must be in [0, {nblocks})")
    return host


def _table_arg(table, batch, nblocks, device):
    host = _host_table_checked(table, batch, nblocks)
    if host is not None:
        return torch.from_numpy(host).to(device)
    bt = _i32_cuda(table)
    if bt.ndim != 2 or bt.shape[0] != batch:
        raise ValueError("block_table must be [B, S] with batch rows")
    return bt


def _as_numpy(x, name):
    """Anything host-side -> float32 C-contiguous numpy (reference: :346-356)."""
    if _is_torch(x):
        if x.is_cuda:
            raise TypeError(f"{name} is a CUDA tensor while another input is host-side; "
                            "move all inputs to the same device")
        return np.ascontiguousarray(x.detach().to(torch.float32).numpy())
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def _no_cpu_path():
    raise RuntimeError(
        "fusedtok_b200 has no CPU implementation: pass CUDA tensors (zero-copy) or cuda=True "
        "(host arrays staged through the GPU)")


# ---------------------------------------------------------------------------
# operators
# ---------------------------------------------------------------------------

def rope(q, k=None, *, theta=10000.0, pos_offset=0, neox=False, cuda=False):
    """Rotary position embedding on (q, k): [seq, dim] with even dim.

    ``neox=False`` rotates interleaved pairs (2j, 2j+1), ``neox=True`` the rotate_half layout (j, j + dim/2).
    ``pos_offset`` is the absolute position of row 0. CUDA tensors may be float32 or bfloat16. Returns
    ``(q_rotated, k_rotated)``; the second element is None if k is.
    Reference: python/fusedtok/__init__.py:645-702.
    """
    if _is_torch(q) and q.is_cuda:
        if q.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("q must be float32 or bfloat16")
        if not q.is_contiguous():
            raise ValueError("q must be contiguous")
        if q.ndim != 2:
            raise ValueError("q must be 2-D [seq, dim]")
        seq, dim = q.shape
        if dim % 2:
            raise ValueError("dim must be even (RoPE pairs elements)")
        if pos_offset < 0:
            raise ValueError("pos_offset must be >= 0")
        q_out = torch.empty_like(q)
        k_out = None
        if k is not None:
            if not (_is_torch(k) and k.is_cuda):
                raise TypeError("k must be a CUDA tensor")
            if k.dtype is not q.dtype:
                raise TypeError("k must have the same dtype as q")
            if k.shape != q.shape:
                raise ValueError("k must have the same shape as q")
            if not k.is_contiguous():
                raise ValueError("k must be contiguous")
            k_out = torch.empty_like(k)
        with _on_device(q.device):
            stream = _cuda_stream()
            for src, dst in ((q, q_out), (k, k_out)):
                if src is None:
                    continue
                if q.dtype is torch.bfloat16:
                    launch = _fusedtok.rope_neox_launch_bf16 if neox else _fusedtok.rope_launch_bf16
                    launch(src.data_ptr(), dst.data_ptr(), seq, dim, theta, pos_offset, stream)
                else:
                    _fusedtok.rope_launch(bool(neox), src.data_ptr(), dst.data_ptr(), seq, dim, theta, pos_offset,
                                          stream)
        return q_out, k_out
    if not cuda:
        _no_cpu_path()
    arr_q = _as_numpy(q, "q")
    arr_k = None if k is None else _as_numpy(k, "k")
    if arr_q.ndim != 2:
        raise ValueError("q must be 2-D [seq, dim]")
    if arr_q.shape[1] % 2:
        raise ValueError("dim must be even (RoPE pairs elements)")
    if pos_offset < 0:
        raise ValueError("pos_offset must be >= 0")
    q_res, k_res = _fusedtok.rope(bool(neox), arr_q, arr_k, theta, pos_offset)
    if _is_torch(q):
        q_res = torch.from_numpy(q_res)
        k_res = None if k_res is None else torch.from_numpy(k_res)
    return q_res, k_res


def attention_decode(q, k_cache, v_cache, lens=None, *, cuda=False):
    """Single-token (decode step) attention with GQA over a contiguous cache:

    ``out[b, h] = softmax(q[b,h] . K[b,kv(h)]^T / sqrt(D)) . V[b,kv(h)]``

    q: [B, Hq, D]; k_cache / v_cache: [B, Hkv, T, D]; lens: optional [B] valid
    lengths (<= T). Query head h uses kv head ``h // (Hq // Hkv)``. A length of
    0 gives a zero row. CUDA tensors may be float32, bfloat16 or float16 (output
    dtype = input dtype, float32 accumulation). Host lens values are validated;
    a CUDA lens tensor is trusted and never read back.
    Reference: python/fusedtok/__init__.py:710-788.
    """
    if _is_torch(q) and q.is_cuda:
        for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache)):
            _check_torch_att(t, name)
        for name, t in (("k_cache", k_cache), ("v_cache", v_cache)):
            if t.dtype is not q.dtype:
                raise TypeError(f"{name} must have the same dtype as q")
        if q.ndim != 3 or k_cache.ndim != 4 or v_cache.ndim != 4:
            raise ValueError("q must be [B, Hq, D]; k/v caches [B, Hkv, T, D]")
        b, hq, d = q.shape
        b2, hkv, t_rows, d2 = k_cache.shape
        if (b2, d2) != (b, d) or v_cache.shape != k_cache.shape:
            raise ValueError("k_cache/v_cache must match q's batch and dim")
        if hq < 1 or hkv < 1:
            raise ValueError("head counts must be >= 1")
        if hq % hkv:
            raise ValueError("q heads must be a multiple of kv heads")
        lens_ptr = None
        if lens is not None:
            lt = _lens_arg(lens, b, t_rows, q.device)
            lens_ptr = lt.data_ptr()
        out = torch.empty((b, hq, d), dtype=q.dtype, device=q.device)
        if b * hq > 0:
            with _on_device(q.device):
                _att_launch_fn(q, "attention_decode_launch")(
                    q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), lens_ptr,
                    out.data_ptr(), b, hq, hkv, t_rows, d, _cuda_stream())
        return out
    if not cuda:
        _no_cpu_path()
    arr_q = _as_numpy(q, "q")
    arr_k = _as_numpy(k_cache, "k_cache")
    arr_v = _as_numpy(v_cache, "v_cache")
    if arr_q.ndim != 3 or arr_k.ndim != 4 or arr_v.ndim != 4:
        raise ValueError("q must be [B, Hq, D]; k/v caches [B, Hkv, T, D]")
    b, hq, d = arr_q.shape
    b2, hkv, t_rows, d2 = arr_k.shape
    if (b2, d2) != (b, d) or arr_v.shape != arr_k.shape:
        raise ValueError("k_cache/v_cache must match q's batch and dim")
    if hq % hkv:
        raise ValueError("q heads must be a multiple of kv heads")
    if lens is None:
        arr_lens = None
    else:
        arr_lens = _host_lens_checked(lens, b, t_rows)
        if arr_lens is None:
            raise TypeError("lens must be a host array on this path")
    res = _fusedtok.attention_decode(arr_q, arr_k, arr_v, arr_lens, b, hq, hkv, t_rows, d)
    return torch.from_numpy(res) if _is_torch(q) else res


def attention_prefill(q, k, v, causal=True, *, cuda=False):
    """Prefill (fresh-sequence) attention over S query rows:

    ``out[b, h, i] = softmax(q[b,h,i] . K[b,kv(h)]^T / sqrt(D)) . V[b,kv(h)]`` where query row i attends key
    rows ``[0, i]`` (``causal=True``) or all S rows (``causal=False``).

    q: [B, Hq, S, D]; k / v: [B, Hkv, S, D]; out: [B, Hq, S, D]; same GQA mapping and dim rules as
    :func:`attention_decode`. CUDA tensors may be float32, bfloat16 or float16 (output dtype = input dtype,
    float32 accumulation). Reference: python/fusedtok/__init__.py:791-846.
    """
    if _is_torch(q) and q.is_cuda:
        for name, t in (("q", q), ("k", k), ("v", v)):
            _check_torch_att(t, name)
        for name, t in (("k", k), ("v", v)):
            if t.dtype is not q.dtype:
                raise TypeError(f"{name} must have the same dtype as q")
        if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
            raise ValueError("q/k/v must be [B, heads, S, D]")
        b, hq, s, d = q.shape
        b2, hkv, s2, d2 = k.shape
        if (b2, s2, d2) != (b, s, d) or v.shape != k.shape:
            raise ValueError("k/v must match q's batch, seq and dim")
        if hq < 1 or hkv < 1:
            raise ValueError("head counts must be >= 1")
        if hq % hkv:
            raise ValueError("q heads must be a multiple of kv heads")
        out = torch.empty((b, hq, s, d), dtype=q.dtype, device=q.device)
        if b * hq * s > 0:
            with _on_device(q.device):
                _att_launch_fn(q, "attention_prefill_launch")(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), b, hq, hkv, s, d, bool(causal),
                    _cuda_stream())
        return out
    if not cuda:
        _no_cpu_path()
    arr_q = _as_numpy(q, "q")
    arr_k = _as_numpy(k, "k")
    arr_v = _as_numpy(v, "v")
    if arr_q.ndim != 4 or arr_k.ndim != 4 or arr_v.ndim != 4:
        raise ValueError("q/k/v must be [B, heads, S, D]")
    b, hq, s, d = arr_q.shape
    b2, hkv, s2, d2 = arr_k.shape
    if (b2, s2, d2) != (b, s, d) or arr_v.shape != arr_k.shape:
        raise ValueError("k/v must match q's batch, seq and dim")
    if hq % hkv:
        raise ValueError("q heads must be a multiple of kv heads")
    res = _fusedtok.attention_prefill(arr_q, arr_k, arr_v, b, hq, hkv, s, d, bool(causal))
    return torch.from_numpy(res) if _is_torch(q) else res


def attention_decode_paged(q, k_pool, v_pool, block_table, lens=None, *, cuda=False):
    """Decode-step attention with GQA over a PAGED cache: pools
    [Nb, Hkv, P, D], block_table [B, S] mapping token t of sequence b to pool
    block ``block_table[b, t // P]`` at offset ``t % P``; lens None = S * P rows.
    GQA group sizes 1/2/4/8/16 (the reference's contract; the native launchers
    accept any group). Host table / lens values are validated, device tensors
    trusted. Reference: python/fusedtok/__init__.py:849-940.
    """
    if _is_torch(q) and q.is_cuda:
        for name, t in (("q", q), ("k_pool", k_pool), ("v_pool", v_pool)):
            _check_torch_att(t, name)
        for name, t in (("k_pool", k_pool), ("v_pool", v_pool)):
            if t.dtype is not q.dtype:
                raise TypeError(f"{name} must have the same dtype as q")
        if q.ndim != 3 or k_pool.ndim != 4 or v_pool.ndim != 4:
            raise ValueError("q must be [B, Hq, D]; pools [Nb, Hkv, P, D]")
        b, hq, d = q.shape
        nb, hkv, page, d2 = k_pool.shape
        if d2 != d or v_pool.shape != k_pool.shape:
            raise ValueError("pools must match q's dim and each other")
        if hq < 1 or hkv < 1:
            raise ValueError("head counts must be >= 1")
        if hq % hkv:
            raise ValueError("q heads must be a multiple of kv heads")
        if hq // hkv not in _PAGED_GROUPS:
            raise ValueError("paged decode supports GQA group sizes 1/2/4/8/16 "
                             "(use attention_decode otherwise)")
        bt = _table_arg(block_table, b, nb, q.device)
        s_width = bt.shape[1]
        lens_ptr = None
        if lens is not None:
            lt = _lens_arg(lens, b, s_width * page, q.device)
            lens_ptr = lt.data_ptr()
        out = torch.empty((b, hq, d), dtype=q.dtype, device=q.device)
        if b * hq > 0:
            with _on_device(q.device):
                _att_launch_fn(q, "attention_decode_paged_launch")(
                    q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), bt.data_ptr(), lens_ptr,
                    out.data_ptr(), b, hq, hkv, page, s_width, d, _cuda_stream())
        return out
    if not cuda:
        _no_cpu_path()
    arr_q = _as_numpy(q, "q")
    arr_k = _as_numpy(k_pool, "k_pool")
    arr_v = _as_numpy(v_pool, "v_pool")
    if arr_q.ndim != 3 or arr_k.ndim != 4 or arr_v.ndim != 4:
        raise ValueError("q must be [B, Hq, D]; pools [Nb, Hkv, P, D]; block_table [B, S]")
    b, hq, d = arr_q.shape
    nb, hkv, page, d2 = arr_k.shape
    arr_t = _host_table_checked(block_table, b, nb)
    if arr_t is None:
        raise TypeError("block_table must be a host array on this path")
    if d2 != d or arr_v.shape != arr_k.shape:
        raise ValueError("pools must match q's dim and each other")
    if hq % hkv:
        raise ValueError("q heads must be a multiple of kv heads")
    if hq // hkv not in _PAGED_GROUPS:
        raise ValueError("paged decode supports GQA group sizes 1/2/4/8/16 "
                         "(use attention_decode otherwise)")
    if lens is None:
        arr_lens = None
    else:
        arr_lens = _host_lens_checked(lens, b, arr_t.shape[1] * page)
        if arr_lens is None:
            raise TypeError("lens must be a host array on this path")
    res = _fusedtok.attention_decode_paged(arr_q, arr_k, arr_v, arr_t, arr_lens, b, hq, hkv, page,
                                           arr_t.shape[1], nb, d)
    return torch.from_numpy(res) if _is_torch(q) else res


def _inplace_host_f32(arr, name):
    """Host caches of the in-place appends must already be float32
    C-contiguous: a converted copy would silently drop the writes."""
    raw = arr.numpy() if _is_torch(arr) else arr
    if not isinstance(raw, np.ndarray) or raw.dtype != np.float32 or not raw.flags["C_CONTIGUOUS"]:
        raise TypeError(f"{name} must be a float32 C-contiguous array "
                        "(in-place op; conversion would drop writes)")
    return raw


def kv_append(k_cache, v_cache, k_new, v_new, lens, *, cuda=False):
    """Append ONE fresh token's k/v rows per sequence into the contiguous cache,
    in place: ``k_new[b]`` / ``v_new[b]`` ([Hkv, D]) land at row ``lens[b]`` of
    ``k_cache[b]`` / ``v_cache[b]`` ([B, Hkv, T, D]). lens is required; host values
    are validated in [0, T), a CUDA lens tensor is trusted. Returns None.
    Reference: python/fusedtok/__init__.py:1029-1112."""
    if _is_torch(k_cache) and k_cache.is_cuda:
        for name, t in (("k_cache", k_cache), ("v_cache", v_cache), ("k_new", k_new), ("v_new", v_new)):
            _check_torch_att(t, name)
        for name, t in (("v_cache", v_cache), ("k_new", k_new), ("v_new", v_new)):
            if t.dtype is not k_cache.dtype:
                raise TypeError(f"{name} must have the cache dtype")
        if k_cache.ndim != 4 or v_cache.ndim != 4:
            raise ValueError("caches must be [B, Hkv, T, D]")
        if k_new.ndim != 3 or v_new.ndim != 3:
            raise ValueError("k_new/v_new must be [B, Hkv, D]")
        b, hkv, t_rows, d = k_cache.shape
        if tuple(k_new.shape) != (b, hkv, d) or v_cache.shape != k_cache.shape or v_new.shape != k_new.shape:
            raise ValueError("k/v operands must match the cache layout")
        if b == 0:
            return None
        lt = _lens_arg(lens, b, t_rows, k_cache.device, upper_inclusive=False)
        with _on_device(k_cache.device):
            _att_launch_fn(k_cache, "kv_append_launch")(
                k_new.data_ptr(), v_new.data_ptr(), lt.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                b, hkv, d, t_rows, _cuda_stream())
        return None
    arr_kc = _inplace_host_f32(k_cache, "k_cache")
    arr_vc = _inplace_host_f32(v_cache, "v_cache")
    if not cuda:
        _no_cpu_path()
    arr_kn = _as_numpy(k_new, "k_new")
    arr_vn = _as_numpy(v_new, "v_new")
    if arr_kc.ndim != 4 or arr_kn.ndim != 3:
        raise ValueError("caches [B,Hkv,T,D]; k_new [B,Hkv,D]")
    b, hkv, t_rows, d = arr_kc.shape
    if arr_kn.shape != (b, hkv, d) or arr_vc.shape != arr_kc.shape or arr_vn.shape != arr_kn.shape:
        raise ValueError("k/v operands must match the cache layout")
    arr_l = _host_lens_checked(lens, b, t_rows, upper_inclusive=False)
    if arr_l is None:
        raise TypeError("lens must be a host array on this path")
    _fusedtok.kv_append(arr_kn, arr_vn, arr_l, arr_kc, arr_vc, b, hkv, d, t_rows)
    return None


def kv_append_paged(k_pool, v_pool, block_table, k_new, v_new, lens, *, cuda=False):
    """Append ONE fresh token's k/v rows per sequence into the paged cache, in
    place: rows land at pool block ``block_table[b, lens[b] // P]``, offset
    ``lens[b] % P``. Pools [Nb, Hkv, P, D]; k_new / v_new [B, Hkv, D]; lens
    required. The table is never modified. Host table / lens values are
    validated, device tensors trusted. Returns None.
    Reference: python/fusedtok/__init__.py:943-1026."""
    if _is_torch(k_pool) and k_pool.is_cuda:
        for name, t in (("k_pool", k_pool), ("v_pool", v_pool), ("k_new", k_new), ("v_new", v_new)):
            _check_torch_att(t, name)
        for name, t in (("v_pool", v_pool), ("k_new", k_new), ("v_new", v_new)):
            if t.dtype is not k_pool.dtype:
                raise TypeError(f"{name} must have the pool dtype")
        if k_pool.ndim != 4 or v_pool.ndim != 4:
            raise ValueError("pools must be [Nb, Hkv, P, D]")
        if k_new.ndim != 3 or v_new.ndim != 3:
            raise ValueError("k_new/v_new must be [B, Hkv, D]")
        nb, hkv, page, d = k_pool.shape
        b = k_new.shape[0]
        if tuple(k_new.shape[1:]) != (hkv, d) or v_pool.shape != k_pool.shape or v_new.shape != k_new.shape:
            raise ValueError("k/v operands must match the pool layout")
        if b == 0:
            return None
        bt = _table_arg(block_table, b, nb, k_pool.device)
        lt = _lens_arg(lens, b, bt.shape[1] * page, k_pool.device, upper_inclusive=False)
        with _on_device(k_pool.device):
            _att_launch_fn(k_pool, "kv_append_paged_launch")(
                k_new.data_ptr(), v_new.data_ptr(), bt.data_ptr(), lt.data_ptr(), k_pool.data_ptr(),
                v_pool.data_ptr(), b, hkv, d, page, bt.shape[1], _cuda_stream())
        return None
    arr_kp = _inplace_host_f32(k_pool, "k_pool")
    arr_vp = _inplace_host_f32(v_pool, "v_pool")
    if not cuda:
        _no_cpu_path()
    arr_kn = _as_numpy(k_new, "k_new")
    arr_vn = _as_numpy(v_new, "v_new")
    if arr_kp.ndim != 4 or arr_kn.ndim != 3:
        raise ValueError("pools [Nb,Hkv,P,D]; k_new [B,Hkv,D]")
    nb, hkv, page, d = arr_kp.shape
    b = arr_kn.shape[0]
    if arr_kn.shape != (b, hkv, d) or arr_vp.shape != arr_kp.shape or arr_vn.shape != arr_kn.shape:
        raise ValueError("k/v operands must match the pool layout")
    arr_t = _host_table_checked(block_table, b, nb)
    if arr_t is None:
        raise TypeError("block_table must be a host array on this path")
    arr_l = _host_lens_checked(lens, b, arr_t.shape[1] * page, upper_inclusive=False)
    if arr_l is None:
        raise TypeError("lens must be a host array on this path")
    _fusedtok.kv_append_paged(arr_kn, arr_vn, arr_t, arr_l, arr_kp, arr_vp, b, hkv, d, page,
                              arr_t.shape[1], nb)
    return None


def _dtype_code(t):
    return {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[t.dtype]


def _rope_append_checks(q, k_new, v_new, cache_k, cache_v, hkv, d, theta, pos_offset, out):
    for name, t in (("q", q), ("k_new", k_new), ("v_new", v_new), ("k cache", cache_k), ("v cache", cache_v)):
        _check_torch_att(t, name)
        if t.dtype is not q.dtype:
            raise TypeError(f"{name} must have the dtype of q")
        if t.device != q.device:
            raise TypeError(f"{name} must be on the device of q")
    if q.ndim != 3 or k_new.ndim != 3 or v_new.ndim != 3:
        raise ValueError("q must be [B, Hq, D]; k_new / v_new [B, Hkv, D]")
    b, hq, dq = q.shape
    if dq != d or tuple(k_new.shape) != (b, hkv, d) or v_new.shape != k_new.shape or cache_v.shape != cache_k.shape:
        raise ValueError("q / k_new / v_new must match the cache layout")
    if hq % hkv:
        raise ValueError("q heads must be a multiple of kv heads")
    if d % 4:
        raise ValueError("head dim must be a multiple of 4")
    if pos_offset < 0:
        raise ValueError("pos_offset must be >= 0")
    if not theta > 0:
        raise ValueError("theta must be positive")
    if out is None:
        return torch.empty_like(q)
    _check_torch_att(out, "out")
    if out.dtype is not q.dtype or out.shape != q.shape or out.device != q.device:
        raise ValueError("out must match q")
    return out


def rope_kv_append(q, k_cache, v_cache, k_new, v_new, lens, *, theta=10000.0, pos_offset=0, neox=False, out=None):
    """The elementwise part of one decode step in a single launch: rotate ``q`` ([B, Hq, D]) and
    ``k_new`` ([B, Hkv, D]) to position ``lens[b] + pos_offset`` and write the rotated key and ``v_new``
    into row ``lens[b]`` of the contiguous caches ([B, Hkv, T, D]), in place. Returns the rotated q (``out``
    if given; ``out=q`` rotates in place). CUDA tensors only, float32 / bfloat16 / float16.

    Equal, bit for bit, to ``rope`` on every head as a one-row matrix at ``pos_offset + lens[b]`` followed by
    ``kv_append`` (reference: python/fusedtok/__init__.py:645-702 and :1029-1112, three to four launches)."""
    if not (_is_torch(k_cache) and k_cache.is_cuda):
        raise TypeError("rope_kv_append takes CUDA tensors (there is no host path)")
    if k_cache.ndim != 4:
        raise ValueError("caches must be [B, Hkv, T, D]")
    b, hkv, t_rows, d = k_cache.shape
    q_out = _rope_append_checks(q, k_new, v_new, k_cache, v_cache, hkv, d, theta, pos_offset, out)
    if q.shape[0] != b:
        raise ValueError("q batch must match the cache batch")
    if b == 0:
        return q_out
    lt = _lens_arg(lens, b, t_rows, q.device, upper_inclusive=False)
    with _on_device(q.device):
        _fusedtok.rope_kv_append_launch(_dtype_code(q), bool(neox), q.data_ptr(), q_out.data_ptr(),
                                        k_new.data_ptr(), v_new.data_ptr(), lt.data_ptr(), k_cache.data_ptr(),
                                        v_cache.data_ptr(), b, q.shape[1], hkv, d, t_rows, theta, pos_offset,
                                        _cuda_stream())
    return q_out


def rope_kv_append_paged(q, k_pool, v_pool, block_table, k_new, v_new, lens, *, theta=10000.0, pos_offset=0,
                         neox=False, out=None):
    """``rope_kv_append`` for a paged cache: the rotated key and ``v_new`` land in pool block
    ``block_table[b, lens[b] // P]`` at offset ``lens[b] % P`` (pools [Nb, Hkv, P, D]).
    Composes ``rope`` and ``kv_append_paged`` (reference: python/fusedtok/__init__.py:645-702, :943-1026)."""
    if not (_is_torch(k_pool) and k_pool.is_cuda):
        raise TypeError("rope_kv_append_paged takes CUDA tensors (there is no host path)")
    if k_pool.ndim != 4:
        raise ValueError("pools must be [Nb, Hkv, P, D]")
    nb, hkv, page, d = k_pool.shape
    q_out = _rope_append_checks(q, k_new, v_new, k_pool, v_pool, hkv, d, theta, pos_offset, out)
    b = q.shape[0]
    if b == 0:
        return q_out
    bt = _table_arg(block_table, b, nb, q.device)
    lt = _lens_arg(lens, b, bt.shape[1] * page, q.device, upper_inclusive=False)
    with _on_device(q.device):
        _fusedtok.rope_kv_append_paged_launch(_dtype_code(q), bool(neox), q.data_ptr(), q_out.data_ptr(),
                                              k_new.data_ptr(), v_new.data_ptr(), bt.data_ptr(), lt.data_ptr(),
                                              k_pool.data_ptr(), v_pool.data_ptr(), b, q.shape[1], hkv, d, page,
                                              bt.shape[1], theta, pos_offset, _cuda_stream())
    return q_out
