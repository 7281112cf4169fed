"""ctypes binding of ``libfusedtok_b200.so`` exposing the function names and
keyword names of the reference's pybind11 module ``fusedtok._fusedtok`` for the
decode-attention path (reference: src/bindings.cpp:2374-2613), so code and
tests written against ``_fusedtok.attention_decode_launch(...)`` run unchanged.

Pointer arguments are Python ints (``tensor.data_ptr()``); ``lens`` may be
``None`` or ``0`` for "all rows valid" (reference: opt_ptr,
src/bindings.cpp:277-283). Status codes of the C ABI are mapped back to the
exceptions the reference raises: invalid argument -> ValueError, runtime
failure -> RuntimeError.

There is no CPU implementation here: the reference's ``*_cpu`` bindings have
no counterpart, and loading fails loudly when the CUDA library is missing.
"""

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
# FUSEDTOK_B200_LIB may point at another build of the same library (e.g. an instrumented one)
_LIB_PATH = os.environ.get("FUSEDTOK_B200_LIB") or os.path.join(_HERE, "libfusedtok_b200.so")

if not os.path.exists(_LIB_PATH):
    raise ImportError(
        "fusedtok_b200: %s is missing - build it with `python fusedtok_b200/_build.py` "
        "(there is no fallback path)" % _LIB_PATH)

_lib = ctypes.CDLL(_LIB_PATH)

_vp = ctypes.c_void_p
_i = ctypes.c_int
_sz = ctypes.c_size_t

_lib.fusedtok_last_error.restype = ctypes.c_char_p
_lib.fusedtok_cuda_available.restype = _i
for _n in ("", "_bf16", "_fp16"):
    getattr(_lib, "fusedtok_attention_decode_launch" + _n).argtypes = [_vp] * 5 + [_i] * 5 + [_sz]
    getattr(_lib, "fusedtok_attention_decode_paged_launch" + _n).argtypes = [_vp] * 6 + [_i] * 6 + [_sz]
for _n in ("", "_bf16", "_fp16"):
    getattr(_lib, "fusedtok_kv_append_launch" + _n).argtypes = [_vp] * 5 + [_i] * 4 + [_sz]
    getattr(_lib, "fusedtok_kv_append_paged_launch" + _n).argtypes = [_vp] * 6 + [_i] * 5 + [_sz]
    getattr(_lib, "fusedtok_attention_prefill_launch" + _n).argtypes = [_vp] * 4 + [_i] * 6 + [_sz]
_lib.fusedtok_attention_prefill.argtypes = [_vp] * 4 + [_i] * 6
_lib.fusedtok_rope_launch.argtypes = [_i, _vp, _vp, _i, _i, ctypes.c_float, _i, _sz]
_lib.fusedtok_rope_launch_bf16.argtypes = [_vp, _vp, _i, _i, ctypes.c_float, _i, _sz]
_lib.fusedtok_rope_neox_launch_bf16.argtypes = [_vp, _vp, _i, _i, ctypes.c_float, _i, _sz]
_lib.fusedtok_rope.argtypes = [_i, _vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _i]
_lib.fusedtok_kv_append.argtypes = [_vp] * 5 + [_i] * 4
_lib.fusedtok_rope_kv_append_launch.argtypes = [_i, _i] + [_vp] * 7 + [_i] * 5 + [ctypes.c_float, _i, _sz]
_lib.fusedtok_rope_kv_append_paged_launch.argtypes = [_i, _i] + [_vp] * 8 + [_i] * 6 + [ctypes.c_float, _i, _sz]
_lib.fusedtok_kv_append_paged.argtypes = [_vp] * 6 + [_i] * 6
_lib.fusedtok_attention_decode.argtypes = [_vp] * 5 + [_i] * 5
_lib.fusedtok_attention_decode_paged.argtypes = [_vp] * 6 + [_i] * 7
_lib.fusedtok_attention_decode_partial_launch.argtypes = [_i] + [_vp] * 5 + [_i] * 5 + [_sz]
_lib.fusedtok_attention_merge_partials_launch.argtypes = [_i, _vp, _i, _vp, _i, _i, _i, _sz]
_lib.fusedtok_attention_partial_floats.argtypes = [_i, _i, _i]
_lib.fusedtok_attention_partial_floats.restype = ctypes.c_longlong
_lib.fusedtok_attention_decode_launch_noalloc.argtypes = [_i] + [_vp] * 5 + [_i] * 5 + [_sz]
_lib.fusedtok_exchange_alloc.argtypes = [_i, _i, _i, _i, ctypes.POINTER(_vp), ctypes.POINTER(ctypes.c_longlong)]
_lib.fusedtok_exchange_free.argtypes = [_vp]
_lib.fusedtok_exchange_export.argtypes = [_vp, ctypes.c_char_p]
_lib.fusedtok_exchange_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(_vp)]
_lib.fusedtok_exchange_close.argtypes = [_vp]
_lib.fusedtok_attention_decode_exchange_launch.argtypes = (
    [_i] + [_vp] * 5 + [ctypes.POINTER(_vp)] + [_i] * 7 + [_sz])
_lib.fusedtok_attention_device_status.argtypes = [ctypes.POINTER(_i)]
_lib.fusedtok_attention_launch_count.argtypes = [_i]
_lib.fusedtok_attention_launch_count.restype = ctypes.c_longlong
_lib.fusedtok_debug_poke_status.argtypes = [_i, _i, _i]
if hasattr(_lib, "fusedtok_debug_read_stream"):           # (measurement aid of bench.py; same remark as below)
    _lib.fusedtok_debug_read_stream.argtypes = [_vp, ctypes.c_ulonglong, _sz]
if hasattr(_lib, "fusedtok_debug_set_pool_blocks"):      # (a test hook: older variant builds lack it; tests/test_abi.py
    _lib.fusedtok_debug_set_pool_blocks.argtypes = [ctypes.c_longlong]      # checks the product library for every export)

# every symbol include/fusedtok_b200.h declares
EXPORTS = (
    "fusedtok_last_error", "fusedtok_cuda_available",
    "fusedtok_attention_decode_launch", "fusedtok_attention_decode_launch_bf16",
    "fusedtok_attention_decode_launch_fp16",
    "fusedtok_attention_decode_paged_launch", "fusedtok_attention_decode_paged_launch_bf16",
    "fusedtok_attention_decode_paged_launch_fp16",
    "fusedtok_attention_decode", "fusedtok_attention_decode_paged",
    "fusedtok_attention_prefill_launch", "fusedtok_attention_prefill_launch_bf16",
    "fusedtok_attention_prefill_launch_fp16", "fusedtok_attention_prefill",
    "fusedtok_rope_launch", "fusedtok_rope_launch_bf16", "fusedtok_rope_neox_launch_bf16", "fusedtok_rope",
    "fusedtok_kv_append_launch", "fusedtok_kv_append_launch_bf16", "fusedtok_kv_append_launch_fp16",
    "fusedtok_kv_append_paged_launch", "fusedtok_kv_append_paged_launch_bf16",
    "fusedtok_kv_append_paged_launch_fp16", "fusedtok_kv_append", "fusedtok_kv_append_paged",
    "fusedtok_rope_kv_append_launch", "fusedtok_rope_kv_append_paged_launch",
    "fusedtok_attention_decode_partial_launch", "fusedtok_attention_partial_floats",
    "fusedtok_attention_merge_partials_launch",
    "fusedtok_exchange_alloc", "fusedtok_exchange_free", "fusedtok_exchange_export",
    "fusedtok_exchange_open", "fusedtok_exchange_close", "fusedtok_attention_decode_exchange_launch",
    "fusedtok_attention_decode_launch_noalloc",
    "fusedtok_attention_device_status", "fusedtok_attention_launch_count", "fusedtok_debug_poke_status",
    "fusedtok_debug_set_pool_blocks", "fusedtok_debug_read_stream",
)


def _check(rc):
    if rc == 0:
        return
    msg = _lib.fusedtok_last_error().decode("utf-8", "replace")
    if rc == 1:
        raise ValueError(msg)
    raise RuntimeError(msg)


def _opt(p):
    return None if (p is None or p == 0) else int(p)


def cuda_available():
    return bool(_lib.fusedtok_cuda_available())


def _make_launch(suffix):
    fn = getattr(_lib, "fusedtok_attention_decode_launch" + suffix)

    def attention_decode_launch(q, k, v, lens, out, batch, hq, hkv, t_seq, dim, stream=0):
        _check(fn(int(q), int(k), int(v), _opt(lens), int(out), batch, hq, hkv, t_seq, dim,
                  int(stream)))
    attention_decode_launch.__name__ = "attention_decode_launch" + suffix
    return attention_decode_launch


def _make_paged_launch(suffix):
    fn = getattr(_lib, "fusedtok_attention_decode_paged_launch" + suffix)

    def attention_decode_paged_launch(q, k_pool, v_pool, table, lens, out, batch, hq, hkv, page,
                                      tbl_width, dim, stream=0):
        _check(fn(int(q), int(k_pool), int(v_pool), int(table), _opt(lens), int(out), batch, hq,
                  hkv, page, tbl_width, dim, int(stream)))
    attention_decode_paged_launch.__name__ = "attention_decode_paged_launch" + suffix
    return attention_decode_paged_launch


attention_decode_launch = _make_launch("")
attention_decode_launch_bf16 = _make_launch("_bf16")
attention_decode_launch_fp16 = _make_launch("_fp16")
attention_decode_paged_launch = _make_paged_launch("")
attention_decode_paged_launch_bf16 = _make_paged_launch("_bf16")
attention_decode_paged_launch_fp16 = _make_paged_launch("_fp16")


def _make_prefill(suffix):
    fn = getattr(_lib, "fusedtok_attention_prefill_launch" + suffix)

    def attention_prefill_launch(q, k, v, out, batch, hq, hkv, seq, dim, causal, stream=0):
        _check(fn(int(q), int(k), int(v), int(out), batch, hq, hkv, seq, dim, 1 if causal else 0, int(stream)))
    attention_prefill_launch.__name__ = "attention_prefill_launch" + suffix
    return attention_prefill_launch


attention_prefill_launch = _make_prefill("")
attention_prefill_launch_bf16 = _make_prefill("_bf16")
attention_prefill_launch_fp16 = _make_prefill("_fp16")


def rope_launch(neox, src, dst, seq, dim, theta, pos_offset, stream=0):
    """float32, layout chosen by the bool (reference: src/bindings.cpp:722-735)."""
    _check(_lib.fusedtok_rope_launch(1 if neox else 0, int(src), int(dst), seq, dim, float(theta), pos_offset,
                                     int(stream)))


def rope_launch_bf16(src, dst, seq, dim, theta, pos_offset, stream=0):
    _check(_lib.fusedtok_rope_launch_bf16(int(src), int(dst), seq, dim, float(theta), pos_offset, int(stream)))


def rope_neox_launch_bf16(src, dst, seq, dim, theta, pos_offset, stream=0):
    _check(_lib.fusedtok_rope_neox_launch_bf16(int(src), int(dst), seq, dim, float(theta), pos_offset, int(stream)))


def _make_append(suffix):
    fn = getattr(_lib, "fusedtok_kv_append_launch" + suffix)

    def kv_append_launch(k_new, v_new, lens, k_cache, v_cache, batch, hkv, dim, t_rows, stream=0):
        _check(fn(int(k_new), int(v_new), int(lens), int(k_cache), int(v_cache), batch, hkv, dim,
                  t_rows, int(stream)))
    kv_append_launch.__name__ = "kv_append_launch" + suffix
    return kv_append_launch


def _make_append_paged(suffix):
    fn = getattr(_lib, "fusedtok_kv_append_paged_launch" + suffix)

    def kv_append_paged_launch(k_new, v_new, table, lens, k_pool, v_pool, batch, hkv, dim, page,
                               tbl_width, stream=0):
        _check(fn(int(k_new), int(v_new), int(table), int(lens), int(k_pool), int(v_pool), batch,
                  hkv, dim, page, tbl_width, int(stream)))
    kv_append_paged_launch.__name__ = "kv_append_paged_launch" + suffix
    return kv_append_paged_launch


# reference: src/bindings.cpp:2698-2748 (paged) and :2802-2845 (contiguous)
kv_append_launch = _make_append("")
kv_append_launch_bf16 = _make_append("_bf16")
kv_append_launch_fp16 = _make_append("_fp16")
kv_append_paged_launch = _make_append_paged("")
kv_append_paged_launch_bf16 = _make_append_paged("_bf16")
kv_append_paged_launch_fp16 = _make_append_paged("_fp16")


def rope_kv_append_launch(dtype, neox, q, q_out, k_new, v_new, lens, k_cache, v_cache, batch, hq, hkv, dim,
                          t_rows, theta, pos_offset, stream=0):
    """RoPE of q and k_new at position lens[b] + pos_offset, rotated key and v_new written into the
    contiguous cache, one launch. dtype: 0 float32, 1 bfloat16, 2 float16."""
    _check(_lib.fusedtok_rope_kv_append_launch(dtype, 1 if neox else 0, int(q), int(q_out), int(k_new),
                                               int(v_new), int(lens), int(k_cache), int(v_cache), batch, hq,
                                               hkv, dim, t_rows, float(theta), pos_offset, int(stream)))


def rope_kv_append_paged_launch(dtype, neox, q, q_out, k_new, v_new, table, lens, k_pool, v_pool, batch, hq,
                                hkv, dim, page, tbl_width, theta, pos_offset, stream=0):
    """The paged-cache form of rope_kv_append_launch."""
    _check(_lib.fusedtok_rope_kv_append_paged_launch(dtype, 1 if neox else 0, int(q), int(q_out), int(k_new),
                                                     int(v_new), int(table), int(lens), int(k_pool),
                                                     int(v_pool), batch, hq, hkv, dim, page, tbl_width,
                                                     float(theta), pos_offset, int(stream)))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def _ptr(a):
    return None if a is None else a.ctypes.data


def attention_decode(q, k, v, lens, batch, hq, hkv, t_seq, dim):
    """Staged path: float32 host arrays in, host array out
    (reference: src/bindings.cpp:2402-2436)."""
    q, k, v, lens = _f32(q), _f32(k), _f32(v), _i32(lens)
    if (q.size != batch * hq * dim or k.size != batch * hkv * t_seq * dim or v.size != k.size):
        raise ValueError("attention operand size mismatch")
    if lens is not None and lens.size != batch:
        raise ValueError("lens must have batch entries")
    out = np.empty((batch, hq, dim), np.float32)
    _check(_lib.fusedtok_attention_decode(_ptr(q), _ptr(k), _ptr(v), _ptr(lens), _ptr(out), batch,
                                          hq, hkv, t_seq, dim))
    return out


def attention_decode_paged(q, k_pool, v_pool, table, lens, batch, hq, hkv, page, tbl_width,
                           num_blocks, dim):
    """Staged paged path (reference: src/bindings.cpp:2507-2565)."""
    q, k_pool, v_pool = _f32(q), _f32(k_pool), _f32(v_pool)
    table, lens = _i32(table), _i32(lens)
    if (q.size != batch * hq * dim or k_pool.size != num_blocks * hkv * page * dim
            or v_pool.size != k_pool.size or table.size != batch * tbl_width):
        raise ValueError("attention operand size mismatch")
    if lens is not None and lens.size != batch:
        raise ValueError("lens must have batch entries")
    out = np.empty((batch, hq, dim), np.float32)
    _check(_lib.fusedtok_attention_decode_paged(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table),
                                                _ptr(lens), _ptr(out), batch, hq, hkv, page,
                                                tbl_width, num_blocks, dim))
    return out


def attention_prefill(q, k, v, batch, hq, hkv, seq, dim, causal):
    """Staged prefill: float32 host arrays in, host array out
    (reference: src/bindings.cpp:2863-2886)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    if q.size != batch * hq * seq * dim or k.size != batch * hkv * seq * dim or v.size != k.size:
        raise ValueError("attention operand size mismatch")
    out = np.empty((batch, hq, seq, dim), np.float32)
    _check(_lib.fusedtok_attention_prefill(_ptr(q), _ptr(k), _ptr(v), _ptr(out), batch, hq, hkv, seq, dim,
                                           1 if causal else 0))
    return out


def rope(neox, q, k, theta, pos_offset):
    """Staged RoPE: float32 host [seq, dim] arrays in, rotated copies out
    (reference: src/bindings.cpp:683-716)."""
    q = _f32(q)
    if q.ndim != 2:
        raise ValueError("q must be 2-D [seq, dim]")
    if k is not None:
        k = _f32(k)
        if k.shape != q.shape:
            raise ValueError("k must have the same shape as q")
    q_out = np.empty_like(q)
    k_out = None if k is None else np.empty_like(k)
    _check(_lib.fusedtok_rope(1 if neox else 0, _ptr(q), _ptr(k), _ptr(q_out), _ptr(k_out), q.shape[0],
                              q.shape[1], float(theta), int(pos_offset)))
    return q_out, k_out


def kv_append(k_new, v_new, lens, k_cache, v_cache, batch, hkv, dim, t_rows):
    """Staged append into float32 C-contiguous host caches, in place
    (reference: src/bindings.cpp:2766-2800)."""
    k_new, v_new, lens = _f32(k_new), _f32(v_new), _i32(lens)
    if k_new.size != batch * hkv * dim or v_new.size != k_new.size or lens.size != batch \
            or k_cache.size != batch * hkv * t_rows * dim or v_cache.size != k_cache.size:
        raise ValueError("kv append operand size mismatch")
    _check(_lib.fusedtok_kv_append(_ptr(k_new), _ptr(v_new), _ptr(lens), _ptr(k_cache), _ptr(v_cache),
                                   batch, hkv, dim, t_rows))


def kv_append_paged(k_new, v_new, table, lens, k_pool, v_pool, batch, hkv, dim, page, tbl_width,
                    num_blocks):
    """Staged paged append into float32 C-contiguous host pools, in place
    (reference: src/bindings.cpp:2636-2696)."""
    k_new, v_new, table, lens = _f32(k_new), _f32(v_new), _i32(table), _i32(lens)
    if k_new.size != batch * hkv * dim or v_new.size != k_new.size or lens.size != batch \
            or table.size != batch * tbl_width \
            or k_pool.size != num_blocks * hkv * page * dim or v_pool.size != k_pool.size:
        raise ValueError("kv append operand size mismatch")
    _check(_lib.fusedtok_kv_append_paged(_ptr(k_new), _ptr(v_new), _ptr(table), _ptr(lens),
                                         _ptr(k_pool), _ptr(v_pool), batch, hkv, dim, page,
                                         tbl_width, num_blocks))


def attention_decode_partial_launch(dtype, q, k, v, lens, partial, batch, hq, hkv, t_seq, dim,
                                    stream=0):
    """Raw (m, l, acc) triples over this GPU's slice of the cache rows
    (multi-GPU KV-length split; dtype 0 f32, 1 bf16, 2 fp16)."""
    _check(_lib.fusedtok_attention_decode_partial_launch(
        dtype, int(q), int(k), int(v), _opt(lens), int(partial), batch, hq, hkv, t_seq, dim,
        int(stream)))


def attention_partial_floats(batch, hq, dim):
    """Length in float32 elements of one triple block for (batch, hq, dim)."""
    return int(_lib.fusedtok_attention_partial_floats(batch, hq, dim))


def attention_merge_partials_launch(dtype, partials, n_parts, out, batch, hq, dim, stream=0):
    """Fold n_parts gathered triple blocks into the normalised output."""
    _check(_lib.fusedtok_attention_merge_partials_launch(
        dtype, int(partials), n_parts, int(out), batch, hq, dim, int(stream)))


def exchange_alloc(n_ranks, batch, hq, dim):
    """Allocate this rank's exchange buffer for the direct peer exchange;
    returns (device pointer, bytes)."""
    ptr, nbytes = _vp(), ctypes.c_longlong()
    _check(_lib.fusedtok_exchange_alloc(n_ranks, batch, hq, dim, ctypes.byref(ptr), ctypes.byref(nbytes)))
    return ptr.value, nbytes.value


def exchange_free(ptr):
    _check(_lib.fusedtok_exchange_free(ptr))


def exchange_export(ptr):
    """64-byte CUDA IPC handle of an exchange buffer (bytes)."""
    buf = ctypes.create_string_buffer(64)
    _check(_lib.fusedtok_exchange_export(ptr, buf))
    return buf.raw


def exchange_open(handle):
    """Map a peer's exchange buffer from its IPC handle; returns the device pointer."""
    ptr = _vp()
    _check(_lib.fusedtok_exchange_open(handle, ctypes.byref(ptr)))
    return ptr.value


def exchange_close(ptr):
    _check(_lib.fusedtok_exchange_close(ptr))


def attention_decode_exchange_launch(dtype, q, k, v, lens, out, buffers, rank, batch, hq, hkv, t_seq,
                                     dim, stream=0):
    """KV-length split step with direct peer exchange, one kernel per rank:
    `buffers` lists every rank's exchange buffer pointer (own at index `rank`)."""
    n = len(buffers)
    arr = (_vp * n)(*buffers)
    _check(_lib.fusedtok_attention_decode_exchange_launch(
        dtype, int(q), int(k), int(v), _opt(lens), int(out), arr, n, rank, batch, hq, hkv, t_seq, dim,
        int(stream)))


def attention_decode_launch_noalloc(dtype, q, k, v, lens, out, batch, hq, hkv, t_seq, dim, stream=0):
    """Contiguous-cache decode for callers that may not allocate device memory
    after start-up (pre-budgeted serving processes, allocator-policed hosts):
    identical results to ``attention_decode_launch*`` but the split-KV scratch
    is a fixed 4 MiB array inside the library, so nothing is allocated. dtype:
    0 f32, 1 bf16, 2 fp16. Larger shapes raise ValueError. Make the first call
    on a device outside stream capture; do not overlap calls on one device."""
    _check(_lib.fusedtok_attention_decode_launch_noalloc(
        dtype, int(q), int(k), int(v), _opt(lens), int(out), batch, hq, hkv, t_seq, dim, int(stream)))


def attention_device_status():
    """Synchronise the current device and return (then clear) the kernels'
    status word; 0 means every bounded device-side wait completed."""
    st = _i(0)
    _check(_lib.fusedtok_attention_device_status(ctypes.byref(st)))
    return st.value


def attention_launch_count(reset=False):
    return int(_lib.fusedtok_attention_launch_count(1 if reset else 0))
