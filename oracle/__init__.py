"""CPU oracle for decode attention - TEST INFRASTRUCTURE ONLY.

ctypes front end over ``liboracle.so`` (the plain-C restatement in
``attention_oracle.c``) and, when it has been built, over
``_ref/libfusedtok_ref.so`` (the reference's own sources behind a C shim).
The shipped package never imports this module: only the tests, the smoke
check and the benchmark's CPU-baseline leg do, and only as the checker.

All functions take and return float32 numpy arrays (the reference's CPU path
is float32 only; half-precision cases are fed the half-rounded values widened
to float32, the reference's own test protocol, tests/test_attention.py:568-571).
"""

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "liboracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libfusedtok_ref.so")

_fp = ctypes.POINTER(ctypes.c_float)
_ip = ctypes.POINTER(ctypes.c_int)
_i = ctypes.c_int

_lib = None
_ref = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_ORACLE_SO):
            from . import build_oracle
            build_oracle.build_oracle()
        _lib = ctypes.CDLL(_ORACLE_SO)
        _lib.oracle_attention_decode.argtypes = [_fp, _fp, _fp, _ip, _fp] + [_i] * 5
        _lib.oracle_attention_decode_paged.argtypes = (
            [_fp, _fp, _fp, _ip, _ip, _fp] + [_i] * 7)
        _lib.oracle_attention_partial.argtypes = [_fp, _fp, _fp, _fp, _fp, _fp, _i, _i, _i]
        _lib.oracle_attention_merge.argtypes = [_fp, _fp, _i, _i, _fp]
        _lib.oracle_attention_prefill.argtypes = [_fp, _fp, _fp, _fp] + [_i] * 6
        _lib.oracle_rope.argtypes = [_fp, _fp, _i, _i, ctypes.c_float, _i, _i]
        _lib.oracle_kv_append.argtypes = [_fp, _fp, _ip, _fp, _fp] + [_i] * 4
        _lib.oracle_kv_append_paged.argtypes = [_fp, _fp, _ip, _ip, _fp, _fp] + [_i] * 6
    return _lib


def ref_available():
    """True when the reference-source build (oracle/_ref) is present."""
    return os.path.exists(_REF_SO)


def _load_ref():
    global _ref
    if _ref is None:
        if not ref_available():
            raise RuntimeError("oracle/_ref/libfusedtok_ref.so has not been built")
        _ref = ctypes.CDLL(_REF_SO)
        _ref.ref_last_error.restype = ctypes.c_char_p
        _ref.ref_attention_decode_cpu.argtypes = [_fp, _fp, _fp, _ip, _fp] + [_i] * 5
        _ref.ref_attention_decode_paged_cpu.argtypes = (
            [_fp, _fp, _fp, _ip, _ip, _fp] + [_i] * 7)
        if hasattr(_ref, "ref_kv_append_cpu"):
            _ref.ref_kv_append_cpu.argtypes = [_fp, _fp, _ip, _fp, _fp] + [_i] * 4
            _ref.ref_kv_append_paged_cpu.argtypes = [_fp, _fp, _ip, _ip, _fp, _fp] + [_i] * 6
        vp = ctypes.c_void_p
        if hasattr(_ref, "ref_attention_prefill_cpu"):
            _ref.ref_attention_prefill_cpu.argtypes = [_fp, _fp, _fp, _fp] + [_i] * 6
            _ref.ref_attention_prefill_launch.argtypes = [_i, vp, vp, vp, vp] + [_i] * 6 + [ctypes.c_size_t]
        if hasattr(_ref, "ref_rope_cpu"):
            _ref.ref_rope_cpu.argtypes = [_fp, _fp, _i, _i, ctypes.c_float, _i, _i]
        _ref.ref_attention_decode_launch.argtypes = (
            [_i, vp, vp, vp, vp, vp] + [_i] * 5 + [ctypes.c_size_t])
        _ref.ref_attention_decode_paged_launch.argtypes = (
            [_i, vp, vp, vp, vp, vp, vp] + [_i] * 6 + [ctypes.c_size_t])
    return _ref


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def _pf(a):
    return a.ctypes.data_as(_fp)


def _pi(a):
    return None if a is None else a.ctypes.data_as(_ip)


def _decode(fn, q, k, v, lens):
    q, k, v, lens = _f32(q), _f32(k), _f32(v), _i32(lens)
    b, hq, d = q.shape
    _, hkv, t, _ = k.shape
    out = np.empty((b, hq, d), np.float32)
    rc = fn(_pf(q), _pf(k), _pf(v), _pi(lens), _pf(out), b, hq, hkv, t, d)
    if rc:
        raise ValueError("oracle rejected the arguments (code %d)" % rc)
    return out


def _decode_paged(fn, q, k_pool, v_pool, table, lens):
    q, k_pool, v_pool = _f32(q), _f32(k_pool), _f32(v_pool)
    table, lens = _i32(table), _i32(lens)
    b, hq, d = q.shape
    nb, hkv, page, _ = k_pool.shape
    width = table.shape[1]
    out = np.empty((b, hq, d), np.float32)
    rc = fn(_pf(q), _pf(k_pool), _pf(v_pool), _pi(table), _pi(lens), _pf(out),
            b, hq, hkv, page, width, nb, d)
    if rc:
        raise ValueError("oracle rejected the arguments (code %d)" % rc)
    return out


def decode(q, k, v, lens=None):
    """Contiguous-cache decode attention through the C restatement."""
    return _decode(_load().oracle_attention_decode, q, k, v, lens)


def decode_paged(q, k_pool, v_pool, table, lens=None):
    """Paged-cache decode attention through the C restatement."""
    return _decode_paged(_load().oracle_attention_decode_paged, q, k_pool,
                         v_pool, table, lens)


def ref_decode(q, k, v, lens=None):
    """The reference's own attention_decode_cpu (src/attention.cu:1318-1373)."""
    return _decode(_load_ref().ref_attention_decode_cpu, q, k, v, lens)


def ref_decode_paged(q, k_pool, v_pool, table, lens=None):
    """The reference's own attention_decode_paged_cpu (src/attention.cu:1382-1456)."""
    return _decode_paged(_load_ref().ref_attention_decode_paged_cpu, q, k_pool,
                         v_pool, table, lens)


def _prefill(fn, q, k, v, causal):
    q, k, v = _f32(q), _f32(k), _f32(v)
    b, hq, s, d = q.shape
    hkv = k.shape[1]
    out = np.empty((b, hq, s, d), np.float32)
    rc = fn(_pf(q), _pf(k), _pf(v), _pf(out), b, hq, hkv, s, d, 1 if causal else 0)
    if rc:
        raise ValueError("oracle rejected the arguments (code %d)" % rc)
    return out


def prefill(q, k, v, causal=True):
    """Fresh-sequence prefill attention through the C restatement."""
    return _prefill(_load().oracle_attention_prefill, q, k, v, causal)


def ref_prefill(q, k, v, causal=True):
    """The reference's own attention_prefill_cpu (src/attention.cu:1591-1638)."""
    return _prefill(_load_ref().ref_attention_prefill_cpu, q, k, v, causal)


def ref_gpu_prefill_launch(dtype_code, q_ptr, k_ptr, v_ptr, out_ptr, b, hq, hkv, s, d, causal, stream):
    """The reference's prefill GPU launcher on raw device pointers (timing only)."""
    r = _load_ref()
    rc = r.ref_attention_prefill_launch(dtype_code, q_ptr, k_ptr, v_ptr, out_ptr, b, hq, hkv, s, d,
                                        1 if causal else 0, stream)
    if rc:
        raise RuntimeError(r.ref_last_error().decode())


def _rope(fn, x, theta, pos_offset, neox):
    x = _f32(x)
    if x.ndim != 2:
        raise ValueError("x must be [seq, dim]")
    y = np.empty_like(x)
    rc = fn(_pf(x), _pf(y), x.shape[0], x.shape[1], float(theta), int(pos_offset), 1 if neox else 0)
    if rc:
        raise ValueError("oracle rejected the arguments (code %d)" % rc)
    return y


def rope(x, theta=10000.0, pos_offset=0, neox=False):
    """Rotary embedding of one [seq, dim] matrix through the C restatement."""
    return _rope(_load().oracle_rope, x, theta, pos_offset, neox)


def ref_rope(x, theta=10000.0, pos_offset=0, neox=False):
    """The reference's own rope_cpu / rope_neox_cpu (src/rope.cu:95-146)."""
    return _rope(_load_ref().ref_rope_cpu, x, theta, pos_offset, neox)


def partial(q_row, k_rows, v_rows, t0, t1):
    """(m, l, acc[D]) of one (b, h) over cache rows [t0, t1)."""
    q_row, k_rows, v_rows = _f32(q_row), _f32(k_rows), _f32(v_rows)
    d = q_row.shape[0]
    m = ctypes.c_float()
    l = ctypes.c_float()
    acc = np.empty(d, np.float32)
    _load().oracle_attention_partial(_pf(q_row), _pf(k_rows), _pf(v_rows),
                                     ctypes.byref(m), ctypes.byref(l), _pf(acc),
                                     int(t0), int(t1), d)
    return np.float32(m.value), np.float32(l.value), acc


def merge(ml, acc):
    """Fold n partial triples (ml [n,2], acc [n,D]) into the output row."""
    ml, acc = _f32(ml), _f32(acc)
    n, d = acc.shape
    out = np.empty(d, np.float32)
    _load().oracle_attention_merge(_pf(ml), _pf(acc), n, d, _pf(out))
    return out


def ref_gpu_decode_launch(dtype_code, q_ptr, k_ptr, v_ptr, lens_ptr, out_ptr,
                          b, hq, hkv, t, d, stream):
    """The reference's GPU launcher on raw device pointers (for timing it
    beside ours). dtype_code: 0 float32, 1 bfloat16, 2 float16."""
    r = _load_ref()
    rc = r.ref_attention_decode_launch(dtype_code, q_ptr, k_ptr, v_ptr,
                                       lens_ptr or None, out_ptr, b, hq, hkv,
                                       t, d, stream)
    if rc:
        raise RuntimeError(r.ref_last_error().decode())


def ref_gpu_decode_paged_launch(dtype_code, q_ptr, k_ptr, v_ptr, table_ptr,
                                lens_ptr, out_ptr, b, hq, hkv, page, width, d,
                                stream):
    """The reference's paged GPU launcher on raw device pointers."""
    r = _load_ref()
    rc = r.ref_attention_decode_paged_launch(dtype_code, q_ptr, k_ptr, v_ptr,
                                             table_ptr, lens_ptr or None,
                                             out_ptr, b, hq, hkv, page, width,
                                             d, stream)
    if rc:
        raise RuntimeError(r.ref_last_error().decode())


def _append(fn, k_cache, v_cache, k_new, v_new, lens):
    k_new, v_new, lens = _f32(k_new), _f32(v_new), _i32(lens)
    kc, vc = _f32(k_cache).copy(), _f32(v_cache).copy()
    b, hkv, t, d = kc.shape
    rc = fn(_pf(k_new), _pf(v_new), _pi(lens), _pf(kc), _pf(vc), b, hkv, d, t)
    if rc:
        raise ValueError("oracle rejected the arguments (code %d)" % rc)
    return kc, vc


def _append_paged(fn, k_pool, v_pool, table, k_new, v_new, lens):
    k_new, v_new, lens, table = _f32(k_new), _f32(v_new), _i32(lens), _i32(table)
    kp, vp = _f32(k_pool).copy(), _f32(v_pool).copy()
    nb, hkv, page, d = kp.shape
    b = k_new.shape[0]
    rc = fn(_pf(k_new), _pf(v_new), _pi(table), _pi(lens), _pf(kp), _pf(vp), b, hkv, d, page,
            table.shape[1], nb)
    if rc:
        raise ValueError("oracle rejected the arguments (code %d)" % rc)
    return kp, vp


def kv_append(k_cache, v_cache, k_new, v_new, lens):
    """Contiguous append through the C restatement; returns the updated copies."""
    return _append(_load().oracle_kv_append, k_cache, v_cache, k_new, v_new, lens)


def kv_append_paged(k_pool, v_pool, table, k_new, v_new, lens):
    """Paged append through the C restatement; returns the updated copies."""
    return _append_paged(_load().oracle_kv_append_paged, k_pool, v_pool, table, k_new, v_new, lens)


def ref_kv_append(k_cache, v_cache, k_new, v_new, lens):
    """The reference's own kv_append_cpu (src/attention.cu:2064-2099)."""
    return _append(_load_ref().ref_kv_append_cpu, k_cache, v_cache, k_new, v_new, lens)


def ref_kv_append_paged(k_pool, v_pool, table, k_new, v_new, lens):
    """The reference's own kv_append_paged_cpu (src/attention.cu:2037-2062)."""
    return _append_paged(_load_ref().ref_kv_append_paged_cpu, k_pool, v_pool, table, k_new, v_new, lens)
