"""CPU-only checks of the C-ABI boundary: the library loads, exports every
symbol include/fusedtok_b200.h declares, and rejects bad arguments with the
reference's error types before touching the GPU
(reference: tests/test_attention.py:118-149, tests/test_attention_paged.py:127-151)."""

import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fusedtok_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fusedtok_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from fusedtok_b200 import _fusedtok
    lib = ctypes.CDLL(_fusedtok._LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_fusedtok.EXPORTS) == names


def test_no_cpu_path():
    import fusedtok_b200 as ft
    q = np.zeros((1, 4, 32), np.float32)
    k = np.zeros((1, 2, 8, 32), np.float32)
    with pytest.raises(RuntimeError):
        ft.attention_decode(q, k, k)
    with pytest.raises(RuntimeError):
        ft.attention_decode_paged(q, np.zeros((2, 2, 16, 32), np.float32),
                                  np.zeros((2, 2, 16, 32), np.float32), np.zeros((1, 1), np.int32))


def test_shape_errors_before_any_launch():
    import fusedtok_b200 as ft
    q = np.zeros((1, 6, 32), np.float32)
    k = np.zeros((1, 2, 8, 32), np.float32)
    v = np.zeros_like(k)
    with pytest.raises(ValueError):      # Hq not a multiple of Hkv
        ft.attention_decode(np.zeros((1, 5, 32), np.float32), k, v, cuda=True)
    with pytest.raises(ValueError):      # v shape mismatch
        ft.attention_decode(q, k, np.zeros((1, 2, 7, 32), np.float32), cuda=True)
    with pytest.raises(ValueError):      # dim mismatch
        ft.attention_decode(q, np.zeros((1, 2, 8, 30), np.float32), v, cuda=True)
    bad = [np.zeros((1, 6, 30), np.float32), np.zeros((1, 2, 8, 30), np.float32),
           np.zeros((1, 2, 8, 30), np.float32)]
    with pytest.raises(ValueError):      # dim not a multiple of 4
        ft.attention_decode(*bad, cuda=True)
    big = [np.zeros((1, 2, 516), np.float32), np.zeros((1, 1, 4, 516), np.float32),
           np.zeros((1, 1, 4, 516), np.float32)]
    with pytest.raises(ValueError):      # dim over 512
        ft.attention_decode(*big, cuda=True)
    for lens in ([9], [-1], [1, 2]):
        with pytest.raises(ValueError):
            ft.attention_decode(q, k, v, np.array(lens, np.int32), cuda=True)
    with pytest.raises(TypeError):       # non-integral lens
        ft.attention_decode(q, k, v, [1.5], cuda=True)


def test_paged_errors_before_any_launch():
    import fusedtok_b200 as ft
    import cases
    rng = np.random.default_rng(46)
    q, kp, vp, tbl, kc, vc, lens = cases.make_paged_case(rng, 2, 4, 2, 32, 8, [16, 32])
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q, kp, vp, tbl, np.array([2 * 16 + 1, 3], np.int32), cuda=True)
    bad = tbl.copy()
    bad[0, 0] = 999
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q, kp, vp, bad, lens, cuda=True)
    with pytest.raises(ValueError):      # GQA group 3 is not in {1,2,4,8,16}
        q3 = rng.standard_normal((1, 3, 32)).astype(np.float32)
        ft.attention_decode_paged(q3, kp[:, :1], vp[:, :1], tbl[:1, :1], np.array([16], np.int32),
                                  cuda=True)
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q, kp, vp, tbl[:1], lens, cuda=True)
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q[:, :, :16], kp, vp, tbl, lens, cuda=True)


def test_c_abi_status_codes():
    from fusedtok_b200 import _fusedtok
    lib = _fusedtok._lib
    # argument validation returns before any CUDA call: dummy pointers are never touched
    rc = lib.fusedtok_attention_decode_launch(1, 1, 1, None, 1, 1, 5, 2, 8, 32, 0)
    assert rc == 1 and b"multiple of kv heads" in lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_launch_bf16(1, 1, 1, None, 1, 1, 4, 2, 8, 30, 0)
    assert rc == 1 and b"multiple of 4" in lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_paged_launch(1, 1, 1, 1, None, 1, 1, 4, 2, 0, 4, 32, 0)
    assert rc == 1
    rc = lib.fusedtok_attention_decode_paged_launch_fp16(1, 1, 1, 1, None, 1, 1, 4, 2, 1 << 20,
                                                         1 << 20, 32, 0)
    assert rc == 1 and b"capacity" in lib.fusedtok_last_error()
    # batch 0 is a no-op
    assert lib.fusedtok_attention_decode_launch(1, 1, 1, None, 1, 0, 4, 2, 8, 32, 0) == 0
    assert _fusedtok.attention_partial_floats(3, 5, 8) == 32 + 3 * 5 * 8


def test_misaligned_operands_are_refused_before_any_launch():
    """Operands must be aligned to 4 elements; a view that starts at an odd element offset is an invalid
    argument, not a device fault. Dummy pointers: the check precedes every CUDA call."""
    from fusedtok_b200 import _fusedtok
    lib = _fusedtok._lib
    ok = 4096
    for bad in ((ok + 2, ok, ok, ok), (ok, ok + 4, ok, ok), (ok, ok, ok + 6, ok), (ok, ok, ok, ok + 2)):
        q, k, v, out = bad
        rc = lib.fusedtok_attention_decode_launch_bf16(q, k, v, None, out, 1, 4, 2, 8, 32, 0)
        assert rc == 1 and b"aligned" in lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_launch(ok + 8, ok, ok, None, ok, 1, 4, 2, 8, 32, 0)      # float32: 16 bytes
    assert rc == 1 and b"aligned" in lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_paged_launch_fp16(ok, ok + 4, ok, ok, None, ok, 1, 4, 2, 16, 4, 32, 0)
    assert rc == 1 and b"aligned" in lib.fusedtok_last_error()
    rc = lib.fusedtok_kv_append_launch_bf16(ok + 4, ok, ok, ok, ok, 1, 2, 32, 8, 0)
    assert rc == 1 and b"aligned" in lib.fusedtok_last_error()
    rc = lib.fusedtok_attention_decode_partial_launch(1, ok, ok + 2, ok, None, ok, 1, 4, 2, 8, 32, 0)
    assert rc == 1 and b"aligned" in lib.fusedtok_last_error()


def test_measurement_and_test_hooks_check_their_arguments():
    """fusedtok_debug_read_stream (bench.py's read-only bandwidth figure) and fusedtok_debug_set_pool_blocks (the
    self-checking build's pool size) refuse bad arguments before any CUDA call."""
    from fusedtok_b200 import _fusedtok
    lib = _fusedtok._lib
    assert lib.fusedtok_debug_read_stream(None, 1 << 20, 0) == 1
    assert lib.fusedtok_debug_read_stream(4096 + 8, 1 << 20, 0) == 1 and b"aligned" in lib.fusedtok_last_error()
    assert lib.fusedtok_debug_read_stream(4096, 8, 0) == 1
    assert lib.fusedtok_debug_set_pool_blocks(-1) == 1
    assert lib.fusedtok_debug_set_pool_blocks(0) == 0


def test_exchange_launch_argument_checks():
    from fusedtok_b200 import _fusedtok
    lib = _fusedtok._lib
    two = (ctypes.c_void_p * 2)(4096, 8192)
    same = (ctypes.c_void_p * 2)(4096, 4096)
    hole = (ctypes.c_void_p * 2)(4096, None)
    args = (1, 4, 2, 64, 32, 0)
    assert lib.fusedtok_attention_decode_exchange_launch(1, 256, 256, 256, None, 256, two, 2, 2, *args) == 1
    assert lib.fusedtok_attention_decode_exchange_launch(1, 256, 256, 256, None, 256, two, 17, 0, *args) == 1
    assert lib.fusedtok_attention_decode_exchange_launch(1, 256, 256, 256, None, 256, hole, 2, 0, *args) == 1
    assert lib.fusedtok_attention_decode_exchange_launch(1, 256, 256, 256, None, 256, same, 2, 0, *args) == 1
    assert b"distinct" in lib.fusedtok_last_error()
    assert lib.fusedtok_attention_decode_exchange_launch(1, 256, 256, 256, None, 256, two, 2, 0, 1, 5, 2, 64, 32, 0) == 1
    assert lib.fusedtok_attention_decode_exchange_launch(9, 256, 256, 256, None, 256, two, 2, 0, *args) == 1


def test_host_route_is_validated_before_it_is_refused():
    import fusedtok_b200 as ft
    k = np.zeros((1, 2, 4, 8), np.float32)
    with pytest.raises(ValueError):                                  # 3 query heads over 2 kv heads
        ft.attention_decode(np.zeros((1, 3, 8), np.float32), k, k.copy())
    with pytest.raises(ValueError, match="head counts"):
        ft.attention_decode(np.zeros((2, 0, 4), np.float32), np.zeros((2, 1, 8, 4), np.float32),
                            np.zeros((2, 1, 8, 4), np.float32))
    with pytest.raises(ValueError):                                  # paged group of 3
        ft.attention_decode_paged(np.zeros((1, 6, 8), np.float32), np.zeros((4, 2, 2, 8), np.float32),
                                  np.zeros((4, 2, 2, 8), np.float32), np.zeros((1, 2), np.int32))
    with pytest.raises(TypeError):                                   # non-integral lens
        ft.attention_decode(np.zeros((1, 4, 8), np.float32), k, k.copy(), [1.5])
    with pytest.raises(ValueError):                                  # lens beyond the cache
        ft.attention_decode(np.zeros((1, 4, 8), np.float32), k, k.copy(), [5])
    with pytest.raises(ft.NoHostPathError):
        ft.attention_decode(np.zeros((1, 4, 8), np.float32), k, k.copy(), [4])
    kc = np.zeros((1, 2, 8, 4), np.float32)
    kn = np.zeros((1, 2, 4), np.float32)
    with pytest.raises(ValueError):                                  # same size, other shape
        ft.kv_append(kc, np.zeros((1, 2, 4, 8), np.float32), kn, np.zeros((1, 2, 8), np.float32), [0])
    with pytest.raises(TypeError):
        ft.kv_append(kc, kc.copy(), kn, kn.copy(), [1.5])
    with pytest.raises(ValueError):                                  # the append bound is exclusive
        ft.kv_append(kc, kc.copy(), kn, kn.copy(), [8])
    assert ft.kv_append(np.zeros((0, 2, 8, 4), np.float32), np.zeros((0, 2, 8, 4), np.float32),
                        np.zeros((0, 2, 4), np.float32), np.zeros((0, 2, 4), np.float32), []) is None
    with pytest.raises(ft.NoHostPathError):
        ft.kv_append(kc, kc.copy(), kn, kn.copy(), [3])
