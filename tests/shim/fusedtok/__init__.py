"""TEST INFRASTRUCTURE, never shipped: a package named ``fusedtok`` so that the reference's own test files
(which ``import fusedtok``) can be pointed at this library unmodified.

* CUDA tensors and ``cuda=True`` go straight to ``fusedtok_b200`` - the product.
* Host arrays without ``cuda=True`` are a CPU computation in the reference. ``fusedtok_b200`` has no host
  implementation: it validates the call and raises ``NoHostPathError``. Here, and only here, that case is then
  answered by the CPU oracle (the reference's own CPU code when it has been built from a reference checkout,
  else the C restatement), so that the reference's CPU-route tests exercise this library's argument contract
  and the oracle's numerics.

``tests/test_reference_suite.py`` runs the reference's attention test files against this package wherever a
reference checkout is available.
"""

import numpy as np

import fusedtok_b200 as _ft
from fusedtok_b200 import (attention_prefill as _prefill, attention_decode as _decode,      # noqa: F401
                           attention_decode_paged as _decode_paged, cuda_available, kv_append, kv_append_paged,
                           rope)
from fusedtok_b200 import _fusedtok                                                         # noqa: F401

import oracle as _oracle

try:
    import torch as _torch
except ImportError:                                                                         # pragma: no cover
    _torch = None

__version__ = _ft.__version__


def _np(x):
    if _torch is not None and _torch.is_tensor(x):
        x = x.detach().to(_torch.float32).numpy()
    return np.ascontiguousarray(x, dtype=np.float32)


def _ints(x):
    if x is None:
        return None
    if _torch is not None and _torch.is_tensor(x):
        x = x.numpy()
    return np.ascontiguousarray(x, dtype=np.int32)


def _like(q, arr):
    return _torch.from_numpy(arr) if (_torch is not None and _torch.is_tensor(q)) else arr


def attention_decode(q, k_cache, v_cache, lens=None, *, cuda=False):
    try:
        return _decode(q, k_cache, v_cache, lens, cuda=cuda)
    except _ft.NoHostPathError:
        fn = _oracle.ref_decode if _oracle.ref_available() else _oracle.decode
        return _like(q, fn(_np(q), _np(k_cache), _np(v_cache), _ints(lens)))


def attention_decode_paged(q, k_pool, v_pool, block_table, lens=None, *, cuda=False):
    try:
        return _decode_paged(q, k_pool, v_pool, block_table, lens, cuda=cuda)
    except _ft.NoHostPathError:
        fn = _oracle.ref_decode_paged if _oracle.ref_available() else _oracle.decode_paged
        return _like(q, fn(_np(q), _np(k_pool), _np(v_pool), _ints(block_table), _ints(lens)))


def attention_prefill(q, k, v, causal=True, *, cuda=False):
    try:
        return _prefill(q, k, v, causal, cuda=cuda)
    except _ft.NoHostPathError:
        fn = _oracle.ref_prefill if _oracle.ref_available() else _oracle.prefill
        return _like(q, fn(_np(q), _np(k), _np(v), bool(causal)))
