"""The argument contract of the attention operators on the GPU routes, case by case after the reference's
tests/test_validation.py (:100-105 GQA on the CUDA route, :123-136 host lens validated before upload,
:139-146 the inclusive decode bound, :149-157 host list == device tensor, :160-183 device lens are trusted and
a call is graph-capturable, :187-205 block-table values, :209-223 the exclusive append bound, :358-380 host
operands on the zero-copy route, :457-476 staged lens / table ranges, :509-515 non-integral lens,
:725-737 zero query heads). Same inputs and seeds; where the reference computes on the CPU this library
raises its "no host path" RuntimeError instead, after the same validation."""

import numpy as np
import pytest
import torch

import fusedtok_b200 as ft

pytestmark = pytest.mark.gpu


def _decode_fixture(device):
    rng = np.random.default_rng(3)
    b, hq, hkv, t, d = 2, 4, 2, 16, 8
    q = torch.tensor(rng.standard_normal((b, hq, d)), dtype=torch.float32, device=device)
    k = torch.tensor(rng.standard_normal((b, hkv, t, d)), dtype=torch.float32, device=device)
    return q, k, b, t


def test_gqa_checked_on_the_cuda_route():
    q = torch.zeros((1, 3, 8), device="cuda")
    k = torch.zeros((1, 2, 4, 8), device="cuda")
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.clone())
    with pytest.raises(ValueError):
        ft.attention_prefill(torch.zeros((1, 3, 4, 8), device="cuda"), k, k.clone())


def test_host_lens_values_validated_before_upload():
    q, k, b, t = _decode_fixture("cuda")
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.clone(), [t + 1, 0])
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.clone(), [0, -1])
    with pytest.raises(ValueError):                   # wrong element count is a shape error
        ft.attention_decode(q, k, k.clone(), [0])
    with pytest.raises(ValueError):                   # host tensors are validated like lists
        ft.attention_decode(q, k, k.clone(), torch.tensor([0, t + 1]))


def test_lens_equal_to_the_capacity_is_valid():
    q, k, b, t = _decode_fixture("cuda")
    out = ft.attention_decode(q, k, k.clone(), [t, t])
    assert out.shape == q.shape
    assert torch.equal(out, ft.attention_decode(q, k, k.clone()))


def test_host_list_and_device_tensor_agree():
    q, k, b, t = _decode_fixture("cuda")
    lens = [t, 7]
    assert torch.equal(ft.attention_decode(q, k, k.clone(), lens),
                       ft.attention_decode(q, k, k.clone(), torch.tensor(lens, device="cuda")))


def test_device_lens_are_trusted_and_the_call_is_graph_capturable():
    q, k, b, t = _decode_fixture("cuda")
    v = k.clone()
    lens = torch.tensor([t, 7], dtype=torch.int32, device="cuda")
    ft.attention_decode(q, k, v, lens)               # warm-up (workspace)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            ft.attention_decode(q, k, v, lens)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g):
        out = ft.attention_decode(q, k, v, lens)
    ref = ft.attention_decode(q, k, v, lens).clone()
    g.replay()
    assert torch.equal(out, ref)
    q.copy_(q * 0.5)                                  # replay reads the same addresses again
    g.replay()
    assert torch.equal(out, ft.attention_decode(q, k, v, lens))


def test_block_table_host_values_validated_device_tables_trusted():
    rng = np.random.default_rng(4)
    b, hq, hkv, nb, p, d = 1, 4, 2, 4, 4, 8
    q = torch.tensor(rng.standard_normal((b, hq, d)), dtype=torch.float32, device="cuda")
    pool = torch.tensor(rng.standard_normal((nb, hkv, p, d)), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):                   # block 4 does not exist in a 4-block pool
        ft.attention_decode_paged(q, pool, pool.clone(), [[0, 4]])
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q, pool, pool.clone(), [[0, -1]])
    out = ft.attention_decode_paged(q, pool, pool.clone(), torch.tensor([[0, 1]], dtype=torch.int32, device="cuda"))
    assert out.shape == q.shape


def test_append_bound_is_exclusive():
    rng = np.random.default_rng(5)
    b, hkv, nb, p, d = 1, 2, 4, 4, 8
    pool = torch.zeros((nb, hkv, p, d), dtype=torch.float32, device="cuda")
    k_new = torch.tensor(rng.standard_normal((b, hkv, d)), dtype=torch.float32, device="cuda")
    table = torch.tensor([[0, 1]], dtype=torch.int32, device="cuda")
    ft.kv_append_paged(pool, pool.clone(), table, k_new, k_new.clone(), [2 * p - 1])    # last slot of block 1
    with pytest.raises(ValueError):
        ft.kv_append_paged(pool, pool.clone(), table, k_new, k_new.clone(), [2 * p])


def test_host_operand_on_the_zero_copy_route_rejected_everywhere():
    q = torch.randn(1, 4, 8, device="cuda")
    k = torch.randn(1, 2, 8, 8, device="cuda")
    with pytest.raises(TypeError):
        ft.attention_decode(q, k.cpu(), k.clone())
    with pytest.raises(TypeError):
        ft.attention_decode(q, k, k.clone().cpu())
    kn = torch.randn(1, 2, 8)
    kc = torch.zeros(1, 2, 8, 8, device="cuda")
    with pytest.raises(TypeError):
        ft.kv_append(kc, kc.clone(), kn, kn.clone(), [0])
    pool = torch.zeros(4, 2, 4, 8, device="cuda")
    with pytest.raises(TypeError):
        ft.attention_decode_paged(q, pool.cpu(), pool.clone(), [[0, 1]])
    out = ft.attention_decode(q, k, k.clone())       # the context is still healthy after the rejections
    torch.cuda.synchronize()
    assert out.shape == q.shape and torch.isfinite(out).all()


def test_staged_lens_and_table_ranges():
    q = np.zeros((1, 4, 8), dtype=np.float32)
    k = np.zeros((1, 2, 8, 8), dtype=np.float32)
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.copy(), [9], cuda=True)
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.copy(), [-1], cuda=True)
    pool = np.zeros((4, 2, 4, 8), dtype=np.float32)
    table = np.zeros((1, 3), dtype=np.int32)
    table[0, 2] = 99
    with pytest.raises(ValueError):
        ft.attention_decode_paged(q, pool, pool.copy(), table, [4], cuda=True)


def test_non_integral_lens_rejected():
    q = torch.zeros((1, 4, 8), device="cuda")
    k = torch.zeros((1, 2, 8, 8), device="cuda")
    with pytest.raises(TypeError):
        ft.attention_decode(q, k, k.clone(), [1.5])


def test_zero_query_heads_rejected_on_both_routes():
    q = np.zeros((2, 0, 4), dtype=np.float32)
    k = np.zeros((2, 1, 8, 4), dtype=np.float32)
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.copy())
    with pytest.raises(ValueError):
        ft.attention_decode(q, k, k.copy(), cuda=True)
    qt = torch.zeros((2, 0, 4), dtype=torch.float32, device="cuda")
    kt = torch.zeros((2, 1, 8, 4), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError, match="head counts"):
        ft.attention_decode(qt, kt, kt.clone())


def test_host_inputs_without_cuda_are_validated_then_refused():
    """The reference computes these on the CPU; here the shapes are checked the same way and the call then
    stops with the library's RuntimeError - there is no host implementation to fall back to."""
    q = np.zeros((1, 3, 8), dtype=np.float32)
    k = np.zeros((1, 2, 4, 8), dtype=np.float32)
    with pytest.raises(ValueError):                   # GQA rule first
        ft.attention_decode(q, k, k.copy())
    with pytest.raises(ValueError):                   # paged group 3
        ft.attention_decode_paged(np.zeros((1, 6, 8), np.float32), np.zeros((4, 2, 2, 8), np.float32),
                                  np.zeros((4, 2, 2, 8), np.float32), np.zeros((1, 2), np.int32))
    with pytest.raises(ft.NoHostPathError):
        ft.attention_decode(np.zeros((1, 4, 8), np.float32), k, k.copy())


def test_read_stream_measurement_kernel_runs():
    """bench.py's read-only bandwidth probe: a launch over a small buffer completes and leaves the status clean."""
    from fusedtok_b200 import _fusedtok
    buf = torch.zeros(1 << 22, dtype=torch.uint8, device="cuda")
    assert _fusedtok._lib.fusedtok_debug_read_stream(buf.data_ptr(), buf.numel(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert _fusedtok.attention_device_status() == 0
