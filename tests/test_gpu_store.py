"""GPU: append-and-quantize parity — codes, scales and every untouched byte bit-exact against the checker."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import assert_extents_equal, chunk_params, dev, struct_to_device
from kvcase import Scenario, f32_to_bf16, make_staging
from richengine_b200 import lib, ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu
FORMATS = [INT4, INT8, FP8E4M3, BF16]


def both_store_verify(s: Scenario, k, v, rows, layer_index=0, committed=None):
    params = chunk_params(s, rows, layer_index, committed)
    o = om.oracle()
    fmt = s.layout.format
    o.rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params)
    max_rows = max(rows) if isinstance(rows, (list, tuple)) else rows
    ops.store_verify(s.layout, dev(k), dev(v), s.table_pointers, struct_to_device(params),
                     s.storage.layers()[layer_index], s.lanes, min(max_rows, 16))
    torch.cuda.synchronize()


@pytest.mark.parametrize("fmt", FORMATS)
def test_verify_store_four_lanes(fmt):
    """4-lane batched verify store, rows straddling page boundaries, two layers
    (dev/tests/engine/q8_chunked_prefill_metal_test.mm:761-862)."""
    s = Scenario(Layout(2, 4, 256, fmt), [0, 27, 64, 1000], extra_tokens=16, device=True)
    rng = np.random.default_rng(fmt)
    for layer in (1, 0):
        k, v = make_staging(rng, s.lanes, s.layout)
        both_store_verify(s, k, v, 8, layer)
    assert_extents_equal(s, "verify store")
    s.close()


@pytest.mark.parametrize("fmt", FORMATS)
def test_decode_append_one_token_at_a_time(fmt):
    s = Scenario(Layout(1, 4, 256, fmt), [30, 31], extra_tokens=40, device=True)
    rng = np.random.default_rng(10 + fmt)
    for step in range(36):  # crosses a page boundary in both lanes
        k, v = make_staging(rng, s.lanes, s.layout)
        both_store_verify(s, k, v, 1, 0, [c + step for c in s.contexts])
    assert_extents_equal(s, "decode append")
    s.close()


@pytest.mark.parametrize("fmt", FORMATS)
def test_commit_index_overwrite_and_ragged_rows(fmt):
    """Rejected rows are overwritten by the next store at the same logical position
    (q8_chunked_prefill_metal_test.mm:723-759); lanes store different row counts."""
    s = Scenario(Layout(1, 4, 256, fmt), [5, 40, 90], extra_tokens=32, device=True)
    rng = np.random.default_rng(20 + fmt)
    k, v = make_staging(rng, s.lanes, s.layout)
    both_store_verify(s, k, v, [16, 8, 3])
    k, v = make_staging(rng, s.lanes, s.layout)
    both_store_verify(s, k, v, [8, 15, 1], 0, [c + 2 for c in s.contexts])  # accept 2, overwrite the rest
    assert_extents_equal(s, "overwrite")
    s.close()


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows,committed", [(1, 0), (70, 13), (33, 31), (2048, 0), (257, 96)])
def test_prefill_chunk_store(fmt, rows, committed):
    s = Scenario(Layout(2, 4, 256, fmt), [committed], extra_tokens=rows, device=True)
    rng = np.random.default_rng(rows)
    stride = (rows + 31) // 32 * 32
    k = f32_to_bf16(rng.standard_normal((4, stride, 256)).astype(np.float32) * 2)
    v = f32_to_bf16(rng.standard_normal((4, 256, stride)).astype(np.float32) * 0.3)
    k[2, min(3, rows - 1), :] = 0  # a zero row: scale 0, codes 0
    v[1, :, 0] = 0x8000  # negative zeros
    params = lib.ChunkParams(committed, rows, stride, len(s.pages[0]), s.host.layer(1))
    assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, s.host_tables[0].ctypes.data,
                                       C.byref(params)) == 0
    gpu_params = lib.ChunkParams(committed, rows, stride, len(s.pages[0]), s.storage.layers()[1])
    ops.store_chunk(s.layout, dev(k), dev(v), s.device_tables[0], gpu_params)
    torch.cuda.synchronize()
    assert_extents_equal(s, "chunk store")
    s.close()


def test_bf16_store_preserves_edge_bits():
    """Signed zero, subnormals, infinities and NaN payloads keep their 16 bits
    (dev/tests/engine/paged_attention_plan_test.mm:681-699)."""
    bits = np.array([0, 0x8000, 1, 0x8001, 0x007f, 0x0080, 0x4960, 0x7f7f, 0xff7f, 0x7f80, 0xff80, 0x7fc3], np.uint16)
    s = Scenario(Layout(1, 4, 256, BF16), [31], extra_tokens=33, device=True)
    k = np.resize(bits, 4 * 64 * 256).reshape(4, 64, 256).copy()
    v = np.resize(bits[::-1], 4 * 256 * 64).reshape(4, 256, 64).copy()
    params = lib.ChunkParams(31, 33, 64, len(s.pages[0]), s.host.layer(0))
    assert om.oracle().rko_store_chunk(BF16, 4, 256, k.ctypes.data, v.ctypes.data, s.host_tables[0].ctypes.data, C.byref(params)) == 0
    ops.store_chunk(s.layout, dev(k), dev(v), s.device_tables[0],
                    lib.ChunkParams(31, 33, 64, len(s.pages[0]), s.storage.layers()[0]))
    torch.cuda.synchronize()
    assert_extents_equal(s, "bf16 edges")
    s.close()


@pytest.mark.parametrize("fmt", [INT8, INT4, FP8E4M3])
def test_quantizer_boundary_values(fmt):
    """Rows built to land on rounding ties and on the e4m3 saturation edge."""
    s = Scenario(Layout(1, 4, 256, fmt), [0], extra_tokens=64, device=True)
    rng = np.random.default_rng(77)
    rows, stride = 64, 64
    base = np.zeros((4, stride, 256), np.float32)
    for r in range(rows):
        amax = np.float32(2.0 ** rng.integers(-8, 8))
        steps = rng.integers(-254, 255, size=(4, 256)).astype(np.float32)
        base[:, r, :] = steps * amax / np.float32(254.0)  # half-steps of the int8 grid: ties
        base[:, r, 0] = amax
    k = f32_to_bf16(base)
    v = f32_to_bf16(base.transpose(0, 2, 1) * np.float32(1.0009765625))
    params = lib.ChunkParams(0, rows, stride, len(s.pages[0]), s.host.layer(0))
    assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, s.host_tables[0].ctypes.data, C.byref(params)) == 0
    ops.store_chunk(s.layout, dev(k), dev(v), s.device_tables[0], lib.ChunkParams(0, rows, stride, len(s.pages[0]), s.storage.layers()[0]))
    torch.cuda.synchronize()
    assert_extents_equal(s, "boundary values")
    s.close()


def test_invalid_params_write_nothing():
    """Kernels given invalid parameters return without writing (paged_store_row.h:14-29);
    the host entry refuses before launching (PagedAttention.cpp:407-408)."""
    s = Scenario(Layout(1, 4, 256, INT8), [0, 0], extra_tokens=8, device=True)
    rng = np.random.default_rng(1)
    k, v = make_staging(rng, 2, s.layout)
    params = chunk_params(s, 8)
    params[0].page_table_entries = 0  # too short: lane 0 must be skipped, lane 1 stored
    om.oracle().rko_store_verify(INT8, 4, 256, 2, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params)
    ops.store_verify(s.layout, dev(k), dev(v), s.table_pointers, struct_to_device(params), s.storage.layers()[0], 2, 8)
    torch.cuda.synchronize()
    assert_extents_equal(s, "invalid lane skipped")
    with pytest.raises(lib.RichKvError):
        ops.store_chunk(s.layout, dev(k), dev(v), s.device_tables[0], lib.ChunkParams(0, 8, 24, 1, s.storage.layers()[0]))
    s.close()
