"""Helpers for the GPU parity tests: run the CUDA path and the CPU checker on the same scenario."""
import ctypes as C

import numpy as np
import torch

import oracle as om
from kvcase import Scenario, bf16_to_f32
from richengine_b200 import abi, lib, ops

TOLERANCE = 2e-3  # max-abs, relative to max(1, max|reference|): the parity bar for attention outputs


def dev(array: np.ndarray) -> torch.Tensor:
    """numpy (any dtype) -> device tensor of the same bytes (uint16 travels as int16)."""
    a = np.ascontiguousarray(array)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    elif a.dtype == np.uint32:
        a = a.view(np.int32)
    elif a.dtype == np.uint64:
        a = a.view(np.int64)
    return torch.from_numpy(a.copy()).cuda()


def host_u16(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def chunk_params(scenario: Scenario, rows, layer_index=0, committed=None, stride=32):
    committed = committed or scenario.contexts
    rows = rows if isinstance(rows, (list, tuple)) else [rows] * scenario.lanes
    array = (lib.ChunkParams * scenario.lanes)()
    for i in range(scenario.lanes):
        array[i] = lib.ChunkParams(committed[i], rows[i], stride, len(scenario.pages[i]), scenario.host.layer(layer_index))
    return array


def verify_params(scenario: Scenario, active_rows, row_capacity, splits=None, layer_index=0, committed=None,
                  score_scale=0.0):
    committed = committed or scenario.contexts
    active = active_rows if isinstance(active_rows, (list, tuple)) else [active_rows] * scenario.lanes
    array = (lib.VerifyParams * scenario.lanes)()
    lane_splits = [splits or abi.verify_attention_splits(c, a) for c, a in zip(committed, active)]
    slot = max(lane_splits)
    for i in range(scenario.lanes):
        array[i] = lib.VerifyParams(committed[i], len(scenario.pages[i]), scenario.host.layer(layer_index),
                                    lane_splits[i], slot, active[i], row_capacity, score_scale)
    return array, slot


def struct_to_device(array) -> torch.Tensor:
    raw = np.frombuffer(bytes(array), dtype=np.uint8)
    return torch.from_numpy(raw.copy()).cuda()


def run_verify_attention_gpu(scenario: Scenario, queries: np.ndarray, active_rows, row_capacity, row_masks=None,
                             splits=None, layer_index=0, committed=None, tensor_core=False):
    """Split + reduce (general tile, or the tcgen05 split). Returns (bf16 bits, fp32) outputs [lane][H][32][G][D]."""
    layout = scenario.layout
    params, slot = verify_params(scenario, active_rows, row_capacity, splits, layer_index, committed)
    d_params = struct_to_device(params)
    lanes, H, D, G = scenario.lanes, layout.kv_heads, layout.head_dimension, 6
    M = row_capacity * G
    partials = torch.full((lanes * H * slot * M * D,), float("nan"), dtype=torch.float32, device="cuda")
    stats = torch.full((lanes * H * slot * M * 2,), float("nan"), dtype=torch.float32, device="cuda")
    q = dev(queries)
    out = torch.zeros_like(q)
    out32 = torch.zeros(q.shape, dtype=torch.float32, device="cuda")
    masks = dev(row_masks) if row_masks is not None else None
    layer = scenario.storage.layers()[layer_index]
    if tensor_core:
        runner = ops.VerifyWindowAttention(layout, 24, scenario.storage.window())
        runner.split(lanes, row_capacity, slot, q, partials, stats, scenario.table_pointers, masks, d_params, layer)
    else:
        ops.attention_verify_split(layout, 24, lanes, row_capacity, slot, q, partials, stats, scenario.table_pointers,
                                   masks, d_params, layer)
    ops.attention_verify_reduce(layout, 24, lanes, row_capacity, partials, stats, out, d_params, output_f32=out32)
    torch.cuda.synchronize()
    if tensor_core:
        runner.check()
        runner.close()
    return host_u16(out), out32.cpu().numpy(), (partials, stats)


def run_verify_attention_oracle(scenario: Scenario, queries: np.ndarray, active_rows, row_capacity, row_masks=None,
                                layer_index=0, committed=None):
    layout = scenario.layout
    params, _ = verify_params(scenario, active_rows, row_capacity, 32, layer_index, committed)
    out16 = np.zeros(queries.shape, np.uint16)
    out32 = np.zeros(queries.shape, np.float32)
    masks = np.ascontiguousarray(row_masks, dtype=np.uint32) if row_masks is not None else None
    status = om.oracle().rko_attention_verify(layout.format, layout.kv_heads, 6, layout.head_dimension, scenario.lanes,
                                              queries.ctypes.data, scenario.host_table_pointers(), params,
                                              masks.ctypes.data if masks is not None else None,
                                              out16.ctypes.data, out32.ctypes.data)
    assert status == 0
    return out16, out32


def assert_attention_close(got32: np.ndarray, want32: np.ndarray, got16: np.ndarray | None = None, what=""):
    scale = max(1.0, float(np.abs(want32).max()))
    error = float(np.abs(got32 - want32).max())
    assert np.isfinite(got32).all(), f"{what}: non-finite output"
    assert error <= TOLERANCE * scale, f"{what}: max-abs error {error:.3e} > {TOLERANCE * scale:.3e}"
    if got16 is not None:
        # the bf16 store adds at most half a bf16 ulp of each element (2^-9 relative)
        bound = TOLERANCE * scale + np.abs(want32) * 2.0 ** -8
        assert (np.abs(bf16_to_f32(got16) - want32) <= bound).all(), f"{what}: bf16 output outside the bound"


def assert_extents_equal(scenario: Scenario, what=""):
    """Device extents == host (checker) extents, byte for byte, including every untouched byte."""
    for extent, got in enumerate(scenario.download()):
        want = scenario.host.bytes[extent]
        if not np.array_equal(got, want):
            where = np.nonzero(got != want)[0]
            raise AssertionError(f"{what}: extent {extent} differs at {len(where)} bytes, first {where[:8]} "
                                 f"got {got[where[:8]]} want {want[where[:8]]}")


def run_decode_attention_gpu(scenario: Scenario, queries: np.ndarray, layer_index=0, committed=None, ctas=0):
    """Streaming decode kernel: one query row per lane. Returns (bf16 bits, fp32) [lane][H][32][G][D]."""
    layout = scenario.layout
    params, _ = verify_params(scenario, 1, 1, 32, layer_index, committed)
    d_params = struct_to_device(params)
    q = dev(queries)
    out = torch.zeros_like(q)
    out32 = torch.zeros(q.shape, dtype=torch.float32, device="cuda")
    runner = ops.DecodeAttention(layout, 24, scenario.lanes, scenario.storage.window(), ctas)
    runner.partials.fill_(float("nan"))
    runner.statistics.fill_(float("nan"))
    runner.run(q, out, scenario.table_pointers, d_params, scenario.storage.layers()[layer_index], output_f32=out32)
    runner.status()
    torch.cuda.synchronize()
    runner.close()
    return host_u16(out), out32.cpu().numpy()
