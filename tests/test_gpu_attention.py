"""GPU: the general split-KV tile + reduce against the checker's dequantized fp64 attention."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (assert_attention_close, chunk_params, dev, host_u16, run_verify_attention_gpu,
                     run_verify_attention_oracle, struct_to_device)
from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
from richengine_b200 import abi, lib, ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu
FORMATS = [INT4, INT8, FP8E4M3, BF16]


def prepared(fmt, contexts, rows, seed=3, layers=1):
    """History + `rows` current rows stored on the host mirror, uploaded to the device."""
    s = Scenario(Layout(layers, 4, 256, fmt), contexts, extra_tokens=16, device=True, seed=seed)
    fill_history_with_store(s, 0, seed=seed)
    rng = np.random.default_rng(seed + 100)
    k, v = make_staging(rng, s.lanes, s.layout)
    params = chunk_params(s, rows)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    return s, make_queries(rng, s.lanes, s.layout)


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows,capacity", [(1, 1), (8, 8), (16, 16), (3, 8)])
def test_verify_attention_matches_checker(fmt, rows, capacity):
    s, q = prepared(fmt, [0, 31, 33, 700], rows)
    got16, got32, _ = run_verify_attention_gpu(s, q, rows, capacity)
    want16, want32 = run_verify_attention_oracle(s, q, rows, capacity)
    assert_attention_close(got32, want32, got16, f"fmt {fmt} rows {rows}")
    assert not got16[:, :, rows:].any()  # rows past the live rows are zeros
    s.close()


@pytest.mark.parametrize("fmt", [INT4, INT8])
def test_long_history_many_splits(fmt):
    s, q = prepared(fmt, [4096 + 5, 9000], 8)
    got16, got32, _ = run_verify_attention_gpu(s, q, 8, 8)
    _, want32 = run_verify_attention_oracle(s, q, 8, 8)
    assert_attention_close(got32, want32, got16, "long history")
    # one split (everything in one tile) gives the same answer within the bar
    _, one32, _ = run_verify_attention_gpu(s, q, 8, 8, splits=1)
    assert_attention_close(one32, want32, None, "single split")
    s.close()


def test_repeat_run_is_bit_identical():
    """Same inputs, same bits: output, partials and statistics
    (dev/tests/engine/q8_flash_attention_metal_test.mm:558-608)."""
    s, q = prepared(INT4, [1500, 333], 8)
    a16, a32, (pa, sa) = run_verify_attention_gpu(s, q, 8, 8)
    b16, b32, (pb, sb) = run_verify_attention_gpu(s, q, 8, 8)
    assert np.array_equal(a16, b16) and np.array_equal(a32, b32)
    assert torch.equal(torch.nan_to_num(pa), torch.nan_to_num(pb)) and torch.equal(torch.nan_to_num(sa), torch.nan_to_num(sb))
    s.close()


@pytest.mark.parametrize("fmt", [INT4, INT8, BF16])
def test_tree_masks(fmt):
    """Ancestor bitmasks over the scratch rows (paged_attention_tile.h:111-114,141-143)."""
    s, q = prepared(fmt, [45, 200], 15)
    rng = np.random.default_rng(8)
    masks = np.zeros((2, 16), np.uint32)
    for lane in range(2):
        for r in range(15):
            masks[lane, r] = (1 << r) | int(rng.integers(0, 1 << r)) if r else 1
    got16, got32, _ = run_verify_attention_gpu(s, q, 15, 16, row_masks=masks)
    _, want32 = run_verify_attention_oracle(s, q, 15, 16, row_masks=masks)
    assert_attention_close(got32, want32, got16, "tree")
    s.close()


@pytest.mark.parametrize("tensor_core", [False, True])
@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows,committed", [(1, 0), (1, 95), (70, 13), (8, 32), (300, 1000)])
def test_prefill_attention(fmt, rows, committed, tensor_core):
    """8-row tiles over a chunk; rows=1 is the plain one-query decode
    (runtime/metal/kernels/prefill/paged_attention.metal:7-67)."""
    s = Scenario(Layout(1, 4, 256, fmt), [committed], extra_tokens=rows, device=True)
    fill_history_with_store(s, 0)
    rng = np.random.default_rng(rows + committed)
    stride = (rows + 31) // 32 * 32
    from kvcase import f32_to_bf16
    k = f32_to_bf16(rng.standard_normal((4, stride, 256)).astype(np.float32))
    v = f32_to_bf16(rng.standard_normal((4, 256, stride)).astype(np.float32))
    params = lib.ChunkParams(committed, rows, stride, len(s.pages[0]), s.host.layer(0))
    assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, s.host_tables[0].ctypes.data, C.byref(params)) == 0
    s.upload()
    q = make_queries(rng, 1, s.layout, stride=stride)[0]  # [H][stride][G][D]
    tiles = (rows + 7) // 8
    splits = abi.prefill_splits(tiles)
    pp = lib.PrefillParams(committed, rows, stride, len(s.pages[0]), s.storage.layers()[0], splits, 0.0)
    partials = torch.zeros(tiles * 4 * splits * 48 * 256, dtype=torch.float32, device="cuda")
    stats = torch.zeros(tiles * 4 * splits * 48 * 2, dtype=torch.float32, device="cuda")
    dq = dev(q)
    out = torch.zeros_like(dq)
    out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
    if tensor_core:
        runner = ops.VerifyWindowAttention(s.layout, 24, s.storage.window())
        runner.prefill_split(dq, partials, stats, s.device_tables[0], pp)
        ops.attention_prefill_reduce(s.layout, 24, partials, stats, out, pp, output_f32=out32)
        runner.check()
        runner.close()
    else:
        ops.attention_prefill(s.layout, 24, dq, out, partials, stats, s.device_tables[0], pp, output_f32=out32)
    torch.cuda.synchronize()
    got32 = out32.cpu().numpy()
    for tile in range(tiles):
        start = tile * 8
        active = min(8, rows - start)
        for head in range(4):
            want = np.zeros((48, 256), np.float32)
            assert om.oracle().rko_attention_tile(fmt, 4, 6, 256, head, q[head, start].ctypes.data,
                                                  s.host_tables[0].ctypes.data, s.host.layer(0), committed + start,
                                                  active, 8, None, 0.0, int(fmt == FP8E4M3), want.ctypes.data) == 0
            got = got32[head, start:start + 8].reshape(-1, 256)[: active * 6]
            assert_attention_close(got, want[: active * 6], None, f"tile {tile} head {head}")
    s.close()


def reduce_gate_checker():
    """The CPU restatement of the gate epilogue lives with the other checkers, under oracle/."""
    import importlib.util
    from pathlib import Path
    path = Path(__file__).resolve().parent.parent / "oracle" / "reduce_gate.py"
    spec = importlib.util.spec_from_file_location("rk_reduce_gate_checker", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("rows,capacity", [(8, 8), (5, 8), (1, 1), (16, 16)])
def test_reduce_gate_and_gather_epilogue(rows, capacity):
    """The merge that also writes the out-projection's input (decode/paged_attention.metal:273-413): the gather
    form is the merged bf16 row re-laid out, bit for bit; the gate form multiplies it by sigmoid(gate) in fp32."""
    from kvcase import bf16_to_f32, f32_to_bf16
    s, q = prepared(INT4, [100, 3000, 40], rows)
    lanes = s.lanes
    from gpuhelp import verify_params
    lane_params, slot = verify_params(s, rows, capacity)
    d_params = struct_to_device(lane_params)
    got16, _, (partials, stats) = run_verify_attention_gpu(s, q, rows, capacity)
    rng = np.random.default_rng(4)
    stride = 2 * 24 * 256 + 2 * 4 * 256
    packed = f32_to_bf16((rng.standard_normal((lanes, capacity, stride)) * 3).astype(np.float32))
    hidden = torch.zeros((lanes, capacity, 24, 256), dtype=torch.int16, device="cuda")
    out = torch.zeros((lanes, 4, 32, 6, 256), dtype=torch.int16, device="cuda")
    ops.attention_verify_reduce_gate(s.layout, 24, lanes, capacity, partials, stats, out, dev(packed), hidden, d_params)
    torch.cuda.synchronize()
    assert np.array_equal(host_u16(out), got16)  # the attention rows are the plain merge's
    merged = got16[:, :, :capacity].transpose(0, 2, 1, 3, 4).reshape(lanes, capacity, 24, 256)  # [lane][row][kv*6+g][D]
    want = reduce_gate_checker().reduce_gate(merged.astype(np.uint16), packed.astype(np.uint16))  # oracle/reduce_gate.py
    got = host_u16(hidden)
    mismatch = got != want
    assert mismatch.mean() < 2e-3  # exp2 of the two libraries may differ in the last place before the bf16 rounding
    close = np.abs(bf16_to_f32(got) - bf16_to_f32(want)) <= np.abs(bf16_to_f32(want)) * 2.0 ** -7 + 1e-30
    assert close.all()
    hidden.zero_()
    ops.attention_verify_reduce_gate(s.layout, 24, lanes, capacity, partials, stats, None, None, hidden, d_params)
    torch.cuda.synchronize()
    assert np.array_equal(host_u16(hidden), merged)
    s.close()
