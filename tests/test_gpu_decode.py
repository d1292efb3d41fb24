"""GPU: the streaming decode kernels (TMA page ring + warp-level MMA; all four formats) against the checker,
against the general tile, and through its size-independent properties."""
import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (assert_attention_close, chunk_params, run_decode_attention_gpu, run_verify_attention_gpu,
                     run_verify_attention_oracle)
from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

STREAMING = [INT4, INT8, FP8E4M3, BF16]

pytestmark = pytest.mark.gpu


def prepared(contexts, seed=3, layers=1, layer=0, fmt=INT4):
    s = Scenario(Layout(layers, 4, 256, fmt), contexts, extra_tokens=1, device=True, seed=seed)
    fill_history_with_store(s, layer, seed=seed)
    rng = np.random.default_rng(seed + 100)
    k, v = make_staging(rng, s.lanes, s.layout)
    params = chunk_params(s, 1, layer)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    return s, make_queries(rng, s.lanes, s.layout)


@pytest.mark.parametrize("fmt", STREAMING)
@pytest.mark.parametrize("contexts", [[0], [1], [31], [32], [33], [0, 31, 32, 700], [4095, 17, 2048, 5, 64, 63, 999]])
def test_decode_matches_checker(contexts, fmt):
    s, q = prepared(contexts, fmt=fmt)
    got16, got32 = run_decode_attention_gpu(s, q)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(got32, want32, got16, f"decode {contexts}")
    assert not got16[:, :, 1:].any()  # only row 0 of each tile is written
    s.close()


@pytest.mark.parametrize("fmt,lanes", [(INT4, 1024), (INT8, 1024), (BF16, 300), (INT4, 9), (FP8E4M3, 12)])
def test_widest_batches_and_the_merge_shapes_between(fmt, lanes):
    """The widest batch a launch takes (1 024 lanes: every CTA's range spans several lanes, most lanes a single
    segment, some none at all) and the widths at which the merge changes shape (up to 6 lanes sixteen slot groups
    per block, up to 12 eight, beyond that the row merge)."""
    rng = np.random.default_rng(lanes)
    contexts = [int(c) for c in rng.integers(0, 260 if lanes > 100 else 3000, size=lanes)]
    contexts[3] = 0  # a lane without history among the others
    s, q = prepared(contexts, seed=lanes, fmt=fmt)
    got16, got32 = run_decode_attention_gpu(s, q)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(got32, want32, got16, f"decode of {lanes} lanes")
    again16, _ = run_decode_attention_gpu(s, q)
    assert np.array_equal(got16, again16)
    s.close()


@pytest.mark.parametrize("fmt", STREAMING)
@pytest.mark.parametrize("ctas", [1, 3, 7, 148, 1000])
def test_partition_independent_of_grid(ctas, fmt):
    """Any number of CTA ranges gives the same attention within the bar; one range is one tile."""
    s, q = prepared([700, 33, 1500, 64], seed=9, fmt=fmt)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    got16, got32 = run_decode_attention_gpu(s, q, ctas=ctas)
    assert_attention_close(got32, want32, got16, f"ctas {ctas}")
    s.close()


@pytest.mark.parametrize("fmt,repeats", [(INT4, 100), (INT8, 30), (FP8E4M3, 30), (BF16, 30)])
@pytest.mark.parametrize("ctas", [1, 3])
@pytest.mark.parametrize("contexts", [[700, 33, 1500, 64], [1500, 1500], [3000, 3000, 3000]])
def test_small_grids_give_the_same_bits_every_time(contexts, ctas, fmt, repeats):
    """One CTA walks several whole lanes back to back: every repeat must give the bits of the first, and those must
    meet the bar. (A build whose page loop was compiled differently gave a wrong partial for the lane BEFORE a lane
    change in up to one run in three on exactly these mixes; single lanes and rows of short lanes never failed.)"""
    if fmt != INT4 and contexts != [700, 33, 1500, 64]:
        repeats = 10
    s, q = prepared(contexts, seed=9, fmt=fmt)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    first16, first32 = run_decode_attention_gpu(s, q, ctas=ctas)
    assert_attention_close(first32, want32, first16, f"ctas {ctas}")
    for repeat in range(repeats):
        got16, got32 = run_decode_attention_gpu(s, q, ctas=ctas)
        assert np.array_equal(got32, first32) and np.array_equal(got16, first16), f"repeat {repeat} differs"
    s.close()


@pytest.mark.parametrize("fmt", STREAMING)
def test_decode_repeatable_and_agrees_with_general_tile(fmt):
    s, q = prepared([3000, 257, 8191], seed=11, layers=2, layer=1, fmt=fmt)
    a16, a32 = run_decode_attention_gpu(s, q, layer_index=1)
    b16, b32 = run_decode_attention_gpu(s, q, layer_index=1)
    assert np.array_equal(a16, b16) and np.array_equal(a32, b32)  # same grid, same bits
    _, tile32, _ = run_verify_attention_gpu(s, q, 1, 1, layer_index=1)
    assert_attention_close(a32, tile32, None, "decode vs general tile")
    s.close()


def test_zero_rows_and_extreme_scales():
    """All-zero K or V rows (scale 0) and very large / very small value magnitudes."""
    s = Scenario(Layout(1, 4, 256, INT4), [95, 40], extra_tokens=1, device=True, seed=4)
    fill_history_with_store(s, 0, seed=4)
    host = s.host
    for lane, pages in enumerate(s.pages):
        for page in pages[:2]:
            vs = host.tensor_view(page, 0, 3).view(np.float32)
            ks = host.tensor_view(page, 0, 1).view(np.float32)
            vs[3] = 0.0; host.tensor_view(page, 0, 2)[3 * 128:(3 + 1) * 128] = 0  # zero V row (head 0, token 3)
            ks[40] = 0.0                                                           # zero K row (head 1, token 8)
            vs[64:96] *= np.float32(3.0e4)                                        # head 2: huge values
            vs[96:128] *= np.float32(1.0e-6)                                       # head 3: tiny values
    rng = np.random.default_rng(1)
    k, v = make_staging(rng, s.lanes, s.layout)
    params = chunk_params(s, 1, 0)
    assert om.oracle().rko_store_verify(INT4, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    q = make_queries(rng, s.lanes, s.layout)
    got16, got32 = run_decode_attention_gpu(s, q)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    for head in range(4):  # per head: magnitudes differ by ten orders
        assert_attention_close(got32[:, head] / max(1e-30, np.abs(want32[:, head]).max()),
                               want32[:, head] / max(1e-30, np.abs(want32[:, head]).max()), None, f"head {head}")
    s.close()


def test_invalid_lane_is_skipped():
    s, q = prepared([100, 50, 70])
    from gpuhelp import dev, host_u16, struct_to_device, verify_params
    from richengine_b200 import ops
    params, _ = verify_params(s, 1, 1, 32)
    params[1].page_table_entries = 0  # contract violation: lane 1 must not be touched
    dq = dev(q)
    out = torch.full_like(dq, 0x1234)
    runner = ops.DecodeAttention(s.layout, 24, 3, s.storage.window())
    runner.run(dq, out, s.table_pointers, struct_to_device(params), s.storage.layers()[0])
    runner.status()
    torch.cuda.synchronize()
    got = host_u16(out)
    assert (got[1] == 0x1234).all()
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    from kvcase import bf16_to_f32
    for lane in (0, 2):
        assert np.abs(bf16_to_f32(got[lane, :, 0]) - want32[lane, :, 0]).max() < 2e-3 * max(1, np.abs(want32).max()) + 2 ** -8 * np.abs(want32).max()
    s.close()


@pytest.mark.parametrize("fmt", [FP8E4M3, BF16])
def test_stale_non_finite_bytes_in_the_tail_page(fmt):
    """Recycled pages: bytes past the last visible token may decode to NaN and must not leak into the output."""
    s = Scenario(Layout(1, 4, 256, fmt), [100, 40, 31], extra_tokens=1, device=True, seed=5)
    for raw in s.host.bytes:
        raw[:] = 0xFF
    fill_history_with_store(s, 0, seed=5)
    rng = np.random.default_rng(105)
    k, v = make_staging(rng, s.lanes, s.layout)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk_params(s, 1)) == 0
    s.upload()
    q = make_queries(rng, s.lanes, s.layout)
    got16, got32 = run_decode_attention_gpu(s, q)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(got32, want32, got16, "stale bytes")
    s.close()
