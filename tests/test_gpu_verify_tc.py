"""GPU: the tcgen05 window kernel (row capacity 1, 8, 16; all four formats) against the checker and the general tile."""
import numpy as np
import pytest
import torch

from gpuhelp import assert_attention_close, run_verify_attention_gpu, run_verify_attention_oracle
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8
from test_gpu_attention import prepared

pytestmark = pytest.mark.gpu
FORMATS = [INT4, INT8, FP8E4M3, BF16]


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows,capacity", [(8, 8), (16, 16), (3, 8), (11, 16), (1, 8), (1, 1)])
def test_window_matches_checker(fmt, rows, capacity):
    s, q = prepared(fmt, [0, 31, 33, 700, 64, 2049], rows)
    got16, got32, _ = run_verify_attention_gpu(s, q, rows, capacity, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, rows, capacity)
    assert_attention_close(got32, want32, got16, f"fmt {fmt} rows {rows}/{capacity}")
    assert not got16[:, :, rows:].any()
    s.close()


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("splits", [1, 3, None])
def test_long_history_any_split_count(fmt, splits):
    s, q = prepared(fmt, [4096 + 5, 9000], 16)
    got16, got32, _ = run_verify_attention_gpu(s, q, 16, 16, splits=splits, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 16, 16)
    assert_attention_close(got32, want32, got16, f"fmt {fmt} splits {splits}")
    tile16, tile32, _ = run_verify_attention_gpu(s, q, 16, 16, splits=splits)
    assert_attention_close(got32, tile32, None, "against the general tile")
    s.close()


@pytest.mark.parametrize("fmt", FORMATS)
def test_one_row_decode_long_history(fmt):
    s, q = prepared(fmt, [5000, 12345, 1], 1)
    got16, got32, _ = run_verify_attention_gpu(s, q, 1, 1, splits=7, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(got32, want32, got16, f"fmt {fmt} decode")
    s.close()


@pytest.mark.parametrize("fmt", [INT4, INT8, BF16])
def test_tree_masks(fmt):
    s, q = prepared(fmt, [45, 200, 1000], 15)
    rng = np.random.default_rng(8)
    masks = np.zeros((3, 16), np.uint32)
    for lane in range(3):
        for r in range(15):
            masks[lane, r] = (1 << r) | int(rng.integers(0, 1 << r)) if r else 1
    got16, got32, _ = run_verify_attention_gpu(s, q, 15, 16, row_masks=masks, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 15, 16, row_masks=masks)
    assert_attention_close(got32, want32, got16, f"fmt {fmt} tree")
    s.close()


def test_repeat_run_is_bit_identical():
    s, q = prepared(INT4, [1500, 333], 8)
    a16, a32, (pa, sa) = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    b16, b32, (pb, sb) = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    assert np.array_equal(a16, b16) and np.array_equal(a32, b32)
    assert torch.equal(torch.nan_to_num(pa), torch.nan_to_num(pb)) and torch.equal(torch.nan_to_num(sa), torch.nan_to_num(sb))
    s.close()


@pytest.mark.parametrize("fmt", [INT4, INT8])
def test_large_value_scales_and_peaked_scores(fmt):
    """Scores with a wide spread (late maxima force the lazy rescale) and big value scales."""
    s, q = prepared(fmt, [3000], 8, seed=11)
    q = (q.view(np.uint16).astype(np.uint32) << 16).view(np.float32) * 6.0
    q = (q.view(np.uint32) >> 16).astype(np.uint16)
    got16, got32, _ = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 8, 8)
    assert_attention_close(got32, want32, got16, "peaked")
    s.close()


@pytest.mark.parametrize("fmt", [FP8E4M3, BF16])
def test_stale_non_finite_bytes_past_the_visible_tokens(fmt):
    """Pages are recycled: bytes past the last visible token may decode to NaN and must not leak."""
    import oracle as om
    from gpuhelp import chunk_params
    from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
    from richengine_b200.abi import Layout
    s = Scenario(Layout(1, 4, 256, fmt), [100, 40, 31], extra_tokens=16, device=True, seed=5)
    for raw in s.host.bytes:
        raw[:] = 0xFF  # e4m3 0xFF and bf16 0xFFFF are NaN; scale bytes 0xFFFFFFFF too
    fill_history_with_store(s, 0, seed=5)
    rng = np.random.default_rng(105)
    k, v = make_staging(rng, s.lanes, s.layout)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk_params(s, 8)) == 0
    s.upload()
    q = make_queries(rng, s.lanes, s.layout)
    got16, got32, _ = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 8, 8)
    assert_attention_close(got32, want32, got16, "stale bytes")
    s.close()
