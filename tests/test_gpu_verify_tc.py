"""GPU: the tcgen05 verify-window split (8 / 16 rows, int4) against the checker and the general tile."""
import numpy as np
import pytest
import torch

from gpuhelp import assert_attention_close, run_verify_attention_gpu, run_verify_attention_oracle
from richengine_b200.abi import INT4
from test_gpu_attention import prepared

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,capacity", [(8, 8), (16, 16), (3, 8), (11, 16), (1, 8)])
def test_window_matches_checker(rows, capacity):
    s, q = prepared(INT4, [0, 31, 33, 700, 64, 2049], rows)
    got16, got32, _ = run_verify_attention_gpu(s, q, rows, capacity, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, rows, capacity)
    assert_attention_close(got32, want32, got16, f"rows {rows}/{capacity}")
    assert not got16[:, :, rows:].any()
    s.close()


@pytest.mark.parametrize("splits", [1, 3, None])
def test_long_history_any_split_count(splits):
    s, q = prepared(INT4, [4096 + 5, 9000], 16)
    got16, got32, _ = run_verify_attention_gpu(s, q, 16, 16, splits=splits, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 16, 16)
    assert_attention_close(got32, want32, got16, f"splits {splits}")
    tile16, tile32, _ = run_verify_attention_gpu(s, q, 16, 16, splits=splits)
    assert_attention_close(got32, tile32, None, "against the general tile")
    s.close()


def test_tree_masks():
    s, q = prepared(INT4, [45, 200, 1000], 15)
    rng = np.random.default_rng(8)
    masks = np.zeros((3, 16), np.uint32)
    for lane in range(3):
        for r in range(15):
            masks[lane, r] = (1 << r) | int(rng.integers(0, 1 << r)) if r else 1
    got16, got32, _ = run_verify_attention_gpu(s, q, 15, 16, row_masks=masks, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 15, 16, row_masks=masks)
    assert_attention_close(got32, want32, got16, "tree")
    s.close()


def test_repeat_run_is_bit_identical():
    s, q = prepared(INT4, [1500, 333], 8)
    a16, a32, (pa, sa) = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    b16, b32, (pb, sb) = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    assert np.array_equal(a16, b16) and np.array_equal(a32, b32)
    assert torch.equal(torch.nan_to_num(pa), torch.nan_to_num(pb)) and torch.equal(torch.nan_to_num(sa), torch.nan_to_num(sb))
    s.close()


def test_large_value_scales_and_peaked_scores():
    """Scores with a wide spread (late maxima force the lazy rescale) and big value scales."""
    s, q = prepared(INT4, [3000], 8, seed=11)
    q = (q.view(np.uint16).astype(np.uint32) << 16).view(np.float32) * 6.0
    q = (q.view(np.uint32) >> 16).astype(np.uint16)
    got16, got32, _ = run_verify_attention_gpu(s, q, 8, 8, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, 8, 8)
    assert_attention_close(got32, want32, got16, "peaked")
    s.close()
