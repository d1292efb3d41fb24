"""CPU: operator plans — kernel names, grids and workspaces against the reference's own
PagedAttention.cpp compiled in place, and the values its tests pin
(dev/tests/engine/paged_attention_plan_test.mm:94-177)."""
import ctypes as C

import pytest

import oracle as om
from richengine_b200 import lib
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout
from richengine_b200 import abi
from richengine_b200.hostplane import prefill_plan, verify_plan

needs_reference = pytest.mark.skipif(om.reference() is None, reason="reference checkout was not compiled here")


def test_plan_known_values():
    names, n = verify_plan(4, 24, Layout(16, 4, 256, INT4), [100, 5000, 32768, 262144])
    assert names == ["verify_attention_int4_split", "verify_attention_reduce", "verify_attention_int4_store"]
    assert n[0] == 128 and n[1:5] == [32, 32, 65, 128] and n[5:8] == [4, 128, 4] and n[8:11] == [4, 48, 4]
    assert n[11] == 4 * 8 * 128 * 24 * 256 * 4 and n[12] == 4 * 8 * 128 * 24 * 2 * 4 and n[13] == 8
    names, n = verify_plan(2, 24, Layout(16, 4, 256, INT8), [10, 20], tree=True)
    assert names[0] == "verify_tree_attention_q8_split" and names[1] == "verify_tree_attention_reduce" and n[13] == 16
    names, n = prefill_plan(2048, 24, Layout(16, 4, 256, INT8))
    assert names == ["prefill_attention_q8_split", "prefill_attention_reduce"] and n[:2] == [2048, 1]
    assert n[2:5] == [4, 256, 1] and n[5:8] == [4, 48, 256]
    with pytest.raises(ValueError):
        verify_plan(1, 24, Layout(16, 4, 256, FP8E4M3), [10], tree=True)  # tree verify has no fp8 kernels
    with pytest.raises(ValueError):
        verify_plan(1, 20, Layout(16, 4, 256, INT8), [10])  # unsupported attention layout
    with pytest.raises(ValueError):
        verify_plan(1, 24, Layout(16, 4, 256, INT8), [262144 + 8])  # history exceeds the physical context
    # the plain decode plan sizes the streaming kernel's scratch instead
    names, n = verify_plan(64, 24, Layout(16, 4, 256, INT4), [32768] * 64, row_capacity=1, ctas=148)
    assert n[13] == 1 and n[14] == 1 and n[11] == (64 + 148) * 4 * 3 * 6 * 256 * 4


def test_window_plan_fills_the_sms_once():
    """8/16-row int4 windows on a B200: (lanes x heads x splits) CTAs <= SMs, whole 64-token groups per split."""
    layout = Layout(16, 4, 256, INT4)
    names, n = verify_plan(4, 24, layout, [65536] * 4, row_capacity=16, ctas=148)
    assert n[15] == 1 and n[0] == 9 and n[1:5] == [9, 9, 9, 9] and n[5:8] == [4, 9, 4]
    pages = abi.pages_for(65536 + 16)
    per_split = -(-pages // 9)
    assert per_split % 2 == 0 and per_split * 9 >= pages
    # short lanes get fewer splits (at least one group each), one lane alone takes up to 37
    names, n = verify_plan(2, 24, layout, [40, 100000], row_capacity=8, ctas=148)
    assert n[15] == 1 and n[1:3] == [1, 18]
    names, n = verify_plan(1, 24, layout, [262144 - 8], row_capacity=8, ctas=148)
    assert n[15] == 1 and n[0] <= 37 and n[0] * 4 <= 148
    # other formats and the host-only default keep the reference's plan
    assert verify_plan(4, 24, Layout(16, 4, 256, INT8), [65536] * 4, row_capacity=16, ctas=148)[1][15] == 0
    assert verify_plan(4, 24, layout, [65536] * 4, row_capacity=16)[1][15] in (0, 1)


@needs_reference
@pytest.mark.parametrize("fmt", [INT8, INT4, BF16, FP8E4M3])
def test_plans_match_reference(fmt):
    r = om.reference()
    library = lib.load()
    layout = Layout(16, 4, 256, fmt)
    names = C.create_string_buffer(256)
    out = (C.c_uint64 * 16)()
    for lanes, history in [(1, [0]), (2, [31, 4096]), (4, [100, 5000, 32768, 262144]), (3, [65535, 65536, 131072])]:
        for tree in (False, True):
            h = (C.c_uint32 * 4)(*history)
            status = r.ref_verify_plan(lanes, 24, 16, 4, 256, fmt, h, int(tree), names, 256, out)
            if status:
                with pytest.raises(ValueError):
                    verify_plan(lanes, 24, layout, history, tree)
                continue
            mine_names, mine = verify_plan(lanes, 24, layout, history, tree)
            assert mine_names[:2] == names.value.decode().split("\n")
            assert mine[:14] == list(out[:14])
    for rows in (1, 7, 8, 9, 70, 256, 2047, 2048):
        assert r.ref_prefill_plan(rows, 24, 16, 4, 256, fmt, names, 256, out) == 0
        mine_names, mine = prefill_plan(rows, 24, layout)
        assert mine_names == names.value.decode().split("\n") and mine == list(out[:10])
    mine_ws = (C.c_uint64 * 4)()
    ref_ws = (C.c_uint64 * 4)()
    for lanes, rows in [(1, 8), (4, 2048), (2, 100)]:
        assert r.ref_workspaces(lanes, rows, 24, 16, 4, 256, fmt, ref_ws) == 0
        assert library.rk_plan_workspaces(lanes, rows, 24, 16, 4, 256, fmt, mine_ws) == 0
        assert list(mine_ws) == list(ref_ws)
    for case in [(0, 0, 32, 1), (0, 8, 24, 1), (30, 8, 32, 1), (262150, 16, 32, 9000), (0, 8, 32, 1), (0, 2049, 2080, 99)]:
        assert library.rk_chunk_validation_error(*case) == r.ref_chunk_validation(*case)
