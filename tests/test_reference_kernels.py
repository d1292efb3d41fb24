"""CPU: the checker against the reference's OWN kernels. The Metal source of runtime/metal/kernels/common/
paged_store_row.h, paged_attention_tile.h, decode/paged_attention_store.metal and prefill/paged_attention_store.metal is
compiled as C++ in place (oracle/ref_metal_kernels.cpp over oracle/metal_shim) and run on the host, one fiber per Metal
thread. Stores and tree compaction: the row decode, the page addressing, the maximum reduction, the quantiser
expressions, the nibble packing and the copy order are the reference's own text, and every byte of every extent must
agree, for int8, int4, bf16 and fp8 (the hardware's fp8 pack is the reference's own C++ e4m3 conversion). Attention: the reference's tile (admission rule, scale folds, online softmax with bf16
probabilities, conditional rescale, partials and statistics per split) and its fixed-order merge, with the tensor
operations stood in for by plain fp32 sums, against the checker's fp64 attention, chain and tree."""
import ctypes as C

import numpy as np
import pytest

import oracle as om
from kvcase import Scenario, make_staging
from richengine_b200 import lib
from richengine_b200.abi import BF16, INT4, INT8, Layout

reference = om.reference()
pytestmark = pytest.mark.skipif(reference is None or not hasattr(reference, "ref_metal_store_verify"),
                                reason="the reference's kernels were not compiled here")
FORMATS = [INT8, INT4, BF16]


def four_tables(scenario):
    pointers = [t.ctypes.data for t in scenario.host_tables]
    return (C.c_void_p * 4)(*(pointers + [pointers[0]] * (4 - len(pointers))))


def pair(layout, contexts, extra, seed=7):
    """Two scenarios with the same geometry and page placement: the checker writes into one, the reference kernels
    into the other."""
    return Scenario(layout, contexts, extra_tokens=extra, seed=seed), Scenario(layout, contexts, extra_tokens=extra, seed=seed)


def assert_same_bytes(mine, theirs, what):
    for extent, (a, b) in enumerate(zip(mine.host.bytes, theirs.host.bytes)):
        if not np.array_equal(a, b):
            where = np.nonzero(a != b)[0]
            raise AssertionError(f"{what}: extent {extent} differs at {len(where)} bytes, first {where[:8]}: {a[where[:8]]} vs {b[where[:8]]}")


def edge_rows(k, v):
    """Rows that decide the rounding: exact ties of x * range / amax (ties go to even), a zero row, a row with one
    non-zero element, the largest finite bf16, negative zero."""
    bf = lambda x: (np.asarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)
    ties7 = np.array([7.0] + [0.5, 1.5, 2.5, 3.5, 4.5, 5.5, 6.5, -0.5, -1.5, -2.5, -6.5] * 23 + [0.0, -7.0], np.float32)[:256]
    ties127 = np.array([127.0] + [0.5, 1.5, 2.5, 63.5, 126.5, -0.5, -63.5, -126.5] * 31 + [1.0] * 7, np.float32)[:256]
    k[0, 0, 0] = bf(ties7); k[0, 1, 0] = bf(ties127); k[0, 2, 0] = 0; k[0, 3, 0] = 0; k[0, 3, 0, 17] = bf([-3.0])[0]
    k[0, 0, 1] = bf(np.full(256, 3.3895313892515355e38, np.float32)); k[0, 1, 1] = 0x8000
    v[0, 0, :, 0] = bf(ties7); v[0, 1, :, 0] = bf(ties127); v[0, 2, :, 0] = 0; v[0, 3, :, 1] = 0x8000


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows", [1, 8, 15])
def test_verify_store_equals_the_reference_kernel(fmt, rows):
    layout = Layout(2, 4, 256, fmt)
    mine, theirs = pair(layout, [77, 5, 0, 31], 16)
    k, v = make_staging(np.random.default_rng(3), 4, layout)
    edge_rows(k, v)
    for layer in range(2):
        chunk = (lib.ChunkParams * 4)(*[lib.ChunkParams(c, rows, 32, len(p), mine.host.layer(layer)) for c, p in zip(mine.contexts, mine.pages)])
        assert om.oracle().rko_store_verify(fmt, 4, 256, 4, k.ctypes.data, v.ctypes.data, mine.host_table_pointers(), chunk) == 0
        chunk = (lib.ChunkParams * 4)(*[lib.ChunkParams(c, rows, 32, len(p), theirs.host.layer(layer)) for c, p in zip(theirs.contexts, theirs.pages)])
        assert reference.ref_metal_store_verify(fmt, k.ctypes.data, v.ctypes.data, four_tables(theirs), chunk, 4) == 0
    assert any(e.any() for e in mine.host.bytes)
    assert_same_bytes(mine, theirs, "verify store")


@pytest.mark.parametrize("fmt", FORMATS)
def test_chunk_store_equals_the_reference_kernel(fmt):
    layout = Layout(1, 4, 256, fmt)
    mine, theirs = pair(layout, [37], 100)
    rng = np.random.default_rng(4)
    k, v = make_staging(rng, 1, layout, stride=128)
    edge_rows(k, v)
    for scenario, store in ((mine, None), (theirs, reference)):
        params = lib.ChunkParams(37, 100, 128, len(scenario.pages[0]), scenario.host.layer(0))
        if store is None:
            assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, scenario.host_tables[0].ctypes.data, C.byref(params)) == 0
        else:
            assert store.ref_metal_store_chunk(fmt, k.ctypes.data, v.ctypes.data, scenario.host_tables[0].ctypes.data, C.byref(params)) == 0
    assert_same_bytes(mine, theirs, "chunk store")


@pytest.mark.parametrize("fmt", FORMATS)
def test_a_store_the_contract_refuses_writes_nothing_in_either(fmt):
    layout = Layout(1, 4, 256, fmt)
    mine, theirs = pair(layout, [30], 8)
    k, v = make_staging(np.random.default_rng(5), 1, layout)
    for bad in (lib.ChunkParams(30, 8, 24, len(mine.pages[0]), mine.host.layer(0)),      # stride no multiple of 32
                lib.ChunkParams(30, 8, 32, 1, mine.host.layer(0)),                          # page table too short
                lib.ChunkParams(30, 0, 32, len(mine.pages[0]), mine.host.layer(0))):        # no rows
        assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, mine.host_tables[0].ctypes.data, C.byref(bad)) == -1
        assert reference.ref_metal_store_chunk(fmt, k.ctypes.data, v.ctypes.data, theirs.host_tables[0].ctypes.data, C.byref(bad)) == 0
    assert not any(e.any() for e in mine.host.bytes) and not any(e.any() for e in theirs.host.bytes)


@pytest.mark.parametrize("fmt", FORMATS)
def test_tree_compaction_equals_the_reference_kernel(fmt):
    layout = Layout(1, 4, 256, fmt)
    mine, theirs = pair(layout, [29, 64, 7], 16)
    k, v = make_staging(np.random.default_rng(12), 3, layout)
    paths = np.zeros((3, 8), np.uint32)
    paths[0, :4] = [0, 1, 9, 10]
    paths[1, :6] = [0, 8, 2, 3, 11, 14]      # crosses a page boundary: 64 + 8 .. 64 + 14
    counts = np.array([4, 6, 0], np.uint32)
    for scenario in (mine, theirs):
        chunk = (lib.ChunkParams * 3)(*[lib.ChunkParams(c, 15, 32, len(p), scenario.host.layer(0)) for c, p in zip(scenario.contexts, scenario.pages)])
        assert om.oracle().rko_store_verify(fmt, 4, 256, 3, k.ctypes.data, v.ctypes.data, scenario.host_table_pointers(), chunk) == 0
        if scenario is mine:
            for lane in range(3):
                assert om.oracle().rko_tree_compact(fmt, 4, 256, scenario.host_tables[lane].ctypes.data, C.byref(chunk[lane]),
                                                    paths[lane].ctypes.data, int(counts[lane])) == 0
        else:
            assert reference.ref_metal_tree_compact(fmt, four_tables(scenario), chunk, paths.ctypes.data, counts.ctypes.data, 3) == 0
    assert_same_bytes(mine, theirs, "tree compaction")


# ---- attention: the reference's tile and its merge, run on host threads, against the checker's fp64 attention -------
from kvcase import bf16_to_f32, fill_history_with_store, make_queries   # noqa: E402


def reference_attention(fmt, rows, scenario, queries, params, masks, group=6, packed=None):
    lanes = scenario.lanes
    slots = max(p.slot_splits for p in params)
    partials = np.zeros((lanes * 4 * slots, rows * group, 256), np.float32)
    statistics = np.zeros((lanes * 4 * slots, rows * group, 2), np.float32)
    out = np.zeros((lanes, 4, 32, group, 256), np.uint16)
    q = queries.copy()
    hidden = None if packed is None else np.zeros((lanes, 8, 4 * group, 256), np.uint16)
    assert reference.ref_metal_attention_verify(fmt, rows, group, q.ctypes.data, four_tables(scenario), params, lanes,
                                                None if masks is None else masks.ctypes.data, partials.ctypes.data,
                                                statistics.ctypes.data, out.ctypes.data,
                                                None if packed is None else packed.ctypes.data, None if hidden is None else hidden.ctypes.data) == 0
    return out if packed is None else (out, hidden)


def checker_attention(fmt, scenario, queries, params, masks, group=6):
    out = np.zeros((scenario.lanes, 4, 32, group, 256), np.float32)
    out16 = np.zeros((scenario.lanes, 4, 32, group, 256), np.uint16)
    assert om.oracle().rko_attention_verify(fmt, 4, group, 256, scenario.lanes, queries.ctypes.data, scenario.host_table_pointers(), params,
                                            None if masks is None else masks.ctypes.data, out16.ctypes.data, out.ctypes.data) == 0
    return out


def store_rows(fmt, scenario, rows, seed):
    k, v = make_staging(np.random.default_rng(seed), scenario.lanes, scenario.layout)
    chunk = (lib.ChunkParams * scenario.lanes)(*[lib.ChunkParams(c, rows, 32, len(p), scenario.host.layer(0))
                                                 for c, p in zip(scenario.contexts, scenario.pages)])
    assert om.oracle().rko_store_verify(fmt, 4, 256, scenario.lanes, k.ctypes.data, v.ctypes.data, scenario.host_table_pointers(), chunk) == 0


def assert_attention_close(theirs16, mine, active, what):
    """The reference rounds each probability (times its value scale) to bf16 before the value contraction, so its own
    output sits within 2^-8 of the largest magnitude of the exact fp64 attention (a convex combination of values each
    off by at most 2^-9 relative, and a bf16 output). The bar is that bound: what is pinned is the algorithm (admission
    rule, scale folds, online softmax across pages and splits, merge order, zero rows), not the last bit."""
    for lane, rows in enumerate(active):
        got, want = bf16_to_f32(theirs16[lane, :, :rows]), mine[lane, :, :rows]
        bound = 2.0 ** -8 * max(1.0, float(np.abs(want).max())) + np.abs(want) * 2.0 ** -8
        worst = float((np.abs(got - want) - bound).max())
        assert worst <= 0, f"{what}: lane {lane} off by {worst} past the bar"
        assert np.abs(want).max() > 0.05, "a comparison of zeros proves nothing"


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("splits,group", [(1, 6), (3, 6), (2, 4)])
def test_chain_verify_attention_agrees_with_the_reference_tile_and_merge(fmt, splits, group):
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [150, 5, 0, 67], extra_tokens=8)
    fill_history_with_store(s, 0)
    store_rows(fmt, s, 8, 21)
    q = make_queries(np.random.default_rng(6), s.lanes, layout, query_heads=4 * group)
    params = (lib.VerifyParams * 4)(*[lib.VerifyParams(c, len(p), s.host.layer(0), splits, 4, 8, 8, 0.0) for c, p in zip(s.contexts, s.pages)])
    theirs = reference_attention(fmt, 8, s, q, params, None, group)
    mine = checker_attention(fmt, s, q, params, None, group)
    assert_attention_close(theirs, mine, [8, 8, 8, 8], "chain verify")


def tree_case(fmt, group):
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [90, 31], extra_tokens=16)
    fill_history_with_store(s, 0)
    store_rows(fmt, s, 15, 22)
    q = make_queries(np.random.default_rng(7), s.lanes, layout, query_heads=4 * group)
    active = [11, 15]
    params = (lib.VerifyParams * 2)(*[lib.VerifyParams(c, len(p), s.host.layer(0), 2, 2, a, 16, 0.0)
                                      for c, p, a in zip(s.contexts, s.pages, active)])
    rng = np.random.default_rng(8)
    masks = np.zeros((2, 16), np.uint32)
    for lane, rows in enumerate(active):       # a comb: every row sees itself and a random subset of the rows before it
        for row in range(rows):
            masks[lane, row] = (1 << row) | (int(rng.integers(0, 1 << row)) if row else 0)
        masks[lane, 3] = 0                      # a row with an empty mask attends only committed history
    return s, q, params, masks, active


@pytest.mark.parametrize("fmt", FORMATS)
def test_tree_verify_attention_agrees_with_the_reference_tile_and_merge(fmt):
    """Four query heads per KV head: 64 fused rows, four softmax lanes of eight tokens per row, the shape the
    reference's page softmax is written for."""
    s, q, params, masks, active = tree_case(fmt, 4)
    theirs = reference_attention(fmt, 16, s, q, params, masks, 4)
    mine = checker_attention(fmt, s, q, params, masks, 4)
    assert_attention_close(theirs, mine, active, "tree verify")
    for lane, rows in enumerate(active):        # rows past the active ones are written as zeros by the reference's merge
        assert not theirs[lane, :, rows:16].any() and not mine[lane, :, rows:16].any()


def test_the_reference_tree_tile_of_six_heads_normalises_pairs_of_rows_together():
    """A finding, recorded so that nobody mistakes it for a defect of this repository: with six query heads per KV head
    a tree tile has 96 fused rows, more than 64, so the reference's page softmax takes sixteen tokens per lane, two
    lanes per row (paged_attention_tile.h:308), but still folds the row maximum and the row sum over FOUR
    neighbouring lanes (`simd_shuffle_xor(.., 1)` and `(.., 2)`, :147-148 and :162-163). Fused rows 2k and 2k+1 (two
    query heads of one query row) therefore share one denominator: each comes out scaled by its share of the pair's
    sum, and the two shares add up to one. The kernels and the checker of this repository normalise every row by its
    own sum; the chain tile (48 rows) and the tree tile of four heads (64 rows) take the four-lane path and agree."""
    s, q, params, masks, active = tree_case(INT8, 6)
    theirs = bf16_to_f32(reference_attention(INT8, 16, s, q, params, masks, 6))
    mine = checker_attention(INT8, s, q, params, masks, 6)
    shares = []
    for lane, rows in enumerate(active):
        for row in range(rows):
            for pair in range(3):
                a, b = 2 * pair, 2 * pair + 1
                strong = np.abs(mine[lane, 0, row, a]) > 1.0, np.abs(mine[lane, 0, row, b]) > 1.0
                share_a = float(np.median(theirs[lane, 0, row, a][strong[0]] / mine[lane, 0, row, a][strong[0]]))
                share_b = float(np.median(theirs[lane, 0, row, b][strong[1]] / mine[lane, 0, row, b][strong[1]]))
                shares.append(share_a + share_b)
    assert np.allclose(shares, 1.0, atol=0.02), (min(shares), max(shares))


@pytest.mark.parametrize("fmt", FORMATS)
@pytest.mark.parametrize("rows,committed,splits", [(21, 70, 2), (1, 150, 3), (1, 0, 1)])
def test_prefill_and_decode_attention_agree_with_the_reference_phases(fmt, rows, committed, splits):
    """The reference's own prefill split and reduce phases place the tiles (tile_start = 8 x tile, committed +
    tile_start, active = min(8, rows - tile_start)); one row is the plain decode step."""
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [committed], extra_tokens=rows)
    fill_history_with_store(s, 0)
    k, v = make_staging(np.random.default_rng(31), 1, layout, stride=32)
    chunk = lib.ChunkParams(committed, rows, 32, len(s.pages[0]), s.host.layer(0))
    assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, s.host_tables[0].ctypes.data, C.byref(chunk)) == 0
    q = make_queries(np.random.default_rng(32), 1, layout)[0]            # [4][32][6][256], chunk stride 32
    params = lib.PrefillParams(committed, rows, 32, len(s.pages[0]), s.host.layer(0), splits, 0.0)
    tiles = (rows + 7) // 8
    partials = np.zeros((tiles * 4 * splits, 48, 256), np.float32)
    statistics = np.zeros((tiles * 4 * splits, 48, 2), np.float32)
    theirs = np.zeros((4, 32, 6, 256), np.uint16)
    assert reference.ref_metal_attention_prefill(fmt, q.copy().ctypes.data, s.host_tables[0].ctypes.data, C.byref(params),
                                                 partials.ctypes.data, statistics.ctypes.data, theirs.ctypes.data) == 0
    for tile in range(tiles):
        start, active = 8 * tile, min(8, rows - 8 * tile)
        for head in range(4):
            mine = np.zeros((48, 256), np.float32)
            assert om.oracle().rko_attention_tile(fmt, 4, 6, 256, head, q[head, start:].ctypes.data, s.host_tables[0].ctypes.data, s.host.layer(0),
                                                  committed + start, active, 8, None, 0.0, 0, mine.ctypes.data) == 0
            got = bf16_to_f32(theirs[head, start:start + 8]).reshape(48, 256)
            bound = 2.0 ** -8 * max(1.0, float(np.abs(mine).max())) + np.abs(mine) * 2.0 ** -8
            assert (np.abs(got - mine) <= bound).all(), (tile, head, float(np.abs(got - mine).max()))
            assert not got[active * 6:].any() and not mine[active * 6:].any()   # rows past the chunk are zeros in both
            assert np.abs(mine[: active * 6]).max() > 0.05


def test_the_reduce_gate_checker_equals_the_reference_phase():
    """The merge with the gate buffers bound (decode/paged_attention.metal:273-311, run on host threads): the merged
    rows it writes equal the plain merge's, and the gated hidden rows equal oracle/reduce_gate.py applied to them, bit
    for bit (both take the logistic function as 1 / (1 + exp2(-log2(e) x)) in fp32)."""
    import importlib.util
    from pathlib import Path
    spec = importlib.util.spec_from_file_location("rk_reduce_gate_checker", Path(__file__).resolve().parent.parent / "oracle" / "reduce_gate.py")
    checker = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(checker)
    layout = Layout(1, 4, 256, INT4)
    s = Scenario(layout, [150, 5, 40], extra_tokens=8)
    fill_history_with_store(s, 0)
    store_rows(INT4, s, 8, 41)
    q = make_queries(np.random.default_rng(42), s.lanes, layout)
    params = (lib.VerifyParams * 3)(*[lib.VerifyParams(c, len(p), s.host.layer(0), 2, 2, 8, 8, 0.0) for c, p in zip(s.contexts, s.pages)])
    stride = 2 * 24 * 256 + 2 * 4 * 256
    packed = ((np.random.default_rng(43).standard_normal((3, 8, stride)).astype(np.float32) * 3).view(np.uint32) >> 16).astype(np.uint16)
    plain = reference_attention(INT4, 8, s, q, params, None)
    merged, hidden = reference_attention(INT4, 8, s, q, params, None, packed=packed)
    assert np.array_equal(merged, plain)
    rows = merged[:, :, :8].transpose(0, 2, 1, 3, 4).reshape(3, 8, 24, 256)      # [lane][row][kv head x group][dim]
    want = checker.reduce_gate(rows, packed)
    assert np.array_equal(hidden, want) and hidden.any()


# ---- fp8 e4m3: the reference's fp8 store rows and fp8 tile, with its own C++ e4m3 conversions as the hardware's pack ----
from richengine_b200.abi import FP8E4M3   # noqa: E402


def test_fp8_stores_equal_the_reference_kernels():
    layout = Layout(2, 4, 256, FP8E4M3)
    mine, theirs = pair(layout, [77, 5, 0, 31], 16)
    k, v = make_staging(np.random.default_rng(3), 4, layout)
    edge_rows(k, v)
    for layer in range(2):
        for scenario, store in ((mine, None), (theirs, reference)):
            chunk = (lib.ChunkParams * 4)(*[lib.ChunkParams(c, 8, 32, len(p), scenario.host.layer(layer)) for c, p in zip(scenario.contexts, scenario.pages)])
            if store is None:
                assert om.oracle().rko_store_verify(FP8E4M3, 4, 256, 4, k.ctypes.data, v.ctypes.data, scenario.host_table_pointers(), chunk) == 0
            else:
                assert store.ref_metal_store_verify(FP8E4M3, k.ctypes.data, v.ctypes.data, four_tables(scenario), chunk, 4) == 0
    assert_same_bytes(mine, theirs, "fp8 verify store")
    mine, theirs = pair(Layout(1, 4, 256, FP8E4M3), [37], 100)
    k, v = make_staging(np.random.default_rng(4), 1, layout, stride=128)
    edge_rows(k, v)
    for scenario, store in ((mine, None), (theirs, reference)):
        params = lib.ChunkParams(37, 100, 128, len(scenario.pages[0]), scenario.host.layer(0))
        if store is None:
            assert om.oracle().rko_store_chunk(FP8E4M3, 4, 256, k.ctypes.data, v.ctypes.data, scenario.host_tables[0].ctypes.data, C.byref(params)) == 0
        else:
            assert store.ref_metal_store_chunk(FP8E4M3, k.ctypes.data, v.ctypes.data, scenario.host_tables[0].ctypes.data, C.byref(params)) == 0
    assert_same_bytes(mine, theirs, "fp8 chunk store")


@pytest.mark.parametrize("splits", [1, 3])
def test_fp8_chain_verify_attention_agrees_with_the_reference_fp8_tile(splits):
    """fp16-staged queries, fp16 probabilities, two passes of half the fused rows (paged_attention_fp8_tile.h:134-265)."""
    layout = Layout(1, 4, 256, FP8E4M3)
    s = Scenario(layout, [150, 5, 0, 67], extra_tokens=8)
    fill_history_with_store(s, 0)
    store_rows(FP8E4M3, s, 8, 21)
    q = make_queries(np.random.default_rng(6), s.lanes, layout)
    params = (lib.VerifyParams * 4)(*[lib.VerifyParams(c, len(p), s.host.layer(0), splits, 4, 8, 8, 0.0) for c, p in zip(s.contexts, s.pages)])
    theirs = reference_attention(FP8E4M3, 8, s, q, params, None)
    mine = checker_attention(FP8E4M3, s, q, params, None)
    assert_attention_close(theirs, mine, [8, 8, 8, 8], "fp8 chain verify")


@pytest.mark.parametrize("norm_f32", [1, 0])
def test_qkv_prepare_checker_equals_the_reference_storage_phase(norm_f32):
    """kernels/common/attention_qkv_prepare.h run on host threads (with rms_inverse.h): per-head RMS norm, norm weights,
    bf16 rounding, rotary on the first 2 x 32 dims, gate skipped, the three stagings' layouts. The one freedom the
    reference leaves, the order of its 32-wide sum, is the xor butterfly on both sides; everything else is its text.
    Every bit of the three stagings must agree."""
    from kvcase import f32_to_bf16
    rng = np.random.default_rng(17)
    lanes, rows, HQ, HKV, D = 3, 7, 24, 4, 256
    packed_stride = HQ * 2 * D + 2 * HKV * D
    packed = f32_to_bf16((rng.standard_normal((lanes, rows, packed_stride)) * 2).astype(np.float32))
    packed[0, 0, : 2 * D] = 0                                       # a zero head: the norm of nothing
    qn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    if not norm_f32:
        qn, kn = f32_to_bf16(qn), f32_to_bf16(kn)
    angle = rng.uniform(0, 6.28, (lanes, rows, 32)).astype(np.float32)
    cosine, sine = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    outputs = []
    for side in ("mine", "theirs"):
        q = np.zeros((lanes, HKV, 32, HQ // HKV, D), np.uint16)
        k = np.zeros((lanes, HKV, 32, D), np.uint16)
        v = np.zeros((lanes, HKV, D, 32), np.uint16)
        if side == "mine":
            assert om.oracle().rko_qkv_prepare(HKV, HQ, D, lanes, rows, packed.ctypes.data, qn.ctypes.data, kn.ctypes.data, norm_f32,
                                               cosine.ctypes.data, sine.ctypes.data, 1e-6, q.ctypes.data, k.ctypes.data, v.ctypes.data) == 0
        else:
            assert reference.ref_metal_qkv_prepare(packed.ctypes.data, qn.ctypes.data, kn.ctypes.data, norm_f32, cosine.ctypes.data,
                                                   sine.ctypes.data, q.ctypes.data, k.ctypes.data, v.ctypes.data, lanes, rows) == 0
        outputs.append((q, k, v))
    for name, a, b in zip(("queries", "keys", "values"), outputs[0], outputs[1]):
        assert np.array_equal(a, b), f"{name}: {int((a != b).sum())} of {a.size} elements differ"
        assert a.any()


@pytest.mark.parametrize("fmt", [INT4, INT8])
def test_long_contexts_and_the_plan_s_split_counts_agree_with_the_reference(fmt):
    """Thousands of tokens over the split counts the reference's plan picks (32 at these lengths; a lane whose pages do
    not fill them leaves splits unwritten, which the merge must skip)."""
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [4100, 777, 33], extra_tokens=8)
    fill_history_with_store(s, 0)
    store_rows(fmt, s, 8, 51)
    q = make_queries(np.random.default_rng(52), s.lanes, layout)
    params = (lib.VerifyParams * 3)(*[lib.VerifyParams(c, len(p), s.host.layer(0), 32, 32, 8, 8, 0.0) for c, p in zip(s.contexts, s.pages)])
    theirs = reference_attention(fmt, 8, s, q, params, None)
    mine = checker_attention(fmt, s, q, params, None)
    assert_attention_close(theirs, mine, [8, 8, 8], "long chain verify")


@pytest.mark.parametrize("fmt", [INT4, INT8])
def test_the_largest_chunk_store_equals_the_reference_kernel(fmt):
    """2 048 rows, the reference's prefill token budget, appended after 6 144 committed tokens (the prefill benchmark's
    shape): 16 384 threadgroups of the reference's chunk store."""
    layout = Layout(1, 4, 256, fmt)
    mine, theirs = pair(layout, [6144], 2048)
    k, v = make_staging(np.random.default_rng(71), 1, layout, stride=2048)
    for scenario, store in ((mine, None), (theirs, reference)):
        params = lib.ChunkParams(6144, 2048, 2048, len(scenario.pages[0]), scenario.host.layer(0))
        if store is None:
            assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, scenario.host_tables[0].ctypes.data, C.byref(params)) == 0
        else:
            assert store.ref_metal_store_chunk(fmt, k.ctypes.data, v.ctypes.data, scenario.host_tables[0].ctypes.data, C.byref(params)) == 0
    assert_same_bytes(mine, theirs, "largest chunk store")
