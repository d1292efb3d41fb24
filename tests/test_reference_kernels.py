"""CPU: the checker's stores and tree compaction against the reference's OWN kernels. The Metal source of
runtime/metal/kernels/common/paged_store_row.h, decode/paged_attention_store.metal and prefill/paged_attention_store.metal
is compiled as C++ in place (oracle/ref_metal_store.cpp over oracle/metal_shim/metal_stdlib) and run on host threads,
one per Metal thread: the row decode, the page addressing, the maximum reduction, the quantiser expressions, the nibble
packing and the copy order are the reference's own text. Every byte of every extent must agree, for int8, int4 and
bf16 (the fp8 store needs the hardware's fp8 pack; its encoder is pinned by the reference's C++ fp8 reference instead)."""
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
