"""GPU: the operator's encoders (ops::PagedAttention::addVerify / addPrefill / addPrefillStore /
addVerifyTreeCompact, runtime/ops/PagedAttention.cpp:399-573) through their C handles: a verify step and a prefill
chunk give the checker's result, and every refusal the reference makes before it encodes anything
(dev/tests/engine/paged_attention_plan_test.mm:717-761,807-812: undersized scratch, aliased queries and output, a
missing tree mask, a plan of another row count) leaves pages and outputs untouched: nothing was launched."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (assert_attention_close, assert_extents_equal, chunk_params, dev, host_u16, run_verify_attention_oracle,
                     struct_to_device, verify_params)
from kvcase import Scenario, bf16_to_f32, fill_history_with_store, make_queries, make_staging
from richengine_b200 import lib, ops
from richengine_b200.abi import INT4, INT8, Layout

pytestmark = pytest.mark.gpu
CANARY = 0x3C3C  # bf16 bit pattern no kernel writes by accident


class VerifyStep:
    """One verify batch bound the way a runtime binds it: stagings, scratch sized from the plan, device parameter blocks."""

    def __init__(self, s: Scenario, rows: int, fmt: int, tree: bool = False, seed: int = 91):
        library = lib.load()
        self.library, self.s, self.rows = library, s, rows
        layout = s.layout
        rng = np.random.default_rng(seed)
        self.k, self.v = make_staging(rng, s.lanes, layout)
        self.q = make_queries(rng, s.lanes, layout)
        history = (C.c_uint32 * s.lanes)(*s.contexts)
        self.plan = library.rk_op_verify_plan(s.lanes, 24, 1, 4, 256, fmt, history, int(tree), rows, 0)
        assert self.plan, library.rk_last_error()
        info = (C.c_uint64 * 6)()
        assert library.rk_op_plan_workspace(self.plan, info) == lib.OK
        self.partials_bytes, self.statistics_bytes, self.splits = int(info[0]), int(info[1]), int(info[2])
        self.streaming, self.window_kernel = bool(info[4] & 1), bool(info[4] & 2)
        self.partials = torch.zeros(max(self.partials_bytes, 4) // 4, dtype=torch.float32, device="cuda")
        self.statistics = torch.zeros(max(self.statistics_bytes, 4) // 4, dtype=torch.float32, device="cuda")
        self.descriptors = torch.zeros(max(int(info[5]), 4) // 4, dtype=torch.int32, device="cuda")
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        base, size = s.storage.window()
        self.window = library.rk_window_create(base, size)
        self.dk, self.dv, self.dq = dev(self.k), dev(self.v), dev(self.q)
        self.out = torch.full_like(self.dq, CANARY)
        self.chunks = chunk_params(s, rows)
        self.d_chunks = struct_to_device(self.chunks)
        lane_splits = [library.rk_op_plan_lane_splits(self.plan, lane) for lane in range(s.lanes)]
        attention = (lib.VerifyParams * s.lanes)()
        for lane in range(s.lanes):
            attention[lane] = lib.VerifyParams(s.contexts[lane], len(s.pages[lane]), s.host.layer(0), lane_splits[lane],
                                               self.splits, rows, rows, 0.0)
        self.d_attention = struct_to_device(attention)
        # sixteen-row windows run the tree kernels (the reference's 16-row tile is its tree tile): a causal chain is the
        # ancestor masks (1 << (row + 1)) - 1
        self.masks = dev(np.tile(((1 << (np.arange(16, dtype=np.uint64) + 1)) - 1).astype(np.uint32), (s.lanes, 1))) if rows == 16 else None

    def buffers(self, **changes) -> lib.VerifyBuffers:
        fields = dict(chunk_keys=self.dk.data_ptr(), chunk_values=self.dv.data_ptr(), queries=self.dq.data_ptr(),
                      output=self.out.data_ptr(), partials=self.partials.data_ptr(), statistics=self.statistics.data_ptr(),
                      descriptors=self.descriptors.data_ptr(), status=self.status.data_ptr(),
                      page_tables=self.s.table_pointers.data_ptr(),
                      tree_masks=self.masks.data_ptr() if self.masks is not None else None, partials_bytes=self.partials_bytes,
                      statistics_bytes=self.statistics_bytes)
        fields.update(changes)
        return lib.VerifyBuffers(**fields)

    def add(self, plan=None, **changes) -> int:
        b = self.buffers(**changes)
        return self.library.rk_op_add_verify(torch.cuda.current_stream().cuda_stream, self.s.storage.layers()[0], C.byref(b),
                                             self.d_chunks.data_ptr(), self.d_attention.data_ptr(), plan or self.plan, self.window)

    def close(self):
        self.library.rk_op_plan_destroy(self.plan)
        self.library.rk_window_destroy(self.window)


def prepared(contexts, fmt, rows, seed=90):
    s = Scenario(Layout(1, 4, 256, fmt), contexts, extra_tokens=rows, device=True, seed=seed)
    fill_history_with_store(s, 0, seed=seed)
    s.upload()
    return s


@pytest.mark.parametrize("fmt,rows", [(INT4, 16), (INT4, 8), (INT8, 8), (INT4, 1)])
def test_add_verify_stores_attends_and_merges(fmt, rows):
    s = prepared([700, 33, 1500, 64], fmt, rows)
    step = VerifyStep(s, rows, fmt)
    assert step.add() == lib.OK, step.library.rk_last_error()
    torch.cuda.synchronize()
    assert int(step.status.item()) == 0
    # the same step on the checker: store, then attention
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, step.k.ctypes.data, step.v.ctypes.data, s.host_table_pointers(), step.chunks) == 0
    assert_extents_equal(s, "addVerify store")
    _, want32 = run_verify_attention_oracle(s, step.q, rows, rows)
    got16 = host_u16(step.out)
    scale = max(1.0, float(np.abs(want32).max()))
    live = bf16_to_f32(got16[:, :, :rows])
    assert (np.abs(live - want32[:, :, :rows]) <= 2e-3 * scale + np.abs(want32[:, :, :rows]) * 2.0 ** -8).all()
    step.close(); s.close()


def test_add_verify_refusals_launch_nothing():
    s = prepared([700, 33, 1500, 64], INT4, 16)
    step = VerifyStep(s, 16, INT4)
    library = step.library
    tree = VerifyStep(s, 16, INT4, tree=True)
    # each refusal carries the reference's text (read right after the call)
    assert step.add(partials_bytes=step.partials_bytes - 4) == lib.INVALID and b"scratch is smaller" in library.rk_last_error()
    assert step.add(statistics_bytes=step.statistics_bytes - 4) == lib.INVALID and b"scratch is smaller" in library.rk_last_error()
    assert step.add(output=step.dq.data_ptr()) == lib.INVALID and b"must not alias" in library.rk_last_error()
    assert tree.add(tree_masks=None) == lib.INVALID and b"ancestor masks" in library.rk_last_error()
    assert step.add(page_tables=None) == lib.INVALID and b"invalid paged verify batch" in library.rk_last_error()
    assert step.window_kernel and step.add(status=None) == lib.INVALID and b"status word" in library.rk_last_error()
    torch.cuda.synchronize()
    # nothing ran: the pages are the history's, the output still holds its canary, the scratch is clean
    assert_extents_equal(s, "refused calls")
    assert (host_u16(step.out) == CANARY).all() and not step.partials.any() and not step.statistics.any()
    # and the same buffers then take the valid call
    assert step.add() == lib.OK
    torch.cuda.synchronize()
    assert not (host_u16(step.out)[:, :, :16] == CANARY).all()
    for x in (step, tree):
        x.close()
    s.close()


@pytest.mark.parametrize("window_kernel", [False, True])
def test_add_prefill_store_and_prefill(window_kernel):
    library = lib.load()
    fmt, history, rows = INT4, 1000, 200
    s = Scenario(Layout(1, 4, 256, fmt), [history], extra_tokens=rows, device=True, seed=95)
    fill_history_with_store(s, 0, seed=95)
    s.upload()
    rng = np.random.default_rng(96)
    stride = (rows + 31) // 32 * 32
    from kvcase import f32_to_bf16
    k = f32_to_bf16(rng.standard_normal((4, stride, 256)).astype(np.float32))
    v = f32_to_bf16(rng.standard_normal((4, 256, stride)).astype(np.float32))
    q = f32_to_bf16(rng.standard_normal((4, stride, 6, 256)).astype(np.float32))
    dk, dv, dq = dev(k), dev(v), dev(q)
    out = torch.full_like(dq, CANARY)
    plan = library.rk_op_prefill_plan(rows, 24, 1, 4, 256, fmt)
    wrong_plan = library.rk_op_prefill_plan(rows - 8, 24, 1, 4, 256, fmt)
    info = (C.c_uint64 * 6)()
    assert library.rk_op_plan_workspace(plan, info) == lib.OK
    partials = torch.zeros(int(info[0]) // 4, dtype=torch.float32, device="cuda")
    statistics = torch.zeros(int(info[1]) // 4, dtype=torch.float32, device="cuda")
    status_word = torch.zeros(1, dtype=torch.int32, device="cuda")
    base, size = s.storage.window()
    window = library.rk_window_create(base, size) if window_kernel else None
    stream = torch.cuda.current_stream().cuda_stream
    place = s.storage.layers()[0]
    table = s.device_tables[0]
    chunk = lib.ChunkParams(history, rows, stride, len(s.pages[0]), place)

    def add_prefill(plan_handle=plan, queries=dq, output=out, partials_bytes=int(info[0])):
        return library.rk_op_add_prefill(stream, place, queries.data_ptr(), output.data_ptr(), partials.data_ptr(), statistics.data_ptr(),
                                         partials_bytes, int(info[1]), table.data_ptr(), C.byref(chunk), plan_handle, window,
                                         status_word.data_ptr() if window_kernel else None)
    # refusals first: a plan of another row count, undersized scratch, aliasing, an invalid chunk — nothing launched
    assert add_prefill(plan_handle=wrong_plan) == lib.INVALID and b"do not match plan" in library.rk_last_error()
    assert add_prefill(partials_bytes=int(info[0]) - 4) == lib.INVALID and b"scratch is smaller" in library.rk_last_error()
    assert add_prefill(output=dq) == lib.INVALID and b"must not alias" in library.rk_last_error()
    bad = lib.ChunkParams(history, rows, stride - 1, len(s.pages[0]), place)
    assert library.rk_op_add_prefill_store(stream, place, dk.data_ptr(), dv.data_ptr(), table.data_ptr(), C.byref(bad), 1, 4, 256, fmt) == lib.INVALID
    torch.cuda.synchronize()
    assert_extents_equal(s, "refused prefill calls")
    assert (host_u16(out) == CANARY).all() and not partials.any()
    # the chunk: store, then causal attention over history + chunk
    assert library.rk_op_add_prefill_store(stream, place, dk.data_ptr(), dv.data_ptr(), table.data_ptr(), C.byref(chunk), 1, 4, 256, fmt) == lib.OK
    assert add_prefill() == lib.OK, library.rk_last_error()
    torch.cuda.synchronize()
    assert int(status_word.item()) == 0
    host_chunk = lib.ChunkParams(history, rows, stride, len(s.pages[0]), s.host.layer(0))
    assert om.oracle().rko_store_chunk(fmt, 4, 256, k.ctypes.data, v.ctypes.data, s.host_tables[0].ctypes.data, C.byref(host_chunk)) == 0
    assert_extents_equal(s, "addPrefillStore")
    got = bf16_to_f32(host_u16(out))
    want = np.zeros((4, stride, 6, 256), np.float32)
    for head in range(4):
        for tile in range((rows + 7) // 8):
            active = min(8, rows - 8 * tile)
            tile_out = np.zeros((8 * 6, 256), np.float32)
            tile_q = np.ascontiguousarray(q[head, 8 * tile:8 * tile + 8])
            assert om.oracle().rko_attention_tile(fmt, 4, 6, 256, head, tile_q.ctypes.data, s.host_tables[0].ctypes.data, s.host.layer(0),
                                                  history + 8 * tile, active, 8, None, 0.0, 0, tile_out.ctypes.data) == 0
            want[head, 8 * tile:8 * tile + active] = tile_out.reshape(8, 6, 256)[:active]
    scale = max(1.0, float(np.abs(want).max()))
    assert (np.abs(got[:, :rows] - want[:, :rows]) <= 2e-3 * scale + np.abs(want[:, :rows]) * 2.0 ** -8).all()
    library.rk_op_plan_destroy(plan); library.rk_op_plan_destroy(wrong_plan)
    if window:
        library.rk_window_destroy(window)
    s.close()


def test_add_verify_tree_compact_moves_the_retained_path():
    library = lib.load()
    fmt = INT4
    s = Scenario(Layout(1, 4, 256, fmt), [90, 40], extra_tokens=16, device=True, seed=97)
    fill_history_with_store(s, 0, seed=97)
    rng = np.random.default_rng(98)
    k, v = make_staging(rng, s.lanes, s.layout)
    params = chunk_params(s, 8)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    paths = np.array([[0, 2, 5, 7, 0, 0, 0, 0], [0, 1, 6, 0, 0, 0, 0, 0]], dtype=np.uint32)
    counts = np.array([4, 3], dtype=np.uint32)
    stream = torch.cuda.current_stream().cuda_stream
    # a batch without lanes is refused before anything moves; fp8 has no tree kernels
    assert library.rk_op_add_verify_tree_compact(stream, s.storage.layers()[0], s.table_pointers.data_ptr(), dev(paths).data_ptr(),
                                                 dev(counts).data_ptr(), struct_to_device(params).data_ptr(), 0, 1, 4, 256, fmt) == lib.INVALID
    assert library.rk_op_add_verify_tree_compact(stream, s.storage.layers()[0], s.table_pointers.data_ptr(), dev(paths).data_ptr(),
                                                 dev(counts).data_ptr(), struct_to_device(params).data_ptr(), s.lanes, 1, 4, 256, 4) == lib.INVALID
    torch.cuda.synchronize()
    assert_extents_equal(s, "refused compaction")
    assert library.rk_op_add_verify_tree_compact(stream, s.storage.layers()[0], s.table_pointers.data_ptr(), dev(paths).data_ptr(),
                                                 dev(counts).data_ptr(), struct_to_device(params).data_ptr(), s.lanes, 1, 4, 256, fmt) == lib.OK
    torch.cuda.synchronize()
    for lane in range(s.lanes):
        host_params = lib.ChunkParams(s.contexts[lane], 8, 32, len(s.pages[lane]), s.host.layer(0))
        assert om.oracle().rko_tree_compact(fmt, 4, 256, s.host_tables[lane].ctypes.data, C.byref(host_params),
                                            paths[lane].ctypes.data, int(counts[lane])) == 0
    assert_extents_equal(s, "addVerifyTreeCompact")
    s.close()
