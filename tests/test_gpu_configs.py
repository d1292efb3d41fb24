"""GPU: the benchmark configurations at their full sizes, as parity cases against the checker.

cfg 0  one int8 layer, 4096 tokens appended one at a time, then one decode query
cfg 1  int4, batch 8, contexts uniform in 8K-32K: append one token, decode (two layers of the stack)
cfg 2  int4, batch 4 x 64K: 16-row verify windows, seeded acceptance, rejected rows overwritten by the next window
cfg 3  format sweep at batch 32 x 16K: decode of every format (the pool filled on the GPU, read back for the checker)
north star  int4, batch 64 x 32K (one layer of the 16): every lane against the checker, the same bits on a second run,
            the same answer within the bar from a grid cut differently
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (assert_attention_close, assert_extents_equal, chunk_params, dev, run_decode_attention_gpu,
                     run_verify_attention_gpu, run_verify_attention_oracle, struct_to_device)
from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
from richengine_b200 import lib, ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu


def fill_on_gpu_and_mirror(s: Scenario, layers, seed=5):
    """History through the CUDA chunk store (fast), then the device extents become the checker's pool too.
    The stores themselves are compared bit for bit elsewhere; here the pages are inputs."""
    generator = torch.Generator(device="cuda").manual_seed(seed)
    H, D = s.layout.kv_heads, s.layout.head_dimension
    k = torch.randn((H, 2048, D), generator=generator, device="cuda")
    v = torch.randn((H, D, 2048), generator=generator, device="cuda")
    k[:, :, 17] *= 20.0
    v[:, 99, :] *= 20.0
    k, v = k.to(torch.bfloat16), v.to(torch.bfloat16)
    places = s.storage.layers()
    for lane, context in enumerate(s.contexts):
        done = 0
        while done < context:
            rows = min(2048, context - done)
            for layer in layers:
                ops.store_chunk(s.layout, k, v, s.device_tables[lane], lib.ChunkParams(done, rows, 2048, len(s.pages[lane]), places[layer]))
            done += rows
    torch.cuda.synchronize()
    for extent, data in enumerate(s.download()):
        s.host.bytes[extent][:] = data


def test_cfg0_int8_appended_token_by_token_then_decode():
    layout = Layout(1, 4, 256, INT8)  # score scale 0 selects 1/sqrt(256) = 1/16
    s = Scenario(layout, [0], extra_tokens=4096, device=True, seed=40)
    rng = np.random.default_rng(41)
    tokens = 4096
    k_all, v_all = make_staging(rng, 1, layout, stride=32)  # pattern source; fresh rows per token below
    o = om.oracle()
    for token in range(tokens):
        k = np.roll(k_all, token, axis=-1).copy()
        v = np.roll(v_all, token, axis=-2).copy()
        params = chunk_params(s, 1, committed=[token])
        assert o.rko_store_verify(INT8, 4, 256, 1, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
        ops.store_verify(layout, dev(k), dev(v), s.table_pointers, struct_to_device(params), s.storage.layers()[0], 1, 1)
    torch.cuda.synchronize()
    assert_extents_equal(s, "cfg0 pages after 4096 appends")
    q = make_queries(rng, 1, layout)
    committed = [tokens - 1]  # the last appended token is the current row
    got16, got32, _ = run_verify_attention_gpu(s, q, 1, 1, committed=committed)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1, committed=committed)
    assert_attention_close(got32, want32, got16, "cfg0 decode (general tile)")
    w16, w32, _ = run_verify_attention_gpu(s, q, 1, 1, committed=committed, splits=3, tensor_core=True)
    assert_attention_close(w32, want32, w16, "cfg0 decode (window kernel)")
    s.close()


def test_cfg1_int4_ragged_batch_append_and_decode():
    contexts = [int(x) for x in np.random.default_rng(1).integers(8192, 32769, size=8)]
    layout = Layout(2, 4, 256, INT4)
    s = Scenario(layout, contexts, extra_tokens=1, device=True, seed=50)
    fill_on_gpu_and_mirror(s, layers=[0, 1])
    rng = np.random.default_rng(51)
    k, v = make_staging(rng, s.lanes, layout)
    q = make_queries(rng, s.lanes, layout)
    for layer in (0, 1):
        params = chunk_params(s, 1, layer_index=layer)
        assert om.oracle().rko_store_verify(INT4, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
        ops.store_verify(layout, dev(k), dev(v), s.table_pointers, struct_to_device(params), s.storage.layers()[layer], s.lanes, 1)
    torch.cuda.synchronize()
    assert_extents_equal(s, "cfg1 append")
    for layer in (0, 1):
        _, want32 = run_verify_attention_oracle(s, q, 1, 1, layer_index=layer)
        d16, d32 = run_decode_attention_gpu(s, q, layer_index=layer)
        assert_attention_close(d32, want32, d16, f"cfg1 decode layer {layer}")
    s.close()


def test_cfg2_int4_verify_windows_with_rollback():
    layout = Layout(1, 4, 256, INT4)
    s = Scenario(layout, [65536] * 4, extra_tokens=64, device=True, seed=60)
    fill_on_gpu_and_mirror(s, layers=[0])
    rng = np.random.default_rng(61)
    committed = list(s.contexts)
    accepted = [5, 16, 0, 11]
    for step in range(2):
        k, v = make_staging(rng, s.lanes, layout)
        q = make_queries(rng, s.lanes, layout)
        params = chunk_params(s, 16, committed=committed)
        assert om.oracle().rko_store_verify(INT4, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
        ops.store_verify(layout, dev(k), dev(v), s.table_pointers, struct_to_device(params), s.storage.layers()[0], s.lanes, 16)
        torch.cuda.synchronize()
        assert_extents_equal(s, f"cfg2 window store, step {step}")
        got16, got32, _ = run_verify_attention_gpu(s, q, 16, 16, committed=committed, splits=9, tensor_core=True)
        _, want32 = run_verify_attention_oracle(s, q, 16, 16, committed=committed)
        assert_attention_close(got32, want32, got16, f"cfg2 window attention, step {step}")
        # the accepted rows stay; the rejected tail is overwritten by the next window
        committed = [c + a for c, a in zip(committed, accepted)]
    s.close()


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
def test_cfg3_format_sweep_decode(fmt):
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [16384] * 32, extra_tokens=1, device=True, seed=70)
    fill_on_gpu_and_mirror(s, layers=[0])
    rng = np.random.default_rng(71)
    q = make_queries(rng, s.lanes, layout)
    committed = [c - 1 for c in s.contexts]  # the last stored token is the current row
    _, want32 = run_verify_attention_oracle(s, q, 1, 1, committed=committed)
    d16, d32 = run_decode_attention_gpu(s, q, committed=committed)
    assert_attention_close(d32, want32, d16, f"cfg3 format {fmt} decode (streaming kernel)")
    w16, w32, _ = run_verify_attention_gpu(s, q, 1, 1, committed=committed, splits=1, tensor_core=True)
    assert_attention_close(w32, want32, w16, f"cfg3 format {fmt} decode (window kernel)")
    s.close()


def test_north_star_size_int4_batch64_ctx32k_decode():
    """The size the headline number is quoted on, one layer of it (2.2 GB of int4 pages): the streaming kernel's
    output of ALL 64 lanes against the checker, bit-identical on a second run (the cut, the folds and the merge order
    depend on the lanes' page counts and the grid alone), and within the bar again when the same pages are cut for 37
    CTAs instead of one per SM (other ranges, other lane boundaries inside a range, other folds)."""
    layout = Layout(1, 4, 256, INT4)
    s = Scenario(layout, [32768] * 64, extra_tokens=1, device=True, seed=90)
    fill_on_gpu_and_mirror(s, layers=[0])
    rng = np.random.default_rng(91)
    q = make_queries(rng, s.lanes, layout)
    committed = [c - 1 for c in s.contexts]
    _, want32 = run_verify_attention_oracle(s, q, 1, 1, committed=committed)
    d16, d32 = run_decode_attention_gpu(s, q, committed=committed)
    assert_attention_close(d32, want32, d16, "north-star size, one CTA per SM")
    again16, again32 = run_decode_attention_gpu(s, q, committed=committed)
    assert np.array_equal(d16, again16) and np.array_equal(d32.view(np.uint32), again32.view(np.uint32))
    other16, other32 = run_decode_attention_gpu(s, q, committed=committed, ctas=37)
    assert_attention_close(other32, want32, other16, "north-star size, 37 CTAs")
    s.close()


class TableView:
    """What the attention helpers need of a scenario, over tables that came from the request cache."""

    def __init__(self, layout, storage, mirror, page_lists, contexts):
        self.layout, self.storage, self.host = layout, storage, mirror
        self.pages, self.contexts, self.lanes = page_lists, contexts, len(page_lists)
        self.device_tables = []
        for pages in page_lists:
            table = torch.zeros(len(pages), dtype=torch.int64, device="cuda")
            storage.write_entries(pages, 0, table)
            self.device_tables.append(table)
        self.table_pointers = ops.table_pointer_array(self.device_tables)
        self.host_tables = [mirror.table(p) for p in page_lists]

    def host_table_pointers(self):
        return (C.c_void_p * self.lanes)(*[t.ctypes.data for t in self.host_tables])


def test_cfg3_prefix_shared_by_32_requests_fork_diverge_decode():
    """32 requests fork one published prefix of 256 refcounted pages (the last one partial: copy-on-write), each
    appends 512 tokens of its own, and every request decodes through its forked table: shared pages stay
    bit-identical to the checker's mirror, refcounts add up, attention through shared + own pages meets the bar."""
    from test_gpu_hostplane import World
    from richengine_b200.hostplane import GRANTED
    layout = Layout(1, 4, 256, INT4)
    w = World(layout, 1024, 128)
    prefix_tokens = 32 * 256 - 9  # 256 pages, the last one holds 23 tokens
    children = list(range(2, 34))
    ids = np.random.default_rng(3).integers(0, 50000, size=prefix_tokens + 1, dtype=np.uint32)
    w.cache.begin_request(1)
    assert w.cache.ensure_tokens(1, prefix_tokens) == GRANTED
    done = 0
    while done < prefix_tokens:  # chunk stores of at most 2048 rows
        rows = min(2048, prefix_tokens - done)
        w.append(1, done, rows)
        done += rows
    w.cache.publish(1, ids, prefix_tokens)
    parent_pages = w.cache.page_table(1)[0]
    assert len(parent_pages) == 256
    for child in children:
        w.cache.begin_request(child)
        assert w.cache.fork(1, child, prefix_tokens) == 1  # one page copied: the partial tail
        pages = w.cache.page_table(child)[0]
        assert pages[:255] == parent_pages[:255] and pages[255] not in parent_pages
        om.oracle().rko_copy_page(INT4, 1, 4, 256, 128, w.mirror.entry(parent_pages[255]), w.mirror.entry(pages[255]))
        assert w.cache.ensure_tokens(child, prefix_tokens + 512 + 1) == GRANTED
        w.append(child, prefix_tokens, 512, seed=child)
    torch.cuda.synchronize()
    snapshot = w.pool.snapshot()
    own = len(w.cache.page_table(2)[0]) - 255
    assert snapshot["pages_active"] == 256 + 32 * own and w.cache.snapshot()["fork_copies"] == 32
    for extent in range(w.mirror.extents):  # every byte of the pool, shared and private pages alike
        if w.storage.is_allocated(extent * 128):
            assert np.array_equal(w.storage.read_extent(extent), w.mirror.bytes[extent]), f"extent {extent}"
    # decode through the forked tables (the parent rides along as lane 0)
    requests = [1] + children
    page_lists = [w.cache.page_table(r)[0] for r in requests]
    committed = [prefix_tokens - 1] + [prefix_tokens + 512 - 1] * 32  # the last stored token is the current row
    view = TableView(layout, w.storage, w.mirror, page_lists, committed)
    q = make_queries(np.random.default_rng(72), view.lanes, layout)
    _, want32 = run_verify_attention_oracle(view, q, 1, 1, committed=committed)
    d16, d32 = run_decode_attention_gpu(view, q, committed=committed)
    assert_attention_close(d32, want32, d16, "cfg3 decode through forked tables")
    # children share 255 pages but not their answers
    assert not np.array_equal(d16[1], d16[2])
    for r in requests:
        w.cache.end_request(r)
    assert w.pool.snapshot()["pages_active"] == 0
    w.close()


@pytest.mark.parametrize("history", [131072, 260096])
def test_long_histories_decode(history):
    """The longest histories the reference's plan tests run (dev/tests/engine/paged_attention_plan_test.mm:999-1012):
    one int4 lane, streaming decode against the checker."""
    layout = Layout(1, 4, 256, INT4)
    s = Scenario(layout, [history], extra_tokens=1, device=True, seed=80, extent_pages=256)
    fill_on_gpu_and_mirror(s, layers=[0])
    q = make_queries(np.random.default_rng(81), 1, layout)
    committed = [history - 1]
    _, want32 = run_verify_attention_oracle(s, q, 1, 1, committed=committed)
    d16, d32 = run_decode_attention_gpu(s, q, committed=committed)
    assert_attention_close(d32, want32, d16, f"decode over {history} tokens")
    s.close()
