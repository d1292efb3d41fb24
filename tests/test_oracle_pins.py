"""CPU: pins the C++ restatement against the reference's own portable code (compiled in
place when the checkout exists) and against the closed-form fixtures of its tests."""
import ctypes as C

import numpy as np
import pytest

import oracle as om
from kvcase import HostPool, Scenario, bf16_to_f32, f32_to_bf16, fill_history_with_store, make_queries
from richengine_b200 import abi, lib
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

needs_reference = pytest.mark.skipif(om.reference() is None, reason="reference checkout was not compiled here")


def layout_for(fmt, layers=1):
    return Layout(layers, 4, 256, fmt)


# ---- byte accounting: dev/tests/engine/q8_paged_kv_test.cc:17-61 -----------------------------------
def test_layout_byte_accounting_matches_reference_asserts():
    q8 = Layout(16, 4, 256, INT8)
    assert q8.elements_per_layer_page() == 32768
    assert q8.bytes_per_layer_page() == 66560 and q8.bytes_per_model_page() == 1064960
    assert q8.extent_alignment_pages() == 128 and q8.extent_pages_for(4096) == 128
    assert Layout(16, 4, 256, INT4).bytes_per_model_page() == 540672
    assert Layout(16, 4, 256, BF16).bytes_per_model_page() == 2097152
    assert Layout(16, 4, 256, FP8E4M3).bytes_per_model_page() == 1064960
    assert [Layout(16, 4, 256, f).bytes_per_token_layer() for f in (INT4, INT8, FP8E4M3, BF16)] == [1056, 2080, 2080, 4096]


@needs_reference
@pytest.mark.parametrize("fmt", [INT8, BF16, INT4, FP8E4M3])
@pytest.mark.parametrize("heads,dim,layers", [(4, 256, 16), (2, 256, 12), (8, 64, 10), (2, 128, 28)])
def test_layout_matches_reference(fmt, heads, dim, layers):
    r = om.reference()
    out = (C.c_uint64 * 8)()
    l = Layout(layers, heads, dim, fmt)
    for pool_pages in (100, 1000, 4096, 50000):
        r.ref_layout(layers, heads, dim, fmt, pool_pages, out)
        assert list(out) == [l.data_bytes_per_layer_page(), l.scale_bytes_per_layer_page(), l.bytes_per_layer_page(),
                             l.bytes_per_model_page(), l.extent_alignment_pages(), l.minimum_extent_pages(),
                             l.maximum_extent_pages(), l.extent_pages_for(pool_pages)]
    rng = np.random.default_rng(0)
    for _ in range(200):
        ep = int(rng.integers(1, 300)); layer = int(rng.integers(0, layers)); tensor = int(rng.integers(0, 4))
        index = int(rng.integers(0, ep))
        d, s = l.data_bytes_per_layer_page(), l.scale_bytes_per_layer_page()
        assert r.ref_kv_offset(ep, d, s, layer, tensor, index) == l.layer_offset(ep, layer, tensor, index)
    for c, rows in [(0, 8), (100, 8), (32768, 8), (65536, 15), (262144, 15), (511, 8), (16 * 32 * 33, 8)]:
        assert r.ref_verify_splits(c, rows) == abi.verify_attention_splits(c, rows)


# ---- scalar conversions ------------------------------------------------------------------------------
@needs_reference
def test_conversions_match_reference():
    o, r = om.oracle(), om.reference()
    for code in range(256):
        a, b = o.rko_e4m3_to_f32(code), r.ref_e4m3_to_f32(code)
        assert (np.isnan(a) and np.isnan(b)) or a == b
        if not np.isnan(a):
            assert o.rko_f32_to_e4m3(a) == code or a == 0.0  # encode(decode) is the identity
    rng = np.random.default_rng(1)
    values = np.concatenate([rng.standard_normal(4000) * 10 ** rng.uniform(-6, 3, 4000),
                             [0.0, -0.0, 448.0, 464.0, 463.99, 480.0, 500.0, 511.9, 512.0, 1e9, 2 ** -6, 2 ** -7,
                              2 ** -9, 2 ** -10, 1.5 * 2 ** -10, 0.0009765625 * 2.5, 240.0, 248.0, 232.0]]).astype(np.float32)
    for v in values:
        for sign in (1.0, -1.0):
            x = float(v) * sign
            assert o.rko_f32_to_e4m3(x) == r.ref_f32_to_e4m3(x), x
            assert o.rko_f32_to_bf16(x) == r.ref_f32_to_bf16(x)
            assert o.rko_query_stage_f16(x) == r.ref_query_stage(x)
    bits = f32_to_bf16(values)
    for v, b in zip(values, bits):  # the numpy helper used by the fixtures agrees too
        assert int(b) == r.ref_f32_to_bf16(float(v))


def test_e4m3_known_answers():
    """Fp8PageFormatReference.hpp:27-52: bias 7, max 448 = 0x7E, subnormal step 2^-9."""
    o = om.oracle()
    assert o.rko_f32_to_e4m3(448.0) == 0x7E and o.rko_f32_to_e4m3(1e6) == 0x7E and o.rko_f32_to_e4m3(-1e6) == 0xFE
    assert o.rko_f32_to_e4m3(1.0) == 0x38 and o.rko_f32_to_e4m3(-1.0) == 0xB8
    assert o.rko_f32_to_e4m3(2.0 ** -9) == 0x01 and o.rko_f32_to_e4m3(2.0 ** -6) == 0x08
    assert o.rko_f32_to_e4m3(0.0) == 0 and o.rko_f32_to_e4m3(-0.0) == 0x80
    assert o.rko_e4m3_to_f32(0x7E) == 448.0 and o.rko_e4m3_to_f32(0x01) == 2.0 ** -9
    assert o.rko_f32_to_e4m3(464.0) == 0x7E and o.rko_f32_to_e4m3(1.0625) == 0x38 and o.rko_f32_to_e4m3(1.1875) == 0x3A


# ---- page quantizers vs the reference's int8 / fp8 references -----------------------------------------
def _store_one_page(fmt, keys_f32, values_f32, valid):
    """Stores `valid` tokens [token][head][dim] through the checker into a one-page pool; returns the pool."""
    layout = layout_for(fmt)
    pool = HostPool(layout, layout.extent_alignment_pages(), 1)
    H, D = 4, 256
    k = np.zeros((H, 32, D), np.uint16); v = np.zeros((H, D, 32), np.uint16)
    k[:, :valid, :] = f32_to_bf16(keys_f32).reshape(valid, H, D).transpose(1, 0, 2)
    v[:, :, :valid] = f32_to_bf16(values_f32).reshape(valid, H, D).transpose(1, 2, 0)
    table = pool.table([5])
    params = lib.ChunkParams(0, valid, 32, 1, pool.layer(0))
    assert om.oracle().rko_store_chunk(fmt, H, D, k.ctypes.data, v.ctypes.data, table.ctypes.data, C.byref(params)) == 0
    return pool


@needs_reference
@pytest.mark.parametrize("fmt", [INT8, FP8E4M3])
@pytest.mark.parametrize("valid", [1, 17, 32])
def test_store_matches_reference_page_quantizer(fmt, valid):
    rng = np.random.default_rng(valid)
    shape = (valid, 4, 256)
    keys = rng.standard_normal(shape).astype(np.float32) * 3
    values = rng.standard_normal(shape).astype(np.float32) * 0.01
    keys[0, 1, :] = 0.0  # an all-zero row stores scale 0 and codes 0
    values[:, :, 7] *= 50.0
    keys, values = bf16_to_f32(f32_to_bf16(keys)), bf16_to_f32(f32_to_bf16(values))  # bf16-exact inputs
    pool = _store_one_page(fmt, keys, values, valid)
    expected = np.zeros(66560, np.uint8)
    fn = om.reference().ref_q8_quantize_page if fmt == INT8 else om.reference().ref_fp8_quantize_page
    assert fn(keys.ctypes.data, values.ctypes.data, valid, expected.ctypes.data) == 0
    got = np.concatenate([pool.tensor_view(5, 0, t) for t in range(4)])
    assert np.array_equal(got, expected)
    assert not pool.bytes[0][: pool.layout.layer_offset(pool.extent_pages, 0, 0, 5)].any()  # other pages untouched


# ---- int4 / bf16 stores: expected bytes as dev/tests/engine/paged_attention_plan_test.mm:573-627,681-699 ----
def test_int4_store_expected_bytes():
    rng = np.random.default_rng(3)
    layout = layout_for(INT4)
    pool = HostPool(layout, 128, 1)
    H, D, rows, committed = 4, 256, 8, 27  # rows straddle a page boundary
    k = f32_to_bf16(rng.standard_normal((H, 32, D)).astype(np.float32))
    v = f32_to_bf16(rng.standard_normal((H, D, 32)).astype(np.float32))
    pages = [9, 3]
    table = pool.table(pages)
    params = lib.ChunkParams(committed, rows, 32, 2, pool.layer(0))
    assert om.oracle().rko_store_chunk(INT4, H, D, k.ctypes.data, v.ctypes.data, table.ctypes.data, C.byref(params)) == 0
    expected = [np.zeros_like(b) for b in pool.bytes]
    shadow = HostPool(layout, 128, 1)
    for tensor, src in ((0, bf16_to_f32(k)), (2, bf16_to_f32(v).transpose(0, 2, 1))):
        for row in range(rows):
            token = committed + row
            page = pages[token // 32]
            for head in range(H):
                x = src[head, row]
                amax = np.float32(np.abs(x).max())
                scale = np.float32(0) if amax == 0 else np.float32(amax / np.float32(7))
                codes = np.clip(np.rint((x * np.float32(7)) / amax), -7, 7).astype(np.int32)
                data = shadow.tensor_view(page, 0, tensor)
                base = (head * 32 + token % 32) * D // 2
                data[base:base + D // 2] = (codes[0::2] & 0xF) | ((codes[1::2] & 0xF) << 4)
                shadow.tensor_view(page, 0, tensor + 1).view(np.float32)[head * 32 + token % 32] = scale
    assert np.array_equal(pool.bytes[0], shadow.bytes[0])


def test_bf16_store_preserves_edge_bit_patterns():
    bits = np.array([0, 0x8000, 1, 0x8001, 0x007f, 0x0080, 0x4960, 0x7f7f, 0xff7f, 0x7f80, 0xff80, 0x7fc3], np.uint16)
    layout = layout_for(BF16)
    pool = HostPool(layout, 4, 1)
    H, D = 4, 256
    k = np.resize(bits, H * 32 * D).reshape(H, 32, D).copy()
    v = np.resize(bits[::-1], H * D * 32).reshape(H, D, 32).copy()
    table = pool.table([2, 1])
    params = lib.ChunkParams(31, 2, 32, 2, pool.layer(0))
    assert om.oracle().rko_store_chunk(BF16, H, D, k.ctypes.data, v.ctypes.data, table.ctypes.data, C.byref(params)) == 0
    for row, (page, pt) in enumerate([(2, 31), (1, 0)]):
        keys = pool.tensor_view(page, 0, 0).view(np.uint16).reshape(H, 32, D)
        values = pool.tensor_view(page, 0, 2).view(np.uint16).reshape(H, D, 32)
        assert np.array_equal(keys[:, pt, :], k[:, row, :]) and np.array_equal(values[:, :, pt], v[:, :, row])


def test_store_contract_rejections_write_nothing():
    """paged_store_row.h:14-29 and PagedAttention.hpp:75-95."""
    layout = layout_for(INT8)
    pool = HostPool(layout, 128, 1)
    k = np.ones((4, 32, 256), np.uint16); v = np.ones((4, 256, 32), np.uint16)
    table = pool.table([1])
    bad = [lib.ChunkParams(0, 0, 32, 1, pool.layer(0)), lib.ChunkParams(0, 33, 32, 2, pool.layer(0)),
           lib.ChunkParams(0, 8, 24, 1, pool.layer(0)), lib.ChunkParams(30, 8, 32, 1, pool.layer(0)),
           lib.ChunkParams(262150, 16, 32, 9000, pool.layer(0)), lib.ChunkParams(0, 8, 32, 1, lib.KvLayer(0, 0))]
    for params in bad:
        assert om.oracle().rko_store_chunk(INT8, 4, 256, k.ctypes.data, v.ctypes.data, table.ctypes.data, C.byref(params)) == -1
    assert not pool.bytes[0].any()
    if om.reference() is not None:
        r = om.reference()
        assert r.ref_chunk_validation(0, 0, 32, 1) == b"chunk_tokens_out_of_range"
        assert r.ref_chunk_validation(0, 8, 24, 1) == b"chunk_stride_invalid"
        assert r.ref_chunk_validation(30, 8, 32, 1) == b"page_table_too_short"
        assert r.ref_chunk_validation(262150, 16, 32, 9000) == b"context_out_of_range"
        assert r.ref_chunk_validation(0, 8, 32, 1) == b""


# ---- attention: the fast (timed) evaluation agrees with the fp64 tile; closed-form cases ------------------
@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
def test_fast_attention_agrees_with_fp64_tile(fmt):
    layout = layout_for(fmt)
    s = Scenario(layout, [77, 5], extra_tokens=8)
    fill_history_with_store(s, 0)
    # the 8 verify rows live in the cache too (stored before attention)
    o = om.oracle()
    rng = np.random.default_rng(5)
    q = make_queries(rng, s.lanes, layout)
    from kvcase import make_staging
    k, v = make_staging(rng, s.lanes, layout)
    chunk = (lib.ChunkParams * 2)(*[lib.ChunkParams(c, 8, 32, len(p), s.host.layer(0)) for c, p in zip(s.contexts, s.pages)])
    assert o.rko_store_verify(fmt, 4, 256, 2, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk) == 0
    params = (lib.VerifyParams * 2)(*[lib.VerifyParams(c, len(p), s.host.layer(0), 32, 32, 8, 8, 0.0)
                                      for c, p in zip(s.contexts, s.pages)])
    out = np.zeros((2, 4, 32, 6, 256), np.float32)
    out16 = np.zeros((2, 4, 32, 6, 256), np.uint16)
    assert o.rko_attention_verify(fmt, 4, 6, 256, 2, q.ctypes.data, s.host_table_pointers(), params, None,
                                  out16.ctypes.data, out.ctypes.data) == 0
    for lane in range(2):
        for head in range(4):
            tile = np.zeros((48, 256), np.float32)
            assert o.rko_attention_tile(fmt, 4, 6, 256, head, q[lane, head].ctypes.data, s.host_tables[lane].ctypes.data,
                                        s.host.layer(0), s.contexts[lane], 8, 8, None, 0.0, int(fmt == FP8E4M3),
                                        tile.ctypes.data) == 0
            got = out[lane, head, :8].reshape(48, 256)
            assert np.abs(got - tile).max() <= 2e-5 * max(1.0, np.abs(tile).max())
    assert np.array_equal(out16, f32_to_bf16(out))
    assert not out[:, :, 8:].any()


def test_attention_single_token_returns_its_value_row():
    """One visible token: softmax is 1, output = dequantized V row (rows=1, history 0:
    dev/tests/engine/paged_attention_plan_test.mm:1019)."""
    layout = layout_for(INT8)
    s = Scenario(layout, [0], extra_tokens=1)
    o = om.oracle()
    rng = np.random.default_rng(9)
    from kvcase import make_staging
    k, v = make_staging(rng, 1, layout)
    chunk = (lib.ChunkParams * 1)(lib.ChunkParams(0, 1, 32, 1, s.host.layer(0)))
    assert o.rko_store_verify(INT8, 4, 256, 1, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk) == 0
    q = make_queries(rng, 1, layout)
    tile = np.zeros((6, 256), np.float32)
    assert o.rko_attention_tile(INT8, 4, 6, 256, 2, q[0, 2].ctypes.data, s.host_tables[0].ctypes.data, s.host.layer(0),
                                0, 1, 1, None, 0.0, 0, tile.ctypes.data) == 0
    page = s.pages[0][0]
    codes = s.host.tensor_view(page, 0, 2).view(np.int8).reshape(4, 256, 32)[2, :, 0].astype(np.float32)
    scale = s.host.tensor_view(page, 0, 3).view(np.float32)[2 * 32]
    for g in range(6):
        assert np.allclose(tile[g], codes * scale, rtol=1e-6, atol=0)


def test_merge_fixture_split_order():
    """Merge of split partials equals attention over the union (q8_flash_attention_metal_test.mm:648-667 shape)."""
    o = om.oracle()
    rng = np.random.default_rng(4)
    for splits in (1, 3, 7, 32, 65, 128):
        D = 256
        maxima = rng.uniform(-5, 5, splits).astype(np.float32)
        sums = rng.uniform(0.5, 20, splits).astype(np.float32)
        partials = rng.standard_normal((splits, D)).astype(np.float32)
        stats = np.stack([maxima, sums], 1).copy()
        out = np.zeros(D, np.float32)
        o.rko_merge_row(partials.ctypes.data, D, stats.ctypes.data, 2, splits, D, out.ctypes.data)
        w = np.exp(maxima.astype(np.float64) - maxima.max())
        want = (w[:, None] * partials).sum(0) / (w * sums).sum()
        assert np.abs(out - want).max() < 1e-5
    empty = np.full((1, 2), [-np.inf, 0.0], np.float32)
    out = np.ones(256, np.float32)
    o.rko_merge_row(np.zeros((1, 256), np.float32).ctypes.data, 256, empty.ctypes.data, 2, 1, 256, out.ctypes.data)
    assert not out.any()  # a zero denominator yields zeros


def test_tree_mask_admission():
    """A tree row attends history plus its ancestor bits (paged_attention_tile.h:111-114,141-143);
    the causal mask (1 << (r+1)) - 1 reproduces the chain."""
    layout = layout_for(INT4)
    s = Scenario(layout, [45], extra_tokens=16)
    fill_history_with_store(s, 0)
    o = om.oracle()
    rng = np.random.default_rng(6)
    from kvcase import make_staging
    k, v = make_staging(rng, 1, layout)
    chunk = (lib.ChunkParams * 1)(lib.ChunkParams(45, 15, 32, len(s.pages[0]), s.host.layer(0)))
    assert o.rko_store_verify(INT4, 4, 256, 1, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk) == 0
    q = make_queries(rng, 1, layout)
    causal = np.array([(1 << (r + 1)) - 1 for r in range(16)], np.uint32)
    a = np.zeros((96, 256), np.float32); b = np.zeros((96, 256), np.float32)
    args = (INT4, 4, 6, 256, 1, q[0, 1].ctypes.data, s.host_tables[0].ctypes.data, s.host.layer(0), 45, 15, 16)
    assert o.rko_attention_tile(*args, None, 0.0, 0, a.ctypes.data) == 0
    assert o.rko_attention_tile(*args, causal.ctypes.data, 0.0, 0, b.ctypes.data) == 0
    assert np.array_equal(a, b)
    only_history = np.zeros(16, np.uint32)
    c = np.zeros((96, 256), np.float32)
    assert o.rko_attention_tile(*args, only_history.ctypes.data, 0.0, 0, c.ctypes.data) == 0
    assert not np.array_equal(a[:6], c[:6])  # without its own bit row 0 loses its own token
    assert np.array_equal(c[:6], c[6:12]) is False  # rows differ by their queries only
