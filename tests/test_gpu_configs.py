"""GPU: the benchmark configurations at their full sizes, as parity cases against the checker.

cfg 0  one int8 layer, 4096 tokens appended one at a time, then one decode query
cfg 1  int4, batch 8, contexts uniform in 8K-32K: append one token, decode (two layers of the stack)
cfg 2  int4, batch 4 x 64K: 16-row verify windows, seeded acceptance, rejected rows overwritten by the next window
cfg 3  format sweep at batch 32 x 16K: decode of every format (the pool filled on the GPU, read back for the checker)
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
    if fmt == INT4:
        d16, d32 = run_decode_attention_gpu(s, q, committed=committed)
        assert_attention_close(d32, want32, d16, "cfg3 int4 decode (streaming kernel)")
    w16, w32, _ = run_verify_attention_gpu(s, q, 1, 1, committed=committed, splits=1, tensor_core=True)
    assert_attention_close(w32, want32, w16, f"cfg3 format {fmt} decode (window kernel)")
    s.close()
