"""GPU: the CUDA path against the reference's OWN kernels, without the checker in between. The library that holds the
reference's Metal kernel source compiled as C++ (oracle/_ref, built where the reference checkout is present) travels
with the tree; where it is absent these tests skip. Stores: every byte of every extent the CUDA kernels write equals
what the reference's store kernels write. Attention: the tcgen05 window kernel, the general tile and the streaming
decode kernel against the reference's tile and merge, within the reference's own rounding bound (it rounds
probabilities to bf16; these kernels keep more bits, so the distance is the reference's rounding)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import chunk_params, dev, run_decode_attention_gpu, run_verify_attention_gpu, struct_to_device, verify_params
from kvcase import Scenario, bf16_to_f32, fill_history_with_store, make_queries, make_staging
from richengine_b200 import ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

reference = om.reference()
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(reference is None or not hasattr(reference, "ref_metal_attention_verify"),
                                                  reason="the reference's kernels were not compiled into oracle/_ref")]


def four_tables(scenario):
    pointers = [t.ctypes.data for t in scenario.host_tables]
    return (C.c_void_p * 4)(*(pointers + [pointers[0]] * (4 - len(pointers))))


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
def test_cuda_verify_store_writes_the_bytes_the_reference_kernel_writes(fmt):
    s = Scenario(Layout(2, 4, 256, fmt), [0, 27, 64, 1000], extra_tokens=16, device=True)
    rng = np.random.default_rng(60 + fmt)
    for layer in (1, 0):
        k, v = make_staging(rng, s.lanes, s.layout)
        params = chunk_params(s, 8, layer)
        assert reference.ref_metal_store_verify(fmt, k.ctypes.data, v.ctypes.data, four_tables(s), params, s.lanes) == 0   # into the host mirror
        ops.store_verify(s.layout, dev(k), dev(v), s.table_pointers, struct_to_device(params), s.storage.layers()[layer], s.lanes, 8)
    torch.cuda.synchronize()
    for extent, got in enumerate(s.download()):
        assert np.array_equal(got, s.host.bytes[extent]), f"extent {extent}"
    assert any(e.any() for e in s.host.bytes)
    s.close()


def reference_chain(fmt, s, q, splits):
    params, slot = verify_params(s, 8, 8, splits)
    partials = np.zeros((s.lanes * 4 * slot, 48, 256), np.float32)
    statistics = np.zeros((s.lanes * 4 * slot, 48, 2), np.float32)
    out = np.zeros(q.shape, np.uint16)
    assert reference.ref_metal_attention_verify(fmt, 8, 6, q.copy().ctypes.data, four_tables(s), params, s.lanes, None,
                                                partials.ctypes.data, statistics.ctypes.data, out.ctypes.data, None, None) == 0
    return bf16_to_f32(out)


def close_to_reference(got32, theirs, rows, what):
    for lane in range(got32.shape[0]):
        a, b = got32[lane, :, :rows], theirs[lane, :, :rows]
        bound = 2.0 ** -8 * max(1.0, float(np.abs(b).max())) + np.abs(b) * 2.0 ** -8
        assert (np.abs(a - b) <= bound).all(), f"{what}: lane {lane} off by {float((np.abs(a - b) - bound).max())}"
        assert np.abs(b).max() > 0.05


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
@pytest.mark.parametrize("tensor_core", [True, False])
def test_cuda_verify_attention_against_the_reference_tile_and_merge(fmt, tensor_core):
    s = Scenario(Layout(1, 4, 256, fmt), [1500, 5, 0, 67], extra_tokens=8, device=True)
    fill_history_with_store(s, 0)
    k, v = make_staging(np.random.default_rng(61), s.lanes, s.layout)
    params = chunk_params(s, 8, 0)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    q = make_queries(np.random.default_rng(62), s.lanes, s.layout)
    theirs = reference_chain(fmt, s, q, 3)
    _, got32, _ = run_verify_attention_gpu(s, q, 8, 8, splits=None, tensor_core=tensor_core)
    close_to_reference(got32, theirs, 8, "verify attention")
    s.close()


@pytest.mark.parametrize("fmt,contexts", [(INT4, [2100, 33, 1]), (INT8, [2100, 33, 1]), (BF16, [2100, 33, 1]), (INT4, [32768, 8191])])
def test_cuda_streaming_decode_against_the_reference_prefill_phases_of_one_row(fmt, contexts):
    """The last case is the north-star context length: 32 768 tokens of int4 history through the reference's page loop."""
    s = Scenario(Layout(1, 4, 256, fmt), contexts, extra_tokens=0, device=True)
    fill_history_with_store(s, 0)
    s.upload()
    q = make_queries(np.random.default_rng(63), s.lanes, s.layout)
    _, got32 = run_decode_attention_gpu(s, q, committed=[c - 1 for c in contexts])   # the row's own token is the last stored one
    from richengine_b200 import lib
    for lane, context in enumerate(contexts):
        params = lib.PrefillParams(context - 1, 1, 32, len(s.pages[lane]), s.host.layer(0), 2, 0.0)
        partials = np.zeros((4 * 2, 48, 256), np.float32)
        statistics = np.zeros((4 * 2, 48, 2), np.float32)
        out = np.zeros((4, 32, 6, 256), np.uint16)
        assert reference.ref_metal_attention_prefill(fmt, q[lane].copy().ctypes.data, s.host_tables[lane].ctypes.data, C.byref(params),
                                                     partials.ctypes.data, statistics.ctypes.data, out.ctypes.data) == 0
        close_to_reference(got32[lane:lane + 1], bf16_to_f32(out)[None], 1, f"decode lane {lane}")
    s.close()
