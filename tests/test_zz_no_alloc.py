"""GPU: the decode entry point that brings its own scratch.

Some users of this library cannot hand it scratch buffers because they cannot allocate any: their
KV pool already owns the device, or the thread that drives decoding is not allowed to call into the
allocator. rk_attention_decode_static serves them from an array built into the library. This test
calls it through the C ABI twice in a row (the array keeps the previous call's contents, so the
second call proves nothing stale leaks through) and compares each result with rk_attention_decode
run on caller-provided scratch, within the attention parity bar of the other tests.
Collected last so that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (TOLERANCE, chunk_params, dev, host_u16, run_decode_attention_gpu, struct_to_device, verify_params)
from kvcase import Scenario, bf16_to_f32, fill_history_with_store, make_queries, make_staging
from richengine_b200 import lib, ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu


def build(contexts, seed, fmt=INT4):
    s = Scenario(Layout(1, 4, 256, fmt), contexts, extra_tokens=1, device=True, seed=seed)
    fill_history_with_store(s, 0, seed=seed)
    rng = np.random.default_rng(seed)
    k, v = make_staging(rng, s.lanes, s.layout)
    params = chunk_params(s, 1)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    return s, make_queries(rng, s.lanes, s.layout)


def run_static(library, window, s, q):
    fmt = s.layout.format
    params, _ = verify_params(s, 1, 1, 32)
    d_params = struct_to_device(params)
    dq = dev(q)
    out = torch.zeros_like(dq)
    out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    status = library.rk_attention_decode_static(window, fmt, s.lanes, dq.data_ptr(), out.data_ptr(), out32.data_ptr(),
                                                s.table_pointers.data_ptr(), d_params.data_ptr(),
                                                s.storage.layers()[0], stream)
    assert status == lib.OK, library.rk_last_error()
    assert library.rk_attention_decode_static_status(stream) == lib.OK  # synchronises; no wait ran out
    free_after, _ = torch.cuda.mem_get_info()
    # the call took no device memory, neither from the driver nor from torch's allocator
    assert free_after >= free_before and torch.cuda.memory_reserved() == reserved_before
    return host_u16(out), out32.cpu().numpy()


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
def test_static_scratch_decode_matches_caller_scratch_decode_twice(fmt):
    library = lib.load()
    for call, (contexts, seed) in enumerate([([900, 33, 4000, 1], 21), ([70, 2500], 22)]):
        s, q = build(contexts, seed, fmt)
        base, size = s.storage.window()
        window = library.rk_window_create(base, size)
        assert window
        want16, want32 = run_decode_attention_gpu(s, q)
        got16, got32 = run_static(library, window, s, q)
        scale = max(1.0, float(np.abs(want32).max()))
        assert np.isfinite(got32).all()
        assert float(np.abs(got32 - want32).max()) <= TOLERANCE * scale, f"call {call}"
        assert (np.abs(bf16_to_f32(got16) - bf16_to_f32(want16)) <= TOLERANCE * scale + np.abs(want32) * 2.0 ** -8).all()
        library.rk_window_destroy(window)
        s.close()


def test_static_scratch_decode_refuses_more_lanes_than_fit():
    library = lib.load()
    s, q = build([40] * 17, 23)
    base, size = s.storage.window()
    window = library.rk_window_create(base, size)
    params, _ = verify_params(s, 1, 1, 32)
    dq = dev(q)
    out = torch.zeros_like(dq)
    status = library.rk_attention_decode_static(window, INT4, 17, dq.data_ptr(), out.data_ptr(), None,
                                                s.table_pointers.data_ptr(), struct_to_device(params).data_ptr(),
                                                s.storage.layers()[0], torch.cuda.current_stream().cuda_stream)
    assert status == lib.INVALID and b"16 lanes" in library.rk_last_error()
    torch.cuda.synchronize()
    assert not host_u16(out).any()  # nothing ran
    library.rk_window_destroy(window)
    s.close()
