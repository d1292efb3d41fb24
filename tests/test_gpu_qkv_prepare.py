"""GPU: the step before the path (packed projection rows -> stagings / pages) against the checker, bit for bit."""
import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import assert_extents_equal, chunk_params, dev, host_u16, struct_to_device
from kvcase import Scenario, f32_to_bf16, fill_history_with_store
from richengine_b200 import ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu
HQ, HKV, D = 24, 4, 256
PACKED = 2 * HQ * D + 2 * HKV * D


def inputs(lanes, rows, seed, norm_f32):
    rng = np.random.default_rng(seed)
    packed = (rng.standard_normal((lanes, rows, PACKED)) * 2).astype(np.float32)
    packed[..., 5::97] *= 15.0   # outliers
    packed[0, 0, 2 * HQ * D: 2 * HQ * D + D] = 0.0  # an all-zero key row: inverse RMS = 1/sqrt(eps), result 0
    packed = f32_to_bf16(packed)
    qn = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kn = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    if not norm_f32:
        qn, kn = f32_to_bf16(qn), f32_to_bf16(kn)
    angle = rng.uniform(0, 6.28, size=(lanes, rows, 32)).astype(np.float32)
    return packed, qn, kn, np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)


def checker(packed, qn, kn, cosine, sine, lanes, rows, norm_f32):
    q = np.zeros((lanes, HKV, 32, HQ // HKV, D), np.uint16)
    k = np.zeros((lanes, HKV, 32, D), np.uint16)
    v = np.zeros((lanes, HKV, D, 32), np.uint16)
    assert om.oracle().rko_qkv_prepare(HKV, HQ, D, lanes, rows, packed.ctypes.data, qn.ctypes.data, kn.ctypes.data,
                                       int(norm_f32), cosine.ctypes.data, sine.ctypes.data, 1e-6, q.ctypes.data,
                                       k.ctypes.data, v.ctypes.data) == 0
    return q, k, v


def norm_tensor(w):
    return torch.from_numpy(w.copy()).cuda() if w.dtype == np.float32 else dev(w)


@pytest.mark.parametrize("norm_f32", [False, True])
@pytest.mark.parametrize("lanes,rows", [(1, 1), (3, 8), (2, 16), (5, 3)])
def test_stagings_equal_the_checker(lanes, rows, norm_f32):
    packed, qn, kn, cosine, sine = inputs(lanes, rows, 10 * lanes + rows, norm_f32)
    want_q, want_k, want_v = checker(packed, qn, kn, cosine, sine, lanes, rows, norm_f32)
    q = torch.zeros((lanes, HKV, 32, HQ // HKV, D), dtype=torch.int16, device="cuda")
    k = torch.zeros((lanes, HKV, 32, D), dtype=torch.int16, device="cuda")
    v = torch.zeros((lanes, HKV, D, 32), dtype=torch.int16, device="cuda")
    ops.qkv_prepare(Layout(1, HKV, D, INT4), HQ, lanes, rows, dev(packed), norm_tensor(qn), norm_tensor(kn),
                    torch.from_numpy(cosine).cuda(), torch.from_numpy(sine).cuda(), q, k, v)
    torch.cuda.synchronize()
    assert np.array_equal(host_u16(q), want_q)
    assert np.array_equal(host_u16(k), want_k)
    assert np.array_equal(host_u16(v), want_v)


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
def test_fused_store_equals_prepare_then_store(fmt):
    rows = 8
    s = Scenario(Layout(1, HKV, D, fmt), [0, 31, 70, 500], extra_tokens=rows, device=True, seed=33)
    fill_history_with_store(s, 0, seed=33)
    packed, qn, kn, cosine, sine = inputs(s.lanes, rows, 77, False)
    want_q, want_k, want_v = checker(packed, qn, kn, cosine, sine, s.lanes, rows, False)
    params = chunk_params(s, rows)
    assert om.oracle().rko_store_verify(fmt, HKV, D, s.lanes, want_k.ctypes.data, want_v.ctypes.data, s.host_table_pointers(), params) == 0
    # device: history as before the window, then the fused kernel
    s2 = Scenario(Layout(1, HKV, D, fmt), [0, 31, 70, 500], extra_tokens=rows, device=False, seed=33)
    fill_history_with_store(s2, 0, seed=33)
    for extent in range(s.host.extents):
        s.storage.write_extent(extent, s2.host.bytes[extent])
    q = torch.zeros((s.lanes, HKV, 32, HQ // HKV, D), dtype=torch.int16, device="cuda")
    ops.qkv_prepare_store(s.layout, HQ, s.lanes, rows, dev(packed), dev(qn), dev(kn), torch.from_numpy(cosine).cuda(),
                          torch.from_numpy(sine).cuda(), q, s.table_pointers, struct_to_device(params), s.storage.layers()[0])
    torch.cuda.synchronize()
    assert np.array_equal(host_u16(q), want_q)
    assert_extents_equal(s, f"fused prepare + store, format {fmt}")
    s.close()
