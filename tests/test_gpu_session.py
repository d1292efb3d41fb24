"""GPU: DecodeSession.step_host — compact host rows in pinned memory in, compact host rows out, pipelined over the copy
streams — against the checker, over several back-to-back calls with their own queries and result buffers."""
import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import chunk_params, struct_to_device, verify_params
from kvcase import Scenario, bf16_to_f32, f32_to_bf16, fill_history_with_store
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout
from richengine_b200.session import DecodeSession

pytestmark = pytest.mark.gpu


def pinned(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(array.view(np.int16).copy()).view(torch.bfloat16).pin_memory()


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
def test_step_host_matches_checker_over_pipelined_calls(fmt):
    layout = Layout(2, 4, 256, fmt)
    s = Scenario(layout, [300, 33, 1500, 64], extra_tokens=1, device=True, seed=11)
    fill_history_with_store(s, 1, seed=11)
    rng = np.random.default_rng(12)
    lanes, H, G, D = s.lanes, 4, 6, 256
    k_rows = f32_to_bf16(rng.standard_normal((lanes, H, D)).astype(np.float32))
    v_rows = f32_to_bf16(rng.standard_normal((lanes, H, D)).astype(np.float32))
    calls = 5
    q_rows = [f32_to_bf16(rng.standard_normal((lanes, H * G, D)).astype(np.float32)) for _ in range(calls)]
    # the checker: stage row 0, append it, attend
    keys = np.zeros((lanes, H, 32, D), np.uint16)
    values = np.zeros((lanes, H, D, 32), np.uint16)
    keys[:, :, 0] = k_rows
    values[:, :, :, 0] = v_rows
    cp = chunk_params(s, 1, layer_index=1)
    assert om.oracle().rko_store_verify(fmt, H, D, lanes, keys.ctypes.data, values.ctypes.data, s.host_table_pointers(), cp) == 0
    s.upload()  # history only differs from the host mirror by the row the session appends itself
    vp, _ = verify_params(s, 1, 1, 32, layer_index=1)
    wants = []
    for q in q_rows:
        staged = np.zeros((lanes, H, 32, G, D), np.uint16)
        staged[:, :, 0] = q.reshape(lanes, H, G, D)
        out16 = np.zeros(staged.shape, np.uint16)
        out32 = np.zeros(staged.shape, np.float32)
        assert om.oracle().rko_attention_verify(fmt, H, G, D, lanes, staged.ctypes.data, s.host_table_pointers(), vp, None,
                                                out16.ctypes.data, out32.ctypes.data) == 0
        wants.append(out32[:, :, 0].reshape(lanes, H * G, D))
    session = DecodeSession(s.storage, H * G, lanes)
    d_cp, d_vp = struct_to_device(cp), struct_to_device(vp)
    k_host, v_host = pinned(k_rows), pinned(v_rows)
    q_hosts = [pinned(q) for q in q_rows]
    outs = [torch.zeros((lanes, H * G, D), dtype=torch.bfloat16).pin_memory() for _ in range(calls)]
    for q_host, out in zip(q_hosts, outs):
        session.step_host(1, q_host, k_host, v_host, out, s.table_pointers, d_cp, d_vp)
    session.finish_host()
    torch.cuda.current_stream().synchronize()
    session.attention.status()
    for call, (out, want) in enumerate(zip(outs, wants)):
        got16 = out.view(torch.int16).numpy().view(np.uint16)
        assert np.isfinite(bf16_to_f32(got16)).all()
        bound = 2e-3 * max(1.0, float(np.abs(want).max())) + np.abs(want) * 2.0 ** -8
        assert (np.abs(bf16_to_f32(got16) - want) <= bound).all(), f"call {call}"
    session.close()
    s.close()
