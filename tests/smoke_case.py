"""The smoke scenario: append one token per lane, then paged decode attention (general tile, streaming decode
kernel, tcgen05 window kernel), on the GPU, compared with the CPU checker (codes bit-exact, attention within the
parity bar)."""
import numpy as np
import torch

import oracle as om
from gpuhelp import (assert_attention_close, assert_extents_equal, chunk_params, dev, run_verify_attention_gpu,
                     run_verify_attention_oracle, struct_to_device)
from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
from richengine_b200 import ops


def run(layout):
    s = Scenario(layout, [40, 700, 1], extra_tokens=1, device=True)
    fill_history_with_store(s, 1)
    s.upload()
    rng = np.random.default_rng(0)
    k, v = make_staging(rng, s.lanes, layout)
    params = chunk_params(s, 1, layer_index=1)
    assert om.oracle().rko_store_verify(layout.format, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data,
                                        s.host_table_pointers(), params) == 0
    ops.store_verify(layout, dev(k), dev(v), s.table_pointers, struct_to_device(params), s.storage.layers()[1], s.lanes, 1)
    torch.cuda.synchronize()
    assert_extents_equal(s, "smoke append")
    q = make_queries(rng, s.lanes, layout)
    got16, got32, _ = run_verify_attention_gpu(s, q, 1, 1, layer_index=1)
    _, want32 = run_verify_attention_oracle(s, q, 1, 1, layer_index=1)
    assert_attention_close(got32, want32, got16, "smoke decode")
    from gpuhelp import run_decode_attention_gpu
    d16, d32 = run_decode_attention_gpu(s, q, layer_index=1)
    assert_attention_close(d32, want32, d16, "smoke decode (streaming kernel)")
    # an 8-row verify window on the tcgen05 kernel over the same pages (7 of its rows read zero staging rows)
    w16, w32, _ = run_verify_attention_gpu(s, q, 1, 8, layer_index=1, tensor_core=True)
    assert_attention_close(w32, want32, w16, "smoke window (tcgen05 kernel)")
    s.close()
