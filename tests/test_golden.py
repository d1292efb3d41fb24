"""Known-answer vectors (tests/golden/golden.json, made by tests/golden/make_golden.py from the reference's compiled
quantisers and the pinned checker): the checker on CPU, the CUDA store and attention kernels on the GPU."""
import json
import sys
from pathlib import Path

import numpy as np
import pytest

import oracle as om
from gpuhelp import TOLERANCE, chunk_params
from richengine_b200.abi import BF16, FP8E4M3, FORMAT_NAMES, INT4, INT8

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))
import make_golden as mg  # noqa: E402

GOLDEN = json.loads((GOLDEN_DIR / "golden.json").read_text())
FORMATS = [INT4, INT8, FP8E4M3, BF16]


def scenario_or_skip(fmt, device=False):
    s, k, v, q = mg.build_scenario(fmt, device=device)
    want = GOLDEN["scenarios"][FORMAT_NAMES[fmt]]
    if mg.digest(k, v, q) != want["input_sha256"]:
        s.close()
        pytest.skip("this numpy draws a different random stream than the one the vectors were made with")
    return s, k, v, q, want


@pytest.mark.parametrize("fmt", FORMATS)
def test_checker_reproduces_the_vectors(fmt):
    s, k, v, q, want = scenario_or_skip(fmt)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(),
                                        chunk_params(s, mg.ROWS)) == 0
    assert [mg.digest(b) for b in s.host.bytes] == want["extent_sha256"]
    from gpuhelp import run_verify_attention_oracle
    _, got32 = run_verify_attention_oracle(s, q, mg.ROWS, 8)
    sample = got32.reshape(-1)[::mg.SAMPLE_STRIDE]
    assert np.abs(sample - np.array(want["attention_sample"], np.float32)).max() <= 1e-5 * max(1.0, want["attention_abs_max"])
    s.close()


@pytest.mark.parametrize("name", ["int8", "fp8e4m3"])
def test_checker_store_equals_the_reference_quantiser_vectors(name):
    """One full page through the checker's chunk store = the page the reference's quantiser produced."""
    import ctypes as C
    from kvcase import HostPool, f32_to_bf16
    from richengine_b200 import lib
    from richengine_b200.abi import Layout
    want = GOLDEN["reference_pages"][name]
    fmt = INT8 if name == "int8" else FP8E4M3
    keys, values = mg.page_inputs(want["seed"])
    if mg.digest(keys, values) != want["input_sha256"]:
        pytest.skip("this numpy draws a different random stream than the one the vectors were made with")
    valid = want["valid_tokens"]
    pool = HostPool(Layout(1, 4, 256, fmt), 128, 1)
    table = pool.table([5])
    params = lib.ChunkParams(0, valid, 32, 1, pool.layer(0))
    k16, v16 = np.zeros((4, 32, 256), np.uint16), np.zeros((4, 256, 32), np.uint16)
    k16[:, :valid, :] = f32_to_bf16(keys).transpose(1, 0, 2)
    v16[:, :, :valid] = f32_to_bf16(values).transpose(1, 2, 0)
    assert om.oracle().rko_store_chunk(fmt, 4, 256, k16.ctypes.data, v16.ctypes.data, table.ctypes.data, C.byref(params)) == 0
    got = np.concatenate([pool.tensor_view(5, 0, t) for t in range(4)])
    assert got[:32].tolist() == want["first_bytes"]
    assert mg.digest(got) == want["page_sha256"]


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", FORMATS)
def test_cuda_store_and_attention_reproduce_the_vectors(fmt):
    import torch
    from gpuhelp import dev, run_verify_attention_gpu, struct_to_device
    from richengine_b200 import ops
    s, k, v, q, want = scenario_or_skip(fmt, device=True)
    s.upload()  # history as the checker stored it; the window rows go through the CUDA store
    ops.store_verify(s.layout, dev(k), dev(v), s.table_pointers, struct_to_device(chunk_params(s, mg.ROWS)),
                     s.storage.layers()[0], s.lanes, mg.ROWS)
    torch.cuda.synchronize()
    assert [mg.digest(b) for b in s.download()] == want["extent_sha256"]
    reference = np.array(want["attention_sample"], np.float32)
    bound = TOLERANCE * max(1.0, want["attention_abs_max"])
    for tensor_core in (False, True):
        _, got32, _ = run_verify_attention_gpu(s, q, mg.ROWS, 8, tensor_core=tensor_core)
        assert np.abs(got32.reshape(-1)[::mg.SAMPLE_STRIDE] - reference).max() <= bound
    s.close()
