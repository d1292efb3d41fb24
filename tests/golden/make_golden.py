"""Generates tests/golden/golden.json: known-answer vectors for the paged KV path.

    python tests/golden/make_golden.py

Run where the reference checkout was compiled (oracle/_ref/librk_ref.so): the int8 and fp8 page quantisation
vectors come from the reference's own quantisers; the scenario vectors (append + quantise into pages, then a
verify window over them) come from the checker, which tests/test_oracle_pins.py pins to the reference.
Inputs are seeded; the file records a digest of the inputs so that a changed random stream is noticed instead
of being compared. Whole extents are recorded as SHA-256 (bit-exact work), attention outputs as a strided
sample of fp32 values (tolerance work).
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

import oracle as om  # noqa: E402
from gpuhelp import chunk_params, run_verify_attention_oracle  # noqa: E402
from kvcase import Scenario, bf16_to_f32, f32_to_bf16, fill_history_with_store, make_queries, make_staging  # noqa: E402
from richengine_b200.abi import BF16, FP8E4M3, FORMAT_NAMES, INT4, INT8, Layout  # noqa: E402

CONTEXTS = [37, 64, 5]
ROWS = 8
SAMPLE_STRIDE = 997


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def build_scenario(fmt, device=False):
    """The fixture's scenario: history through the chunk store, then ROWS window rows through the verify store."""
    s = Scenario(Layout(1, 4, 256, fmt), CONTEXTS, extra_tokens=16, device=device, seed=21)
    fill_history_with_store(s, 0, seed=21)
    rng = np.random.default_rng(121)
    k, v = make_staging(rng, s.lanes, s.layout)
    q = make_queries(rng, s.lanes, s.layout)
    return s, k, v, q


PAGE_TOKENS_VALID = 29


def page_inputs(seed):
    """Token-major fp32 rows [token][head][dim] (bf16-exact), as the reference's page quantisers take them."""
    rng = np.random.default_rng(seed)
    keys = rng.standard_normal((PAGE_TOKENS_VALID, 4, 256)).astype(np.float32)
    values = rng.standard_normal((PAGE_TOKENS_VALID, 4, 256)).astype(np.float32) * 0.05
    keys[:, :, 7] *= 20.0
    values[:, :, 100] *= 20.0
    keys[3, 1, :] = 0.0  # a zero row: scale 0, codes 0
    return bf16_to_f32(f32_to_bf16(keys)), bf16_to_f32(f32_to_bf16(values))


def main():
    out = {"contexts": CONTEXTS, "rows": ROWS, "sample_stride": SAMPLE_STRIDE, "scenarios": {}, "reference_pages": {}}
    reference = om.reference()
    if reference is None:
        raise SystemExit("oracle/_ref/librk_ref.so is missing: build it with `make -C oracle` next to the reference checkout")
    for name, fn in (("int8", reference.ref_q8_quantize_page), ("fp8e4m3", reference.ref_fp8_quantize_page)):
        keys, values = page_inputs(77)
        expected = np.zeros(66560, np.uint8)
        assert fn(keys.ctypes.data, values.ctypes.data, PAGE_TOKENS_VALID, expected.ctypes.data) == 0
        out["reference_pages"][name] = {"seed": 77, "valid_tokens": PAGE_TOKENS_VALID, "input_sha256": digest(keys, values),
                                        "page_sha256": digest(expected), "first_bytes": expected[:32].tolist(),
                                        "first_key_scales": expected[32768:32768 + 16].view(np.float32).tolist()}
    for fmt in (INT4, INT8, FP8E4M3, BF16):
        s, k, v, q = build_scenario(fmt)
        assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(),
                                            chunk_params(s, ROWS)) == 0
        _, want32 = run_verify_attention_oracle(s, q, ROWS, 8)
        out["scenarios"][FORMAT_NAMES[fmt]] = {
            "input_sha256": digest(k, v, q),
            "extent_sha256": [digest(b) for b in s.host.bytes],
            "attention_sample": [float(x) for x in want32.reshape(-1)[::SAMPLE_STRIDE]],
            "attention_abs_max": float(np.abs(want32).max()),
        }
        s.close()
    (HERE / "golden.json").write_text(json.dumps(out, indent=1) + "\n")
    print("wrote", HERE / "golden.json")


if __name__ == "__main__":
    main()
