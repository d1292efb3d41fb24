"""CPU: the checker's QKV-prepare against a plain float64 restatement of the reference's formulas
(kernels/common/attention_qkv_prepare.h:52-82) and against closed-form cases."""
import numpy as np

import oracle as om
from kvcase import bf16_to_f32, f32_to_bf16

HQ, HKV, D = 24, 4, 256
PACKED = 2 * HQ * D + 2 * HKV * D


def run(packed, qn, kn, cosine, sine, lanes, rows):
    q = np.zeros((lanes, HKV, 32, HQ // HKV, D), np.uint16)
    k = np.zeros((lanes, HKV, 32, D), np.uint16)
    v = np.zeros((lanes, HKV, D, 32), np.uint16)
    assert om.oracle().rko_qkv_prepare(HKV, HQ, D, lanes, rows, packed.ctypes.data, qn.ctypes.data, kn.ctypes.data, 1,
                                       cosine.ctypes.data, sine.ctypes.data, 1e-6, q.ctypes.data, k.ctypes.data, v.ctypes.data) == 0
    return q, k, v


def test_against_float64_formulas_and_layouts():
    rng = np.random.default_rng(0)
    lanes, rows = 2, 5
    packed = f32_to_bf16((rng.standard_normal((lanes, rows, PACKED)) * 2).astype(np.float32))
    qn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    angle = rng.uniform(0, 6.28, (lanes, rows, 32)).astype(np.float32)
    cosine, sine = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    q, k, v = run(packed, qn, kn, cosine, sine, lanes, rows)
    x = bf16_to_f32(packed).astype(np.float64)
    for lane in range(lanes):
        for row in range(rows):
            for head in range(HQ + HKV):
                query = head < HQ
                start = head * 2 * D if query else 2 * HQ * D + (head - HQ) * D
                e = x[lane, row, start:start + D]
                normed = bf16_to_f32(f32_to_bf16((e / np.sqrt((e * e).mean() + 1e-6) * (qn if query else kn)).astype(np.float32))).astype(np.float64)
                want = normed.copy()
                c, s = cosine[lane, row].astype(np.float64), sine[lane, row].astype(np.float64)
                want[:32] = normed[:32] * c - normed[32:64] * s
                want[32:64] = normed[32:64] * c + normed[:32] * s
                got = bf16_to_f32(q[lane, head // 6, row, head % 6] if query else k[lane, head - HQ, row]).astype(np.float64)
                # a double rounding at a bf16 tie may move one unit in the last place
                assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -7 + 1e-6).all()
                if not query:
                    source = packed[lane, row, 2 * HQ * D + HKV * D + (head - HQ) * D:][:D]
                    assert np.array_equal(v[lane, head - HQ, :, row], source)  # the value bits, untouched
    assert not q[:, :, rows:].any() and not k[:, :, rows:].any() and not v[:, :, :, rows:].any()


def test_identity_rotation_and_unit_weights_are_a_pure_norm():
    lanes, rows = 1, 1
    packed = np.zeros((lanes, rows, PACKED), np.float32)
    packed[0, 0, :D] = 3.0  # query head 0: constant row -> x / sqrt(9 + eps) = 1 (to bf16)
    packed = f32_to_bf16(packed)
    ones = np.ones(D, np.float32)
    q, k, _ = run(packed, ones, ones, np.ones((1, 1, 32), np.float32), np.zeros((1, 1, 32), np.float32), lanes, rows)
    assert (bf16_to_f32(q[0, 0, 0, 0]) == 1.0).all()
    assert not k.any()  # all-zero key rows stay zero: 0 * (1 / sqrt(eps))
