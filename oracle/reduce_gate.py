"""CPU restatement of the reference's reduce -> gate epilogue. Test infrastructure only: nothing in the product
imports this file; tests/test_gpu_attention.py uses it as the checker of `rk_attention_verify_reduce_gate`.

Follows kernels/decode/paged_attention.metal:273-413 (the split merge with the gate buffers bound): the merged
attention row of (lane, row, query head) is multiplied, in fp32, by the logistic function of the gate value the packed
projection row carries beside that head's query (packed row layout per token: 24 heads x {query[256], gate[256]},
then 4 key heads x 256, then 4 value heads x 256; indexing as :300-308), and stored as bf16 in the order the
out-projection reads, [lane][row][query head][dim]. sigmoid(x) = 1 / (1 + exp2(-log2(e) * x)) as the shader writes
it. Parity pinned: tests/test_reference_kernels.py runs the reference's own reduce/gate phase (its Metal source
compiled as C++ on host threads) and finds these rows bit for bit; against the GPU the exp2 of numpy and of the device
may differ in the last place before the bf16 rounding, which that test bounds.
"""
import numpy as np

LOG2_E = np.float32(1.44269504089)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round to nearest even, as the store of the merged row does."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounded = bits + np.uint32(0x7FFF) + ((bits >> 16) & np.uint32(1))
    return (rounded >> 16).astype(np.uint16)


def gate_values(packed: np.ndarray, query_heads: int = 24, head_dim: int = 256) -> np.ndarray:
    """packed [lanes][rows][stride] bf16 bits -> gate [lanes][rows][query_heads][head_dim] fp32."""
    lanes, rows, _ = packed.shape
    pairs = packed[:, :, : 2 * query_heads * head_dim].reshape(lanes, rows, query_heads, 2, head_dim)
    return bf16_to_f32(pairs[:, :, :, 1, :])


def reduce_gate(merged: np.ndarray, packed: np.ndarray) -> np.ndarray:
    """merged [lanes][rows][query_heads][head_dim] bf16 bits (the plain merge's rows) -> gated hidden rows, bf16 bits."""
    gate = gate_values(packed, merged.shape[2], merged.shape[3])
    sigmoid = (np.float32(1.0) / (np.float32(1.0) + np.exp2(-LOG2_E * gate))).astype(np.float32)
    return f32_to_bf16((bf16_to_f32(merged) * sigmoid).astype(np.float32))
