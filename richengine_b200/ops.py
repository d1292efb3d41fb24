"""Kernel entry points over torch device tensors (thin: pointers and sizes only).

Buffer layouts are the reference kernels' (runtime/metal/kernels/decode/
paged_attention_store.metal:32-35, decode/paged_attention.metal:39-47):
  chunk_keys   bf16 [lane][kv_head][stride][D]
  chunk_values bf16 [lane][kv_head][D][stride]          (dimension-major)
  queries/out  bf16 [lane][kv_head][stride][group][D]
  tables       one device array of uint64 entries per lane; `table_pointers`
               is a device array of their addresses
  params       device array of the 24/36-byte parameter blocks, one per lane
torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import lib
from .abi import CHUNK_PARAMS, VERIFY_PARAMS, Layout


def _stream(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def params_to_device(array: np.ndarray, device="cuda") -> torch.Tensor:
    """Uploads a numpy structured array of parameter blocks as raw bytes."""
    raw = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
    return torch.from_numpy(raw.copy()).to(device)


def table_pointer_array(tables, device="cuda") -> torch.Tensor:
    return torch.tensor([t.data_ptr() for t in tables], dtype=torch.int64, device=device)


def store_verify(layout: Layout, chunk_keys, chunk_values, table_pointers, params, layer: lib.KvLayer,
                 lanes: int, max_rows: int, stream=None) -> None:
    status = lib.load().rk_store_verify(layout.format, layout.kv_heads, layout.head_dimension, lanes, max_rows,
                                        chunk_keys.data_ptr(), chunk_values.data_ptr(), table_pointers.data_ptr(),
                                        params.data_ptr(), layer, _stream(stream))
    lib.check(status, "rk_store_verify")


def store_chunk(layout: Layout, chunk_keys, chunk_values, table, params: lib.ChunkParams, stream=None) -> None:
    status = lib.load().rk_store_chunk(layout.format, layout.kv_heads, layout.head_dimension, chunk_keys.data_ptr(),
                                       chunk_values.data_ptr(), table.data_ptr(), C.byref(params), _stream(stream))
    lib.check(status, "rk_store_chunk")


def attention_verify_split(layout: Layout, query_heads: int, lanes: int, row_capacity: int, grid_splits: int,
                           queries, partials, statistics, table_pointers, row_masks, params, layer: lib.KvLayer,
                           stream=None) -> None:
    status = lib.load().rk_attention_verify_split(
        layout.format, layout.kv_heads, query_heads, layout.head_dimension, lanes, row_capacity, grid_splits,
        queries.data_ptr(), partials.data_ptr(), statistics.data_ptr(), table_pointers.data_ptr(),
        row_masks.data_ptr() if row_masks is not None else None, params.data_ptr(), layer, _stream(stream))
    lib.check(status, "rk_attention_verify_split")


class VerifyWindowAttention:
    """8/16-row int4 verify windows on the tcgen05 split kernel (rk_attention_verify_split_tc).

    Holds the pool window's tensor maps and the status word; partials and statistics stay the
    caller's, in the layout of attention_verify_split, and attention_verify_reduce merges them."""

    def __init__(self, layout: Layout, query_heads: int, window: tuple[int, int]):
        self._lib = lib.load()
        self.layout, self.query_heads = layout, query_heads
        self._window = self._lib.rk_window_create(window[0], window[1])
        if not self._window:
            raise lib.RichKvError(lib.INVALID, "rk_window_create")
        self.status_word = torch.zeros(1, dtype=torch.int32, device="cuda")

    def close(self) -> None:
        if self._window:
            self._lib.rk_window_destroy(self._window)
            self._window = None

    def __del__(self):
        self.close()

    def split(self, lanes: int, row_capacity: int, grid_splits: int, queries, partials, statistics, table_pointers,
              row_masks, params, layer: lib.KvLayer, stream=None) -> None:
        status = self._lib.rk_attention_verify_split_tc(
            self._window, self.layout.format, self.layout.kv_heads, self.query_heads, self.layout.head_dimension,
            lanes, row_capacity, grid_splits, queries.data_ptr(), partials.data_ptr(), statistics.data_ptr(),
            table_pointers.data_ptr(), row_masks.data_ptr() if row_masks is not None else None, params.data_ptr(),
            layer, self.status_word.data_ptr(), _stream(stream))
        lib.check(status, "rk_attention_verify_split_tc")

    def prefill_split(self, queries, partials, statistics, table, params: lib.PrefillParams, stream=None) -> None:
        """The 8-row tiles of a prefill chunk (rk_attention_prefill_split_tc); merge with attention_prefill_reduce."""
        status = self._lib.rk_attention_prefill_split_tc(
            self._window, self.layout.format, self.layout.kv_heads, self.query_heads, self.layout.head_dimension,
            queries.data_ptr(), partials.data_ptr(), statistics.data_ptr(), table.data_ptr(), C.byref(params),
            self.status_word.data_ptr(), _stream(stream))
        lib.check(status, "rk_attention_prefill_split_tc")

    def check(self) -> None:
        """Synchronises and raises if a bounded wait ran out in a launched step."""
        if int(self.status_word.item()) != 0:
            raise lib.RichKvError(lib.TIMEOUT, "rk_attention_verify_split_tc: a bounded wait ran out")


class WindowDecodeAttention:
    """One-query decode on the tcgen05 window kernel (row capacity 1) + the split merge: the decode path of the
    int8, fp8 and bf16 pools (int4 has the streaming kernel, DecodeAttention). Same call shape as DecodeAttention;
    the lanes' parameters carry split_count = slot_splits = `splits`."""

    def __init__(self, layout: Layout, query_heads: int, lanes: int, window: tuple[int, int], splits: int = 1):
        self.layout, self.query_heads, self.lanes, self.splits = layout, query_heads, lanes, splits
        self.inner = VerifyWindowAttention(layout, query_heads, window)
        group = query_heads // layout.kv_heads
        slots = lanes * layout.kv_heads * splits * group
        self.partials = torch.empty(slots * layout.head_dimension, dtype=torch.float32, device="cuda")
        self.statistics = torch.empty(slots * 2, dtype=torch.float32, device="cuda")

    def close(self) -> None:
        self.inner.close()

    def run(self, queries, output, table_pointers, params, layer: lib.KvLayer, output_f32=None, stream=None) -> None:
        self.inner.split(self.lanes, 1, self.splits, queries, self.partials, self.statistics, table_pointers, None, params,
                         layer, stream)
        attention_verify_reduce(self.layout, self.query_heads, self.lanes, 1, self.partials, self.statistics, output,
                                params, output_f32, stream)

    def status(self) -> None:
        self.inner.check()


def attention_verify_reduce(layout: Layout, query_heads: int, lanes: int, row_capacity: int, partials, statistics,
                            output, params, output_f32=None, stream=None) -> None:
    status = lib.load().rk_attention_verify_reduce(
        layout.kv_heads, query_heads, layout.head_dimension, lanes, row_capacity, partials.data_ptr(),
        statistics.data_ptr(), output.data_ptr(), output_f32.data_ptr() if output_f32 is not None else None,
        params.data_ptr(), _stream(stream))
    lib.check(status, "rk_attention_verify_reduce")


def attention_prefill(layout: Layout, query_heads: int, queries, output, partials, statistics, table,
                      params: lib.PrefillParams, output_f32=None, stream=None) -> None:
    library = lib.load()
    lib.check(library.rk_attention_prefill_split(layout.format, layout.kv_heads, query_heads, layout.head_dimension,
                                                 queries.data_ptr(), partials.data_ptr(), statistics.data_ptr(),
                                                 table.data_ptr(), C.byref(params), _stream(stream)),
              "rk_attention_prefill_split")
    lib.check(library.rk_attention_prefill_reduce(layout.kv_heads, query_heads, layout.head_dimension,
                                                  partials.data_ptr(), statistics.data_ptr(), output.data_ptr(),
                                                  output_f32.data_ptr() if output_f32 is not None else None,
                                                  C.byref(params), _stream(stream)),
              "rk_attention_prefill_reduce")


def qkv_prepare(layout: Layout, query_heads: int, lanes: int, rows: int, packed_qkv, q_norm, k_norm, rope_cos, rope_sin,
                queries, chunk_keys, chunk_values, eps: float = 1e-6, stream=None) -> None:
    """Packed projection rows -> the stagings of the store and the attention (rk_qkv_prepare)."""
    status = lib.load().rk_qkv_prepare(layout.kv_heads, query_heads, layout.head_dimension, lanes, rows,
                                       packed_qkv.data_ptr(), q_norm.data_ptr(), k_norm.data_ptr(),
                                       int(q_norm.dtype == torch.float32), rope_cos.data_ptr(), rope_sin.data_ptr(), eps,
                                       queries.data_ptr(), chunk_keys.data_ptr(), chunk_values.data_ptr(), _stream(stream))
    lib.check(status, "rk_qkv_prepare")


def qkv_prepare_store(layout: Layout, query_heads: int, lanes: int, rows: int, packed_qkv, q_norm, k_norm, rope_cos,
                      rope_sin, queries, table_pointers, params, layer: lib.KvLayer, eps: float = 1e-6, stream=None) -> None:
    """The same with the page store merged in: K/V rows go straight into their page slots (rk_qkv_prepare_store)."""
    status = lib.load().rk_qkv_prepare_store(layout.format, layout.kv_heads, query_heads, layout.head_dimension, lanes, rows,
                                             packed_qkv.data_ptr(), q_norm.data_ptr(), k_norm.data_ptr(),
                                             int(q_norm.dtype == torch.float32), rope_cos.data_ptr(), rope_sin.data_ptr(),
                                             eps, queries.data_ptr(), table_pointers.data_ptr(), params.data_ptr(), layer,
                                             _stream(stream))
    lib.check(status, "rk_qkv_prepare_store")


def attention_verify_reduce_gate(layout: Layout, query_heads: int, lanes: int, row_capacity: int, partials, statistics,
                                 output, packed_qkv, hidden, params, stream=None) -> None:
    """Merge + out-projection input: hidden [lane][row][query head][D] = merged row x sigmoid(gate of packed_qkv), or
    the merged row itself when packed_qkv is None (rk_attention_verify_reduce_gate)."""
    status = lib.load().rk_attention_verify_reduce_gate(
        layout.kv_heads, query_heads, layout.head_dimension, lanes, row_capacity, partials.data_ptr(),
        statistics.data_ptr(), output.data_ptr() if output is not None else None,
        packed_qkv.data_ptr() if packed_qkv is not None else None, hidden.data_ptr(), params.data_ptr(), _stream(stream))
    lib.check(status, "rk_attention_verify_reduce_gate")


def attention_prefill_reduce(layout: Layout, query_heads: int, partials, statistics, output, params: lib.PrefillParams,
                             output_f32=None, stream=None) -> None:
    lib.check(lib.load().rk_attention_prefill_reduce(layout.kv_heads, query_heads, layout.head_dimension,
                                                     partials.data_ptr(), statistics.data_ptr(), output.data_ptr(),
                                                     output_f32.data_ptr() if output_f32 is not None else None,
                                                     C.byref(params), _stream(stream)),
              "rk_attention_prefill_reduce")


def tree_compact(layout: Layout, lanes: int, table_pointers, params, layer: lib.KvLayer, retained_path,
                 retained_count, stream=None) -> None:
    status = lib.load().rk_tree_compact(layout.format, layout.kv_heads, layout.head_dimension, lanes,
                                        table_pointers.data_ptr(), params.data_ptr(), layer,
                                        retained_path.data_ptr(), retained_count.data_ptr(), _stream(stream))
    lib.check(status, "rk_tree_compact")


def chunk_params_array(lanes: int) -> np.ndarray:
    return np.zeros(lanes, dtype=CHUNK_PARAMS)


def verify_params_array(lanes: int) -> np.ndarray:
    return np.zeros(lanes, dtype=VERIFY_PARAMS)


class DecodeAttention:
    """Streaming decode attention over one pool's address window (rk_attention_decode).

    Holds the window's tensor map and the step's scratch, sized by the plan:
    one query row per lane, row capacity 1; the lane parameter blocks and the
    page tables live on the device.
    """

    def __init__(self, layout: Layout, query_heads: int, lanes: int, window: tuple[int, int], ctas: int = 0):
        self._lib = lib.load()
        self.layout, self.query_heads, self.lanes = layout, query_heads, lanes
        self.plan = lib.DecodePlan()
        lib.check(self._lib.rk_decode_plan_make(layout.format, layout.kv_heads, query_heads, layout.head_dimension,
                                                lanes, ctas, C.byref(self.plan)), "rk_decode_plan_make")
        self._window = self._lib.rk_window_create(window[0], window[1])
        if not self._window:
            raise lib.RichKvError(lib.INVALID, "rk_window_create")
        self.partials = torch.empty(self.plan.partials_bytes // 4, dtype=torch.float32, device="cuda")
        self.statistics = torch.empty(self.plan.statistics_bytes // 4, dtype=torch.float32, device="cuda")
        self.descriptors = torch.zeros(self.plan.descriptor_bytes // 4, dtype=torch.int32, device="cuda")

    def close(self):
        if self._window:
            self._lib.rk_window_destroy(self._window)
            self._window = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def run(self, queries, output, table_pointers, params, layer: lib.KvLayer, output_f32=None, stream=None):
        status = self._lib.rk_attention_decode(
            self._window, C.byref(self.plan), self.layout.format, queries.data_ptr(), output.data_ptr(),
            output_f32.data_ptr() if output_f32 is not None else None, self.partials.data_ptr(),
            self.statistics.data_ptr(), self.descriptors.data_ptr(), table_pointers.data_ptr(), params.data_ptr(),
            layer, _stream(stream))
        lib.check(status, "rk_attention_decode")

    def status(self, stream=None) -> None:
        """Raises if a bounded device wait ran out during the steps launched so far."""
        lib.check(self._lib.rk_attention_decode_status(C.byref(self.plan), self.descriptors.data_ptr(), _stream(stream)),
                  "rk_attention_decode_status")
