"""One decode step's worth of buffers and launches: append each lane's new K/V row and
attend its one query row over the paged history, layer by layer.

This is the step the reference encodes per attention layer as store -> split ->
reduce (runtime/ops/PagedAttention.cpp:467-545, called from
runtime/model/QwenTarget.cpp:799-812), with the lanes generalised from the
reference's four to any batch width. Two entry points:
  step_device(...)  inputs already staged on the device (what a model runtime calls);
  step_host(...)    compact host rows in pinned memory in, compact host rows out
                    (copies, staging scatter and output gather inside the call).
step_host is one call into the library (rk_session_step_host, include/richkv.h): calls pipeline there — the upload
of a call's rows runs on a copy stream while the previous call's kernels run, and a call's result goes back on a
second copy stream while the next call computes. finish_host() makes the compute stream wait for the copies still
in flight.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib, ops
from .abi import VERIFY_CHUNK_STRIDE, Layout
from .storage import PageStorage


def _stream_handle(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if isinstance(stream, torch.cuda.Stream) else int(stream)


class DecodeSession:
    def __init__(self, storage: PageStorage, query_heads: int, lanes: int, ctas: int = 0):
        layout = storage.layout
        self.storage, self.layout, self.query_heads, self.lanes = storage, layout, query_heads, lanes
        self._lib = lib.load()
        H, D, G = layout.kv_heads, layout.head_dimension, query_heads // layout.kv_heads
        stride = VERIFY_CHUNK_STRIDE
        device = "cuda"
        self.queries = torch.zeros((lanes, H, stride, G, D), dtype=torch.bfloat16, device=device)
        self.output = torch.zeros_like(self.queries)
        self.chunk_keys = torch.zeros((lanes, H, stride, D), dtype=torch.bfloat16, device=device)
        self.chunk_values = torch.zeros((lanes, H, D, stride), dtype=torch.bfloat16, device=device)
        self._c_session, self._ctas = None, ctas  # the host-rows pipeline lives in the library (rk_session_*)
        # every format decodes on its streaming kernel
        self.attention = ops.DecodeAttention(layout, query_heads, lanes, storage.window(), ctas)
        self.layers = storage.layers()
        self.kernel_launches = 0

    def close(self):
        if self._c_session:
            self._lib.rk_session_destroy(self._c_session)
            self._c_session = None
        self.attention.close()

    def step_device(self, layer: int, table_pointers, chunk_params, verify_params, stream=None) -> None:
        """Store row 0 of the stagings at each lane's committed position, then attend (3 kernels)."""
        place = self.layers[layer]
        ops.store_verify(self.layout, self.chunk_keys, self.chunk_values, table_pointers, chunk_params, place,
                         self.lanes, 1, stream)
        self.attention.run(self.queries, self.output, table_pointers, verify_params, place, stream=stream)
        self.kernel_launches += 3

    def attend_device(self, layer: int, table_pointers, verify_params, stream=None) -> None:
        self.attention.run(self.queries, self.output, table_pointers, verify_params, self.layers[layer], stream=stream)
        self.kernel_launches += 2

    def step_host(self, layer: int, q_host, k_host, v_host, out_host, table_pointers, chunk_params, verify_params,
                  stream=None) -> None:
        """q_host [lanes][query_heads][D], k_host / v_host [lanes][kv_heads][D], out_host like q_host:
        pinned bf16 host tensors. One C call (rk_session_step_host: uploads, append, attention, download, all
        asynchronous); out_host is valid after finish_host() and a synchronise of the stream. The host tensors must
        stay unchanged until then."""
        lib.check(self._lib.rk_session_step_host(self._host_session(), layer, q_host.data_ptr(), k_host.data_ptr(),
                                                 v_host.data_ptr(), out_host.data_ptr(), table_pointers.data_ptr(),
                                                 chunk_params.data_ptr(), verify_params.data_ptr(), _stream_handle(stream)),
                  "rk_session_step_host")
        self.kernel_launches += 5

    def finish_host(self, stream=None) -> None:
        """Orders `stream` after every result copy step_host has started: synchronising it then makes out_host valid."""
        lib.check(self._lib.rk_session_finish_host(self._host_session(), _stream_handle(stream)), "rk_session_finish_host")

    def host_status(self, stream=None) -> None:
        """Raises when a bounded wait ran out in any host step since the last call (sticky; cleared by this read)."""
        lib.check(self._lib.rk_session_status(self._host_session(), _stream_handle(stream)), "rk_session_status")

    def _host_session(self):
        if self._c_session is None:
            layers = (lib.KvLayer * len(self.layers))(*self.layers)
            layout = self.layout
            self._c_session = self._lib.rk_session_create(layout.format, layout.kv_heads, self.query_heads,
                                                          layout.head_dimension, self.lanes, self.attention._window,
                                                          layers, len(self.layers), self._ctas)
            if not self._c_session:
                raise lib.RichKvError(lib.INVALID, "rk_session_create")
        return self._c_session

    def host_bytes_per_layer(self) -> tuple[int, int]:
        """(host->device, device->host) bytes one step_host call moves."""
        D, H = self.layout.head_dimension, self.layout.kv_heads
        return self.lanes * (self.query_heads + 2 * H) * D * 2, self.lanes * self.query_heads * D * 2
