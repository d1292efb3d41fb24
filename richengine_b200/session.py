"""One decode step's worth of buffers and launches: append each lane's new K/V row and
attend its one query row over the paged history, layer by layer.

This is the step the reference encodes per attention layer as store -> split ->
reduce (runtime/ops/PagedAttention.cpp:467-545, called from
runtime/model/QwenTarget.cpp:799-812), with the lanes generalised from the
reference's four to any batch width. Two entry points:
  step_device(...)  inputs already staged on the device (what a model runtime calls);
  step_host(...)    compact host rows in pinned memory in, compact host rows out
                    (copies, staging scatter and output gather inside the call).
step_host calls pipeline: the upload of a call's rows runs on a copy stream while the previous call's kernels run,
and a call's result goes back on a second copy stream while the next call computes (two sets of row buffers,
events between the streams). finish_host() makes the compute stream wait for the copies still in flight.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib, ops
from .abi import VERIFY_CHUNK_STRIDE, Layout
from .storage import PageStorage


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
        # two sets of compact rows: one being filled or drained by a copy stream while the other is in use
        self.q_rows = [torch.zeros((lanes, query_heads, D), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.k_rows = [torch.zeros((lanes, H, D), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.v_rows = [torch.zeros((lanes, H, D), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.out_rows = [torch.zeros((lanes, query_heads, D), dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.upload_stream, self.download_stream = torch.cuda.Stream(), torch.cuda.Stream()
        self.uploaded = [torch.cuda.Event() for _ in range(2)]    # the set's rows have arrived
        self.consumed = [torch.cuda.Event() for _ in range(2)]    # the staging kernel has read the set
        self.gathered = [torch.cuda.Event() for _ in range(2)]    # the set's output rows are complete
        self.downloaded = [torch.cuda.Event() for _ in range(2)]  # the set's output rows have left
        self.host_calls = 0
        # every format decodes on its streaming kernel
        self.attention = ops.DecodeAttention(layout, query_heads, lanes, storage.window(), ctas)
        self.layers = storage.layers()
        self.kernel_launches = 0

    def close(self):
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
        pinned bf16 host tensors. Asynchronous; out_host is valid after finish_host() and a synchronise of the stream.
        The host tensors must stay unchanged until then."""
        compute = torch.cuda.current_stream() if stream is None else (
            stream if isinstance(stream, torch.cuda.Stream) else torch.cuda.ExternalStream(int(stream)))
        s = compute.cuda_stream
        slot = self.host_calls & 1
        self.host_calls += 1
        with torch.cuda.stream(self.upload_stream):
            self.upload_stream.wait_event(self.consumed[slot])  # the call before last has read this set
            self.q_rows[slot].copy_(q_host, non_blocking=True)
            self.k_rows[slot].copy_(k_host, non_blocking=True)
            self.v_rows[slot].copy_(v_host, non_blocking=True)
            self.uploaded[slot].record(self.upload_stream)
        compute.wait_event(self.uploaded[slot])
        layout = self.layout
        lib.check(self._lib.rk_stage_decode_rows(layout.kv_heads, self.query_heads, layout.head_dimension, self.lanes,
                                                 self.q_rows[slot].data_ptr(), self.k_rows[slot].data_ptr(),
                                                 self.v_rows[slot].data_ptr(), self.queries.data_ptr(),
                                                 self.chunk_keys.data_ptr(), self.chunk_values.data_ptr(), s),
                  "rk_stage_decode_rows")
        self.consumed[slot].record(compute)
        self.step_device(layer, table_pointers, chunk_params, verify_params, compute)
        compute.wait_event(self.downloaded[slot])  # the call before last has sent this set's output rows
        lib.check(self._lib.rk_gather_decode_rows(layout.kv_heads, self.query_heads, layout.head_dimension, self.lanes,
                                                  self.output.data_ptr(), self.out_rows[slot].data_ptr(), s),
                  "rk_gather_decode_rows")
        self.gathered[slot].record(compute)
        with torch.cuda.stream(self.download_stream):
            self.download_stream.wait_event(self.gathered[slot])
            out_host.copy_(self.out_rows[slot], non_blocking=True)
            self.downloaded[slot].record(self.download_stream)
        self.kernel_launches += 2

    def finish_host(self, stream=None) -> None:
        """Orders `stream` after every result copy step_host has started: synchronising it then makes out_host valid."""
        compute = torch.cuda.current_stream() if stream is None else (
            stream if isinstance(stream, torch.cuda.Stream) else torch.cuda.ExternalStream(int(stream)))
        for event in self.downloaded:
            compute.wait_event(event)

    def host_bytes_per_layer(self) -> tuple[int, int]:
        """(host->device, device->host) bytes one step_host call moves."""
        h2d = (self.q_rows[0].numel() + self.k_rows[0].numel() + self.v_rows[0].numel()) * 2
        return h2d, self.out_rows[0].numel() * 2
