"""Multi-GPU operation of the KV path: one process per GPU, torch.distributed for the plumbing.

Two ways to shard (the reference is single-GPU; both are new here):
  * by request — sequences are independent, each rank owns its pool, tables and tier, and the data
    path has NO collective (`partition_requests` balances ranks by total context);
  * by sequence — one long context's pages are dealt to the ranks in contiguous ranges
    (`shard_page_range`); each rank attends its pages (rk_attention_decode_shard), the per-rank
    {max, sum, un-normalised output} triples (24 768 bytes per lane at 24 heads x 256) are
    all-gathered (NCCL over NVLink on GPUs, gloo in CPU tests) into local memory, and every rank
    merges them in rank order (rk_attention_merge_shards), so all ranks hold identical bits.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import lib
from .abi import PAGE_TOKENS, Layout, pages_for


def partition_requests(contexts, ranks: int) -> list[list[int]]:
    """Request ids per rank, balanced by total context: longest first onto the lightest rank
    (ties: lowest rank). Deterministic, so every rank computes the same assignment."""
    order = sorted(range(len(contexts)), key=lambda i: (-int(contexts[i]), i))
    load = [0] * ranks
    assignment = [[] for _ in range(ranks)]
    for i in order:
        r = min(range(ranks), key=lambda k: (load[k], k))
        assignment[r].append(i)
        load[r] += int(contexts[i])
    return [sorted(a) for a in assignment]


def shard_page_range(pages: int, rank: int, ranks: int) -> tuple[int, int]:
    """Rank r owns logical pages [r*P/R, (r+1)*P/R)."""
    return rank * pages // ranks, (rank + 1) * pages // ranks


def shard_tokens(visible_tokens: int, rank: int, ranks: int) -> tuple[int, int]:
    """First token and token count of rank r's shard of a sequence with `visible_tokens` tokens."""
    first, last = shard_page_range(pages_for(visible_tokens), rank, ranks)
    begin = first * PAGE_TOKENS
    end = min(last * PAGE_TOKENS, visible_tokens)
    return begin, max(0, end - begin)


def tail_owner(visible_tokens: int, ranks: int) -> int:
    """The rank whose shard holds the last token: new K/V rows are appended there."""
    pages = pages_for(visible_tokens)
    for r in range(ranks):
        first, last = shard_page_range(pages, r, ranks)
        if first <= pages - 1 < last:
            return r
    return ranks - 1


def gather_shards(triples: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gathers each rank's [lanes][query_heads][2 + D] fp32 triples into [ranks][...], in rank order.
    `out` ([ranks * lanes][query_heads][2 + D]) avoids an allocation per call."""
    world = dist.get_world_size(group)
    flat = out if out is not None else torch.empty((world * triples.shape[0], *triples.shape[1:]), dtype=triples.dtype,
                                                   device=triples.device)
    dist.all_gather_into_tensor(flat, triples, group=group)  # concatenated along dim 0, rank by rank
    return flat.view(world, *triples.shape)


class SequenceSplitDecoder:
    """One rank's part of a sequence-split decode step (int4, 27B geometry)."""

    def __init__(self, layout: Layout, query_heads: int, lanes: int, window, ctas: int = 0):
        from . import ops
        self._lib = lib.load()
        self.layout, self.query_heads, self.lanes = layout, query_heads, lanes
        self.inner = ops.DecodeAttention(layout, query_heads, lanes, window, ctas)
        self.triples = torch.zeros((lanes, query_heads, layout.head_dimension + 2), dtype=torch.float32, device="cuda")
        self.gathered = None  # the all-gather's destination, allocated once the group size is known

    def close(self):
        self.inner.close()

    def shard(self, queries, table_pointers, params, layer: lib.KvLayer, stream=None) -> torch.Tensor:
        from .ops import _stream
        a = self.inner
        status = self._lib.rk_attention_decode_shard(a._window, C.byref(a.plan), self.layout.format, queries.data_ptr(),
                                                     self.triples.data_ptr(), a.partials.data_ptr(), a.statistics.data_ptr(),
                                                     a.descriptors.data_ptr(), table_pointers.data_ptr(), params.data_ptr(),
                                                     layer, _stream(stream))
        lib.check(status, "rk_attention_decode_shard")
        return self.triples

    def merge(self, gathered: torch.Tensor, output, output_f32=None, stream=None) -> None:
        from .ops import _stream
        status = self._lib.rk_attention_merge_shards(self.layout.kv_heads, self.query_heads, self.layout.head_dimension,
                                                     self.lanes, gathered.shape[0], gathered.data_ptr(), output.data_ptr(),
                                                     output_f32.data_ptr() if output_f32 is not None else None, _stream(stream))
        lib.check(status, "rk_attention_merge_shards")

    def step(self, queries, output, table_pointers, params, layer, group=None, output_f32=None):
        """shard -> all-gather -> merge; every rank ends with the same output."""
        world = dist.get_world_size(group)
        if self.gathered is None or self.gathered.shape[0] != world * self.lanes:
            self.gathered = torch.empty((world * self.lanes, *self.triples.shape[1:]), dtype=torch.float32, device="cuda")
        gathered = gather_shards(self.shard(queries, table_pointers, params, layer), group, self.gathered)
        self.merge(gathered, output, output_f32)
        return gathered


class PeerExchangeDecoder:
    """The sequence split with the combine inside the library's own kernel (rk_attention_decode_exchange): per step
    two launches, no collective library on the data path. Each rank's triple goes into every rank's exchange buffer
    by plain peer stores over NVLink; the buffers are shared through CUDA IPC handles that the ranks gather once,
    at construction, over `group` (a torch.distributed group; None with world size 1 needs no group at all)."""

    def __init__(self, layout: Layout, query_heads: int, lanes: int, window, rank: int = 0, ranks: int = 1, group=None,
                 ctas: int = 0, connect: bool = True):
        from . import ops
        self._lib = lib.load()
        self.layout, self.query_heads, self.lanes, self.rank, self.ranks = layout, query_heads, lanes, rank, ranks
        self.inner = ops.DecodeAttention(layout, query_heads, lanes, window, ctas)
        handle = (C.c_ubyte * 64)()
        self._exchange = self._lib.rk_exchange_create(rank, ranks, lanes, handle)
        if not self._exchange:
            raise lib.RichKvError(lib.CUDA_ERROR, "rk_exchange_create")
        if ranks > 1 and connect:
            mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
            everyone = torch.empty(ranks * 64, dtype=torch.uint8, device="cuda")
            dist.all_gather_into_tensor(everyone, mine, group=group)
            handles = bytes(everyone.cpu().numpy().tobytes())
            lib.check(self._lib.rk_exchange_connect(self._exchange, handles), "rk_exchange_connect")
            dist.barrier(group)  # every rank has mapped every buffer before anyone's first step

    def close(self):
        if self._exchange:
            self._lib.rk_exchange_destroy(self._exchange)
            self._exchange = None
        self.inner.close()

    def step(self, queries, output, table_pointers, params, layer: lib.KvLayer, output_f32=None, loopback_rank: int = -1,
             stream=None) -> None:
        from .ops import _stream
        a = self.inner
        status = self._lib.rk_attention_decode_exchange(
            a._window, C.byref(a.plan), self.layout.format, queries.data_ptr(), output.data_ptr(),
            output_f32.data_ptr() if output_f32 is not None else None, a.partials.data_ptr(), a.statistics.data_ptr(),
            a.descriptors.data_ptr(), table_pointers.data_ptr(), params.data_ptr(), layer, self._exchange, loopback_rank,
            _stream(stream))
        lib.check(status, "rk_attention_decode_exchange")

    def status(self, stream=None) -> None:
        self.inner.status(stream)
