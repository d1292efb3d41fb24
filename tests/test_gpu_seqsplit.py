"""GPU: sequence-split decode on one GPU — the shards of one long context run one after another
(each over its own slice of the page table), their triples are stacked as an all-gather would, and the
rank-order merge equals the checker's attention over the whole sequence and the unsplit kernel."""
import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (assert_attention_close, chunk_params, dev, host_u16, run_decode_attention_gpu,
                     run_verify_attention_oracle, struct_to_device)
from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
from richengine_b200 import lib, ops, parallel
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("context,ranks,fmt", [(5000, 2, INT4), (5000, 4, INT4), (40, 8, INT4), (1023, 3, INT4),
                                                (5000, 4, INT8), (1023, 3, FP8E4M3), (5000, 2, BF16)])
def test_sequence_split_matches_whole_sequence(context, ranks, fmt):
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [context], extra_tokens=1, device=True, seed=5)
    fill_history_with_store(s, 0, seed=5)
    rng = np.random.default_rng(9)
    k, v = make_staging(rng, 1, layout)
    params = chunk_params(s, 1)
    assert om.oracle().rko_store_verify(fmt, 4, 256, 1, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    q = make_queries(rng, 1, layout)
    visible = context + 1
    dq = dev(q)
    decoder = parallel.SequenceSplitDecoder(layout, 24, 1, s.storage.window())
    shards = []
    for r in range(ranks):
        first, last = parallel.shard_page_range(len(s.pages[0]), r, ranks)
        begin, count = parallel.shard_tokens(visible, r, ranks)
        if count == 0:  # a rank without pages contributes an empty triple
            empty = torch.zeros((1, 24, 258), dtype=torch.float32, device="cuda")
            empty[:, :, 0] = float("-inf")
            shards.append(empty)
            continue
        table = s.device_tables[0][first:last].contiguous()
        pointers = ops.table_pointer_array([table])
        lane = (lib.VerifyParams * 1)(lib.VerifyParams(count - 1, last - first, s.storage.layers()[0], 1, 1, 1, 1, 0.0))
        shards.append(decoder.shard(dq, pointers, struct_to_device(lane), s.storage.layers()[0]).clone())
        decoder.inner.status()
    gathered = torch.stack(shards).contiguous()
    out = torch.zeros_like(dq)
    out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
    decoder.merge(gathered, out, out32)
    torch.cuda.synchronize()
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(out32.cpu().numpy(), want32, host_u16(out), f"seqsplit {ranks}")
    _, whole32 = run_decode_attention_gpu(s, q)
    assert_attention_close(out32.cpu().numpy(), whole32, None, "split vs whole")
    decoder.close(); s.close()


@pytest.mark.parametrize("context,ranks,fmt", [(5000, 2, INT4), (9000, 8, INT4), (40, 8, INT4), (1023, 3, INT8), (5000, 4, BF16)])
def test_peer_exchange_step_emulated_on_one_gpu(context, ranks, fmt):
    """The fused reduce -> peer stores -> flags -> merge kernel with every "peer" buffer being the local one: the
    emulated ranks run one after another (all but the last only publish, the last finds every flag set, waits for
    nothing and merges). Two steps in a row use both parities of the buffer; the result equals the all-gather
    variant's bit for bit and the checker's within the bar."""
    layout = Layout(1, 4, 256, fmt)
    s = Scenario(layout, [context], extra_tokens=1, device=True, seed=6)
    fill_history_with_store(s, 0, seed=6)
    rng = np.random.default_rng(10)
    k, v = make_staging(rng, 1, layout)
    assert om.oracle().rko_store_verify(fmt, 4, 256, 1, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk_params(s, 1)) == 0
    s.upload()
    visible = context + 1
    place = s.storage.layers()[0]
    shards = []
    for r in range(ranks):
        first, last = parallel.shard_page_range(len(s.pages[0]), r, ranks)
        begin, count = parallel.shard_tokens(visible, r, ranks)
        if count == 0:  # no pages on this rank: an invalid lane, which publishes an empty triple
            table = s.device_tables[0][:1].contiguous()
            lane = (lib.VerifyParams * 1)(lib.VerifyParams(0, 0, place, 1, 1, 1, 1, 0.0))
        else:
            table = s.device_tables[0][first:last].contiguous()
            lane = (lib.VerifyParams * 1)(lib.VerifyParams(count - 1, last - first, place, 1, 1, 1, 1, 0.0))
        shards.append((table, ops.table_pointer_array([table]), struct_to_device(lane), count))
    exchange = parallel.PeerExchangeDecoder(layout, 24, 1, s.storage.window(), rank=0, ranks=ranks, connect=False)
    reference = parallel.SequenceSplitDecoder(layout, 24, 1, s.storage.window())
    for step in range(2):
        q = make_queries(rng, 1, layout)
        dq = dev(q)
        out = torch.zeros_like(dq)
        out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
        for r, (_, pointers, lane, _) in enumerate(shards):
            exchange.step(dq, out, pointers, lane, place, output_f32=out32, loopback_rank=r)
        exchange.status()
        torch.cuda.synchronize()
        # the all-gather variant on the same shards
        triples = []
        for _, pointers, lane, count in shards:
            if count == 0:
                empty = torch.zeros((1, 24, 258), dtype=torch.float32, device="cuda")
                empty[:, :, 0] = float("-inf")
                triples.append(empty)
            else:
                triples.append(reference.shard(dq, pointers, lane, place).clone())
        want = torch.zeros_like(dq)
        want32 = torch.zeros_like(out32)
        reference.merge(torch.stack(triples).contiguous(), want, want32)
        torch.cuda.synchronize()
        assert torch.equal(out32, want32) and torch.equal(out, want), f"step {step}: exchange and all-gather variants differ"
        _, oracle32 = run_verify_attention_oracle(s, q, 1, 1)
        assert_attention_close(out32.cpu().numpy(), oracle32, host_u16(out), f"peer exchange, step {step}")
    exchange.close(); reference.close(); s.close()


def _peer_exchange_rank(rank, ranks, port, context, fmt, results):
    """One rank of the real thing: its own GPU, its own process, the exchange buffers mapped through CUDA IPC."""
    import os
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=ranks, device_id=torch.device("cuda", rank))
    try:
        layout = Layout(1, 4, 256, fmt)
        s = Scenario(layout, [context], extra_tokens=1, device=True, seed=6)  # every rank builds the same pages
        fill_history_with_store(s, 0, seed=6)
        rng = np.random.default_rng(10)
        k, v = make_staging(rng, 1, layout)
        assert om.oracle().rko_store_verify(fmt, 4, 256, 1, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), chunk_params(s, 1)) == 0
        s.upload()
        visible, place = context + 1, s.storage.layers()[0]
        first, last = parallel.shard_page_range(len(s.pages[0]), rank, ranks)
        _, count = parallel.shard_tokens(visible, rank, ranks)
        table = s.device_tables[0][first:last].contiguous()  # this rank attends only its token range
        lane = struct_to_device((lib.VerifyParams * 1)(lib.VerifyParams(count - 1, last - first, place, 1, 1, 1, 1, 0.0)))
        pointers = ops.table_pointer_array([table])
        exchange = parallel.PeerExchangeDecoder(layout, 24, 1, s.storage.window(), rank=rank, ranks=ranks)
        worst = 0.0
        for step in range(3):  # three steps: both parities of the buffers, and one reuse
            q = make_queries(rng, 1, layout)
            dq = dev(q)
            out = torch.zeros_like(dq)
            out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
            exchange.step(dq, out, pointers, lane, place, output_f32=out32)
            exchange.status()
            torch.cuda.synchronize()
            _, oracle32 = run_verify_attention_oracle(s, q, 1, 1)
            assert_attention_close(out32.cpu().numpy(), oracle32, host_u16(out), f"rank {rank}, step {step}")
            everyone = [torch.zeros_like(out32) for _ in range(ranks)]
            dist.all_gather(everyone, out32)
            assert all(torch.equal(everyone[0], other) for other in everyone), "the ranks hold different bits"
            worst = max(worst, float(np.abs(out32.cpu().numpy() - oracle32).max()))
        dist.barrier()  # nobody leaves while a peer may still store into its buffer
        exchange.close(); s.close()
        results[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
@pytest.mark.parametrize("context,fmt", [(5000, INT4), (70000, INT4), (3000, INT8)])
def test_peer_exchange_across_two_gpus(context, fmt):
    """The sequence split as it runs in production: two processes, two GPUs, triples stored into the peer's buffer
    over NVLink, flags, rank-order merge. Every rank's output equals the checker's answer over the WHOLE sequence
    within the bar, and the ranks hold the same bits."""
    import torch.multiprocessing as mp
    manager = mp.get_context("spawn").Manager()
    results = manager.dict()
    port = 29600 + (context % 97)
    mp.spawn(_peer_exchange_rank, args=(2, port, context, fmt, results), nprocs=2, join=True)
    assert len(results) == 2
