"""CPU (gloo, world size 2 and 3): request partitioning and the sequence-split combine — each rank
computes its shard's {max, sum, un-normalised output} with the checker's arithmetic, the triples are
all-gathered through torch.distributed, and the rank-order merge equals attention over the whole
sequence on every rank, bit-identically across ranks."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from richengine_b200 import parallel  # noqa: E402


def test_request_partition_is_balanced_and_deterministic():
    rng = np.random.default_rng(0)
    contexts = rng.integers(4096, 65537, size=256)
    for ranks in (1, 2, 4, 8):
        parts = parallel.partition_requests(contexts, ranks)
        assert sorted(i for p in parts for i in p) == list(range(256))
        loads = [int(sum(contexts[i] for i in p)) for p in parts]
        assert max(loads) - min(loads) <= int(contexts.max())  # within one request of each other
        assert parts == parallel.partition_requests(list(contexts), ranks)
    assert parallel.partition_requests([5, 5, 5], 2) == [[0, 2], [1]]


def test_sequence_shards_tile_the_pages():
    for visible in (1, 31, 32, 33, 4097, 262145):
        for ranks in (1, 2, 3, 4, 8):
            pages = parallel.pages_for(visible)
            covered, tokens = 0, 0
            for r in range(ranks):
                first, last = parallel.shard_page_range(pages, r, ranks)
                assert first == covered
                covered = last
                begin, count = parallel.shard_tokens(visible, r, ranks)
                assert begin == min(first * 32, begin) and count >= 0
                tokens += count
            assert covered == pages and tokens == visible
            owner = parallel.tail_owner(visible, ranks)
            begin, count = parallel.shard_tokens(visible, owner, ranks)
            assert begin <= visible - 1 < begin + count


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _shard_triples(q, k, v, begin, count):
    """{max, sum, un-normalised output} of softmax(q.k/16).v over tokens [begin, begin+count), fp32 like the kernels."""
    heads, d = q.shape
    out = np.zeros((heads, d + 2), np.float32)
    out[:, 0] = -np.inf
    if count == 0:
        return out
    s = (q.astype(np.float32) @ k[begin:begin + count].T.astype(np.float32)) * np.float32(0.0625)
    m = s.max(axis=1)
    p = np.exp(s - m[:, None]).astype(np.float32)
    out[:, 0], out[:, 1], out[:, 2:] = m, p.sum(axis=1), p @ v[begin:begin + count]
    return out


def _merge(gathered):
    """Rank-order merge (paged_attention_tile.h:362-404 with split = rank), fp32, sequential."""
    ranks = gathered.shape[0]
    maximum = gathered[:, :, 0].max(axis=0)
    numerator = np.zeros(gathered.shape[1:2] + (gathered.shape[2] - 2,), np.float32)
    denominator = np.zeros(gathered.shape[1], np.float32)
    for r in range(ranks):
        own = gathered[r, :, 0]
        weight = np.where(np.isneginf(own), np.float32(0), np.exp(own - maximum)).astype(np.float32)
        numerator += weight[:, None] * gathered[r, :, 2:]
        denominator += weight * gathered[r, :, 1]
    return numerator / denominator[:, None]


def _worker(rank, world, port, visible, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)  # every rank holds the query; K/V stand for the rank's own pages
    q = rng.standard_normal((24, 256)).astype(np.float32)
    k = rng.standard_normal((visible, 256)).astype(np.float32)
    v = rng.standard_normal((visible, 256)).astype(np.float32)
    begin, count = parallel.shard_tokens(visible, rank, world)
    mine = torch.from_numpy(_shard_triples(q, k, v, begin, count)[None])  # [lanes=1][24][258]
    gathered = parallel.gather_shards(mine).numpy()
    assert gathered.shape == (world, 1, 24, 258)
    merged = _merge(gathered[:, 0])
    s = (q @ k.T) * 0.0625
    p = np.exp(s - s.max(axis=1, keepdims=True))
    want = (p / p.sum(axis=1, keepdims=True)) @ v
    assert np.abs(merged - want).max() < 2e-5
    np.save(os.path.join(result_dir, f"merged{rank}.npy"), merged)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,visible", [(2, 1000), (2, 33), (3, 4097), (2, 20)])
def test_sequence_split_combine_over_gloo(world, visible, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, visible, str(tmp_path)), nprocs=world, join=True)
    results = [np.load(tmp_path / f"merged{r}.npy") for r in range(world)]
    for r in range(1, world):
        assert np.array_equal(results[0], results[r])  # identical bits on every rank
