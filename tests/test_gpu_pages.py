"""GPU: page copies, packing, tree compaction, table entries, extents and the pinned-host tier."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import assert_extents_equal, chunk_params, dev, struct_to_device
from kvcase import Scenario, fill_history_with_store, make_staging
from richengine_b200 import lib, ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout
from richengine_b200.storage import PageStorage

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", [INT4, INT8, BF16])
def test_copy_pages_bit_exact(fmt):
    """Every tensor of every layer moves, nothing else changes (runtime/ops/PageStorage.mm:95-114)."""
    s = Scenario(Layout(3, 4, 256, fmt), [100, 64], extra_tokens=0, device=True)
    for layer in range(3):
        fill_history_with_store(s, layer, seed=layer)
    s.upload()
    copies = [(s.pages[0][0], s.spare_pages[0]), (s.pages[1][1], s.spare_pages[1]), (s.pages[0][3], s.spare_pages[5])]
    for a, b in copies:
        om.oracle().rko_copy_page(fmt, 3, 4, 256, s.extent_pages, s.host.entry(a), s.host.entry(b))
    s.storage.copy_pages(copies)
    torch.cuda.synchronize()
    assert_extents_equal(s, "copy pages")
    s.close()


def test_copy_refuses_unallocated_extent_and_copies_nothing():
    layout = Layout(1, 4, 256, INT8)
    storage = PageStorage(layout, 256, 128)
    assert storage.allocate_extent(0)
    before = storage.read_extent(0)
    with pytest.raises(RuntimeError):
        storage.copy_pages([(0, 1), (2, 130)])  # page 130 lies in extent 1, which holds no memory
    torch.cuda.synchronize()
    assert np.array_equal(before, storage.read_extent(0))
    with pytest.raises(RuntimeError):
        storage.entry(130)
    with pytest.raises(RuntimeError):
        storage.allocate_extent(0)  # already allocated
    with pytest.raises(RuntimeError):
        storage.release_extent(1)  # not allocated
    storage.close()


def test_storage_geometry_validation_and_entries():
    """PageStorage.mm:24-36,116-141: alignment units, whole extents, entries from `first`."""
    layout = Layout(16, 4, 256, INT4)
    for pages, extent in [(256, 100), (200, 128), (0, 128), (128, 0)]:
        with pytest.raises(ValueError):
            PageStorage(layout, pages, extent)
    storage = PageStorage(layout, 384, 128)
    assert storage.bytes_per_page() == 540672 and storage.extent_bytes() == 128 * 540672
    assert storage.allocate_extent(0) and storage.allocate_extent(2)
    base, size = storage.window()
    assert base % (1 << 21) == 0 and size >= 3 * storage.extent_bytes()
    assert storage.entry(5) == base | 5
    assert storage.entry(300) & 0x3FFF == 300 - 256 and storage.entry(300) > storage.entry(5)
    assert storage.actual_allocated_bytes() == 2 * storage.extent_bytes()
    table = torch.full((8,), -1, dtype=torch.int64, device="cuda")
    storage.write_entries([1, 2, 260, 3], 2, table)
    torch.cuda.synchronize()
    host = table.cpu().numpy().view(np.uint64)
    assert host[0] == host[1] == 0xFFFFFFFFFFFFFFFF and host[2] == storage.entry(260) and host[3] == storage.entry(3)
    with pytest.raises(RuntimeError):
        storage.write_entries([1, 130], 0, table)  # extent 1 holds no memory
    with pytest.raises(RuntimeError):
        storage.write_entries([1, 2], 3, table)  # first past the pages
    storage.set_budget(2 * storage.extent_bytes())
    assert storage.allocate_extent(1) is False  # budget refusal is a value, not an error
    storage.release_extent(2)
    assert storage.allocate_extent(1)
    fresh = storage.read_extent(1)
    assert not fresh.any()  # a fresh extent reads as zeros
    storage.close()


@pytest.mark.parametrize("fmt", [INT4, INT8, BF16])
def test_tree_compaction(fmt):
    """Retained path rows move to their path slots, byte-exact with their scales
    (runtime/metal/kernels/decode/paged_attention_store.metal:198-278)."""
    s = Scenario(Layout(1, 4, 256, fmt), [29, 64, 7], extra_tokens=16, device=True)
    rng = np.random.default_rng(12)
    k, v = make_staging(rng, s.lanes, s.layout)
    params = chunk_params(s, 15)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(), params) == 0
    s.upload()
    paths = np.zeros((3, 8), np.uint32)
    paths[0, :4] = [0, 1, 9, 10]
    paths[1, :6] = [0, 8, 2, 3, 11, 14]
    counts = np.array([4, 6, 0], np.uint32)
    for lane in range(3):
        assert om.oracle().rko_tree_compact(fmt, 4, 256, s.host_tables[lane].ctypes.data, C.byref(params[lane]),
                                            paths[lane].ctypes.data, int(counts[lane])) == 0
    ops.tree_compact(s.layout, 3, s.table_pointers, struct_to_device(params), s.storage.layers()[0], dev(paths), dev(counts))
    torch.cuda.synchronize()
    assert_extents_equal(s, "tree compaction")
    s.close()


def test_host_tier_round_trip_and_limits():
    """Demote -> drop -> restore through pinned host memory is bit-exact; transfers are bounded
    (runtime/engine/cache/KvPageTier.cpp:38-132); a failed demotion keeps the page
    (runtime/engine/cache/KvTier.hpp:17-22)."""
    library = lib.load()
    s = Scenario(Layout(2, 4, 256, INT4), [96], extra_tokens=0, device=True)
    for layer in range(2):
        fill_history_with_store(s, layer, seed=layer + 5)
    s.upload()
    tier = library.rk_tier_create(s.storage.handle, 4, 4)
    assert tier and library.rk_tier_slot_bytes(tier) == s.storage.bytes_per_page()
    pages = s.pages[0]
    slots = [library.rk_tier_acquire_slot(tier) for _ in range(4)]
    assert slots == [0, 1, 2, 3] and library.rk_tier_acquire_slot(tier) == -1  # quota full
    ids = [library.rk_tier_demote(tier, pages[i], slots[i], None) for i in range(2)]
    assert all(i >= 0 for i in ids)
    assert library.rk_tier_demote(tier, pages[2], slots[2], None) == lib.REFUSED  # demotions take at most half
    assert library.rk_tier_drain(tier) >= 0
    assert all(library.rk_tier_transfer_ready(tier, i) for i in ids)
    assert [library.rk_tier_transfer_finish(tier, i) for i in ids] == [1, 1]
    # the host slot holds the page's spans in layer, tensor order
    slot0 = np.ctypeslib.as_array(C.cast(library.rk_tier_slot_host_pointer(tier, 0), C.POINTER(C.c_uint8)),
                                  shape=(s.storage.bytes_per_page(),))
    want = np.concatenate([s.host.tensor_view(pages[0], layer, t) for layer in range(2) for t in range(4)])
    assert np.array_equal(slot0, want)
    # wipe the pages on the device, restore them elsewhere and in place
    wiped = [np.zeros_like(b) for b in s.host.bytes]
    for extent in range(s.host.extents):
        s.storage.write_extent(extent, wiped[extent])
    target = s.spare_pages[0]
    r0 = library.rk_tier_restore(tier, slots[0], target, None)
    r1 = library.rk_tier_restore(tier, slots[1], pages[1], None)
    assert r0 >= 0 and r1 >= 0
    library.rk_tier_drain(tier)
    assert library.rk_tier_transfer_finish(tier, r0) == 1 and library.rk_tier_transfer_finish(tier, r1) == 1
    for extent in range(s.host.extents):
        s.host.bytes[extent][:] = 0
    om.oracle()  # rebuild the expectation: only the two restored pages hold data
    shadow = Scenario(Layout(2, 4, 256, INT4), [96], extra_tokens=0, device=False)
    for layer in range(2):
        fill_history_with_store(shadow, layer, seed=layer + 5)
    for source, destination in ((pages[0], target), (pages[1], pages[1])):
        for layer in range(2):
            for t in range(4):
                s.host.tensor_view(destination, layer, t)[:] = shadow.host.tensor_view(source, layer, t)
    assert_extents_equal(s, "tier restore")
    # a failed demotion reports failure and closes the tier to further demotions
    library.rk_tier_fail_next(tier, 1)
    bad = library.rk_tier_demote(tier, pages[1], slots[2], None)
    assert bad >= 0
    library.rk_tier_drain(tier)
    assert library.rk_tier_transfer_finish(tier, bad) == 0
    assert not library.rk_tier_writable(tier) and not library.rk_tier_can_demote(tier)
    assert library.rk_tier_can_restore(tier)  # existing copies stay readable
    library.rk_tier_destroy(tier)
    s.close()


def test_host_tier_batches_of_transfers():
    """Transfers go out in batches of up to 16 of a kind: 40 demotions (two full batches and a rest that leaves at the
    poll) into host slots that are only partly neighbours, every slot's bytes and CRC-32C (taken by the pack kernel)
    against the host's own routine, then all 40 pages wiped and restored in another order, three of them to other
    pages, with a demotion of a further page in flight beside the restores."""
    library = lib.load()
    tokens = 41 * 32
    s = Scenario(Layout(2, 4, 256, INT4), [tokens], extra_tokens=0, device=True, seed=12)
    for layer in range(2):
        fill_history_with_store(s, layer, seed=layer + 21)
    s.upload()
    page_bytes = s.storage.bytes_per_page()
    tier = library.rk_tier_create(s.storage.handle, 64, 128)
    pages = s.pages[0]
    everything = [library.rk_tier_acquire_slot(tier) for _ in range(64)]
    rng = np.random.default_rng(5)
    chosen = sorted(rng.choice(64, size=41, replace=False).tolist())  # runs of neighbours and gaps between them
    for slot in everything:
        if slot not in chosen:
            library.rk_tier_release_slot(tier, slot)
    order = rng.permutation(40)
    ids = {}
    for i in order:  # asked for in any order: a batch sorts its pages by host slot
        ids[i] = library.rk_tier_demote(tier, pages[i], chosen[i], None)
        assert ids[i] >= 0, library.rk_last_error()
    assert not any(library.rk_tier_transfer_ready(tier, t) for t in ids.values())
    while not all(library.rk_tier_transfer_ready(tier, t) for t in ids.values()):
        library.rk_tier_poll(tier)
    assert all(library.rk_tier_transfer_finish(tier, t) == 1 for t in ids.values())
    for i in range(40):
        slot = np.ctypeslib.as_array(C.cast(library.rk_tier_slot_host_pointer(tier, chosen[i]), C.POINTER(C.c_uint8)), shape=(page_bytes,))
        want = np.concatenate([s.host.tensor_view(pages[i], layer, t) for layer in range(2) for t in range(4)])
        assert np.array_equal(slot, want), f"slot of page {i}"
        assert library.rk_tier_slot_checksum(tier, chosen[i]) == library.rk_crc32c_host(want.ctypes.data, page_bytes, 0)
    # wipe, then bring everything back: pages 0..2 land on each other's places, and a demotion runs beside the restores
    for extent in range(s.host.extents):
        s.storage.write_extent(extent, np.zeros_like(s.host.bytes[extent]))
    destinations = {i: pages[i] for i in range(40)}
    destinations[0], destinations[1], destinations[2] = pages[1], pages[2], pages[0]
    restores = [library.rk_tier_restore(tier, chosen[i], destinations[i], None) for i in rng.permutation(40)]
    assert all(r >= 0 for r in restores), library.rk_last_error()
    beside = library.rk_tier_demote(tier, pages[40], chosen[40], None)  # its own batch, on another stream
    assert beside >= 0
    library.rk_tier_drain(tier)
    assert all(library.rk_tier_transfer_finish(tier, r) == 1 for r in restores)
    assert library.rk_tier_transfer_finish(tier, beside) == 1
    assert library.rk_tier_slot_checksum(tier, chosen[40]) == library.rk_crc32c_host(np.zeros(page_bytes, np.uint8).ctypes.data, page_bytes, 0)
    for extent in range(s.host.extents):
        s.host.bytes[extent][:] = 0
    shadow = Scenario(Layout(2, 4, 256, INT4), [tokens], extra_tokens=0, device=False, seed=12)
    for layer in range(2):
        fill_history_with_store(shadow, layer, seed=layer + 21)
    for i in range(40):
        for layer in range(2):
            for t in range(4):
                s.host.tensor_view(destinations[i], layer, t)[:] = shadow.host.tensor_view(pages[i], layer, t)
    assert_extents_equal(s, "tier batches")
    library.rk_tier_destroy(tier)
    s.close()


@pytest.mark.gpu
def test_host_tier_restores_a_chain_demoted_leaf_first():
    """A chain demoted leaf first sits in descending host slots; restored root first, a batch of its restores is one
    run of neighbouring slots once sorted and crosses PCIe as one copy into the staging area (runs of four or more),
    the rest of the chain (a run of three) is unpacked straight out of pinned memory. Every byte of every extent
    after: the chain's pages are back, everything else stays wiped."""
    library = lib.load()
    tokens = 22 * 32
    s = Scenario(Layout(2, 4, 256, INT4), [tokens], extra_tokens=0, device=True, seed=14)
    for layer in range(2):
        fill_history_with_store(s, layer, seed=layer + 31)
    s.upload()
    tier = library.rk_tier_create(s.storage.handle, 32, 128)
    pages = s.pages[0]
    chain = list(range(19))                      # 19 = a full batch of 16 and a run of three
    slots = {}
    for i in reversed(chain):                    # leaf first: the leaf takes the lowest slot
        slots[i] = library.rk_tier_acquire_slot(tier)
        assert library.rk_tier_demote(tier, pages[i], slots[i], None) >= 0, library.rk_last_error()
    assert [slots[i] for i in reversed(chain)] == list(range(19))
    library.rk_tier_drain(tier)
    for extent in range(s.host.extents):
        s.storage.write_extent(extent, np.zeros_like(s.host.bytes[extent]))
    restores = [library.rk_tier_restore(tier, slots[i], pages[i], None) for i in chain]   # root first
    assert all(r >= 0 for r in restores), library.rk_last_error()
    library.rk_tier_drain(tier)
    assert all(library.rk_tier_transfer_finish(tier, r) == 1 for r in restores)
    kept = {(i, layer, t): s.host.tensor_view(pages[i], layer, t).copy() for i in chain for layer in range(2) for t in range(4)}
    for extent in range(s.host.extents):         # only the chain's pages come back; everything else stays wiped
        s.host.bytes[extent][:] = 0
    for (i, layer, t), content in kept.items():
        s.host.tensor_view(pages[i], layer, t)[:] = content
    assert_extents_equal(s, "chain restore")
    library.rk_tier_destroy(tier)
    s.close()
