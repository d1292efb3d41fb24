"""GPU: CRC-32C of packed payloads on the device against the checker, bit-exact, and its size-independent properties."""
import numpy as np
import pytest
import torch

import oracle as om
from richengine_b200 import lib

pytestmark = pytest.mark.gpu


def device_crc(data: torch.Tensor, stride: int, payload: int, count: int, ctas=0) -> np.ndarray:
    out = torch.full((count,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    status = lib.load().rk_crc32c_pages(data.data_ptr(), stride, payload, count, out.data_ptr(), ctas,
                                        torch.cuda.current_stream().cuda_stream)
    assert status == lib.OK, lib.load().rk_last_error()
    torch.cuda.synchronize()
    return out.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("payload,count,stride_pad,ctas", [
    (512, 1, 0, 0), (512, 5, 512, 0), (1024, 3, 0, 1), (1536, 2, 16, 0), (33792, 7, 0, 0), (33792, 300, 0, 7),
    (540672, 1, 0, 0), (540672, 9, 1024, 0), (1064960, 2, 0, 0), (2097152, 3, 0, 0), (65536 * 3 + 512, 2, 0, 148)])
def test_device_crc_matches_checker(payload, count, stride_pad, ctas):
    rng = np.random.default_rng(payload + count)
    stride = payload + stride_pad
    host = rng.integers(0, 256, stride * count, dtype=np.uint8)
    got = device_crc(torch.from_numpy(host).cuda(), stride, payload, count, ctas)
    o = om.oracle()
    for i in range(count):
        want = o.rko_crc32c(host[i * stride:].ctypes.data, payload, 0)
        assert got[i] == want, f"payload {i}: {got[i]:08x} != {want:08x}"


def test_known_answer_rows():
    zeros = torch.zeros(512, dtype=torch.uint8, device="cuda")
    ones = torch.full((512,), 255, dtype=torch.uint8, device="cuda")
    o = om.oracle()
    z = np.zeros(512, np.uint8)
    f = np.full(512, 255, np.uint8)
    assert device_crc(zeros, 512, 512, 1)[0] == o.rko_crc32c(z.ctypes.data, 512, 0)
    assert device_crc(ones, 512, 512, 1)[0] == o.rko_crc32c(f.ctypes.data, 512, 0)


def test_affine_over_xor_at_full_size():
    """crc(a ^ b) ^ crc(a) ^ crc(b) == crc(0...0) for equal lengths, whatever the size: 1 024 model pages of an int4 pool."""
    payload, count = 540672, 1024
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randint(0, 256, (count * payload,), dtype=torch.uint8, device="cuda", generator=g)
    b = torch.randint(0, 256, (count * payload,), dtype=torch.uint8, device="cuda", generator=g)
    ca, cb, cx = (device_crc(t, payload, payload, count) for t in (a, b, a ^ b))
    zero = device_crc(torch.zeros(payload, dtype=torch.uint8, device="cuda"), payload, payload, 1)[0]
    assert ((ca ^ cb ^ cx) == zero).all()
    # and one payload of the batch against the checker
    host = a[5 * payload:6 * payload].cpu().numpy()
    assert ca[5] == om.oracle().rko_crc32c(host.ctypes.data, payload, 0)


def test_refusals():
    library = lib.load()
    data = torch.zeros(2048, dtype=torch.uint8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert library.rk_crc32c_pages(data.data_ptr(), 1000, 1000, 1, out.data_ptr(), 0, None) == lib.INVALID  # not whole rows
    assert library.rk_crc32c_pages(data.data_ptr() + 4, 512, 512, 1, out.data_ptr(), 0, None) == lib.INVALID  # unaligned
    assert library.rk_crc32c_pages(data.data_ptr(), 256, 512, 2, out.data_ptr(), 0, None) == lib.INVALID  # overlapping


@pytest.mark.parametrize("fmt,layers,count", [(3, 16, 5), (1, 2, 3), (4, 3, 2), (2, 2, 2)])
def test_seal_packs_and_checksums_in_one_pass(fmt, layers, count):
    """rk_storage_seal_pages: the slots equal rk_storage_pack_pages byte for byte and every checksum equals the
    checker's CRC-32C of its slot (int4, int8, fp8, bf16 pools; random page ids; pages of different extents)."""
    from richengine_b200.abi import Layout
    from richengine_b200.storage import PageStorage
    library = lib.load()
    layout = Layout(layers, 4, 256, fmt)
    extent_pages = layout.minimum_extent_pages()
    storage = PageStorage(layout, 2 * extent_pages, extent_pages)
    rng = np.random.default_rng(fmt * 100 + layers)
    for extent in range(2):
        assert storage.allocate_extent(extent)
        storage.write_extent(extent, rng.integers(0, 256, size=storage.extent_bytes(), dtype=np.uint8))
    page_bytes = storage.bytes_per_page()
    ids = rng.permutation(2 * extent_pages)[:count].astype(np.uint32)
    packed = torch.zeros(count * page_bytes, dtype=torch.uint8, device="cuda")
    sealed = torch.zeros(count * page_bytes, dtype=torch.uint8, device="cuda")
    sums = torch.zeros(count, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    lib.check(library.rk_storage_pack_pages(storage.handle, ids.ctypes.data, count, packed.data_ptr(), 0, stream), "pack")
    lib.check(library.rk_storage_seal_pages(storage.handle, ids.ctypes.data, count, sealed.data_ptr(), sums.data_ptr(), stream), "seal")
    torch.cuda.synchronize()
    assert torch.equal(packed, sealed)
    host = sealed.cpu().numpy()
    for i in range(count):
        want = om.oracle().rko_crc32c(host[i * page_bytes:].ctypes.data, page_bytes, 0)
        assert int(sums[i].item()) & 0xffffffff == want, f"slot {i}"
    storage.close()
