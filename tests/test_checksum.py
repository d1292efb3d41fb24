"""CRC-32C: the checker against published known answers, and the library's host routine against the checker."""
import ctypes as C

import numpy as np

import oracle as om
from richengine_b200 import lib


def checker(data: bytes, crc=0) -> int:
    buffer = np.frombuffer(data, dtype=np.uint8)
    return om.oracle().rko_crc32c(buffer.ctypes.data if len(data) else None, len(data), crc)


def test_checker_known_answers():
    # the check value of the CRC catalogue and the iSCSI examples (RFC 3720 B.4)
    assert checker(b"123456789") == 0xE3069283
    assert checker(bytes(32)) == 0x8A9136AA
    assert checker(b"\xff" * 32) == 0x62A8AB43
    assert checker(bytes(range(32))) == 0x46DD794E
    assert checker(bytes(range(31, -1, -1))) == 0x113FDB5C
    assert checker(b"") == 0


def test_running_value_continues():
    data = np.random.default_rng(1).integers(0, 256, 1000, dtype=np.uint8).tobytes()
    for cut in (0, 1, 7, 8, 500, 999, 1000):
        assert checker(data[cut:], checker(data[:cut])) == checker(data)


def test_host_routine_matches_checker():
    library = lib.load()
    rng = np.random.default_rng(2)
    for size in list(range(0, 70)) + [255, 256, 4095, 4096, 33792, 100001]:
        data = rng.integers(0, 256, size, dtype=np.uint8)
        want = checker(data.tobytes())
        assert library.rk_crc32c_host(data.ctypes.data if size else None, size, 0) == want
        if size > 3:  # unaligned start and a running value
            head = library.rk_crc32c_host(data.ctypes.data, 3, 0)
            assert library.rk_crc32c_host(data.ctypes.data + 3, size - 3, head) == want
