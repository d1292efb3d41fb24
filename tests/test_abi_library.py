"""CPU: the C-ABI library loads without a GPU and exports every symbol include/richkv.h declares;
the POD blocks keep the reference's sizes and offsets; misuse is refused on the host."""
import ctypes as C
import re
from pathlib import Path

import numpy as np

from richengine_b200 import abi, lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "richkv.h").read_text() + (ROOT / "include" / "richkv_host.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    library = lib.load()
    names = declared_symbols()
    assert len(names) > 40
    for name in names:
        assert hasattr(library, name), f"{name} is declared in richkv.h but not exported"
        assert name in lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(lib.SIGNATURES) == names  # and nothing is bound that the header does not declare


def test_parameter_blocks_match_reference_sizes():
    """runtime/metal/abi/PagedAttention.h:19,30,47,63,86 and KvExtent.h:98."""
    assert C.sizeof(lib.KvLayer) == 8 and C.sizeof(lib.ChunkParams) == 24
    assert C.sizeof(lib.PrefillParams) == 32 and C.sizeof(lib.VerifyParams) == 36 and C.sizeof(lib.PageCopy) == 8
    assert lib.VerifyParams.kv.offset == 8 and lib.VerifyParams.split_count.offset == 16
    assert lib.VerifyParams.score_scale.offset == 32 and lib.PrefillParams.score_scale.offset == 28
    assert abi.VERIFY_PARAMS.fields["score_scale"][1] == 32 and abi.CHUNK_PARAMS.fields["kv"][1] == 16


def test_host_side_refusals_without_a_gpu():
    library = lib.load()
    assert library.rk_extent_alignment_pages(abi.INT8, 4, 256) == 128
    assert library.rk_extent_alignment_pages(abi.INT4, 4, 256) == 128
    assert library.rk_extent_alignment_pages(abi.BF16, 4, 256) == 1
    assert library.rk_extent_alignment_pages(abi.INT8, 2, 256) == 256
    bad = lib.ChunkParams(0, 8, 24, 1, lib.KvLayer(128, 0))  # stride not a multiple of 32
    assert library.rk_store_chunk(abi.INT8, 4, 256, 1, 1, 1, C.byref(bad), None) == lib.INVALID
    assert b"contract" in library.rk_last_error()
    assert library.rk_storage_create(abi.INT8, 16, 4, 256, 256, 100) is None  # not whole alignment units
    assert b"geometry" in library.rk_last_error()
    plan = lib.DecodePlan()
    assert library.rk_decode_plan_make(abi.BF16, 4, 24, 256, 4, 148, C.byref(plan)) == lib.OK
    assert library.rk_decode_plan_make(abi.INT4, 8, 24, 256, 4, 148, C.byref(plan)) == lib.UNSUPPORTED  # another geometry
    assert library.rk_decode_plan_make(abi.INT8, 4, 24, 256, 4, 148, C.byref(plan)) == lib.OK
    assert library.rk_decode_plan_make(abi.INT4, 4, 24, 256, 64, 148, C.byref(plan)) == lib.OK
    assert plan.max_segments == 64 + 148 and plan.partials_bytes == (64 + 148) * 4 * 3 * 6 * 256 * 4
    assert library.rk_window_create(12345, 1 << 20) is None  # unaligned window
