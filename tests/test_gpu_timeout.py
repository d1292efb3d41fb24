"""GPU: the bounded waits of the streaming decode kernels and of the tcgen05 window kernel run out on purpose.

Nothing faults and nothing hangs: the probe entry points launch the production kernels with a poll limit of a few
thousand and a producer that never streams the last pages of its range, so the warps that wait for those pages give
up after microseconds, the kernel raises its status word, lets the copies in flight land (and releases tensor
memory) and returns. The tests check the reported status, that the word is sticky across later launches until it
is read, that reading clears it, and that the next ordinary step on the same buffers is correct again.
The reference's analogue is its command watchdog (runtime/metal/CommandWatchdog.hpp:11-35).
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as om
from gpuhelp import (assert_attention_close, chunk_params, dev, host_u16, run_verify_attention_gpu,
                     run_verify_attention_oracle, struct_to_device, verify_params)
from kvcase import Scenario, fill_history_with_store, make_queries, make_staging
from richengine_b200 import lib, ops
from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout

pytestmark = pytest.mark.gpu

SPIN_LIMIT = 4096


def prepared(contexts, fmt, seed=31):
    s = Scenario(Layout(1, 4, 256, fmt), contexts, extra_tokens=1, device=True, seed=seed)
    fill_history_with_store(s, 0, seed=seed)
    rng = np.random.default_rng(seed + 100)
    k, v = make_staging(rng, s.lanes, s.layout)
    assert om.oracle().rko_store_verify(fmt, 4, 256, s.lanes, k.ctypes.data, v.ctypes.data, s.host_table_pointers(),
                                        chunk_params(s, 1)) == 0
    s.upload()
    return s, make_queries(rng, s.lanes, s.layout)


@pytest.mark.parametrize("fmt", [INT4, INT8, FP8E4M3, BF16])
@pytest.mark.parametrize("ctas", [1, 148])
def test_decode_wait_runs_out_is_reported_sticky_and_recovers(fmt, ctas):
    library = lib.load()
    s, q = prepared([1500, 700, 90], fmt)
    params, _ = verify_params(s, 1, 1, 32)
    d_params, dq = struct_to_device(params), dev(q)
    out = torch.zeros_like(dq)
    out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
    runner = ops.DecodeAttention(s.layout, 24, s.lanes, s.storage.window(), ctas)
    layer = s.storage.layers()[0]
    stream = torch.cuda.current_stream().cuda_stream

    runner.run(dq, out, s.table_pointers, d_params, layer, output_f32=out32)
    runner.status()  # an ordinary step reports nothing
    status = library.rk_attention_decode_probe_timeout(
        runner._window, C.byref(runner.plan), fmt, dq.data_ptr(), out.data_ptr(), runner.partials.data_ptr(),
        runner.statistics.data_ptr(), runner.descriptors.data_ptr(), s.table_pointers.data_ptr(), d_params.data_ptr(),
        layer, SPIN_LIMIT, 1, stream)
    assert status == lib.OK, library.rk_last_error()
    torch.cuda.synchronize()  # the kernel came back: no wait was unbounded
    # two ordinary steps later the word still tells of the wait that ran out
    runner.run(dq, out, s.table_pointers, d_params, layer, output_f32=out32)
    runner.run(dq, out, s.table_pointers, d_params, layer, output_f32=out32)
    with pytest.raises(lib.RichKvError) as caught:
        runner.status()
    assert caught.value.status == lib.TIMEOUT
    runner.status()  # reading cleared it
    torch.cuda.synchronize()
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(out32.cpu().numpy(), want32, host_u16(out), "the step after a timeout")
    runner.close(); s.close()


def test_static_entry_reports_a_wait_that_ran_out():
    library = lib.load()
    s, q = prepared([900, 40], INT4, seed=33)
    params, _ = verify_params(s, 1, 1, 32)
    d_params, dq = struct_to_device(params), dev(q)
    out = torch.zeros_like(dq)
    out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
    base, size = s.storage.window()
    window = library.rk_window_create(base, size)
    layer = s.storage.layers()[0]
    stream = torch.cuda.current_stream().cuda_stream
    plan = lib.DecodePlan()
    lib.check(library.rk_decode_plan_make(INT4, 4, 24, 256, s.lanes, 0, C.byref(plan)), "plan")

    assert library.rk_attention_decode_static(window, INT4, s.lanes, dq.data_ptr(), out.data_ptr(), out32.data_ptr(),
                                              s.table_pointers.data_ptr(), d_params.data_ptr(), layer, stream) == lib.OK
    assert library.rk_attention_decode_static_status(stream) == lib.OK
    # the probe on the library's own array (null scratch pointers)
    assert library.rk_attention_decode_probe_timeout(window, C.byref(plan), INT4, dq.data_ptr(), out.data_ptr(), None, None,
                                                     None, s.table_pointers.data_ptr(), d_params.data_ptr(), layer,
                                                     SPIN_LIMIT, 1, stream) == lib.OK, library.rk_last_error()
    assert library.rk_attention_decode_static(window, INT4, s.lanes, dq.data_ptr(), out.data_ptr(), out32.data_ptr(),
                                              s.table_pointers.data_ptr(), d_params.data_ptr(), layer, stream) == lib.OK
    assert library.rk_attention_decode_static_status(stream) == lib.TIMEOUT
    assert library.rk_attention_decode_static_status(stream) == lib.OK
    torch.cuda.synchronize()
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(out32.cpu().numpy(), want32, host_u16(out), "static entry after a timeout")
    library.rk_window_destroy(window)
    s.close()


@pytest.mark.parametrize("fmt,rows", [(INT4, 16), (INT8, 8), (BF16, 16), (INT4, 1)])
def test_window_kernel_wait_runs_out_is_reported_and_recovers(fmt, rows):
    library = lib.load()
    s, q = prepared([3000, 500], fmt, seed=35)
    committed = [c - rows + 1 for c in s.contexts]  # the window's rows are the last stored tokens
    splits = 3
    params, slot = verify_params(s, rows, rows, splits, committed=committed)
    d_params, dq = struct_to_device(params), dev(q)
    M = rows * 6
    partials = torch.zeros(s.lanes * 4 * slot * M * 256, dtype=torch.float32, device="cuda")
    stats = torch.zeros(s.lanes * 4 * slot * M * 2, dtype=torch.float32, device="cuda")
    runner = ops.VerifyWindowAttention(s.layout, 24, s.storage.window())
    layer = s.storage.layers()[0]
    status = library.rk_attention_verify_probe_timeout(
        runner._window, fmt, 4, 24, 256, s.lanes, rows, slot, dq.data_ptr(), partials.data_ptr(), stats.data_ptr(),
        s.table_pointers.data_ptr(), d_params.data_ptr(), layer, runner.status_word.data_ptr(), SPIN_LIMIT, 1,
        torch.cuda.current_stream().cuda_stream)
    assert status == lib.OK, library.rk_last_error()
    torch.cuda.synchronize()  # the kernel came back and released its tensor memory
    with pytest.raises(lib.RichKvError) as caught:
        runner.check()
    assert caught.value.status == lib.TIMEOUT
    runner.status_word.zero_()
    runner.close()
    # the next ordinary launch (which needs the tensor memory the failed CTAs held) is correct
    got16, got32, _ = run_verify_attention_gpu(s, q, rows, rows, committed=committed, splits=splits, tensor_core=True)
    _, want32 = run_verify_attention_oracle(s, q, rows, rows, committed=committed)
    assert_attention_close(got32, want32, got16, "window kernel after a timeout")
    s.close()


def test_exchange_wait_for_a_peer_runs_out_is_reported_and_recovers():
    """The sequence split's fused exchange kernel waits for every rank's flag with a bounded number of polls (about a
    second). Three emulated ranks on one GPU: rank 0 publishes, rank 1 never runs, rank 2 waits for a flag that nothing
    sets, gives up, raises the step's status word and writes zeros; the next complete step on the same buffers is
    right again. Nothing spins without a bound and nothing faults."""
    from richengine_b200 import parallel
    s, q = prepared([2600], INT4, seed=41)
    ranks, visible, place = 3, 2601, None
    place = s.storage.layers()[0]
    shards = []
    for r in range(ranks):
        first, last = parallel.shard_page_range(len(s.pages[0]), r, ranks)
        _, count = parallel.shard_tokens(visible, r, ranks)
        table = s.device_tables[0][first:last].contiguous()
        lane = struct_to_device((lib.VerifyParams * 1)(lib.VerifyParams(count - 1, last - first, place, 1, 1, 1, 1, 0.0)))
        shards.append((table, ops.table_pointer_array([table]), lane))
    exchange = parallel.PeerExchangeDecoder(s.layout, 24, 1, s.storage.window(), rank=0, ranks=ranks, connect=False)
    dq = dev(q)
    out = torch.zeros_like(dq)
    out32 = torch.zeros(dq.shape, dtype=torch.float32, device="cuda")
    out32[:, :, 0] = 1.0  # the rows the step writes
    for r in (0, 2):  # rank 1 stays away
        exchange.step(dq, out, shards[r][1], shards[r][2], place, output_f32=out32, loopback_rank=r)
    torch.cuda.synchronize()  # the kernel came back on its own
    with pytest.raises(lib.RichKvError) as caught:
        exchange.status()
    assert caught.value.status == lib.TIMEOUT
    assert not out32[:, :, 0].any()  # a step that gave up leaves zeros, not a partial answer
    for r in range(ranks):
        exchange.step(dq, out, shards[r][1], shards[r][2], place, output_f32=out32, loopback_rank=r)
    exchange.status()
    torch.cuda.synchronize()
    _, want32 = run_verify_attention_oracle(s, q, 1, 1)
    assert_attention_close(out32.cpu().numpy(), want32, host_u16(out), "the complete step after a timeout")
    exchange.close(); s.close()
