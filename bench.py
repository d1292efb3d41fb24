"""Benchmark of the paged, quantized KV-cache hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch B] [--context T] [--layers L] [--ragged] [--format int4|int8|fp8e4m3|bf16]
                    [--mode decode|verify|prefill|seqsplit|seal|evict|prepare] [--skip-config4] [--skip-check]

A step is one decode pass over the batch: for each attention layer, append one
new K/V token per sequence (quantize into its page) and run one-query paged
decode attention over the whole history. The default workload is the headline
one: int4 KV, 27B geometry (16 layers x 4 KV heads x 256, 24 query heads),
batch 64, 32 768-token contexts, random non-contiguous page tables, synthetic
bf16 N(0,1) K/V with four x20 outlier channels per head (stored through the
library's own append path).

Prints ONE JSON line (rank 0). `value` is KV GB/s with everything resident in
HBM; `e2e` the same metric through the host-buffer call; `roofline` the decode
kernel against the measured HBM peak; `cpu_baseline` the CPU checker timed on a
bounded sample of the same workload. With N > 1 (torchrun) every rank runs its
own batch (requests are sharded, no collective on the data path): weak scaling.
The default line also carries `checked` (two lanes of the measured pool recomputed by the CPU checker in fp64 and held
to the parity bar) and two blocks for the multi-GPU configuration of the baseline: `config4_requests` (one global
batch of 256 ragged requests dealt to the ranks by balanced total context; strong scaling) and `config4_seqsplit`
(one 262 144-token sequence split along the sequence over the ranks, combined by one fused exchange kernel, with the
NCCL all-gather variant timed beside it and compared bit for bit). The other modes print their own line: `verify`
(16-row speculative window), `prefill` (2 048-row chunk), `seqsplit` (the sequence split alone), `seal` (pack +
CRC-32C of model pages), `evict` (coldest quarter of a pool to pinned host memory and back through the request
cache), `prepare` (QKV-prepare fused with the page store).
"""
from __future__ import annotations

import argparse
import ctypes as C
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

KV_HEADS, QUERY_HEADS, HEAD_DIM = 4, 24, 256
METRIC = "int4_paged_decode_attention_kv_gbps"
# dram__bytes_read.sum + dram__bytes_write.sum of the decode kernel per algorithmic KV byte, from the ncu
# capture summarised under profiles/ (a smaller case of the same kernel; traffic grows with the pages read).
DRAM_BYTES_PER_ALGORITHMIC_BYTE = 1.013
TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of decode_int4_kernel on the 16 x 32768-token case "
                  "(profiles/decode_int4_kernel_ncu_b16_ctx32k.md), scaled by the pages read")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--layers", type=int, default=16)
    ap.add_argument("--ragged", action="store_true", help="contexts uniform in [context/4, context]")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--format", default="int4", choices=["int4", "int8", "fp8e4m3", "bf16"],
                    help="stored KV format of the decode workload (the headline is int4)")
    ap.add_argument("--rows", type=int, default=16, choices=[8, 16], help="--mode verify: window rows per sequence")
    ap.add_argument("--chunk", type=int, default=2048, help="--mode prefill: rows of the prefill chunk")
    ap.add_argument("--pages", type=int, default=2048, help="--mode seal: model pages sealed per step")
    ap.add_argument("--skip-config4", action="store_true", help="leave the config-4 blocks (batch 256 dealt to the ranks, "
                    "262144-token sequence split) out of the line")
    ap.add_argument("--skip-check", action="store_true", help="leave the sampled comparison with the CPU checker out")
    ap.add_argument("--mode", default="requests", choices=["requests", "seqsplit", "verify", "prefill", "seal", "evict", "prepare"],
                    help="requests: every rank runs its own batch (default); seqsplit: ONE sequence of --context "
                         "tokens split along the sequence over the ranks, all-gather of (max, sum, O), rank-order merge")
    return ap.parse_args()


def contexts_for(args, rank: int) -> list[int]:
    if not args.ragged:
        return [args.context] * args.batch
    rng = np.random.default_rng(1000 + rank)
    return [int(x) for x in rng.integers(args.context // 4, args.context + 1, size=args.batch)]


def workload_name(args) -> str:
    shape = f"ctx U[{args.context // 4},{args.context}]" if args.ragged else f"ctx {args.context}"
    return (f"{args.format} KV, 27B geometry ({args.layers} layers x {KV_HEADS} KV heads x {HEAD_DIM}, {QUERY_HEADS} query heads), "
            f"batch {args.batch}, {shape}, random page tables; per layer: append 1 token + 1-query decode attention")


# ------------------------------------------------------------------------------------------------
# CPU leg (the checker): bounded sample of the same workload. Used by cpu_baseline and --impl reference.
# ------------------------------------------------------------------------------------------------
class CpuSample:
    """`lanes` sequences of `context` tokens, one layer of int4 pages in host memory with the production addressing.
    The history is bf16 N(0,1) with four x20 outlier channels per head (the generator of the GPU arm's inputs, seeded),
    quantised into the pages by the checker's own store; one-query decode attention through the checker, all host
    threads."""

    def __init__(self, lanes: int, context: int, seed: int = 5):
        sys.path.insert(0, str(ROOT / "tests"))
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "-s"], check=True)
        import oracle as om
        from concurrent.futures import ThreadPoolExecutor
        from kvcase import HostPool, f32_to_bf16
        from richengine_b200 import lib
        from richengine_b200.abi import INT4, Layout, pages_for
        self.om, self.lib = om, lib
        self.layout = Layout(1, KV_HEADS, HEAD_DIM, INT4)
        self.lanes, self.context = lanes, context
        rng = np.random.default_rng(seed)
        pages_per_lane = pages_for(context + 1)
        extent_pages = 256
        extents = (lanes * pages_per_lane + extent_pages - 1) // extent_pages
        self.pool = HostPool(self.layout, extent_pages, extents)
        order = rng.permutation(self.pool.page_count)
        self.pages = [order[i * pages_per_lane:(i + 1) * pages_per_lane] for i in range(lanes)]
        self.tables = [self.pool.table(p) for p in self.pages]
        # four stagings of 2048 rows, reused in rotation like the GPU arm's fill
        chunk = 2048
        stagings = []
        for index in range(4):
            k = rng.standard_normal((KV_HEADS, chunk, HEAD_DIM), dtype=np.float32)
            v = rng.standard_normal((KV_HEADS, HEAD_DIM, chunk), dtype=np.float32)
            for head in range(KV_HEADS):
                channels = rng.choice(HEAD_DIM, size=4, replace=False)
                k[head][:, channels] *= 20.0
                v[head][channels, :] *= 20.0
            stagings.append((f32_to_bf16(k), f32_to_bf16(v)))
        layer = self.pool.layer(0)
        store = om.oracle().rko_store_chunk

        def fill(lane: int) -> None:
            done = 0
            while done < context + 1:
                rows = min(chunk, context + 1 - done)
                k, v = stagings[(lane + done // chunk) % len(stagings)]
                params = lib.ChunkParams(done, rows, chunk, pages_per_lane, layer)
                if store(INT4, KV_HEADS, HEAD_DIM, k.ctypes.data, v.ctypes.data, self.tables[lane].ctypes.data, C.byref(params)) != 0:
                    raise RuntimeError("the checker's store refused the chunk")
                done += rows
        with ThreadPoolExecutor(max_workers=max(1, len(os.sched_getaffinity(0)))) as pool:  # lanes own disjoint pages
            list(pool.map(fill, range(lanes)))
        self.table_pointers = (C.c_void_p * lanes)(*[t.ctypes.data for t in self.tables])
        self.params = (lib.VerifyParams * lanes)(*[
            lib.VerifyParams(context, pages_per_lane, layer, 32, 32, 1, 1, 0.0) for _ in range(lanes)])
        self.queries = f32_to_bf16(rng.standard_normal((lanes, KV_HEADS, 32, QUERY_HEADS // KV_HEADS, HEAD_DIM)).astype(np.float32))
        self.output = np.zeros(self.queries.shape, np.uint16)
        self.kv_bytes = lanes * (context + 1) * self.layout.bytes_per_token_layer()
        self.threads = om.oracle().rko_threads()

    def run_once(self) -> float:
        start = time.perf_counter()
        status = self.om.oracle().rko_attention_verify(self.layout.format, KV_HEADS, QUERY_HEADS // KV_HEADS, HEAD_DIM,
                                                       self.lanes, self.queries.ctypes.data, self.table_pointers,
                                                       self.params, None, self.output.ctypes.data, None)
        assert status == 0
        return time.perf_counter() - start

    def describe(self) -> str:
        return (f"{self.lanes} sequences x {self.context} tokens, 1 layer, int4 pages quantised by the checker's store from "
                f"bf16 N(0,1) rows with four x20 outlier channels per head; one-query decode attention "
                f"(checker port of the reference tile, OpenMP)")


CPU_SAMPLE_LANES = 16


def cpu_baseline(args, budget_seconds: float) -> dict:
    lanes = min(args.batch, CPU_SAMPLE_LANES)
    sample = CpuSample(lanes, args.context)
    sample.run_once()  # warm-up
    times, spent = [], 0.0
    while spent < budget_seconds and len(times) < 64:
        times.append(sample.run_once())
        spent += times[-1]
    median = statistics.median(times)
    return {"value": round(sample.kv_bytes / median / 1e9, 3), "unit": "GB/s", "cores": sample.threads, "kind": "port",
            "sample": f"{sample.describe()}; median of {len(times)} passes, {median * 1e3:.1f} ms each"}


def run_reference(args):
    """The reference's CPU implementation of the path = the checker port (its kernels are Metal and do not
    build here). Rank 0 only. Each step is one pass over a bounded sample of the headline geometry; the line's
    config says what the sample is."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    # all the host threads it can use: torchrun presets OMP_NUM_THREADS=1 for its workers
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    lanes = min(args.batch, CPU_SAMPLE_LANES)
    sample = CpuSample(lanes, args.context)
    for _ in range(max(args.warmup, 1)):
        sample.run_once()
    times = [sample.run_once() for _ in range(args.steps)]
    total = sum(times)
    value = sample.kv_bytes * args.steps / total / 1e9
    line = {
        "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "impl": "reference", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4 codes, fp32 math",
        "data": "synthetic",
        "config": {"workload": f"bounded sample of the headline workload on the host cores: int4 KV, 27B geometry ({KV_HEADS} KV heads x "
                               f"{HEAD_DIM}, {QUERY_HEADS} query heads), batch {lanes} of the {args.batch}, ctx {args.context}, 1 layer of the "
                               f"{args.layers}, random page tables; one step = one 1-query decode attention pass over the sample "
                               f"(GB/s is a rate: the full workload is {args.batch // max(lanes, 1) * args.layers} such passes per step)",
                   "sample_lanes": lanes, "sample_layers": 1, "full_workload": workload_name(args)},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": sample.threads, "kind": "port",
                         "sample": sample.describe() + "; each step is one pass over the sample"},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU leg
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.samples = []
        self.process = None
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--id={device_index}", f"--query-gpu={self.QUERY}",
                                             "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                            stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def keep_loaded(self, begin: float, work, minimum: int = 3, budget_seconds: float = 3.0) -> None:
        """nvidia-smi samples every 100 ms; a timed region shorter than that sees none. Repeat the same work,
        untimed, until `minimum` samples fall inside the window that started at `begin`."""
        if self.process is None:
            return
        deadline = time.perf_counter() + budget_seconds
        while time.perf_counter() < deadline and sum(1 for stamp, _ in self.samples if stamp >= begin) < minimum:
            work()

    def stop(self, begin: float, end: float) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, line in self.samples:
            if stamp < begin or stamp > end:
                continue
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 7:
                continue
            try:
                clocks.append(float(fields[0])); maxima.append(float(fields[1]))
            except ValueError:
                continue
            for name, flag in zip(names, fields[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(maxima) if maxima else None,
                "samples": len(clocks), "reasons": sorted(reasons)}


def peak_hbm() -> tuple[float, str]:
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        return float(json.loads(peaks_path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def build_pool(layout, lane_pages, seed: int):
    """A pool just large enough for `lane_pages` pages per lane, with random non-contiguous page tables."""
    import torch
    from richengine_b200 import ops
    from richengine_b200.storage import PageStorage
    total = sum(lane_pages)
    extent_pages = layout.extent_pages_for(total) or layout.minimum_extent_pages()
    extents = (total + extent_pages - 1) // extent_pages
    storage = PageStorage(layout, extents * extent_pages, extent_pages)
    for extent in range(extents):
        if not storage.allocate_extent(extent):
            raise RuntimeError("KV pool does not fit in device memory")
    order = np.random.default_rng(seed).permutation(extents * extent_pages)
    tables, page_ids, cursor = [], [], 0
    for count in lane_pages:
        table = torch.zeros(max(count, 1), dtype=torch.int64, device="cuda")
        storage.write_entries(order[cursor:cursor + count], 0, table)
        tables.append(table)
        page_ids.append(order[cursor:cursor + count])
        cursor += count
    return storage, tables, ops.table_pointer_array(tables), extent_pages, page_ids


def make_stagings(generator, count: int = 4, chunk: int = 2048):
    """bf16 N(0,1) K/V chunk stagings with four x20 outlier channels per head."""
    import torch
    out = []
    for _ in range(count):
        k = torch.randn((KV_HEADS, chunk, HEAD_DIM), generator=generator, device="cuda")
        v = torch.randn((KV_HEADS, HEAD_DIM, chunk), generator=generator, device="cuda")
        for head in range(KV_HEADS):
            channels = torch.randperm(HEAD_DIM, generator=generator, device="cuda")[:4]
            k[head][:, channels] *= 20.0
            v[head][channels, :] *= 20.0
        out.append((k.to(torch.bfloat16).contiguous(), v.to(torch.bfloat16).contiguous()))
    return out


def fill_history(layout, storage, tables, lane_pages, contexts, layers: int, stagings, first_token=None):
    """Stores every lane's history through the library's own chunk store (all `layers` layers)."""
    from richengine_b200 import lib, ops
    places = storage.layers()
    chunk = stagings[0][0].shape[1]
    for lane, context in enumerate(contexts):
        done = 0
        while done < context:
            rows = min(chunk, context - done)
            k, v = stagings[(lane + done // chunk) % len(stagings)]
            for layer in range(layers):
                ops.store_chunk(layout, k, v, tables[lane], lib.ChunkParams(done, rows, chunk, lane_pages[lane], places[layer]))
            done += rows


def sampled_check(storage, layout, page_ids, lanes_to_check, committed, queries, output, layer: int = 0) -> dict:
    """Untimed: the decode output of a few lanes of the benchmark's own pool against the CPU checker. The lanes'
    pages of one layer are packed on the device, copied to the host and laid out as a small host pool with the
    production addressing; the checker attends them with the same queries."""
    import torch
    sys.path.insert(0, str(ROOT / "tests"))
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "-s"], check=True)
    import oracle as om  # the checker, used here only to check
    from kvcase import HostPool, bf16_to_f32
    from richengine_b200 import lib
    from richengine_b200.abi import Layout, pages_for
    library = lib.load()
    one_layer = Layout(1, layout.kv_heads, layout.head_dimension, layout.format)
    layer_bytes = one_layer.bytes_per_model_page()
    slot_bytes = storage.bytes_per_page()
    worst, scale_seen = 0.0, 1.0
    for lane in lanes_to_check:
        count = pages_for(committed[lane] + 1)
        ids = np.ascontiguousarray(page_ids[lane][:count], dtype=np.uint32)
        host = HostPool(one_layer, 256, (count + 255) // 256)
        for begin in range(0, count, 256):  # 256 pages x all layers at a time on the device
            batch = ids[begin:begin + 256]
            slots = torch.empty(len(batch) * slot_bytes, dtype=torch.uint8, device="cuda")
            lib.check(library.rk_storage_pack_pages(storage.handle, batch.ctypes.data, len(batch), slots.data_ptr(), 0,
                                                    torch.cuda.current_stream().cuda_stream), "pack")
            rows = slots.view(len(batch), slot_bytes)[:, layer * layer_bytes:(layer + 1) * layer_bytes].contiguous().cpu().numpy()
            data, scale = one_layer.data_bytes_per_layer_page(), one_layer.scale_bytes_per_layer_page()
            for i in range(len(batch)):
                cursor = 0
                for tensor in range(4):
                    size = scale if tensor % 2 else data
                    host.tensor_view(begin + i, 0, tensor)[:] = rows[i, cursor:cursor + size]
                    cursor += size
        table = host.table(range(count))
        pointers = (C.c_void_p * 1)(table.ctypes.data)
        params = (lib.VerifyParams * 1)(lib.VerifyParams(committed[lane], count, host.layer(0), 32, 32, 1, 1, 0.0))
        q = queries[lane:lane + 1].contiguous().cpu().view(torch.int16).numpy().view(np.uint16)
        want = np.zeros(q.shape, np.float32)
        out16 = np.zeros(q.shape, np.uint16)
        status = om.oracle().rko_attention_verify(layout.format, KV_HEADS, QUERY_HEADS // KV_HEADS, HEAD_DIM, 1, q.ctypes.data,
                                                  pointers, params, None, out16.ctypes.data, want.ctypes.data)
        if status != 0:
            raise RuntimeError("the checker refused the sampled lane")
        got = bf16_to_f32(output[lane:lane + 1].contiguous().cpu().view(torch.int16).numpy().view(np.uint16))
        scale_seen = max(scale_seen, float(np.abs(want[:, :, 0]).max()))
        worst = max(worst, float(np.abs(got[:, :, 0] - want[:, :, 0]).max()))
    # the device output is bf16: the bar of the parity tests plus half a bf16 ulp of the largest value
    bound = 2e-3 * scale_seen + 2.0 ** -8 * scale_seen
    return {"lanes": list(lanes_to_check), "layer": layer, "max_abs_error": round(worst, 6), "bound": round(bound, 6),
            "ok": bool(worst <= bound), "against": "CPU checker (fp64 attention over the dequantised pages of the same pool)"}


CONFIG4_BATCH, CONFIG4_LAYERS, CONFIG4_SEQUENCE = 256, 4, 262144


def config4_requests(args, rank: int, world: int) -> dict:
    """BASELINE config 4(i): ONE global batch of 256 int4 sequences, contexts uniform in 4096..65536 from a fixed
    seed, dealt to the ranks by balanced total context (parallel.partition_requests); strong scaling, no collective
    on the data path. A step = per layer append one token per sequence + one-query decode attention."""
    import torch
    import torch.distributed as dist
    from richengine_b200 import parallel
    from richengine_b200.abi import INT4, Layout, pages_for
    from richengine_b200.session import DecodeSession

    layers = CONFIG4_LAYERS
    steps, warmup = max(2, min(args.steps, 5)), 3
    contexts_all = [int(x) for x in np.random.default_rng(4004).integers(4096, 65537, size=CONFIG4_BATCH)]
    mine = parallel.partition_requests(contexts_all, world)[rank]
    contexts = [contexts_all[i] for i in mine]
    layout = Layout(layers, KV_HEADS, HEAD_DIM, INT4)
    total_steps = warmup + steps
    lane_pages = [pages_for(c + total_steps + 2) for c in contexts]
    storage, tables, pointers, extent_pages, _ = build_pool(layout, lane_pages, 400 + rank)
    generator = torch.Generator(device="cuda").manual_seed(40 + rank)
    fill_history(layout, storage, tables, lane_pages, contexts, layers, make_stagings(generator))
    lanes = len(contexts)
    session = DecodeSession(storage, QUERY_HEADS, lanes)
    session.queries.normal_(generator=generator)
    session.chunk_keys.normal_(generator=generator)
    session.chunk_values.normal_(generator=generator)
    from richengine_b200 import ops
    device_params = []
    for step in range(total_steps):
        chunk_params = np.zeros(lanes, dtype=ops.CHUNK_PARAMS)
        verify_params = np.zeros(lanes, dtype=ops.VERIFY_PARAMS)
        for lane, context in enumerate(contexts):
            chunk_params[lane] = (context + step, 1, 32, lane_pages[lane], (extent_pages, 0))
            verify_params[lane] = (context + step, lane_pages[lane], (extent_pages, 0), 1, 1, 1, 1, 0.0)
        device_params.append((ops.params_to_device(chunk_params), ops.params_to_device(verify_params)))

    def run(step: int):
        cp, vp = device_params[step]
        for layer in range(layers):
            session.step_device(layer, pointers, cp, vp)

    for step in range(warmup):
        run(step)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(warmup, total_steps):
        run(step)
    stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    session.attention.status()
    my_ms = start.elapsed_time(stop)
    my_bytes = sum(sum(c + step + 1 for c in contexts) for step in range(warmup, total_steps)) * layout.bytes_per_token_layer() * layers
    stats = torch.tensor([my_ms, float(my_bytes)], dtype=torch.float64, device="cuda")
    if world > 1:
        gathered = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(gathered, stats)
    else:
        gathered = [stats]
    session.close()
    storage.close()
    times = [float(g[0]) for g in gathered]
    sizes = [float(g[1]) for g in gathered]
    slowest = max(times)
    peak, _ = peak_hbm()
    value = sum(sizes) / (slowest * 1e-3) / 1e9
    return {
        "workload": f"one global batch of {CONFIG4_BATCH} int4 sequences, contexts uniform in 4096..65536 (seed 4004, "
                    f"{sum(contexts_all)} tokens), {layers} layers resident, dealt to {world} rank(s) by balanced total context; "
                    f"per layer: append 1 token + 1-query decode attention",
        "scaling": "strong", "steps": steps, "warmup": warmup, "value": round(value, 1), "unit": "GB/s",
        "us_per_layer_step": round(slowest / steps / layers * 1e3, 2),
        "requests_per_rank": [len(a) for a in parallel.partition_requests(contexts_all, world)],
        "kv_gb_per_layer_step_per_rank": [round(b / steps / layers / 1e9, 4) for b in sizes],
        "ms_per_rank": [round(t, 3) for t in times],
        "imbalance_max_over_mean_bytes": round(max(sizes) / (sum(sizes) / len(sizes)), 4),
        "hbm_frac_per_gpu": round(value / world / peak, 4),
    }


def config4_seqsplit(args, rank: int, world: int, sequence: int = CONFIG4_SEQUENCE, layers: int = 16) -> dict:
    """BASELINE config 4(ii): ONE int4 sequence of 262 144 tokens split along the sequence over the ranks (world 1
    included: the same kernels, one shard). Two combines are timed: the library's own fused kernel (reduce -> peer
    stores over NVLink -> flags -> rank-order merge; the product) and, for world > 1, the NCCL all-gather of the
    per-rank {max, sum, O} triples + merge kernel (the baseline it is measured against)."""
    import torch
    import torch.distributed as dist
    from richengine_b200 import lib, ops, parallel
    from richengine_b200.abi import INT4, Layout, pages_for

    steps, warmup = max(2, min(args.steps, 10)), 3
    layout = Layout(layers, KV_HEADS, HEAD_DIM, INT4)
    visible = sequence + 1
    begin, count = parallel.shard_tokens(visible, rank, world)
    first, last = parallel.shard_page_range(pages_for(visible), rank, world)
    local_pages = max(last - first, 1)
    storage, tables, pointers, extent_pages, _ = build_pool(layout, [local_pages], 30 + rank)
    generator = torch.Generator(device="cuda").manual_seed(11 + rank)
    fill_history(layout, storage, tables, [local_pages], [count], layers, make_stagings(generator, 2))
    places = storage.layers()
    queries = torch.randn((1, KV_HEADS, 32, QUERY_HEADS // KV_HEADS, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    if world > 1:
        dist.broadcast(queries, 0)  # every rank attends with the same query
    lane = np.zeros(1, dtype=ops.VERIFY_PARAMS)
    lane[0] = (max(count, 1) - 1, local_pages if count else 0, (extent_pages, 0), 1, 1, 1, 1, 0.0)  # no pages: an empty shard
    params = ops.params_to_device(lane)
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn) -> float:
        for _ in range(warmup):
            step_fn()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            step_fn()
        stop.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item())

    def agree(tensor) -> bool:
        check = tensor.view(torch.int16).to(torch.int64).sum().reshape(1)
        if world == 1:
            return True
        sums = [torch.zeros_like(check) for _ in range(world)]
        dist.all_gather(sums, check)
        return bool(all(int(x) == int(sums[0]) for x in sums))

    result = {
        "workload": f"one int4 sequence of {sequence} tokens split along the sequence over {world} GPU(s), {layers} layers; "
                    f"per layer: streaming decode over the rank's pages, exchange of {QUERY_HEADS * (HEAD_DIM + 2) * 4} B of "
                    f"(max, sum, O) per rank, rank-order merge on every rank",
        "scaling": "strong", "steps": steps, "warmup": warmup,
        "kv_mb_per_layer_step_per_rank": round(count * layout.bytes_per_token_layer() / 1e6, 2),
    }
    total_bytes = visible * layout.bytes_per_token_layer() * layers * steps
    peak, _ = peak_hbm()

    # ---- the product: fused reduce + peer stores + merge ------------------------------------------------------
    out_peer = torch.zeros_like(queries)
    try:
        peer = parallel.PeerExchangeDecoder(layout, QUERY_HEADS, 1, storage.window(), rank=rank, ranks=world)

        def peer_step():
            for layer in range(layers):
                peer.step(queries, out_peer, pointers, params, places[layer])
        ms = timed(peer_step)
        peer.status()
        result.update({"us_per_layer_step": round(ms / steps / layers * 1e3, 2), "value": round(total_bytes / (ms * 1e-3) / 1e9, 1),
                       "unit": "GB/s", "hbm_frac_per_gpu": round(total_bytes / (ms * 1e-3) / 1e9 / world / peak, 4),
                       "combine": "fused reduce + peer stores + flags + merge (one kernel of the library, no collective library)",
                       "ranks_agree": agree(out_peer)})
        peer.close()
    except Exception as error:  # e.g. CUDA IPC unavailable in this container: the NCCL variant below still reports
        result["peer_exchange_error"] = str(error)[:300]

    # ---- the baseline: NCCL all-gather + merge kernel -------------------------------------------------------------
    if world > 1:
        out_nccl = torch.zeros_like(queries)
        decoder = parallel.SequenceSplitDecoder(layout, QUERY_HEADS, 1, storage.window())

        def nccl_step():
            for layer in range(layers):
                decoder.step(queries, out_nccl, pointers, params, places[layer])
        ms = timed(nccl_step)
        decoder.inner.status()
        # the all-gather's share: CUDA events around it on this rank's stream, one untimed pass
        spans = []
        for layer in range(layers):
            triples = decoder.shard(queries, pointers, params, places[layer])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            gathered = parallel.gather_shards(triples, None, decoder.gathered)
            b.record()
            decoder.merge(gathered, out_nccl)
            spans.append((a, b))
        torch.cuda.synchronize()
        gather_us = statistics.mean(a.elapsed_time(b) for a, b in spans) * 1e3
        result["nccl_variant"] = {"us_per_layer_step": round(ms / steps / layers * 1e3, 2), "allgather_us": round(gather_us, 2),
                                  "allgather_share": round(gather_us / (ms / steps / layers * 1e3), 3),
                                  "ranks_agree": agree(out_nccl),
                                  "same_bits_as_fused": bool(torch.equal(out_nccl, out_peer)) if "us_per_layer_step" in result else None}
        if "us_per_layer_step" not in result:  # the fused variant could not run: the NCCL variant is the number
            result.update({"us_per_layer_step": result["nccl_variant"]["us_per_layer_step"], "ranks_agree": result["nccl_variant"]["ranks_agree"],
                           "value": round(total_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "combine": "NCCL all-gather + merge kernel"})
        decoder.close()
    storage.close()
    return result


def run_ours(args):
    import torch
    import torch.distributed as dist

    from richengine_b200 import lib, ops
    from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout, pages_for
    from richengine_b200.session import DecodeSession
    from richengine_b200.storage import PageStorage

    fmt = {"int4": INT4, "int8": INT8, "fp8e4m3": FP8E4M3, "bf16": BF16}[args.format]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        # a short timeout: a rank that failed must end the others' next collective, not leave them spinning
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=240))
    lib.load()

    layout = Layout(args.layers, KV_HEADS, HEAD_DIM, fmt)
    contexts = contexts_for(args, rank)
    lanes = len(contexts)
    steps_total = args.warmup + args.steps
    # every lane keeps room for the tokens the run appends
    lane_pages = [pages_for(c + 2 * steps_total + 2) for c in contexts]
    extent_pages = layout.extent_pages_for(sum(lane_pages)) or layout.minimum_extent_pages()
    extents = (sum(lane_pages) + extent_pages - 1) // extent_pages
    storage = PageStorage(layout, extents * extent_pages, extent_pages)
    for extent in range(extents):
        if not storage.allocate_extent(extent):
            raise RuntimeError("KV pool does not fit in device memory")
    rng = np.random.default_rng(42 + rank)
    order = rng.permutation(extents * extent_pages)
    tables, lane_page_ids, cursor = [], [], 0
    for count in lane_pages:
        table = torch.zeros(count, dtype=torch.int64, device="cuda")
        storage.write_entries(order[cursor:cursor + count], 0, table)
        tables.append(table)
        lane_page_ids.append(order[cursor:cursor + count])
        cursor += count
    table_pointers = ops.table_pointer_array(tables)
    places = storage.layers()

    # ---- fill the history through the library's own chunk store -------------------------------
    chunk = 2048
    generator = torch.Generator(device="cuda").manual_seed(7 + rank)
    def staging():
        k = torch.randn((KV_HEADS, chunk, HEAD_DIM), generator=generator, device="cuda")
        v = torch.randn((KV_HEADS, HEAD_DIM, chunk), generator=generator, device="cuda")
        for head in range(KV_HEADS):
            channels = torch.randperm(HEAD_DIM, generator=generator, device="cuda")[:4]
            k[head][:, channels] *= 20.0
            v[head][channels, :] *= 20.0
        return k.to(torch.bfloat16).contiguous(), v.to(torch.bfloat16).contiguous()
    stagings = [staging() for _ in range(4)]
    for lane, context in enumerate(contexts):
        done = 0
        while done < context:
            rows = min(chunk, context - done)
            k, v = stagings[(lane + done // chunk) % len(stagings)]
            for layer in range(args.layers):
                ops.store_chunk(layout, k, v, tables[lane], lib.ChunkParams(done, rows, chunk, lane_pages[lane], places[layer]))
            done += rows
    torch.cuda.synchronize()

    session = DecodeSession(storage, QUERY_HEADS, lanes)
    session.queries.normal_(generator=generator)
    session.chunk_keys.normal_(generator=generator)
    session.chunk_values.normal_(generator=generator)

    def params_for(step: int):
        chunk_params = np.zeros(lanes, dtype=ops.CHUNK_PARAMS)
        verify_params = np.zeros(lanes, dtype=ops.VERIFY_PARAMS)
        for lane, context in enumerate(contexts):
            committed = context + step
            chunk_params[lane] = (committed, 1, 32, lane_pages[lane], (extent_pages, 0))
            verify_params[lane] = (committed, lane_pages[lane], (extent_pages, 0), 1, 1, 1, 1, 0.0)
        return ops.params_to_device(chunk_params), ops.params_to_device(verify_params)
    device_params = [params_for(step) for step in range(2 * steps_total + 1)]
    kv_bytes_per_step = lambda step: sum(c + step + 1 for c in contexts) * layout.bytes_per_token_layer() * args.layers

    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def device_step(step: int):
        cp, vp = device_params[step]
        for layer in range(args.layers):
            session.step_device(layer, table_pointers, cp, vp)

    # ---- device-resident timing: `value` -------------------------------------------------------
    for step in range(args.warmup):
        device_step(step)
        if step == 0:
            session.attention.status()  # a device-side timeout stops the run here, not after every launch
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches_before = session.kernel_launches
    begin_wall = time.perf_counter()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(args.warmup, steps_total):
        device_step(step)
    stop.record()
    barrier()
    end_wall = time.perf_counter()
    elapsed_ms = start.elapsed_time(stop)
    launches = session.kernel_launches - launches_before
    session.attention.status()
    timed_bytes = sum(kv_bytes_per_step(s) for s in range(args.warmup, steps_total))

    # ---- decode kernel alone: roofline -----------------------------------------------------------
    # Two figures. Back to back, as the launches run inside a step: one event pair around all layers' launches, divided
    # by their number (the merge is a programmatic dependent launch and the next layer's launch follows it without a
    # gap) — the roofline's duration. Isolated: one event pair per launch, which ends that overlap and adds the events'
    # own cost; reported beside it.
    cp, vp = device_params[steps_total]
    events = []
    for repeat in range(2):
        for layer in range(args.layers):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            session.attend_device(layer, table_pointers, vp)
            b.record()
            if repeat:
                events.append((a, b))
    run_begin, run_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    run_begin.record()
    for layer in range(args.layers):
        session.attend_device(layer, table_pointers, vp)
    run_end.record()
    torch.cuda.synchronize()
    isolated_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    kernel_ms = run_begin.elapsed_time(run_end) / args.layers
    layer_bytes = sum(c + steps_total + 1 for c in contexts) * layout.bytes_per_token_layer()

    # ---- end to end through the host-buffer call: `e2e` -----------------------------------------
    q_host = torch.randn((lanes, QUERY_HEADS, HEAD_DIM)).to(torch.bfloat16).pin_memory()
    k_host = torch.randn((lanes, KV_HEADS, HEAD_DIM)).to(torch.bfloat16).pin_memory()
    v_host = torch.randn((lanes, KV_HEADS, HEAD_DIM)).to(torch.bfloat16).pin_memory()
    out_host = torch.zeros((lanes, QUERY_HEADS, HEAD_DIM), dtype=torch.bfloat16).pin_memory()

    enqueue_seconds = [0.0]  # host time spent issuing the steps' calls (the device runs behind)

    def host_step(step: int):
        cp, vp = device_params[step]
        t0 = time.perf_counter()
        for layer in range(args.layers):
            session.step_host(layer, q_host, k_host, v_host, out_host, table_pointers, cp, vp)
        session.finish_host()
        enqueue_seconds[0] += time.perf_counter() - t0
        torch.cuda.current_stream().synchronize()  # the step's result is read on the host
        return float(out_host[0, 0, 0])

    base = steps_total
    for step in range(args.warmup):
        host_step(base + step)
    barrier()
    enqueue_seconds[0] = 0.0
    e2e_start = time.perf_counter()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for step in range(args.warmup, steps_total):
        host_step(base + step)
    e2.record()
    barrier()
    e2e_ms = max(s2.elapsed_time(e2), 0.0)
    e2e_wall_ms = (time.perf_counter() - e2e_start) * 1e3
    e2e_bytes = sum(kv_bytes_per_step(base + s) for s in range(args.warmup, steps_total))
    h2d, d2h = session.host_bytes_per_layer()
    session.attention.status()
    # clocks over all three timed regions (device-resident steps, decode kernel alone, host-buffer steps)
    if sampler:
        def same_load():
            device_step(steps_total)
            torch.cuda.synchronize()
        sampler.keep_loaded(begin_wall, same_load)
    clocks = sampler.stop(begin_wall, time.perf_counter()) if sampler else None

    # ---- untimed: two lanes of the workload that was just timed, against the CPU checker -----------------------
    check = None
    if rank == 0 and not args.skip_check:
        try:
            cp, vp = device_params[steps_total]
            session.attend_device(0, table_pointers, vp)
            torch.cuda.synchronize()
            check = sampled_check(storage, layout, lane_page_ids, [0, lanes - 1] if lanes > 1 else [0],
                                  [c + steps_total for c in contexts], session.queries, session.output)
        except Exception as error:
            check = {"ok": False, "error": str(error)[:300]}

    # ---- reduce over ranks: max time, summed bytes --------------------------------------------------
    stats = torch.tensor([elapsed_ms, float(timed_bytes), max(e2e_ms, e2e_wall_ms), float(e2e_bytes)], dtype=torch.float64, device="cuda")
    if world > 1:
        times = stats[[0, 2]].clone(); sums = stats[[1, 3]].clone()
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        stats = torch.stack([times[0], sums[0], times[1], sums[1]])
    elapsed_ms, timed_bytes, e2e_time_ms, e2e_bytes = [float(x) for x in stats.cpu()]

    # ---- BASELINE config 4 on the same ranks (the headline pool is released first) ------------------------------
    session.close()
    storage.close()
    del tables, table_pointers
    torch.cuda.empty_cache()
    config4 = {}
    if fmt == INT4 and not args.skip_config4:
        for name, block in (("config4_requests", config4_requests), ("config4_seqsplit", config4_seqsplit)):
            try:
                config4[name] = block(args, rank, world)
            except Exception as error:  # a failed block never hides the headline numbers
                config4[name] = {"error": str(error)[:300]}
            torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_source = peak_hbm()
        achieved = layer_bytes / (kernel_ms * 1e-3) / 1e9
        value = timed_bytes / (elapsed_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC if fmt == INT4 else METRIC.replace("int4", args.format), "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(elapsed_ms / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": f"{args.format} codes, {'bf16' if fmt == BF16 else 'fp16'} tensor operands, fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": workload_name(args), "l2": "inputs larger than L2 (KV per step >> 126 MB)",
                       "us_per_layer_step": round(elapsed_ms / args.steps / args.layers * 1e3, 2),
                       "kv_gb_per_step": round(timed_bytes / args.steps / world / 1e9, 3), "sharding": "by request"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         "traffic": round(DRAM_BYTES_PER_ALGORITHMIC_BYTE * layer_bytes) if fmt == INT4 else None,
                         "traffic_source": TRAFFIC_SOURCE if fmt == INT4 else None, "peak_source": peak_source,
                         "kernel": {INT4: "decode_int4_kernel", INT8: "decode_bytes_kernel<int8>", FP8E4M3: "decode_bytes_kernel<fp8>",
                                    BF16: "decode_bf16_kernel"}[fmt] + " (+ its merge)", "us_per_launch": round(kernel_ms * 1e3, 2),
                         "timing": f"{args.layers} launches back to back between one pair of CUDA events, divided by their number",
                         "us_per_launch_isolated": round(isolated_ms * 1e3, 2), "algorithmic_bytes_per_launch": layer_bytes},
            "e2e": {"value": round(e2e_bytes / (e2e_time_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "h2d_bytes_per_step": h2d * args.layers, "d2h_bytes_per_step": d2h * args.layers,
                    "ms_per_step": round(e2e_time_ms / args.steps, 4),
                    "host_issue_ms_per_step": round(enqueue_seconds[0] * 1e3 / args.steps, 4)},
            "gpu_launches": launches,
            "clocks": clocks,
            "checked": check,
            **config4,
        }
        try:
            line["cpu_baseline"] = cpu_baseline(args, args.cpu_seconds) if world == 1 and args.cpu_seconds > 0 and fmt == INT4 else None
        except Exception as error:  # the CPU leg never hides the GPU numbers
            line["cpu_baseline"] = {"error": str(error)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_seqsplit(args):
    """`--mode seqsplit`: the config-4 sequence-split block alone (one int4 sequence of --context tokens over the ranks)."""
    import datetime
    import torch
    import torch.distributed as dist

    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=240))
    sequence = CONFIG4_SEQUENCE if (args.batch == 64 and args.context == 32768) else args.context  # the headline defaults: take this mode's own
    block = config4_seqsplit(args, rank, world, sequence=sequence, layers=args.layers)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": block.get("value"), "unit": "GB/s", "n_gpus": world, "steps": block["steps"],
            "warmup": block["warmup"], "ms_per_step": round(block.get("us_per_layer_step", 0.0) * args.layers / 1e3, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 codes, fp16 tensor operands, fp32 accumulate", "data": "synthetic", "config": block,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_verify(args):
    """Speculative verify on int4 pages: per step and layer, append the window's rows (quantize into the pages)
    and attend them causally over the whole history on the tcgen05 window kernel; then a seeded number of rows
    is accepted and the rest rolled back (the next step starts at committed + accepted). One GPU."""
    import torch

    from richengine_b200 import hostplane, lib, ops
    from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout, pages_for
    from richengine_b200.storage import PageStorage

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rows, lanes = args.rows, args.batch
    fmt = {"int4": INT4, "int8": INT8, "fp8e4m3": FP8E4M3, "bf16": BF16}[args.format]
    layout = Layout(args.layers, KV_HEADS, HEAD_DIM, fmt)
    steps_total = args.warmup + args.steps
    lane_pages = pages_for(args.context + rows * (steps_total + 1))
    extent_pages = layout.extent_pages_for(lanes * lane_pages) or layout.minimum_extent_pages()
    extents = (lanes * lane_pages + extent_pages - 1) // extent_pages
    storage = PageStorage(layout, extents * extent_pages, extent_pages)
    for extent in range(extents):
        if not storage.allocate_extent(extent):
            raise RuntimeError("KV pool does not fit in device memory")
    order = np.random.default_rng(42).permutation(extents * extent_pages)
    tables = []
    for lane in range(lanes):
        table = torch.zeros(lane_pages, dtype=torch.int64, device="cuda")
        storage.write_entries(order[lane * lane_pages:(lane + 1) * lane_pages], 0, table)
        tables.append(table)
    pointers = ops.table_pointer_array(tables)
    places = storage.layers()
    generator = torch.Generator(device="cuda").manual_seed(7)
    k = torch.randn((KV_HEADS, 2048, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    v = torch.randn((KV_HEADS, HEAD_DIM, 2048), generator=generator, device="cuda").to(torch.bfloat16)
    for lane in range(lanes):
        done = 0
        while done < args.context:
            count = min(2048, args.context - done)
            for layer in range(args.layers):
                ops.store_chunk(layout, k, v, tables[lane], lib.ChunkParams(done, count, 2048, lane_pages, places[layer]))
            done += count
    group = QUERY_HEADS // KV_HEADS
    queries = torch.randn((lanes, KV_HEADS, 32, group, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    chunk_keys = torch.randn((lanes, KV_HEADS, 32, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    chunk_values = torch.randn((lanes, KV_HEADS, HEAD_DIM, 32), generator=generator, device="cuda").to(torch.bfloat16)
    output = torch.zeros_like(queries)
    runner = ops.VerifyWindowAttention(layout, QUERY_HEADS, storage.window())

    # accepted rows per (step, lane), seeded 0..rows; a step's committed length = context + what was accepted before
    accepted = np.random.default_rng(9).integers(0, rows + 1, size=(steps_total, lanes))
    committed = args.context + np.concatenate([np.zeros((1, lanes), np.int64), np.cumsum(accepted, axis=0)[:-1]])
    step_params, slots = [], 0
    for step in range(steps_total):
        history = [int(x) for x in committed[step]]
        _, plan = hostplane.verify_plan(lanes, QUERY_HEADS, layout, history, row_capacity=rows, ctas=0)
        assert fmt != INT4 or plan[15] == 1, "the window plan was not selected"
        lane_splits = [hostplane.window_splits(lanes, KV_HEADS, h + rows, 0) for h in history]
        chunk_params = np.zeros(lanes, dtype=ops.CHUNK_PARAMS)
        verify_params = np.zeros(lanes, dtype=ops.VERIFY_PARAMS)
        slot = max(lane_splits)
        for lane in range(lanes):
            chunk_params[lane] = (history[lane], rows, 32, lane_pages, (extent_pages, 0))
            verify_params[lane] = (history[lane], lane_pages, (extent_pages, 0), lane_splits[lane], slot, rows, rows, 0.0)
        step_params.append((ops.params_to_device(chunk_params), ops.params_to_device(verify_params), slot))
        slots = max(slots, slot)
    fused = rows * group
    partials = torch.empty(lanes * KV_HEADS * slots * fused * HEAD_DIM, dtype=torch.float32, device="cuda")
    statistics_buffer = torch.empty(lanes * KV_HEADS * slots * fused * 2, dtype=torch.float32, device="cuda")

    def step_once(step: int):
        cp, vp, slot = step_params[step]
        for layer in range(args.layers):
            ops.store_verify(layout, chunk_keys, chunk_values, pointers, cp, places[layer], lanes, rows)
            runner.split(lanes, rows, slot, queries, partials, statistics_buffer, pointers, None, vp, places[layer])
            ops.attention_verify_reduce(layout, QUERY_HEADS, lanes, rows, partials, statistics_buffer, output, vp)

    for step in range(args.warmup):
        step_once(step)
    torch.cuda.synchronize()
    runner.check()
    sampler = ClockSampler(torch.cuda.current_device())
    begin_wall = time.perf_counter()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for step in range(args.warmup, steps_total):
        step_once(step)
    stop.record()
    torch.cuda.synchronize()
    elapsed_ms = start.elapsed_time(stop)
    # the window kernel alone, per layer
    cp, vp, slot = step_params[steps_total - 1]
    events = []
    for repeat in range(3):
        for layer in range(args.layers):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            runner.split(lanes, rows, slot, queries, partials, statistics_buffer, pointers, None, vp, places[layer])
            b.record()
            if repeat:
                events.append((a, b))
    torch.cuda.synchronize()
    runner.check()
    def same_load():
        step_once(steps_total - 1)
        torch.cuda.synchronize()
    sampler.keep_loaded(begin_wall, same_load)
    clocks = sampler.stop(begin_wall, time.perf_counter())
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    tokens = [int(committed[s].sum()) + rows * lanes for s in range(args.warmup, steps_total)]
    timed_bytes = sum(tokens) * layout.bytes_per_token_layer() * args.layers
    layer_tokens = int(committed[steps_total - 1].sum()) + rows * lanes
    flops = 4.0 * rows * QUERY_HEADS * HEAD_DIM * layer_tokens  # QK^T and PV, 2 flop per multiply-add
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["bf16_tflops"]) if peaks_path.exists() else 1590.0
    print(json.dumps({
        "metric": f"{args.format}_paged_verify_attention_kv_gbps", "value": round(timed_bytes / (elapsed_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(elapsed_ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"{args.format} codes, {'bf16' if fmt == BF16 else 'fp16'} tcgen05 operands, fp32 accumulate in tensor memory", "data": "synthetic",
        "config": {"workload": f"speculative verify, {args.format} KV, 27B geometry ({args.layers} layers), batch {lanes}, {args.context}-token contexts, "
                               f"{rows}-row window: per layer append {rows} rows + window attention + merge; seeded acceptance 0..{rows}, rejected rows rolled back",
                   "l2": "inputs larger than L2", "us_per_layer_step": round(elapsed_ms / args.steps / args.layers * 1e3, 2),
                   "splits_per_lane": slot},
        "roofline": {"bound": "tensor", "achieved": round(flops / (kernel_ms * 1e-3) / 1e12, 1), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(flops / (kernel_ms * 1e-3) / 1e12 / peak, 4), "traffic": None,
                     "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops)" if peaks_path.exists() else "fallback",
                     "kernel": "window_attention_kernel", "us_per_launch": round(kernel_ms * 1e3, 2),
                     "algorithmic_flops_per_launch": flops,
                     "kv_gbps_of_launch": round(layer_tokens * layout.bytes_per_token_layer() / (kernel_ms * 1e-3) / 1e9, 1)},
        "gpu_launches": 3 * args.layers * args.steps, "clocks": clocks,
    }), flush=True)
    runner.close()


def run_prefill(args):
    """Chunked prefill of one sequence on int4 pages: per step and layer, append the chunk's rows (quantize into the
    pages) and attend them causally over the history in 8-row tiles on the tcgen05 window kernel. One GPU."""
    import torch

    from richengine_b200 import lib, ops
    from richengine_b200.abi import INT4, Layout, pages_for, prefill_splits
    from richengine_b200.storage import PageStorage

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rows, history = args.chunk, args.context
    layout = Layout(args.layers, KV_HEADS, HEAD_DIM, INT4)
    pages = pages_for(history + rows)
    extent_pages = layout.minimum_extent_pages()
    extents = (pages + extent_pages - 1) // extent_pages
    storage = PageStorage(layout, extents * extent_pages, extent_pages)
    for extent in range(extents):
        if not storage.allocate_extent(extent):
            raise RuntimeError("KV pool does not fit in device memory")
    table = torch.zeros(pages, dtype=torch.int64, device="cuda")
    storage.write_entries(np.random.default_rng(42).permutation(extents * extent_pages)[:pages], 0, table)
    places = storage.layers()
    generator = torch.Generator(device="cuda").manual_seed(7)
    group = QUERY_HEADS // KV_HEADS
    stride = (rows + 31) // 32 * 32
    k = torch.randn((KV_HEADS, 2048, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    v = torch.randn((KV_HEADS, HEAD_DIM, 2048), generator=generator, device="cuda").to(torch.bfloat16)
    done = 0
    while done < history:
        count = min(2048, history - done)
        for layer in range(args.layers):
            ops.store_chunk(layout, k, v, table, lib.ChunkParams(done, count, 2048, pages, places[layer]))
        done += count
    chunk_keys = torch.randn((KV_HEADS, stride, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    chunk_values = torch.randn((KV_HEADS, HEAD_DIM, stride), generator=generator, device="cuda").to(torch.bfloat16)
    queries = torch.randn((KV_HEADS, stride, group, HEAD_DIM), generator=generator, device="cuda").to(torch.bfloat16)
    output = torch.zeros_like(queries)
    tiles = (rows + 7) // 8
    splits = prefill_splits(tiles)
    partials = torch.empty(tiles * KV_HEADS * splits * 8 * group * HEAD_DIM, dtype=torch.float32, device="cuda")
    statistics_buffer = torch.empty(tiles * KV_HEADS * splits * 8 * group * 2, dtype=torch.float32, device="cuda")
    runner = ops.VerifyWindowAttention(layout, QUERY_HEADS, storage.window())

    def step_once():  # the same chunk position every step: the rows are overwritten in place
        for layer in range(args.layers):
            ops.store_chunk(layout, chunk_keys, chunk_values, table, lib.ChunkParams(history, rows, stride, pages, places[layer]))
            params = lib.PrefillParams(history, rows, stride, pages, places[layer], splits, 0.0)
            runner.prefill_split(queries, partials, statistics_buffer, table, params)
            ops.attention_prefill_reduce(layout, QUERY_HEADS, partials, statistics_buffer, output, params)

    for _ in range(args.warmup):
        step_once()
    torch.cuda.synchronize()
    runner.check()
    sampler = ClockSampler(torch.cuda.current_device())
    begin_wall = time.perf_counter()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step_once()
    stop.record()
    torch.cuda.synchronize()
    elapsed_ms = start.elapsed_time(stop)
    events = []
    params = lib.PrefillParams(history, rows, stride, pages, places[0], splits, 0.0)
    for repeat in range(4):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.prefill_split(queries, partials, statistics_buffer, table, params)
        b.record()
        if repeat:
            events.append((a, b))
    torch.cuda.synchronize()
    runner.check()

    def same_load():
        step_once()
        torch.cuda.synchronize()
    sampler.keep_loaded(begin_wall, same_load)
    clocks = sampler.stop(begin_wall, time.perf_counter())
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    flops = 4.0 * QUERY_HEADS * HEAD_DIM * sum(history + r + 1 for r in range(rows))  # causal: row r sees history + r + 1 tokens
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["bf16_tflops"]) if peaks_path.exists() else 1590.0
    print(json.dumps({
        "metric": "int4_paged_prefill_rows_per_s", "value": round(rows * args.steps / (elapsed_ms * 1e-3), 1), "unit": "rows/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(elapsed_ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 codes, fp16 tcgen05 operands, fp32 accumulate in tensor memory", "data": "synthetic",
        "config": {"workload": f"chunked prefill, int4 KV, 27B geometry ({args.layers} layers), one sequence, {history} tokens of history, "
                               f"chunk of {rows} rows: per layer append the chunk + causal attention in 8-row tiles + merge",
                   "l2": "the history is re-read by every tile; the KV of one layer fits L2", "us_per_layer_step": round(elapsed_ms / args.steps / args.layers * 1e3, 2),
                   "tiles": tiles, "splits": splits},
        "roofline": {"bound": "tensor", "achieved": round(flops / (kernel_ms * 1e-3) / 1e12, 1), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(flops / (kernel_ms * 1e-3) / 1e12 / peak, 4), "traffic": None,
                     "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops)" if peaks_path.exists() else "fallback",
                     "kernel": "window_attention_kernel (prefill tiles)", "us_per_launch": round(kernel_ms * 1e3, 2),
                     "algorithmic_flops_per_launch": flops},
        "gpu_launches": 3 * args.layers * args.steps, "clocks": clocks,
    }), flush=True)
    runner.close()


def run_seal(args):
    """Sealing model pages for the persistent tier: per step, pack --pages pages of an int4 pool (all layers) into
    contiguous slots and take each slot's CRC-32C on the GPU; end to end the slots and checksums also cross to pinned
    host memory. The dominant kernel is the checksum. One GPU."""
    import torch

    from richengine_b200 import lib
    from richengine_b200.abi import INT4, Layout
    from richengine_b200.storage import PageStorage

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    library = lib.load()
    layout = Layout(args.layers, KV_HEADS, HEAD_DIM, INT4)
    count = args.pages
    extent_pages = layout.minimum_extent_pages()
    extents = (count + extent_pages - 1) // extent_pages
    storage = PageStorage(layout, extents * extent_pages, extent_pages)
    for extent in range(extents):
        if not storage.allocate_extent(extent):
            raise RuntimeError("KV pool does not fit in device memory")
        raw = torch.randint(0, 256, (storage.extent_bytes(),), dtype=torch.uint8, device="cuda")
        storage.write_extent(extent, raw.cpu().numpy())
    page_bytes = storage.bytes_per_page()
    ids = np.random.default_rng(3).permutation(extents * extent_pages)[:count].astype(np.uint32)
    slots = torch.empty(count * page_bytes, dtype=torch.uint8, device="cuda")
    sums = torch.zeros(count, dtype=torch.int32, device="cuda")
    host_slots = torch.empty(count * page_bytes, dtype=torch.uint8, pin_memory=True)
    host_sums = torch.zeros(count, dtype=torch.int32, pin_memory=True)
    stream = torch.cuda.current_stream().cuda_stream

    def seal_two_passes():  # pack, then checksum the packed slots: the page is read twice
        lib.check(library.rk_storage_pack_pages(storage.handle, ids.ctypes.data, count, slots.data_ptr(), 0, stream), "pack")
        lib.check(library.rk_crc32c_pages(slots.data_ptr(), page_bytes, page_bytes, count, sums.data_ptr(), 0, stream), "checksum")

    def seal():  # one pass: every row is read from its span, written to its slot and folded into the checksum
        lib.check(library.rk_storage_seal_pages(storage.handle, ids.ctypes.data, count, slots.data_ptr(), sums.data_ptr(), stream), "seal")

    def seal_to_host():
        seal()
        host_slots.copy_(slots, non_blocking=True)
        host_sums.copy_(sums, non_blocking=True)

    for _ in range(args.warmup):
        seal_to_host()
    torch.cuda.synchronize()
    # one slot against the checker before anything is timed
    probe = host_slots[:page_bytes].numpy()
    sys.path.insert(0, str(ROOT / "tests"))
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "-s"], check=True)
    import oracle as om  # the checker: the cpu_baseline leg and one probe
    want = om.oracle().rko_crc32c(probe.ctypes.data, page_bytes, 0)
    if int(host_sums[0].item()) & 0xffffffff != want:
        raise RuntimeError("device CRC-32C differs from the checker")
    sampler = ClockSampler(torch.cuda.current_device())
    begin_wall = time.perf_counter()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        seal()
    stop.record()
    torch.cuda.synchronize()
    device_ms = start.elapsed_time(stop) / args.steps
    start.record()
    for _ in range(args.steps):
        seal_two_passes()
    stop.record()
    torch.cuda.synchronize()
    two_pass_ms = start.elapsed_time(stop) / args.steps
    start.record()
    for _ in range(args.steps):
        seal_to_host()
    stop.record()
    torch.cuda.synchronize()
    host_ms = start.elapsed_time(stop) / args.steps
    events = []
    for repeat in range(6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        lib.check(library.rk_crc32c_pages(slots.data_ptr(), page_bytes, page_bytes, count, sums.data_ptr(), 0, stream), "checksum")
        b.record()
        if repeat:
            events.append((a, b))
    torch.cuda.synchronize()

    def same_load():
        seal()
        torch.cuda.synchronize()
    sampler.keep_loaded(begin_wall, same_load)
    clocks = sampler.stop(begin_wall, time.perf_counter())
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    total = count * page_bytes
    # the checker on the host cores, one thread, on a bounded sample of the same slots
    sample_pages = max(1, min(count, int(args.cpu_seconds * 0.25e9) // page_bytes))
    view = host_slots[:sample_pages * page_bytes].numpy()
    t0 = time.perf_counter()
    for i in range(sample_pages):
        om.oracle().rko_crc32c(view[i * page_bytes:].ctypes.data, page_bytes, 0)
    cpu_seconds = time.perf_counter() - t0
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else 6650.0
    print(json.dumps({
        "metric": "int4_model_page_seal_gbps", "value": round(total / (device_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(device_ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8 (CRC-32C over GF(2), 32-bit remainders)", "data": "synthetic",
        "config": {"workload": f"seal {count} model pages of an int4 pool ({args.layers} layers, {page_bytes} B each): pack the page's spans "
                               f"into a slot + CRC-32C of the slot in one pass over the page, on the device",
                   "l2": f"{total / 1e6:.0f} MB per step, larger than L2",
                   "two_pass_ms_per_step": round(two_pass_ms, 4), "two_pass_gbps": round(total / (two_pass_ms * 1e-3) / 1e9, 1)},
        "roofline": {"bound": "hbm", "achieved": round(total / (kernel_ms * 1e-3) / 1e9, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(total / (kernel_ms * 1e-3) / 1e9 / peak, 4), "traffic": None,
                     "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks_path.exists() else "fallback",
                     "kernel": "crc32c_kernel (checksum of packed slots alone)", "us_per_launch": round(kernel_ms * 1e3, 2),
                     "algorithmic_bytes_per_launch": total},
        "e2e": {"value": round(total / (host_ms * 1e-3) / 1e9, 2), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": total + 4 * count, "ms_per_step": round(host_ms, 4)},
        "cpu_baseline": {"value": round(sample_pages * page_bytes / cpu_seconds / 1e9, 3), "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": f"bit-at-a-time CRC-32C of {sample_pages} of the same slots"},
        "gpu_launches": 2 * args.steps, "clocks": clocks,
    }), flush=True)
    storage.close()


def run_prepare(args):
    """The step before the path: packed projection rows -> query staging + K/V quantised straight into their page slots
    (rk_qkv_prepare_store), for a decode batch (one row per lane) and for 16-row verify windows. One GPU."""
    import torch

    from richengine_b200 import lib, ops
    from richengine_b200.abi import BF16, FP8E4M3, INT4, INT8, Layout, pages_for

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    fmt = {"int4": INT4, "int8": INT8, "fp8e4m3": FP8E4M3, "bf16": BF16}[args.format]
    rows, lanes = (1 if args.rows == 16 and args.batch == 64 else args.rows), args.batch
    layout = Layout(args.layers, KV_HEADS, HEAD_DIM, fmt)
    contexts = [1024] * lanes
    lane_pages = [pages_for(c + rows + 1) for c in contexts]
    storage, tables, pointers, extent_pages, _ = build_pool(layout, lane_pages, 5)
    places = storage.layers()
    generator = torch.Generator(device="cuda").manual_seed(5)
    packed_width = 2 * QUERY_HEADS * HEAD_DIM + 2 * KV_HEADS * HEAD_DIM
    packed = torch.randn((lanes, rows, packed_width), generator=generator, device="cuda").to(torch.bfloat16)
    q_norm = torch.ones(HEAD_DIM, device="cuda").to(torch.bfloat16)
    k_norm = torch.ones(HEAD_DIM, device="cuda").to(torch.bfloat16)
    angle = torch.rand((lanes, rows, 32), generator=generator, device="cuda") * 6.28
    cosine, sine = torch.cos(angle).contiguous(), torch.sin(angle).contiguous()
    queries = torch.zeros((lanes, KV_HEADS, 32, QUERY_HEADS // KV_HEADS, HEAD_DIM), dtype=torch.bfloat16, device="cuda")
    chunk = np.zeros(lanes, dtype=ops.CHUNK_PARAMS)
    for lane, context in enumerate(contexts):
        chunk[lane] = (context, rows, 32, lane_pages[lane], (extent_pages, 0))
    params = ops.params_to_device(chunk)

    def step():
        for layer in range(args.layers):
            ops.qkv_prepare_store(layout, QUERY_HEADS, lanes, rows, packed, q_norm, k_norm, cosine, sine, queries, pointers, params, places[layer])

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    begin_wall = time.perf_counter()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    elapsed_ms = start.elapsed_time(stop)

    def same_load():
        step(); torch.cuda.synchronize()
    sampler.keep_loaded(begin_wall, same_load)
    clocks = sampler.stop(begin_wall, time.perf_counter())
    per_row = packed_width * 2 + QUERY_HEADS * HEAD_DIM * 2 + layout.bytes_per_token_layer()  # packed row in, query rows + page bytes out
    total = per_row * lanes * rows * args.layers * args.steps
    peak, source = peak_hbm()
    us = elapsed_ms / args.steps / args.layers * 1e3
    print(json.dumps({
        "metric": "qkv_prepare_store_rows_per_s", "value": round(lanes * rows * args.layers * args.steps / (elapsed_ms * 1e-3), 1), "unit": "rows/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(elapsed_ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": f"bf16 rows, fp32 norm and rotary, {args.format} pages", "data": "synthetic",
        "config": {"workload": f"{lanes} lanes x {rows} row(s): per layer one fused RMS-norm + rotary + split + quantise-into-pages launch "
                               f"({args.layers} layers, {args.format} pool)", "us_per_layer_step": round(us, 2),
                   "l2": "tiny: launch-latency bound, the rows fit L2"},
        "roofline": {"bound": "hbm", "achieved": round(total / (elapsed_ms * 1e-3) / 1e9, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(total / (elapsed_ms * 1e-3) / 1e9 / peak, 4), "traffic": None, "peak_source": source,
                     "kernel": "qkv_prepare_kernel (fused store)", "us_per_launch": round(us, 2), "algorithmic_bytes_per_launch": per_row * lanes * rows},
        "gpu_launches": args.layers * args.steps, "clocks": clocks,
    }), flush=True)
    storage.close()


def run_evict(args):
    """BASELINE config 4(iii): evict the coldest quarter of a resident int4 pool to pinned host memory and fetch it
    back on access, through the request cache (oldest idle leaf first, page valid until its copy lands, at most 128
    transfers in flight of which demotions at most half and restores at most three quarters:
    runtime/engine/cache/KvPageTier.cpp:38-132). One GPU. Reported against a plain pinned copy of the same bytes
    measured in the same run (the PCIe bound)."""
    import torch

    from richengine_b200 import lib
    from richengine_b200.abi import INT4, Layout
    from richengine_b200.hostplane import GRANTED, Cache, KvPool
    from richengine_b200.storage import PageStorage

    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    layout = Layout(args.layers, KV_HEADS, HEAD_DIM, INT4)
    requests, pages_each = 64, max(4, args.pages // 16)  # --pages = pages evicted; the pool holds four times as many
    total_pages = requests * pages_each
    evict = total_pages // 4
    extent_pages = layout.extent_pages_for(total_pages) or layout.minimum_extent_pages()
    pool_pages = (total_pages + extent_pages - 1) // extent_pages * extent_pages
    storage = PageStorage(layout, pool_pages, extent_pages)
    pool = KvPool(storage=storage, runway_pages=extent_pages)
    transfers = 128
    cache = Cache(pool, Cache.HOST_TIER, evict, transfers)
    page_bytes = storage.bytes_per_page()
    rng = np.random.default_rng(17)
    prompts = [rng.integers(0, 50000, size=pages_each * 32 + 1, dtype=np.uint32) for _ in range(requests)]
    junk = torch.randint(0, 256, (page_bytes,), dtype=torch.uint8, device="cuda")
    library = lib.load()
    for r in range(requests):  # every request's pages hold (any) bytes; published so that they are evictable blocks
        cache.begin_request(r + 1)
        if cache.ensure_tokens(r + 1, pages_each * 32) != GRANTED:
            raise RuntimeError("KV pool does not fit in device memory")
        cache.publish(r + 1, prompts[r], pages_each * 32)
    torch.cuda.synchronize()
    for r in range(requests):
        cache.end_request(r + 1)

    # the PCIe bound of this box: a plain pinned copy of the same number of bytes, each way
    bytes_moved = evict * page_bytes
    pinned = torch.empty(bytes_moved, dtype=torch.uint8, pin_memory=True)
    device = torch.empty(bytes_moved, dtype=torch.uint8, device="cuda")
    rates = {}
    for name, (dst, src) in (("d2h", (pinned, device)), ("h2d", (device, pinned))):
        dst.copy_(src, non_blocking=True); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); dst.copy_(src, non_blocking=True); b.record(); torch.cuda.synchronize()
        rates[name] = bytes_moved / (a.elapsed_time(b) * 1e-3) / 1e9
    del pinned, device

    sampler = ClockSampler(torch.cuda.current_device())
    begin_wall = time.perf_counter()
    # ---- demote the coldest quarter --------------------------------------------------------------------------
    t0 = time.perf_counter()
    peak_in_flight = 0
    target_free = pool.snapshot()["pages_free"] + evict
    idle_rounds = 0
    while pool.snapshot()["pages_free"] < target_free:
        started = cache.reclaim_for_pages(target_free)  # the loop over the candidates runs in the library
        in_flight = cache.snapshot()["transfers"]
        peak_in_flight = max(peak_in_flight, in_flight)
        idle_rounds = 0 if (started or in_flight) else idle_rounds + 1
        if idle_rounds > 1000:
            raise RuntimeError("nothing left to evict before the quarter was reached")
        cache.poll_transfers()  # retire what has landed: its pages return to the pool
    while cache.snapshot()["transfers"]:
        cache.poll_transfers()
    demote_seconds = time.perf_counter() - t0
    snapshot = cache.snapshot()
    if snapshot["tier_blocks"] != evict:
        raise RuntimeError(f"expected {evict} blocks in the host tier, found {snapshot['tier_blocks']}")
    # ---- fetch them back on access: requests with the evicted prompts attach their chains ------------------
    t0 = time.perf_counter()
    restored_pages, request_id = 0, 1000
    # Requests arrive as fast as the tier takes them: a request whose chain does not fit the transfers in flight waits
    # its turn, the others' restores keep the link busy meanwhile (a request is done when none of its restores is pending).
    waiting = list(range(requests))
    running, blocked = [], None  # blocked: the request that asked and was told to wait (it asks again, as itself)
    while waiting or running or blocked:
        while waiting or blocked:
            if blocked is None:  # one match per request, made while the earlier requests' pages are on the link
                chain = cache.lookup(prompts[waiting.pop(0)])
                if not chain:
                    continue
                request_id += 1
                cache.begin_request(request_id)
                blocked = (request_id, chain)
            status, _ = cache.attach_prefix(*blocked)
            if status != GRANTED:  # out of pages or transfers for now: retire some, then ask again
                break
            running.append(blocked[0])
            blocked = None
        cache.poll_transfers()
        still = []
        for rid in running:
            if cache.restores_pending(rid):
                still.append(rid)
            else:
                cache.end_request(rid)
        running = still
    restore_seconds = time.perf_counter() - t0
    after = cache.snapshot()
    restored_pages = after["restores"]
    clocks = sampler.stop(begin_wall, time.perf_counter())
    print(json.dumps({
        "metric": "int4_kv_eviction_gbps", "value": round(bytes_moved / demote_seconds / 1e9, 2), "unit": "GB/s", "n_gpus": 1,
        "steps": 1, "warmup": 0, "ms_per_step": round(demote_seconds * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8 (page bytes; CRC-32C taken while a page is packed)", "data": "synthetic",
        "config": {"workload": f"int4 pool of {total_pages} resident model pages ({args.layers} layers, {page_bytes} B each) in {requests} published "
                               f"chains; the coldest quarter ({evict} pages, {bytes_moved / 1e9:.2f} GB) goes to pinned host memory through the "
                               f"request cache (oldest idle leaf first), then every evicted chain is matched again and fetched back",
                   "transfer_limit": transfers, "peak_transfers_in_flight": int(peak_in_flight),
                   "timing": "host wall clock around each phase (the transfers are asynchronous DMA on the tier's own stream)"},
        "demote": {"gbps": round(bytes_moved / demote_seconds / 1e9, 2), "us_per_page": round(demote_seconds / evict * 1e6, 2),
                   "of_pinned_copy": round(bytes_moved / demote_seconds / 1e9 / rates["d2h"], 3)},
        "restore": {"gbps": round(restored_pages * page_bytes / restore_seconds / 1e9, 2), "pages": int(restored_pages),
                    "us_per_page": round(restore_seconds / max(restored_pages, 1) * 1e6, 2),
                    "of_pinned_copy": round(restored_pages * page_bytes / restore_seconds / 1e9 / rates["h2d"], 3)},
        "roofline": {"bound": "pcie", "achieved": round(bytes_moved / demote_seconds / 1e9, 2), "peak": round(rates["d2h"], 2), "unit": "GB/s",
                     "frac": round(bytes_moved / demote_seconds / 1e9 / rates["d2h"], 4), "traffic": None,
                     "peak_source": "a pinned cudaMemcpyAsync of the same bytes in the same run", "pinned_copy_gbps": {k: round(v, 2) for k, v in rates.items()}},
        "failed_transfers": int(after["failed_transfers"]), "gpu_launches": int(evict + restored_pages), "clocks": clocks,
    }), flush=True)
    cache.close(); pool.close(); storage.close()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.mode == "verify":
        if args.batch == 64 and args.context == 32768:  # the headline defaults: take this mode's own
            args.batch, args.context = 4, 65536
        run_verify(args)
    elif args.mode == "prefill":
        if args.batch == 64 and args.context == 32768:  # the headline defaults: take this mode's own
            args.context = 6144
        run_prefill(args)
    elif args.mode == "seqsplit":
        run_seqsplit(args)
    elif args.mode == "seal":
        run_seal(args)
    elif args.mode == "evict":
        run_evict(args)
    elif args.mode == "prepare":
        run_prepare(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
