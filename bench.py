#!/usr/bin/env python
"""Benchmark of the W4A16 projection path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): the full M=1 projection set of the 24-layer
hybrid stack -- 132 projections, 237,981,696 algorithmic bytes per pass -- with
seeded synthetic weights (bf16 ~N(0, 0.02), quantized by this library's GPU
quantizer) and activations (bf16 ~N(0, 1)).  One step = one pass over the set.
Several distinct copies of the weights are rotated so that every step reads
weights that left L2 long ago (the set is 238 MB, L2 is 126 MB).

Printed: ONE JSON line.  ``value`` is algorithmic GB/s with all inputs resident
in HBM (one grouped launch per step); ``e2e`` is the same metric through the
host-buffer call (activations copied in from pinned host memory and outputs
copied back inside the timed region, synchronised every step); ``roofline``
relates the grouped kernel to the measured HBM copy bandwidth; ``cpu_baseline``
is the reference's CPU GEMV on this box's cores; ``lm_head`` reports the
vocabulary projection (rows/s), vocabulary-parallel when N > 1.

With ``--gpus N`` (N > 1, under torchrun) every rank runs its own replica of the
projection set (the set does not shard: replicas only, no collective), and the
248320-row lm_head is sharded over the ranks with one all-gather of candidates.

``--impl reference`` times the reference's own CPU implementation of the path
(``oracle/_ref`` when it was built from the reference's sources, otherwise the
oracle port) with all host threads, on the same workload and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# (N, K, count): DeltaNet in-proj, DeltaNet out-proj, attn q+gate, k, v, o, gate, up, down
PROJECTION_SET = [(6144, 1024, 18), (1024, 2048, 18), (4096, 1024, 6), (512, 1024, 6),
                  (512, 1024, 6), (1024, 2048, 6), (3584, 1024, 24), (3584, 1024, 24),
                  (1024, 3584, 24)]
VOCAB, HIDDEN, TOP_K = 248320, 1024, 50
SEED = 20250922
METRIC = "w4a16_gemv_hbm_gbps_m1_projection_set"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one grouped launch, from an ncu
# capture of this command with --only set (None until a capture exists)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 242_111_232


def set_bytes(M: int = 1) -> int:
    return sum(c * (N * K // 2 + N * (K // 128) * 2 + M * K * 2 + M * N * 2)
               for N, K, c in PROJECTION_SET)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML from a thread while
    the timed region runs (an NVML query plus 0.5 ms of sleep between samples)."""

    def __init__(self, index: int):
        self.index, self.sm, self.reasons, self.smax = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._err = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            # NVML indexes physical devices; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            idx = self.index
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                idx = int(vis.split(",")[self.index])
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.smax = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons",
                                  getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None))
            while not self._stop.is_set():
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                if get_reasons is not None:
                    mask = int(get_reasons(h))
                    for bit, name in names.items():
                        if mask & bit:
                            self.reasons.add(name)
                time.sleep(0.0005)
        except Exception as e:  # NVML missing or refused: report, do not fail the bench
            self._err = repr(e)

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        time.sleep(0.05)  # let the first samples land before the timed region

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None,
               "sm_max_mhz": self.smax, "samples": len(self.sm), "reasons": sorted(self.reasons)}
        if self._err:
            out["error"] = self._err
        return out


# ---------------------------------------------------------------------------
# reference arm: the reference's CPU GEMV on the host cores
# ---------------------------------------------------------------------------
def cpu_pass(orc, use_ref, weights, xs, threads):
    """One pass of the projection set on the CPU; rows split over threads."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor

    if not use_ref:
        for (W, S), x in zip(weights, xs):
            orc.batch_gemv_bf16(W, S, x[None, :], threads=threads)
        return

    def work(args):
        W, S, x = args
        orc.ref_gemv_bf16(W, S, x)

    jobs = []
    for (W, S), x in zip(weights, xs):
        rows = W.shape[0]
        step = max(16, (rows + threads - 1) // threads)
        for r0 in range(0, rows, step):
            jobs.append((W[r0:r0 + step], S[r0:r0 + step], x))
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(work, jobs))


def cpu_inputs(orc, distinct_layers: int = 1):
    """Raw packed bytes are enough for timing the CPU GEMV (its cost does not
    depend on the values); one layer of each kind is built and reused."""
    import numpy as np
    rng = np.random.default_rng(SEED)
    weights, xs = [], []
    for N, K, c in PROJECTION_SET:
        W = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
        S = (0.001 + 0.02 * rng.random((N, K // 128))).astype(np.float16).view(np.uint16)
        x = orc.f32_to_bf16_bits(rng.standard_normal(K).astype(np.float32))
        for _ in range(c):
            weights.append((W, S))
            xs.append(x)
    return weights, xs


def time_cpu(steps: int, warmup: int, budget_s: float):
    from oracle import cpu_oracle as orc
    orc.build()
    use_ref = orc.have_ref()
    threads = os.cpu_count() or 1
    weights, xs = cpu_inputs(orc)
    for _ in range(max(1, min(warmup, 1))):
        cpu_pass(orc, use_ref, weights, xs, threads)
    times = []
    t_start = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_pass(orc, use_ref, weights, xs, threads)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    sec = statistics.median(times)
    return {"value": set_bytes() / sec / 1e9, "unit": UNIT, "cores": threads,
            "kind": "reference" if use_ref else "port",
            "sample": f"{len(times)} full passes of the 132-projection set (237,981,696 B each), "
                      f"rows split over {threads} threads; median pass {sec * 1e3:.1f} ms"}, sec, len(times)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec, n = time_cpu(max(1, args.steps), args.warmup, budget_s=120.0)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
            "n_gpus": args.gpus, "steps": n, "warmup": min(args.warmup, 1),
            "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int4 weights x bf16 activations, fp32 accumulate",
            "data": "synthetic", "config": workload_config(args.gpus),
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(n_gpus: int, copies: int = 0):
    return {"workload": "configuration 1 of the benchmark plan: full M=1 projection set of the 24-layer hybrid "
                        "stack (132 projections: 1024->6144 x18, 2048->1024 x24, 1024->4096 x6, "
                        "1024->512 x12, 1024->3584 x48, 3584->1024 x24), G=128 int4 + fp16 scales",
            "bytes_per_step": set_bytes(), "M": 1,
            "l2": "distinct weight copies rotated (each 238 MB > 126 MB L2); on the CPU arm the set "
                  "itself exceeds every cache",
            "parallelism": "replicas only (one per GPU, no collective)" if n_gpus > 1 else "1 GPU"}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def build_projection_set(eng, torch, copies: int, seed: int):
    """Device-resident weights (quantized on the GPU by the library), one
    contiguous activation buffer and one contiguous output buffer per copy."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x_elems = sum(c * K for N, K, c in PROJECTION_SET)
    y_elems = sum(c * N for N, K, c in PROJECTION_SET)
    x_dev = torch.randn(x_elems, generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    y_dev = torch.zeros(y_elems, device="cuda", dtype=torch.bfloat16)
    groups, keep = [], []
    for _ in range(copies):
        items, xo, yo = [], 0, 0
        for N, K, c in PROJECTION_SET:
            for _ in range(c):
                w = (torch.randn((N, K), generator=gen, device="cuda", dtype=torch.float32) * 0.02
                     ).to(torch.bfloat16)
                packed, scale = eng.quantize_w4a16(w)
                lin = eng.W4A16Linear(packed, scale)
                items.append((lin, x_dev[xo:xo + K], y_dev[yo:yo + N]))
                xo += K
                yo += N
        keep.append(items)
        groups.append(eng.LinearGroup(items))
    return groups, keep, x_dev, y_dev


def time_steps(torch, fn, steps, warmup, dist=None, min_seconds=0.0, max_repeats=2000):
    """Times `steps` calls of fn after `warmup` untimed ones, with CUDA events on the
    current stream and a barrier + synchronize on both sides.  The timed region of
    `steps` calls is repeated until at least `min_seconds` of GPU time have been timed
    (every repeat bracketed the same way), so that a figure quoted as sustained has run
    for that long.  Returns (median region ms, list of region ms)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    regions, total, call = [], 0.0, warmup
    while True:
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        # Only two events per region: an event recorded between two launches would stop the
        # second kernel from starting while the first drains (the kernels use programmatic
        # dependent launch), which is how a caller issues them.
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            fn(call + i)
        ev1.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        call += steps
        ms = ev0.elapsed_time(ev1)
        regions.append(ms)
        total += ms
        more = total < min_seconds * 1e3 and len(regions) < max_repeats
        if dist is not None:  # every rank repeats as long as any rank wants to
            t = torch.tensor([1.0 if more else 0.0], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            more = bool(t.item() > 0)
        if not more:
            break
    return statistics.median(regions), regions


def max_over_ranks(torch, dist, ms: float) -> float:
    if dist is None:
        return ms
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def build_vocab_shard(eng, torch, lo, hi):
    """Rows [lo, hi) of the synthetic vocabulary matrix, quantized on the GPU; every rank
    draws the whole matrix from one generator stream so that all ranks see the same one."""
    gen = torch.Generator(device="cuda").manual_seed(SEED + 3)
    block = 31040
    packs, scales = [], []
    for r0 in range(0, VOCAB, block):
        w = (torch.randn((block, HIDDEN), generator=gen, device="cuda", dtype=torch.float32) * 0.02
             ).to(torch.bfloat16)
        a, b = max(lo, r0), min(hi, r0 + block)
        if a < b:
            p, s = eng.quantize_w4a16(w[a - r0:b - r0].contiguous())
            packs.append(p)
            scales.append(s)
    return eng.W4A16Linear(torch.cat(packs), torch.cat(scales)), gen


def lm_head_timings(eng, torch, dist, lins, lo, x, M, mode, steps, warmup, in_flight=None):
    """One configuration of the vocabulary projection: per-call latency (calls back to
    back on one stream) and pipelined throughput (`in_flight` calls under way at once, each
    on its own stream with its own workspace and exchange buffers, as a server with several
    decode steps in flight issues them; the next call's projection overlaps the previous
    call's exchange and merge) and the latency again with the calls replayed from a CUDA
    graph (two calls per graph, one per weight copy), which takes the host's issue time out
    of it: with the vocabulary split over eight GPUs a call is shorter than the time the
    host needs to issue its two launches through Python.  Returns (latency ms per call,
    pipelined ms per call, last outputs, calls in flight, graph latency ms per call)."""
    vp = dist is not None and mode is not None
    if in_flight is None:
        # With the peer exchange every activation row of a call in flight may hold a CTA that
        # waits for the other ranks' candidates, and a projection CTA needs an SM to itself:
        # calls in flight x rows stays well below the number of SMs, so that no rank can fill
        # its GPU with waiting CTAs while the calls they wait for cannot start elsewhere.
        in_flight = max(2, min(8, 64 // M))

    def make_head(i):
        h = eng.LmHead(lins[i % len(lins)], TOP_K, id_offset=lo, max_rows=M)
        return eng.VocabParallelLmHead(h, exchange=mode) if vp else h
    heads = [make_head(i) for i in range(2)]
    res = {}

    def step(i):
        res["out"] = heads[i % 2].forward(x)

    lat_ms, _ = time_steps(torch, step, steps, warmup, dist, min_seconds=0.05)
    out = [t.clone() for t in res["out"]]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step(0)
        step(1)
    replays = max(2, steps // 2)
    graph_ms, _ = time_steps(torch, lambda i: graph.replay(), replays, 2, dist, min_seconds=0.05)
    graph_ms /= replays * 2
    if not all(torch.equal(a, b) for a, b in zip(out, res["out"])):
        raise RuntimeError("the graph replay of the vocabulary projection picked different tokens")
    del graph
    # pipelined: in_flight streams, each with its own head; weights alternate between the copies
    pipe = [make_head(i) for i in range(in_flight)]
    streams = [torch.cuda.Stream() for _ in range(in_flight)]
    torch.cuda.synchronize()

    width = [in_flight]

    def region(i):
        cur = torch.cuda.current_stream()
        for st in streams[:width[0]]:
            st.wait_stream(cur)
        for j in range(width[0]):
            with torch.cuda.stream(streams[j]):
                pipe[j].forward(x)
        for st in streams[:width[0]]:
            cur.wait_stream(st)

    rounds = max(2, steps // in_flight)
    pipe_ms, _ = time_steps(torch, region, rounds, 2, dist, min_seconds=0.05)
    best = (pipe_ms / (rounds * in_flight), in_flight)
    if in_flight > 2:
        # fewer calls in flight: more of them does not always help, since their kernels share the SMs
        width[0] = 2
        rounds2 = max(2, steps // 2)
        pipe2_ms, _ = time_steps(torch, region, rounds2, 2, dist, min_seconds=0.05)
        width[0] = in_flight
        if pipe2_ms / (rounds2 * 2) < best[0]:
            best = (pipe2_ms / (rounds2 * 2), 2)
    for h in heads + pipe:
        if vp:
            h.close()
    return lat_ms / steps, best[0], out, best[1], graph_ms


def bench_lm_head(eng, torch, dist, rank, world, steps, warmup):
    """Vocabulary projection: rows/s at M=1 and M=32, vocabulary-parallel over `world`
    ranks (strong scaling: the 248320 rows are split).  Two figures per configuration:
    single-call latency and pipelined throughput (8 calls in flight).  With world > 1, rank 0
    also runs the whole vocabulary on its one GPU inside the same run, which gives the
    efficiencies against one GPU."""
    lo, hi = eng.shard_rows(VOCAB, world, rank)
    lin, gen = build_vocab_shard(eng, torch, lo, hi)
    # a second copy of the shard so consecutive steps do not reuse L2 lines
    lins = [lin, eng.W4A16Linear(lin.weight.clone(), lin.scale.clone())]
    full = None
    if world > 1 and rank == 0:
        f, _ = build_vocab_shard(eng, torch, 0, VOCAB)
        full = [f, eng.W4A16Linear(f.weight.clone(), f.scale.clone())]
    out = {}
    for M in (1, 32):
        x = torch.randn((M, HIDDEN), generator=gen, device="cuda", dtype=torch.float32)
        x = (x / x.pow(2).mean(dim=1, keepdim=True).sqrt()).to(torch.bfloat16)
        if world > 1:
            dist.broadcast(x, 0)  # one activation matrix for every rank
        modes = ["peer", "collective"] if world > 1 else [None]
        entry, picks = {}, {}
        for mode in list(modes):
            try:
                lat, pipe, res, in_flight, glat = lm_head_timings(eng, torch, dist if world > 1 else None,
                                                                  lins, lo, x, M, mode, steps, warmup)
                failed, why = 0, ""
            except Exception as exc:  # e.g. the ranks' GPUs cannot map one another's memory
                if mode != "peer":
                    raise
                failed, why = 1, f"{type(exc).__name__}: {exc}"
            if failed:  # PeerExchange raises on every rank or on none
                modes.remove("peer")
                entry["note"] = f"peer exchange unavailable ({why})"
                continue
            lat = max_over_ranks(torch, dist, lat)
            pipe = max_over_ranks(torch, dist, pipe)
            glat = max_over_ranks(torch, dist, glat)
            picks[mode] = res
            if mode == modes[0]:
                entry.update({
                    "us_per_call": lat * 1e3, "rows_per_s": M / (lat * 1e-3),
                    "graph_us_per_call": glat * 1e3,
                    "pipelined_us_per_call": pipe * 1e3, "pipelined_rows_per_s": M / (pipe * 1e-3),
                    "calls_in_flight": in_flight, "shard_rows": hi - lo,
                    "shard_gbps": (lin.N * lin.K // 2 + lin.N * 16) / (lat * 1e-3) / 1e9,
                    "argmax_row0": int(res[0][0].item()),
                    "exchange": ("peer memory, by the CTA that ranks the row" if mode == "peer"
                                 else "none")})
            else:
                entry["collective_us_per_call"] = lat * 1e3
                entry["collective_graph_us_per_call"] = glat * 1e3
                entry["collective_pipelined_us_per_call"] = pipe * 1e3
                same = all(torch.equal(a, b) for a, b in zip(picks[modes[0]], picks[mode]))
                if not same:
                    raise RuntimeError("peer exchange and all-gather picked different tokens")
                entry["same_pick_as_collective"] = True
        if world > 1:
            # the whole vocabulary on rank 0's GPU alone, inside this run
            one = torch.zeros(4, device="cuda", dtype=torch.float64)
            if rank == 0:
                lat1, pipe1, res1, _, glat1 = lm_head_timings(eng, torch, None, full, 0, x, M, None, steps,
                                                              warmup, in_flight=entry.get("calls_in_flight"))
                one = torch.tensor([lat1, pipe1, float(res1[0][0].item()), glat1], device="cuda",
                                   dtype=torch.float64)
            dist.broadcast(one, 0)
            lat1, pipe1, arg1, glat1 = (float(v) for v in one.tolist())
            entry["one_gpu_us_per_call"] = lat1 * 1e3
            entry["one_gpu_pipelined_us_per_call"] = pipe1 * 1e3
            entry["one_gpu_graph_us_per_call"] = glat1 * 1e3
            entry["efficiency_vs_1gpu"] = {"latency": lat1 / (entry["us_per_call"] * 1e-3) / world,
                                           "pipelined": pipe1 / (entry["pipelined_us_per_call"] * 1e-3) / world,
                                           "graph_latency": glat1 / (entry["graph_us_per_call"] * 1e-3) / world}
            if int(arg1) != entry["argmax_row0"]:
                raise RuntimeError("the vocabulary-parallel argmax differs from the single-GPU one")
            entry["same_argmax_as_one_gpu"] = True
        out[f"M{M}"] = entry
    return out


# the eight (N, K) of the reference's kernel table plus the DeltaNet z projection and the
# N=16 b/a projections (benchmarks/v07b_w4a16_microbench_run1.txt:25-130 of CUDALM; its
# mean time per call on an RTX 2080 Ti in microseconds, where it publishes one)
SHAPE_TABLE = [(16, 1024, 7.27), (512, 1024, 6.90), (1024, 2048, 7.29), (1024, 3584, 8.56),
               (2048, 1024, 7.09), (3584, 1024, 9.92), (4096, 1024, 10.21), (6144, 1024, 13.00)]


def random_packed(torch, gen, copies, N, K):
    """`copies` projections of one shape with random packed bytes and scales (the timing
    does not depend on the values), as one contiguous allocation each."""
    W = torch.randint(0, 256, (copies, N, K // 2), generator=gen, device="cuda", dtype=torch.uint8)
    S = (0.001 + 0.02 * torch.rand((copies, N, K // 128), generator=gen, device="cuda")).to(torch.float16)
    return W, S


def bench_shapes(eng, torch, steps, warmup, peak):
    """Per shape at M=1: (a) streamed GB/s -- one grouped launch over enough distinct copies
    of the shape to hold at least twice the L2 (so every byte comes from HBM), and
    (b) latency per call -- the copies called one by one, each a launch of its own, replayed
    from a CUDA graph (no host time) and issued eagerly from Python (host-bound)."""
    gen = torch.Generator(device="cuda").manual_seed(SEED + 6)
    l2 = torch.cuda.get_device_properties(0).L2_cache_size
    out = {}
    for N, K, ref_us in SHAPE_TABLE:
        per = N * K // 2 + N * (K // 128) * 2
        copies = max(2, min(2048, -(-2 * l2 // per)))
        W, S = random_packed(torch, gen, copies, N, K)
        x = torch.randn(K, generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        y = torch.empty((copies, N), device="cuda", dtype=torch.bfloat16)
        lins = [eng.W4A16Linear(W[i], S[i]) for i in range(copies)]
        grp = eng.LinearGroup([(lins[i], x, y[i]) for i in range(copies)])
        ms, _ = time_steps(torch, lambda i: grp.run(), steps, warmup, min_seconds=0.05)
        sec = ms * 1e-3 / steps
        gbps = grp.bytes / sec / 1e9
        grp.close()
        # latency: one launch per projection; a bounded number of distinct copies
        n_lat = min(copies, 128)
        def calls(i):
            for j in range(n_lat):
                eng.int4_gemv_bf16(lins[j].weight, lins[j].scale, x, y[j])
        eager_ms, _ = time_steps(torch, calls, 3, 1)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            calls(0)
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=side):
                calls(0)
        torch.cuda.current_stream().wait_stream(side)
        graph_ms, _ = time_steps(torch, lambda i: g.replay(), 10, 2, min_seconds=0.02)
        entry = {"streamed_gbps": gbps, "streamed_frac_of_peak": gbps / peak, "copies": copies,
                 "l2_resident": copies * per < 2 * l2,
                 "us_per_call_graph": graph_ms * 1e3 / 10 / n_lat,
                 "us_per_call_eager_python": eager_ms * 1e3 / 3 / n_lat,
                 "reference_2080ti_us_per_call": ref_us}
        out[f"{N}x{K}"] = entry
        del grp, lins, W, S, y, g
        torch.cuda.empty_cache()
    return out


def bench_cohorts(eng, torch, steps, warmup, rows=(8, 16, 32, 64)):
    """Batched decode (configuration 2 of the benchmark plan): M = 8, 16, 32, 64 rows through the
    MLP projections of 24 layers -- fused gate+up (K=1024 -> 2 x 3584) and down
    (K=3584 -> 1024), distinct weights per layer (137 MB of weights > L2)."""
    gen = torch.Generator(device="cuda").manual_seed(SEED + 2)
    layers = []
    for _ in range(24):
        ws = []
        for N, K in ((3584, 1024), (3584, 1024), (1024, 3584)):
            w = (torch.randn((N, K), generator=gen, device="cuda", dtype=torch.float32) * 0.02
                 ).to(torch.bfloat16)
            ws.append(eng.W4A16Linear(*eng.quantize_w4a16(w)))
        layers.append(ws)
    out = {}
    for M in rows:
        x = torch.randn((M, 1024), generator=gen, device="cuda", dtype=torch.float32)
        x[torch.rand((M, 1024), generator=gen, device="cuda") < 0.01] *= 20.0
        x = x.to(torch.bfloat16)
        h = torch.randn((M, 3584), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        gy = torch.empty((M, 3584), device="cuda", dtype=torch.bfloat16)
        uy = torch.empty((M, 3584), device="cuda", dtype=torch.bfloat16)
        dy = torch.empty((M, 1024), device="cuda", dtype=torch.bfloat16)

        # one grouped launch for all gate and up projections, one for the down projections
        items_gu, items_d = [], []
        for g, u, d in layers:
            items_gu += [(g, x, gy), (u, x, uy)]
            items_d.append((d, h, dy))
        grp_gu, grp_d = eng.LinearGroup(items_gu), eng.LinearGroup(items_d)

        def step(i):
            grp_gu.run()
            grp_d.run()

        l0 = eng.launch_count()
        total_ms, _ = time_steps(torch, step, steps, warmup)
        launches = (eng.launch_count() - l0) // (steps + warmup)
        nbytes = sum(g.bytes(M) + u.bytes(M) - M * 1024 * 2 + d.bytes(M) for g, u, d in layers)
        flops = 2 * M * 24 * (2 * 3584 * 1024 + 1024 * 3584)
        sec = total_ms * 1e-3 / steps
        grp_gu.close()
        grp_d.close()
        out[f"M{M}"] = {"gbps": nbytes / sec / 1e9, "tflops": flops / sec / 1e12,
                        "us_per_pass": sec * 1e6, "launches_per_pass": int(launches),
                        "bytes_per_pass": nbytes}
    return out


def bench_mlp(eng, torch, steps, warmup):
    """One layer's MLP at M = 1, 8, 32 and 64 (the fused-epilogue row of the scope table): the reference's five launches
    (gate, up, silu_mul, down, add) as this library's two fused ones, against the same
    work through the unfused entry points plus torch elementwise kernels."""
    gen = torch.Generator(device="cuda").manual_seed(SEED + 5)
    layers = []
    for _ in range(24):
        ws = []
        for N, K in ((3584, 1024), (3584, 1024), (1024, 3584)):
            w = (torch.randn((N, K), generator=gen, device="cuda", dtype=torch.float32) * 0.02
                 ).to(torch.bfloat16)
            ws.append(eng.W4A16Linear(*eng.quantize_w4a16(w)))
        layers.append(ws)
    out = {}
    for M in (1, 8, 32, 64):
        x = torch.randn((M, 1024), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
        act = torch.empty((M, 3584), device="cuda", dtype=torch.bfloat16)
        gy, uy = torch.empty_like(act), torch.empty_like(act)
        h = torch.zeros((M, 1024), device="cuda", dtype=torch.bfloat16)
        dy = torch.empty_like(h)

        def fused(i):
            for g, u, d in layers:
                eng.gate_up_silu_bf16(g, u, x, out=act)
                eng.linear_residual_bf16(d, act, h, y=h)

        def unfused(i):
            for g, u, d in layers:
                eng.gate_up_bf16(g, u, x, gy, uy)
                torch.mul(torch.nn.functional.silu(gy), uy, out=act)
                eng.batch_int4_gemv_bf16(d.weight, d.scale, act, dy)
                h.add_(dy)

        res = {}
        for name, fn in (("fused", fused), ("unfused", unfused)):
            total_ms, _ = time_steps(torch, fn, steps, warmup)
            res[name + "_eager_us_per_layer"] = total_ms * 1e3 / steps / 24
            # the same 24 layers replayed from a CUDA graph: the GPU side without the host's
            # cost of issuing each call from Python
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn(0)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    fn(0)
            torch.cuda.current_stream().wait_stream(side)
            total_ms, _ = time_steps(torch, lambda i: graph.replay(), steps, warmup, min_seconds=0.02)
            res[name + "_us_per_layer"] = total_ms * 1e3 / steps / 24
            del graph
        nbytes = sum(g.bytes(M) + u.bytes(M) + d.bytes(M) for g, u, d in layers) / 24
        res["fused_gbps"] = nbytes / (res["fused_us_per_layer"] * 1e-6) / 1e9
        res["launches_per_layer"] = {"fused": 2, "unfused": 5}
        out[f"M{M}"] = res
    return out


def bench_quantize(eng, torch, steps, warmup):
    """GPU quantize+pack (configuration 4 of the benchmark plan): GB/s of bf16 input consumed."""
    gen = torch.Generator(device="cuda").manual_seed(SEED + 4)
    out = {}
    for N, K in ((248320, 1024), (6144, 1024), (1024, 3584)):
        ws = [(torch.randn((N, K), generator=gen, device="cuda", dtype=torch.float32) * 0.02
               ).to(torch.bfloat16) for _ in range(2 if N > 100000 else 8)]
        total_ms, _ = time_steps(torch, lambda i: eng.quantize_w4a16(ws[i % len(ws)]), steps, warmup)
        sec = total_ms * 1e-3 / steps
        out[f"{N}x{K}"] = {"input_gbps": N * K * 2 / sec / 1e9,
                           "traffic_gbps": N * K * 2.515625 / sec / 1e9, "us": sec * 1e6}
    return out


def run_ours(args):
    import torch
    import cudalm_agent_b200 as eng

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    eng.load_library()

    copies = max(2, args.copies)
    if args.only == "batched":
        out = bench_cohorts(eng, torch, max(2, min(args.steps, 20)), max(1, min(args.warmup, 3)),
                            rows=(args.rows,))
        print(json.dumps({"batched_decode": out}), flush=True)
        return
    if args.only == "mlp":
        print(json.dumps({"mlp": bench_mlp(eng, torch, max(2, min(args.steps, 20)),
                                           max(1, min(args.warmup, 3)))}), flush=True)
        return
    if args.only == "quantize":
        print(json.dumps({"quantize": bench_quantize(eng, torch, max(2, min(args.steps, 20)),
                                                     max(1, min(args.warmup, 3)))}), flush=True)
        return
    if args.only == "lm_head":
        lm = bench_lm_head(eng, torch, dist, rank, world, max(5, min(args.steps, 50)), 3)
        if rank == 0:
            print(json.dumps({"lm_head": lm}), flush=True)
        return
    groups, keep, x_dev, y_dev = build_projection_set(eng, torch, copies, SEED + 1 + rank)
    bytes_step = groups[0].bytes
    assert bytes_step == set_bytes(), (bytes_step, set_bytes())

    # ---- resident-in-HBM timing: one grouped launch per step ----------------
    # The timed region of --steps steps is repeated until a second of GPU time has been
    # timed; `value` comes from the median region, so it is a sustained figure, and the
    # clock sampler sees the GPU under load for that long.
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = eng.launch_count()
    total_ms, regions = time_steps(torch, lambda i: groups[i % copies].run(), args.steps,
                                   args.warmup, dist, min_seconds=args.min_seconds)
    launches = (eng.launch_count() - launches0 - args.warmup) // len(regions)
    clocks = sampler.stop()
    best_ms = max_over_ranks(torch, dist, min(regions))
    total_ms = max_over_ranks(torch, dist, total_ms)
    value = world * bytes_step * args.steps / (total_ms * 1e-3) / 1e9
    kernel_ms = total_ms / args.steps
    timed_region = {"repeats": len(regions), "gpu_seconds_timed": sum(regions) * 1e-3,
                    "weight_copies_rotated": copies,
                    "ms_per_step_median": total_ms / args.steps, "ms_per_step_min": best_ms / args.steps,
                    # an issue-bound kernel's time scales with the clock: compare across boxes by this
                    "us_per_step_x_sm_mhz": (total_ms / args.steps * 1e3 * clocks["sm_mhz"]
                                             if clocks.get("sm_mhz") else None)}

    # ---- end to end through the host-buffer call ------------------------------
    x_host = torch.empty_like(x_dev, device="cpu").pin_memory()
    x_host.copy_(x_dev)
    y_host = torch.empty_like(y_dev, device="cpu").pin_memory()

    def e2e_step(i):
        x_dev.copy_(x_host, non_blocking=True)
        groups[i % copies].run()
        y_host.copy_(y_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(args.warmup):
        e2e_step(i)
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        e2e_step(args.warmup + i)
    ev1.record()
    torch.cuda.synchronize()
    serial_ms = max_over_ranks(torch, dist, max(ev0.elapsed_time(ev1), (time.perf_counter() - t0) * 1e3))
    serial_value = world * bytes_step * args.steps / (serial_ms * 1e-3) / 1e9

    # The same with two steps in flight, as a serving loop issues them: each step
    # has its own stream, pinned host buffers and device buffers; the copies of
    # one step overlap the kernel of the other.  Every step still copies its
    # inputs in and its outputs out, and the host waits for a step's outputs
    # before it reuses that step's buffers.
    slots = []
    for b in range(2):
        xb, yb = torch.empty_like(x_dev), torch.empty_like(y_dev)
        grp_b = []
        for items in keep:
            its, xo, yo = [], 0, 0
            for lin, x, y in items:
                its.append((lin, xb[xo:xo + lin.K], yb[yo:yo + lin.N]))
                xo += lin.K
                yo += lin.N
            grp_b.append(eng.LinearGroup(its))
        slots.append({"x": xb, "y": yb, "groups": grp_b, "stream": torch.cuda.Stream(),
                      "xh": torch.empty_like(x_dev, device="cpu").pin_memory(),
                      "yh": torch.empty_like(y_dev, device="cpu").pin_memory(),
                      "done": torch.cuda.Event()})
        slots[b]["xh"].copy_(x_dev)
    torch.cuda.synchronize()

    waited = [0.0]

    def piped_step(i):
        sl = slots[i % 2]
        w0 = time.perf_counter()
        sl["done"].synchronize()  # the outputs of the step that last used these buffers are on the host
        waited[0] += time.perf_counter() - w0
        with torch.cuda.stream(sl["stream"]):
            sl["x"].copy_(sl["xh"], non_blocking=True)
            sl["groups"][i % copies].run()
            sl["yh"].copy_(sl["y"], non_blocking=True)
            sl["done"].record()

    for i in range(max(args.warmup, 2)):
        piped_step(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e2e_steps = args.steps
    if args.min_seconds > 0:  # as long as the headline: about a quarter of a second at least
        e2e_steps = max(args.steps, int(0.25 / max(kernel_ms * 1e-3, 1e-6)))
    t0 = time.perf_counter()
    host_busy = 0.0
    waited[0] = 0.0
    for i in range(e2e_steps):
        h0 = time.perf_counter()
        piped_step(i)
        host_busy += time.perf_counter() - h0
    for sl in slots:
        sl["done"].synchronize()
    torch.cuda.synchronize()
    e2e_local_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(torch, dist, e2e_local_ms) * args.steps / e2e_steps
    e2e_value = world * bytes_step * args.steps / (e2e_ms * 1e-3) / 1e9
    # where a step's time goes on the host: issuing it (copies + launch) or waiting for the GPU
    e2e_host_issue_ms = max_over_ranks(torch, dist, (host_busy - waited[0]) * 1e3 / e2e_steps)
    e2e_host_wait_ms = max_over_ranks(torch, dist, waited[0] * 1e3 / e2e_steps)
    # the pipelined steps must have produced what the serial call produces
    last = e2e_steps - 1
    for b in range(2):
        i_b = last if last % 2 == b else last - 1
        if i_b < 0:
            continue
        x_dev.copy_(x_host)
        groups[i_b % copies].run()
        torch.cuda.synchronize()
        if not torch.equal(slots[b]["yh"].view(torch.int16), y_dev.cpu().view(torch.int16)):
            raise SystemExit("pipelined end-to-end outputs differ from the serial call's")
    for sl in slots:
        for g in sl["groups"]:
            g.close()

    # ---- latency mode: one launch per projection, as the reference calls it ----
    def per_call(i):
        for lin, x, y in keep[i % copies]:
            eng.int4_gemv_bf16(lin.weight, lin.scale, x, y)

    lat_steps = max(3, min(args.steps, 10))
    lat_ms, _ = time_steps(torch, per_call, lat_steps, 2, dist)
    lat_ms = max_over_ranks(torch, dist, lat_ms)
    # the same 132 calls replayed from a CUDA graph: the GPU side of a call without the
    # host's cost of issuing it (the eager figure is bound by the Python wrapper)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        per_call(0)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for c in range(copies):
                per_call(c)
    torch.cuda.current_stream().wait_stream(side)
    glat_ms, _ = time_steps(torch, lambda i: graph.replay(), lat_steps, 2, dist, min_seconds=0.05)
    glat_ms = max_over_ranks(torch, dist, glat_ms)
    del graph

    status = eng.device_status()
    if status != 0:
        raise SystemExit(f"device status word = {status}: a bounded wait ran out")

    for g in groups:
        g.close()
    del groups, keep
    torch.cuda.empty_cache()

    lm = {} if args.only == "set" else bench_lm_head(eng, torch, dist, rank, world,
                                                      max(5, min(args.steps, 50)), 3)

    cohorts, quant, mlp, shapes = {}, {}, {}, {}
    if args.only == "all" and rank == 0:
        cohorts = bench_cohorts(eng, torch, max(5, min(args.steps, 20)), 3)
        quant = bench_quantize(eng, torch, max(5, min(args.steps, 20)), 3)
        mlp = bench_mlp(eng, torch, max(5, min(args.steps, 20)), 3)
        shapes = bench_shapes(eng, torch, max(5, min(args.steps, 20)), 3, measured_peaks()[0])
    if dist is not None:
        dist.barrier()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peaks()
    achieved = bytes_step / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 weights x bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": workload_config(world, copies),
        "clocks": clocks,
        "timed_region": timed_region,
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": x_dev.numel() * 2, "d2h_bytes_per_step": y_dev.numel() * 2,
                "ms_per_step": e2e_ms / args.steps,
                "steps_timed": e2e_steps,
                # the host's share of a step: issuing it (two copies and a launch through Python)
                # and waiting for the step that last used the same buffers
                "host_issue_ms_per_step": e2e_host_issue_ms,
                "host_wait_ms_per_step": e2e_host_wait_ms,
                "serial_value": serial_value, "serial_ms_per_step": serial_ms / args.steps,
                "what": "per step: pinned-host activations copied in, one grouped launch, outputs "
                        "copied back to pinned host; two steps in flight on two streams (the host "
                        "waits for a step's outputs before reusing its buffers); wall clock; "
                        "weights resident",
                "serial": {"value": serial_value, "ms_per_step": serial_ms / args.steps,
                           "what": "the same, one step at a time, stream synchronised every step"}},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "w4a16_stream_kernel<NT=1> (grouped launch)",
                     "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                     "peak_source": peak_src + ", of measured",
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "algorithmic_bytes_per_launch": bytes_step,
                     "avg_launch_ms": kernel_ms},
        "latency_mode": {"what": "132 separate launches per pass (one per projection, the lean kernel); "
                                 "us_per_call: replayed from a CUDA graph (GPU side only); "
                                 "eager: issued one by one from Python (bound by the host wrapper)",
                         "us_per_call": glat_ms * 1e3 / lat_steps / (132 * copies),
                         "gbps": bytes_step * copies * lat_steps / (glat_ms * 1e-3) / 1e9,
                         "eager_ms_per_pass": lat_ms / lat_steps,
                         "eager_us_per_call": lat_ms * 1e3 / lat_steps / 132,
                         "per_shape": shapes},
        "batched_decode": {"what": "24 layers x (fused gate+up 1024->2x3584, down 3584->1024), "
                                   "bf16 activations with 1% x20 outliers", **cohorts},
        "quantize": quant,
        "mlp": mlp,
        "lm_head": {"vocab": VOCAB, "K": HIDDEN, "top_k": TOP_K, "n_gpus": world,
                    "scaling": "strong (vocabulary rows split over ranks, one all-gather of "
                               "candidates)" if world > 1 else "single GPU", **lm},
    }
    if world == 1 and not args.skip_cpu:
        base, _, _ = time_cpu(5, 1, budget_s=25.0)
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="all", choices=["all", "set", "lm_head", "batched", "quantize", "mlp"],
                    help="profiling aid: run only the projection set, the lm_head, batched decode "
                         "or the quantizer")
    ap.add_argument("--rows", type=int, default=64, help="with --only batched: activation rows M")
    ap.add_argument("--copies", type=int, default=3, help="distinct weight copies rotated")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling aid: no CPU baseline")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="repeat the timed region of --steps steps until this much GPU time has been "
                         "timed (0: exactly one region, for captures under a profiler)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
