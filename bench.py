"""Benchmark of the sparse-MLA attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2|target|cfg2_tp16|cfg5[:s_q]] [--no-more] [--extras]

Headline.  One "step" is `calls_per_step` sparse decode calls (decode kernel + split-KV
combine) over a batch of synthetic requests: batch 16, h_q 64, d_qk 576 / d_v 512,
32 768-token contexts in the 644-byte FP8 + UE8M0 + BF16-RoPE paged cache behind a random
page table, top-k 2048.  The metric is achieved HBM GB/s = algorithmic bytes per call / time
per call.  With N GPUs every rank decodes its own batch of 16 from its own cache
(request-parallel, no collective): weak scaling.  The calls per step are chosen so that the
timed region lasts at least 50 ms.

The timed loop rotates through 16 independent top-k index sets, so the rows gathered between
two uses of the same set (16 x ~21 MB) exceed the 126 MB L2.

The JSON line carries: `value` (inputs resident in HBM), `roofline` (decode kernel alone
against the measured copy bandwidth; `traffic` is read from the committed ncu summary),
`e2e` (same metric through the public operator with q / indices in pinned host memory copied
in and out / lse copied back every step, plus the latency of one eager call on one stream),
`cpu_baseline` (the CPU oracle, a port of the reference's torch path, on the host cores),
the SM clocks sampled during the timed loop, and under `more` the rest of the metric on the
same GPUs: the batch-64 target shape, one tensor-parallel shard (h_q 16), the 128-request
mixed-length decode split over the ranks (strong scaling), sparse prefill in TFLOP/s with the
query rows balanced over the ranks, and for N >= 2 the head-sharded decode step with its
all-gather.

`--impl reference` times the CPU path alone (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "deepseek-v4-flash-sm120_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

N_INDEX_SETS = 16
METRIC = "sparse_decode_achieved_hbm_bandwidth"


# Committed ncu summary of the decode kernel on the headline workload; it carries a line
# "traffic_bytes_per_launch: <dram__bytes_read.sum + dram__bytes_write.sum>".
NCU_SUMMARY = {"cfg2": os.path.join(ROOT, "profiles", "sm100_attn_kernel_decode_cfg2.md")}
MIN_REGION_S = 0.05           # every timed region lasts at least this long


def ncu_traffic_bytes(workload: str):
    """DRAM bytes per launch of the decode kernel from the committed ncu summary, or None."""
    import re
    try:
        with open(NCU_SUMMARY[workload]) as f:
            m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)", f.read())
        return float(m.group(1)) if m else None
    except Exception:  # noqa: BLE001
        return None


def measured_peaks():
    """(HBM GB/s, sustained BF16 TFLOP/s, source) from the driver-written peaks file."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops_sustained"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while a timed region runs
    (read-only queries: NVML in a thread, or an `nvidia-smi -lms` child when NVML cannot be
    loaded).  The GPU is found by UUID so CUDA_VISIBLE_DEVICES remapping cannot pick another."""
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    SMI_FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: torch.device, period_s: float = 0.005):
        self.uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
        self.period, self.rows, self.stop = period_s, [], threading.Event()
        self.thread, self.proc, self.source = None, None, None

    def _nvml_loop(self, nv, h):
        bits = [(nv.nvmlClocksEventReasonHwSlowdown, "hw_slowdown"),
                (nv.nvmlClocksEventReasonHwThermalSlowdown, "hw_thermal_slowdown"),
                (nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_thermal_slowdown"),
                (nv.nvmlClocksEventReasonSwPowerCap, "sw_power_cap")]
        mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        while not self.stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.rows.append((float(sm), float(mx), [n for b, n in bits if mask & b]))
            except Exception:  # noqa: BLE001
                pass
            self.stop.wait(self.period)

    def _smi_loop(self):
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            try:
                self.rows.append((float(c[0]), float(c[1]),
                                  [n for n, v in zip(self.NAMES, c[2:6])
                                   if v.lower().startswith("active")]))
            except Exception:  # noqa: BLE001
                continue

    def __enter__(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByUUID(self.uuid)
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.source = "nvml"
        except Exception:  # noqa: BLE001
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.SMI_FIELDS}",
                     "--format=csv,noheader,nounits", "-lms", "50"],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
                self.thread = threading.Thread(target=self._smi_loop, daemon=True)
                self.source = "nvidia-smi"
            except Exception:  # noqa: BLE001
                self.thread = None
        if self.thread is not None:
            self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:  # noqa: BLE001
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0,
                    "source": self.source}
        reasons = sorted({n for r in self.rows for n in r[2]})
        return {"sm_mhz": statistics.median(r[0] for r in self.rows),
                "sm_min_mhz": min(r[0] for r in self.rows),
                "sm_max_mhz": max(r[1] for r in self.rows), "reasons": reasons,
                "samples": len(self.rows), "source": self.source}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def workload_params(name: str):
    if name == "cfg2":
        return dict(b=16, h_q=64, ctx=32768, topk=2048), "configs[1]: decode b=16 h_q=64 ctx=32768 topk=2048, 644-B FP8 paged KV"
    if name == "target":
        return dict(b=64, h_q=64, ctx=32768, topk=2048), "north_star target: decode b=64 h_q=64 ctx=32768 topk=2048, 644-B FP8 paged KV"
    if name == "cfg2_tp16":
        return dict(b=16, h_q=16, ctx=32768, topk=2048), "configs[1] as one TP shard: h_q=16"
    raise SystemExit(f"unknown workload {name}")


# ----------------------------------------------------------------------------
# CPU path (the oracle): used by --impl reference and by the cpu_baseline leg.
# ----------------------------------------------------------------------------
def time_cpu_oracle(q, kv4, idx, sm_scale, steps: int, warmup: int):
    from oracle import sparse_mla as O           # CPU baseline leg only
    layout = O.V32 if kv4.size(3) == 644 else O.MODEL1
    pages = kv4.view(kv4.size(0), -1)
    for _ in range(warmup):
        O.sparse_decode(q, pages, idx, None, None, sm_scale, kv4.size(1), layout)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.sparse_decode(q, pages, idx, None, None, sm_scale, kv4.size(1), layout)
        times.append(time.perf_counter() - t0)
    return times


def run_reference(args):
    """The reference's CPU torch path (ported in oracle/), all host threads."""
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may run on.
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:  # noqa: BLE001
        pass
    rank, world, _ = dist_env()
    if rank != 0:
        return
    import bench_workloads as W
    from oracle import sparse_mla as O

    def cpu_quantize(k_nope, k_rope, slots, kv):
        layout = O.V32 if kv.size(3) == 644 else O.MODEL1
        body, scales = O.quantize_rows(k_nope, k_rope, layout)
        nrb = layout.nope_rope_bytes
        nb, P = kv.size(0), kv.size(1)
        arena = kv.view(nb, -1)
        p0 = int(slots[0]) // P                 # fill_cache hands over whole pages in order
        n_pages = k_nope.size(0) // P
        arena[p0:p0 + n_pages, : P * nrb] = body.view(n_pages, P * nrb)
        arena[p0:p0 + n_pages, P * nrb: P * layout.bytes_per_token] = \
            scales.view(n_pages, P * layout.scale_slots)

    params, desc = workload_params(args.workload)
    wl = W.config2(torch.device("cpu"), cpu_quantize, n_index_sets=1, **params)
    # One step = one full call of the workload.  The step count asked for is honoured up to
    # about 90 s of CPU time (a warm-up call gives the time of one step).
    t_probe = time_cpu_oracle(wl.q, wl.kv, wl.indices[0], wl.sm_scale, 1, 1)[0]
    steps = max(1, min(args.steps, int(90.0 / max(t_probe, 1e-3))))
    times = time_cpu_oracle(wl.q, wl.kv, wl.indices[0], wl.sm_scale, steps, 0)
    t = statistics.mean(times)
    value = wl.algorithmic_bytes() / t / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1),
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc, "layout": "V32 (576/512, 644 B/token)",
                   "note": "CPU torch port of the reference's tests/reference.py decode path; "
                           "it dequantises the whole cache every call, as the reference does"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} full calls of the workload ({t:.2f} s each)"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# GPU path
# ----------------------------------------------------------------------------
def timed_calls(stream, dev, fn, est_us, barrier, max_over_ranks, min_calls=20):
    """Time back-to-back calls of fn(i) on `stream` with one CUDA-event pair around a region
    of at least MIN_REGION_S; returns microseconds per call (max over ranks)."""
    n = max(min_calls, int(MIN_REGION_S * 1e6 / max(est_us, 1.0)) + 1)
    for i in range(5):
        fn(i)
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for i in range(n):
        fn(i)
    b.record(stream)
    barrier()
    return max_over_ranks(a.elapsed_time(b)) / n * 1e3, n


def run_ours(args):
    rank, world, local = dist_env()
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from deepseek_v4_kernel import cuda as K
    from deepseek_v4_kernel import ops
    import bench_workloads as W

    params, desc = workload_params(args.workload)
    wl = W.config2(dev, ops.kv_store, n_index_sets=N_INDEX_SETS, seed=rank, **params)
    stream = torch.cuda.current_stream(dev)
    call = K.DecodeCall(wl.q, wl.kv, wl.indices[0], wl.sm_scale)
    alg_bytes = [wl.algorithmic_bytes(i) for i in range(N_INDEX_SETS)]
    mean_bytes = sum(alg_bytes) / len(alg_bytes)
    hbm_peak, tf_peak, peak_src = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- (1) inputs resident in HBM: K steps of `inner` whole calls each ----------------
    def one_call(i):
        call.set_indices(wl.indices[i % N_INDEX_SETS])
        call.decode(stream.cuda_stream, with_combine=True)

    for i in range(max(args.warmup, 3) * 4):
        one_call(i)
    barrier()
    # a short probe sizes the step so that the timed region reaches MIN_REGION_S
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(stream)
    for i in range(64):
        one_call(i)
    p1.record(stream)
    torch.cuda.synchronize(dev)
    est_us = max_over_ranks(p0.elapsed_time(p1)) / 64 * 1e3
    inner = max(1, int(MIN_REGION_S * 1e6 / (est_us * args.steps)) + 1)

    def step(s):
        for j in range(inner):
            one_call(s * inner + j)

    for s_ in range(args.warmup):
        step(s_)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def same_load(seconds: float, i0: int):
        """Untimed steps of the same loop, so the clock samples bracket the timed region
        under the load it runs at (the region alone can be shorter than one sample)."""
        t_end, i = time.perf_counter() + seconds, i0
        while time.perf_counter() < t_end:
            for _ in range(64):
                one_call(i)
                i += 1
            stream.synchronize()
        return i

    with ClockSampler(dev) as clocks:
        same_load(args.clock_window / 2, 0)
        barrier()
        ev0.record(stream)
        for s_ in range(args.steps):
            step(s_)
        ev1.record(stream)
        barrier()
        same_load(args.clock_window / 2, 0)
        barrier()
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_per_step = ms_total / args.steps
    us_per_call = ms_per_step / inner * 1e3
    value = world * mean_bytes / (us_per_call * 1e-6) / 1e9

    # ---- (2) the decode kernel alone: back-to-back launches without the combine ------
    # (the partials of one launch are overwritten by the next; one event pair around the
    # whole run, so no per-launch event overhead is counted as kernel time)
    def kernel_only(i):
        call.set_indices(wl.indices[i % N_INDEX_SETS])
        call.decode(stream.cuda_stream, with_combine=False)
    k_us, n_k = timed_calls(stream, dev, kernel_only, est_us, barrier, lambda x: x)
    achieved = mean_bytes / (k_us * 1e-6) / 1e9

    # ---- (2b) the same calls replayed from a CUDA graph (one graph = one pass over the
    # index sets), as a serving loop with captured decode steps would issue them
    graph_us = None
    try:
        side = torch.cuda.Stream(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(N_INDEX_SETS):
                    call.set_indices(wl.indices[i])
                    call.decode(side.cuda_stream, with_combine=True)
        torch.cuda.synchronize(dev)
        reps = max(3, int(MIN_REGION_S * 1e6 / (est_us * N_INDEX_SETS)) + 1)
        for _ in range(2):
            g.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(reps):
            g.replay()
        g1.record(stream)
        torch.cuda.synchronize(dev)
        graph_us = g0.elapsed_time(g1) / (reps * N_INDEX_SETS) * 1e3
    except Exception as exc:  # noqa: BLE001
        graph_us = f"unavailable: {exc}"

    # ---- (3) end to end through the public operator, host buffers -------------------
    # Every step copies its q and indices from pinned host memory, calls the operator and
    # copies out and lse back to pinned host memory.  As a serving framework does for decode,
    # the step (upload, operator, download) is captured once per index set as a CUDA graph
    # and replayed; consecutive steps go round-robin over three streams with a buffer set
    # each, so the upload of one step overlaps the download of another (PCIe is full
    # duplex).  Nothing is skipped or reused between steps.
    q_host = wl.q.cpu().pin_memory()
    idx_host = [t.cpu().pin_memory() for t in wl.indices]
    NBUF = int(os.environ.get("DSV4_BENCH_E2E_STREAMS", "3"))
    out_host = [torch.empty((params["b"], 1, params["h_q"], 512), dtype=torch.bfloat16).pin_memory()
                for _ in range(NBUF)]
    lse_host = [torch.empty((params["b"], params["h_q"], 1), dtype=torch.float32).pin_memory()
                for _ in range(NBUF)]
    q_dev = [torch.empty_like(wl.q) for _ in range(NBUF)]
    idx_dev = [torch.empty_like(wl.indices[0]) for _ in range(NBUF)]
    lanes = [torch.cuda.Stream(dev) for _ in range(NBUF)]

    def e2e_body(k, j):
        q_dev[k].copy_(q_host, non_blocking=True)
        idx_dev[k].copy_(idx_host[j], non_blocking=True)
        out, lse, _, _ = ops.sparse_decode_fwd(q_dev[k], wl.kv, idx_dev[k], None, None, None,
                                               None, None, None, None, 512, wl.sm_scale)
        out_host[k].copy_(out, non_blocking=True)
        lse_host[k].copy_(lse, non_blocking=True)

    graphs = [[None] * N_INDEX_SETS for _ in range(NBUF)]
    for k in range(NBUF):
        pool = None
        with torch.cuda.stream(lanes[k]):
            e2e_body(k, 0)                                    # warm the allocator outside capture
            lanes[k].synchronize()
            for j in range(N_INDEX_SETS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, pool=pool, stream=lanes[k]):
                    e2e_body(k, j)
                pool = g.pool()
                graphs[k][j] = g
    torch.cuda.synchronize(dev)

    def e2e_step(i):
        k = i % NBUF
        with torch.cuda.stream(lanes[k]):
            graphs[k][i % N_INDEX_SETS].replay()

    n_e2e = max(args.steps, int(MIN_REGION_S * 1e6 / (2.5 * est_us)) + 1)
    for i in range(max(args.warmup, NBUF)):
        e2e_step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for k in range(NBUF):
        lanes[k].wait_stream(stream)
    e0.record(stream)
    for k in range(NBUF):
        lanes[k].wait_event(e0)
    for i in range(n_e2e):
        e2e_step(i)
    for k in range(NBUF):
        stream.wait_stream(lanes[k])
    e1.record(stream)
    barrier()
    e2e_us = max_over_ranks(e0.elapsed_time(e1)) / n_e2e * 1e3
    e2e_value = world * mean_bytes / (e2e_us * 1e-6) / 1e9
    h2d = q_host.numel() * 2 + idx_host[0].numel() * 4
    d2h = out_host[0].numel() * 2 + lse_host[0].numel() * 4
    # the last step's result really is in host memory
    assert torch.isfinite(out_host[(n_e2e - 1) % NBUF].float()).all()

    # ---- (3b) one eager call at a time on one stream: upload, operator, download, wait.
    # This is the latency a caller sees, host cost of the operator wrapper included.
    def eager_call(j):
        q_dev[0].copy_(q_host, non_blocking=True)
        idx_dev[0].copy_(idx_host[j % N_INDEX_SETS], non_blocking=True)
        out, lse, _, _ = ops.sparse_decode_fwd(q_dev[0], wl.kv, idx_dev[0], None, None, None,
                                               None, None, None, None, 512, wl.sm_scale)
        out_host[0].copy_(out, non_blocking=True)
        lse_host[0].copy_(lse, non_blocking=True)
        stream.synchronize()
    for j in range(10):
        eager_call(j)
    n_eager = max(50, int(MIN_REGION_S * 1e6 / 150.0))
    t_e = time.perf_counter()
    for j in range(n_eager):
        eager_call(j)
    eager_us = max_over_ranks((time.perf_counter() - t_e) / n_eager * 1e6)

    # ---- (4) CPU baseline (rank 0, single-GPU run only) -----------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
        except Exception:  # noqa: BLE001
            pass
        n_cpu = 40
        times = time_cpu_oracle(wl.q.cpu(), wl.kv.cpu(), wl.indices[0].cpu(), wl.sm_scale, n_cpu, 1)
        cpu = {"value": alg_bytes[0] / statistics.mean(times) / 1e9, "unit": "GB/s",
               "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"{n_cpu} full calls of the same workload after 1 warm-up "
                         f"({statistics.mean(times):.2f} s per call)"}

    headline_cfg = {"workload": desc, "per_gpu_batch": params["b"], "n_splits": call.n_splits,
                    "kv_pool_mb": wl.kv.numel() / 1e6,
                    "l2_policy": f"rotates {N_INDEX_SETS} index sets (~{N_INDEX_SETS * wl.kv_gather_bytes() / 1e6:.0f} MB of distinct rows) so inputs exceed L2",
                    "parallelism": f"request-parallel x{world}, no collective"}
    kv_gather = wl.kv_gather_bytes()
    flops = wl.flops()
    launches_per_call = call.launches_per_call
    n_splits_used = call.n_splits
    del call, wl, graphs, q_dev, idx_dev
    torch.cuda.empty_cache()

    more = {}
    if not args.no_more:
        if not args.head_tp_only:
            more.update(run_more(dev, K, ops, W, stream, rank, world, barrier, max_over_ranks,
                                 hbm_peak, tf_peak))
        if world > 1:
            more.update(run_head_tp(dev, K, ops, W, stream, rank, world, max_over_ranks))
    extras = {}
    if args.extras and rank == 0:
        extras.update(run_extras(dev, K, ops, W, stream))

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "calls_per_step": inner, "us_per_call": us_per_call, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": headline_cfg,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak,
                         "traffic": ncu_traffic_bytes(args.workload),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, "
                                           "from the committed capture summary of this workload",
                         "peak_source": peak_src,
                         "kernel": "sparse decode (gather+dequant+QK^T+softmax+PV)",
                         "kernel_us": k_us, "launches_timed": n_k,
                         "algorithmic_bytes_per_launch": mean_bytes,
                         "kv_gather_gbs": kv_gather / (k_us * 1e-6) / 1e9,
                         "tflops": flops / (k_us * 1e-6) / 1e12},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "us_per_call": e2e_us, "calls_timed": n_e2e,
                    "eager_single_stream_us_per_call": eager_us,
                    "how": "one e2e step is ONE call (the byte counts are per call): "
                           "ops.sparse_decode_fwd with host buffers: upload + operator + download "
                           "captured per index set as a CUDA graph, steps round-robin over 3 streams; "
                           "eager_single_stream_us_per_call is one uncaptured call at a time "
                           "(upload, operator, download, synchronise), wall clock"},
            "cuda_graph_us_per_call": graph_us,
            "gpu_launches": args.steps * inner * launches_per_call,
            "clocks": clocks.summary(),
        }
        line["config"]["n_splits"] = n_splits_used
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if more:
            line["more"] = more
        if extras:
            line["extras"] = extras
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_more(dev, K, ops, W, stream, rank, world, barrier, max_over_ranks, hbm_peak, tf_peak):
    """The rest of the metric, each in a region of at least MIN_REGION_S: the batch-64 target
    shape and one tensor-parallel shard (per rank), the 128-request mixed-length decode split
    over the ranks (strong scaling) and sparse prefill with its query rows balanced (by modelled time) over
    the ranks."""
    from deepseek_v4_kernel import sharding
    out = {}

    def decode_case(wl, est_us, n_splits=None):
        call = K.DecodeCall(wl.q, wl.kv, wl.indices[0], wl.sm_scale, n_splits=n_splits)
        ns = len(wl.indices)

        def fn(i):
            call.set_indices(wl.indices[i % ns])
            call.decode(stream.cuda_stream)
        us, n = timed_calls(stream, dev, fn, est_us, barrier, max_over_ranks)
        return us, n, call

    # target: batch 64 per rank (the shape the 70 %-of-HBM goal is worded on)
    wl = W.config2(dev, ops.kv_store, b=64, h_q=64, n_index_sets=4, seed=100 + rank)
    us, n, call = decode_case(wl, 55.0)
    gbs = wl.algorithmic_bytes() / (us * 1e-6) / 1e9
    out["target_b64"] = {"us_per_call": us, "gbs_per_gpu": gbs, "frac_of_measured_hbm": gbs / hbm_peak,
                         "kv_gather_gbs_per_gpu": wl.kv_gather_bytes() / (us * 1e-6) / 1e9,
                         "n_splits": call.n_splits, "partial_sets": call.partial_sets,
                         "calls_timed": n, "scaling": "weak"}
    del wl, call
    torch.cuda.empty_cache()
    # one tensor-parallel shard of the headline workload: 16 of 64 heads
    wl = W.config2(dev, ops.kv_store, b=16, h_q=16, n_index_sets=16, seed=200 + rank)
    us, n, call = decode_case(wl, 20.0)
    gbs = wl.algorithmic_bytes() / (us * 1e-6) / 1e9
    out["cfg2_tp16"] = {"us_per_call": us, "gbs_per_gpu": gbs, "frac_of_measured_hbm": gbs / hbm_peak,
                        "n_splits": call.n_splits, "calls_timed": n, "scaling": "weak"}
    del wl, call
    torch.cuda.empty_cache()
    # 128 requests in total, contexts 4096..65536, half of every list clustered: 128 / N per rank
    b_total = 128
    b_rank = len(range(*sharding.request_slice(b_total, world, rank).indices(b_total)))
    wl = W.config3(dev, ops.kv_store, b=b_rank, n_index_sets=2, seed=300 + rank)
    us, n, call = decode_case(wl, 100.0 * b_rank / 128 + 10)
    total_bytes = wl.algorithmic_bytes()
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([float(total_bytes)], device=dev, dtype=torch.float64)
        dist.all_reduce(t)
        total_bytes = float(t.item())
    gbs = total_bytes / (us * 1e-6) / 1e9
    out["cfg3_b128_total"] = {"us_per_step": us, "requests_per_s": b_total / (us * 1e-6),
                              "gbs_total": gbs, "frac_of_measured_hbm_per_gpu": gbs / world / hbm_peak,
                              "requests_per_gpu": b_rank, "n_splits": call.n_splits,
                              "calls_timed": n, "scaling": "strong"}
    del wl, call
    torch.cuda.empty_cache()
    # sparse prefill: 8192 causal queries, top-k 2048, FP8 pages; rows balanced by modelled time
    pw = W.config5(dev, ops.kv_store)
    lo, hi = sharding.balanced_query_blocks(pw.q.size(0), pw.indices.size(1), world)[rank]
    q_l, idx_l = pw.q[lo:hi].contiguous(), pw.indices[lo:hi].contiguous()
    res = {}
    for name, fn in (("fp8_pages", lambda i: ops.sparse_prefill_fwd_fp8(q_l, pw.kv_pages, idx_l, pw.sm_scale, 512)),
                     ("bf16_workspace", lambda i: ops.sparse_prefill_fwd(q_l, pw.kv_bf16, idx_l, pw.sm_scale, 512))):
        us, n = timed_calls(stream, dev, fn, 4000.0 / world, barrier, max_over_ranks, min_calls=5)
        tf = pw.flops() / (us * 1e-6) / 1e12
        res[name] = {"ms_per_call": us / 1e3, "tflops_total": tf,
                     "frac_of_measured_bf16_sustained_per_gpu": tf / world / tf_peak, "calls_timed": n}
    res["pairs"] = pw.pairs()
    res["rows_of_rank0"] = hi - lo if rank == 0 else None
    res["scaling"] = "strong"
    out["cfg5_prefill"] = res
    # KV store / quantise of the same 8192 tokens (BF16 latent + RoPE in, 644-byte tokens out);
    # sixteen copies of the input rotate so that the rows read come from HBM, not from L2
    d_nope = pw.kv_bf16.size(1) - 64
    n_tok = pw.q.size(0)
    nope = [pw.kv_bf16[:, :d_nope].contiguous() for _ in range(16)]
    rope = [pw.kv_bf16[:, d_nope:].contiguous() for _ in range(16)]
    slots = torch.arange(n_tok, device=dev, dtype=torch.int64)
    eager_us, _ = timed_calls(stream, dev, lambda i: ops.kv_store(nope[i % 16], rope[i % 16], slots, pw.kv_pages),
                              10.0, barrier, max_over_ranks)
    # the sixteen stores as one CUDA graph: the kernel's own rate, without the host's launch cost
    side = torch.cuda.Stream(dev)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(16):
                ops.kv_store(nope[i], rope[i], slots, pw.kv_pages)
    us16, n = timed_calls(stream, dev, lambda i: g.replay(), 16 * 5.0, barrier, max_over_ranks)
    us = us16 / 16
    sbytes = n_tok * (d_nope * 2 + 128 + 644)
    out["kv_store_8192_tokens"] = {"us_per_call": us, "gbs_per_gpu": sbytes / (us * 1e-6) / 1e9,
                                   "frac_of_measured_hbm": sbytes / (us * 1e-6) / 1e9 / hbm_peak,
                                   "eager_us_per_call": eager_us,
                                   "bytes_per_call": sbytes, "calls_timed": n * 16, "scaling": "weak",
                                   "l2_policy": "16 input copies (151 MB) rotate; graph of 16 stores replayed"}
    del g
    del pw, nope, rope
    torch.cuda.empty_cache()
    return out


def run_head_tp(dev, K, ops, W, stream, rank, world, max_over_ranks):
    """Head-sharded (tensor-parallel) decode of configs[1] and configs[3]: every rank holds
    the same KV cache and index lists (MQA: one KV head), computes h_q / world heads and the
    per-head results are exchanged with one all-gather over NVLink.  KV traffic is not
    reduced by this sharding; the figure of interest is the time of a step."""
    import torch.distributed as dist
    from deepseek_v4_kernel import sharding
    out = {}
    for name, make in (("cfg2", lambda: W.config2(dev, ops.kv_store, n_index_sets=16, seed=0)),
                       ("cfg4", lambda: W.config4(dev, ops.kv_store, seed=0))):
        wl = make()                                  # same seed on every rank: replicated inputs
        hs = sharding.head_slice(wl.q.size(2), world, rank)
        q_loc = wl.q[:, :, hs].contiguous()
        call = K.DecodeCall(q_loc, wl.kv, wl.indices[0], wl.sm_scale, n_splits=wl.force_splits)
        lse_loc = call.lse
        ns = len(wl.indices)

        def step(i, gather=True):
            call.set_indices(wl.indices[i % ns])
            call.decode(stream.cuda_stream)
            if gather:
                return sharding.all_gather_heads(call.out, lse_loc)

        p2p = sharding.HeadGather(wl.q.size(0), 1, wl.q.size(2), dev)

        def step_p2p(i, _gather=True):
            call.set_indices(wl.indices[i % ns])
            call.decode(stream.cuda_stream)
            return p2p.gather(call.out, lse_loc, stream.cuda_stream)

        def step_fused(i, _gather=True):
            call.set_indices(wl.indices[i % ns])
            return p2p.decode_gather(call, stream.cuda_stream)

        # the floor of any exchange built on flags in peer memory: no rows, flags only
        flags_only = sharding.HeadGather(0, 1, wl.q.size(2), dev)

        def step_flags(i, _gather=True):
            call.set_indices(wl.indices[i % ns])
            call.decode(stream.cuda_stream)
            return flags_only.gather(call.out, lse_loc, stream.cuda_stream)

        res = {}
        for label, gather in (("decode_plus_nccl_all_gather", True), ("decode_only", False),
                              ("decode_plus_peer_memory_gather", None),
                              ("decode_and_exchange_in_one_call", "fused"),
                              ("decode_plus_flag_barrier_without_rows", "flags")):
            fn = {"fused": step_fused, "flags": step_flags, None: step_p2p}.get(gather, step)
            n_tp = 1000                                 # >= 50 ms per region at 50 us per step
            for i in range(5):
                fn(i, gather)
            dist.barrier()
            torch.cuda.synchronize(dev)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for i in range(n_tp):
                fn(i, gather)
            b.record(stream)
            dist.barrier()
            torch.cuda.synchronize(dev)
            res[label + "_us"] = max_over_ranks(a.elapsed_time(b)) / n_tp * 1e3
        res["peer_gather_timed_out"] = p2p.timed_out()
        res.update(heads_per_rank=hs.stop - hs.start, n_splits=call.n_splits,
                   gathered_bytes_per_rank=call.out.numel() * 2 + lse_loc.numel() * 4)
        out[f"{name}_head_tp{world}"] = res
        del wl, call
        torch.cuda.empty_cache()

    return out


def run_extras(dev, K, ops, W, stream):
    """Secondary measurements (opt-in): the other configurations of the same path.
    Decode shapes: the batch-64 target, one TP shard (h_q = 16), the reference's own
    584-byte layout, the single-token case, the forced-128-split long context (with its
    combine alone).  Then sparse prefill (TFLOP/s, both KV entries) and the KV store."""
    out = {}
    peak, tf_peak, _ = measured_peaks()

    def time_calls(fn, n=50, warm=5):
        for i in range(warm):
            fn(i)
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for i in range(n):
            fn(i)
        b.record(stream)
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / n

    def decode_case(name, wl, n_splits=None):
        call = K.DecodeCall(wl.q, wl.kv, wl.indices[0], wl.sm_scale, n_splits=n_splits)
        ns = len(wl.indices)

        def fn(i):
            call.set_indices(wl.indices[i % ns])
            call.decode(stream.cuda_stream)
        ms = time_calls(fn)
        gbs = wl.algorithmic_bytes() / (ms * 1e-3) / 1e9
        out[name] = {"us_per_call": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peak,
                     "n_splits": call.n_splits, "partial_sets": call.partial_sets}
        return call

    for name in ("target", "cfg2_tp16"):
        params, _ = workload_params(name)
        wl = W.config2(dev, ops.kv_store, n_index_sets=4 if name == "target" else 16, **params)
        decode_case(name, wl)
        del wl
        torch.cuda.empty_cache()
    wl = W.config2(dev, ops.kv_store, n_index_sets=16, layout="MODEL1")
    decode_case("cfg2_layout_584B", wl)
    del wl
    wl = W.config1(dev, ops.kv_store)
    decode_case("cfg1", wl)
    del wl
    wl = W.config3(dev, ops.kv_store, b=128, n_index_sets=2)     # mixed context lengths, half clustered
    decode_case("cfg3_b128", wl)
    del wl
    torch.cuda.empty_cache()
    wl = W.config4(dev, ops.kv_store)
    call = decode_case("cfg4_128_splits", wl, n_splits=wl.force_splits)
    if call.partial_sets > 1:
        ms = time_calls(lambda i: call.combine(stream.cuda_stream))
        b_, h_q = wl.q.size(0), wl.q.size(2)
        cbytes = call.partial_sets * b_ * h_q * (512 * 4 + 4) + b_ * h_q * (512 * 2 + 4)
        out["cfg4_combine_alone"] = {"us_per_call": ms * 1e3, "gbs": cbytes / (ms * 1e-3) / 1e9,
                                     "bytes": cbytes, "partial_sets": call.partial_sets}
    del wl, call
    torch.cuda.empty_cache()

    # sparse prefill (configs[4]): s_q = s_kv = 8192, causal top-2048
    pw = W.config5(dev, ops.kv_store)
    for name, fn in (("cfg5_prefill_bf16_kv", lambda i: ops.sparse_prefill_fwd(pw.q, pw.kv_bf16, pw.indices, pw.sm_scale, 512)),
                     ("cfg5_prefill_fp8_pages", lambda i: ops.sparse_prefill_fwd_fp8(pw.q, pw.kv_pages, pw.indices, pw.sm_scale, 512))):
        ms = time_calls(fn, n=5, warm=2)
        tf = pw.flops() / (ms * 1e-3) / 1e12
        out[name] = {"ms_per_call": ms, "tflops": tf, "frac_of_measured_bf16_sustained": tf / tf_peak,
                     "pairs": pw.pairs()}
    # KV store / quantise of the same 8192 tokens
    d_nope = pw.kv_bf16.size(1) - 64
    k_nope, k_rope = pw.kv_bf16[:, :d_nope].contiguous(), pw.kv_bf16[:, d_nope:].contiguous()
    slots = torch.arange(pw.q.size(0), device=dev, dtype=torch.int64)
    ms = time_calls(lambda i: ops.kv_store(k_nope, k_rope, slots, pw.kv_pages), n=50)
    sbytes = pw.q.size(0) * (d_nope * 2 + 128 + 644)      # BF16 in, one 644-byte token out
    out["kv_store_8192_tokens"] = {"us_per_call": ms * 1e3, "gbs": sbytes / (ms * 1e-3) / 1e9,
                                   "frac_of_measured_hbm": sbytes / (ms * 1e-3) / 1e9 / peak}

    # CPU oracle beside it, bounded samples: the single-token case as it is, the long
    # context on its one request, prefill on one block of 256 query rows (the last rows:
    # full 2048-entry lists) scaled to the pair count.
    from oracle import sparse_mla as O
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:  # noqa: BLE001
        pass
    cpu = {"cores": torch.get_num_threads()}
    for name, wl in (("cfg1", W.config1(dev, ops.kv_store)), ("cfg4", W.config4(dev, ops.kv_store))):
        t = min(time_cpu_oracle(wl.q.cpu(), wl.kv.cpu(), wl.indices[0].cpu(), wl.sm_scale, 2, 1))
        cpu[name + "_ms_per_call"] = t * 1e3
        del wl
    rows = slice(pw.q.size(0) - 256, pw.q.size(0))
    q_c, kv_c, idx_c = pw.q[rows].cpu(), pw.kv_bf16.cpu(), pw.indices[rows].cpu()
    t0 = time.perf_counter()
    O.sparse_prefill(q_c, kv_c, idx_c, pw.sm_scale, 512)
    t = time.perf_counter() - t0
    pairs = int((idx_c >= 0).sum())
    cpu["cfg5_prefill_tflops"] = pairs * pw.q.size(1) * 2 * (pw.q.size(2) + 512) / t / 1e12
    cpu["cfg5_sample"] = f"last 256 of {pw.q.size(0)} query rows, {t:.2f} s"
    out["cpu_oracle"] = cpu
    return out


def run_prefill(args):
    """`--workload cfg5[:s_q]`: sparse prefill (configs[4]) on one GPU, one JSON line.
    The secondary metric of the path (TFLOP/s against the measured BF16 peak); not the line
    the default run prints."""
    rank, world, local = dist_env()
    if rank != 0:
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from deepseek_v4_kernel import ops
    import bench_workloads as W
    s_q = int(args.workload.split(":")[1]) if ":" in args.workload else 8192
    pw = W.config5(dev, ops.kv_store, s_q=s_q, with_pages=False)
    stream = torch.cuda.current_stream(dev)
    fn = lambda: ops.sparse_prefill_fwd(pw.q, pw.kv_bf16, pw.indices, pw.sm_scale, 512)
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.steps):
        fn()
    b.record(stream)
    torch.cuda.synchronize(dev)
    ms = a.elapsed_time(b) / args.steps
    try:
        tf_peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"]
        src = "measured"
    except Exception:  # noqa: BLE001
        tf_peak, src = 1400.0, "fallback"
    tf = pw.flops() / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "sparse_prefill_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"configs[4]: sparse prefill s_q=s_kv={s_q} h_q=64 causal top-k 2048, BF16 KV workspace",
                   "pairs": pw.pairs()},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": tf_peak, "unit": "TFLOP/s",
                     "frac": tf / tf_peak, "traffic": None, "peak_source": src},
        "gpu_launches": args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--extras", action="store_true")
    ap.add_argument("--no-more", action="store_true",
                    help="headline only: skip the target shape, the strong-scaling decode, prefill "
                         "and the head-sharded step")
    ap.add_argument("--head-tp-only", action="store_true",
                    help="of the additional measurements keep only the head-sharded step (N >= 2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--clock-window", type=float, default=1.0,
                    help="seconds of identical untimed load around the timed region over which "
                         "SM clocks are sampled")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload.startswith("cfg5"):
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
