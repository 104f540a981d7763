#!/usr/bin/env python3
"""Benchmark of the PTO hot path on B200: fp16 -> fp32 GEMM at m = n = k = 6144 (headline), with
flash-attention forward and the vector tile ops measured in the same run as extras.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is REPEATS (20) passes over one batch of independent problems: PROBLEMS_PER_RANK (8) GEMMs of
6144^3 per GPU, each with its own A, B and C (the batch's inputs, 1.2 GB, exceed the 126 MB L2, so operands
come from HBM every time): 160 launches, about 56 ms, so that 20 steps fill more than a second, the
regime of the measured sustained peak, with hundreds of clock samples.  At 8 GPUs the batch is the
64-problem configuration; work per GPU is fixed (weak scaling) and no collective is on the data path; the
all-gather of the outputs is measured both after the step and overlapped with it (`with_allgather`).
Under torchrun every rank runs its own problems; the time of the timed region is the maximum over ranks.

One JSON line is printed by rank 0.  `value` is whole-job TFLOP/s with operands resident in HBM;
`e2e` is the same metric through the C ABI's host-buffer entry point (pinned host operands, copies in
and out inside the timed region); `roofline` describes the GEMM kernel (tensor bound) from CUDA-event
launch durations measured inside the timed loop; `cpu_baseline` is the reference's CPU-simulation tile
program timed on this box's host cores on a bounded sample of the same problem.

`--impl reference` times that CPU-simulation program alone (all host threads), on the same metric.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 6144
PROBLEMS_PER_RANK = 8
REPEATS = 20  # passes over the batch per step
FLOPS_PER_PROBLEM = 2.0 * M * N * K
TILE_M, TILE_N = 128, 256
TILE_FLOPS = 2.0 * TILE_M * TILE_N * K
# dram__bytes_read.sum + dram__bytes_write.sum of one 6144^3 launch, from the ncu capture summarised in
# profiles/gemm2_f16f32_6144_ncu.md
GEMM_DRAM_TRAFFIC_BYTES = 571.3e6
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------ clock sampling during the timed region

class ClockSampler:
    """Samples the SM clock and the clock event reasons of one GPU while the timed region runs: NVML polled from a
    thread every few milliseconds (read-only queries), or an `nvidia-smi -lms` child when NVML cannot be loaded."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                   0x80: "hw_power_brake_slowdown"}

    def __init__(self, index, uuid=None):
        self.index = index
        self.uuid = uuid
        self.samples = []      # (sm_mhz, reasons bitmask) from NVML, or csv fields from nvidia-smi
        self.max_mhz = None
        self.proc = None
        self.thread = None
        self.nvml = None
        self.handle = None
        self.stop_flag = threading.Event()

    def _open_nvml(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = None
            if self.uuid:
                try:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
                except Exception:
                    handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.nvml, self.handle = pynvml, handle
            return True
        except Exception:
            return False

    def start(self):
        if self._open_nvml():
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _poll_nvml(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                bits = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, bits))
            except Exception:
                pass
            time.sleep(0.003)

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            sm = [s[0] for s in self.samples]
            bits = 0
            for s in self.samples:
                bits |= s[1]
            reasons = sorted(name for bit, name in self.REASON_BITS.items() if bits & bit)
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "samples": len(sm),
                    "sm_mhz_min": min(sm) if sm else None, "reasons": reasons, "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


# ------------------------------------------------------------------ CPU side (reference arm / cpu_baseline)

def cpu_gemm_sample(budget_s, min_tiles=1, max_tiles=64):
    """Runs the CPU tile program on C tiles of the 6144^3 problem for about `budget_s` seconds.
    Returns (tflops, info dict).  Uses the reference's own CPU simulation when its build is present."""
    import ctypes

    import numpy as np

    import oracle
    use_ref = oracle.ref is not None
    lib = oracle.ref if use_ref else oracle.port
    P = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    r = np.random.default_rng(0)
    # a strip of the problem: the A rows of one tile row and the B rows (n x k layout) of `max_tiles` tile columns
    tiles_n = min(max_tiles, N // TILE_N)
    a = r.uniform(-1, 1, (TILE_M, K)).astype(np.float16)
    b = r.uniform(-1, 1, (tiles_n * TILE_N, K)).astype(np.float16)
    c = np.zeros((TILE_M, tiles_n * TILE_N), np.float32)

    def run(n_tiles):
        t0 = time.perf_counter()
        if use_ref:
            rc = lib.lib.pto_ref_gemm_f16f32_tiles(P(a), P(b), P(c), TILE_M, tiles_n * TILE_N, K, 1, 0, n_tiles)
        else:
            rc = lib.lib.pto_oracle_gemm_f16f32_window(P(a), P(b), P(c), TILE_M, tiles_n * TILE_N, K, 1, 0, TILE_M, 0,
                                                       n_tiles * TILE_N)
        assert rc == 0
        return time.perf_counter() - t0

    t1 = run(1)  # calibration (also warms the thread pool / page faults)
    n_tiles = int(max(min_tiles, min(tiles_n, budget_s / max(t1, 1e-6))))
    dt = run(n_tiles)
    cores = (lib.lib.pto_ref_hardware_threads() if use_ref else lib.lib.pto_oracle_threads())
    info = {"kind": "reference" if use_ref else "port", "cores": int(cores),
            "sample": f"{n_tiles} C tiles of 128x256 at full k=6144 of the 6144^3 problem ({dt:.2f} s)",
            "tiles": n_tiles, "seconds": dt}
    return n_tiles * TILE_FLOPS / dt / 1e12, info


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    total_steps = args.steps + args.warmup
    per_step_budget = max(0.5, min(10.0, 150.0 / max(total_steps, 1)))
    vals, info = [], None
    for i in range(total_steps):
        v, info = cpu_gemm_sample(per_step_budget)
        if i >= args.warmup:
            vals.append((v, info["seconds"], info["tiles"]))
    flops = sum(t * TILE_FLOPS for _, _, t in vals)
    secs = sum(s for _, s, _ in vals)
    value = flops / secs / 1e12
    line = {
        "impl": "reference", "metric": "fp16 GEMM TFLOPS (m=n=k=6144, fp32 accumulate and output)", "value": value,
        "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * secs / max(len(vals), 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": "gemm_f16f32 m=n=k=6144, B stored n x k (Layout::DN), uniform[-1,1) seeded",
                   "note": "CPU simulation of the reference's tile program (TLOAD/TEXTRACT/TMATMUL/TSTORE, base "
                           "128x256, k step 64) on host cores; each step is a bounded sample of C tiles"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
                         "sample": info["sample"]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------ GPU arm

def bench_loop(torch, fn, warm, iters):
    """Average duration (ms) of `fn` over `iters` calls, CUDA events on the launching stream, after `warm` calls."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def stamps_summary(torch, stamps, blocks):
    """Per-block profile stamps (pto_b200_set_profile_buffer) of the last launch reduced as the reference's host does
    (kernels/manual/common/flash_atten/main.cpp:616-660): earliest start, latest end, and the clock the blocks ran at."""
    st = stamps[:blocks].cpu()
    t0, t1, c0, c1 = st[:, 0], st[:, 1], st[:, 2], st[:, 3]
    ok = (t1 > t0) & (c1 > c0)
    if not bool(ok.any()):
        return None
    dur_ns = (t1 - t0)[ok].double()
    mhz = ((c1 - c0)[ok].double() / dur_ns * 1e3)
    return {"blocks": int(ok.sum()), "kernel_us": float((t1[ok].max() - t0[ok].min()).item()) / 1e3,
            "block_us_median": float(dur_ns.median().item()) / 1e3,
            "sm_mhz_median": float(mhz.median().item()), "sm_mhz_min": float(mhz.min().item()),
            "source": "clock64 / %globaltimer per block (pto_b200_set_profile_buffer)"}


def cpu_vector_and_attention_baselines():
    """The reference's CPU simulation (its own build when present, else the port) on the vector configs and on one
    attention head, timed on this box's host cores; bounded (a few seconds each)."""
    import numpy as np

    import oracle
    lib = oracle.ref if oracle.ref is not None else oracle.port
    kind = "reference" if oracle.ref is not None else "port"
    r = np.random.default_rng(1)
    n = 1 << 24
    x = r.standard_normal(n).astype(np.float32)
    out = {}
    t0 = time.perf_counter()
    lib.tcvt_f32_f16(x)
    dt = time.perf_counter() - t0
    out["tcvt_f16"] = {"value": 6.0 * n / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
                       "sample": f"TCVT f32->f16, 16M elements, {dt:.2f} s (the simulation's TCVT loop is single-threaded)"}
    idx = r.integers(0, n, n).astype(np.int32)
    src = x.reshape(4096, 4096)
    t0 = time.perf_counter()
    lib.tgather(src, idx)
    dt = time.perf_counter() - t0
    out["tgather"] = {"value": 12.0 * n / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
                      "sample": f"TGATHER f32 by int32 index, 16M of 16M, {dt:.2f} s (single-threaded loop)"}
    S, D = 2048, 128
    q = (r.standard_normal((S, D)) / np.sqrt(D)).astype(np.float16)
    k = r.standard_normal((S, D)).astype(np.float16)
    v = r.standard_normal((S, D)).astype(np.float16)
    # the reference build's attention program is instantiated for its unit-test shapes only: the head is timed on the
    # C restatement of the same instruction sequence (bit-identical to it where both exist)
    t0 = time.perf_counter()
    oracle.port.attn_head_f16(q, k, v, 0, 1.0)
    dt = time.perf_counter() - t0
    try:
        cores = int(oracle.port.lib.pto_oracle_threads())
    except Exception:
        cores = os.cpu_count() or 1
    out["attention"] = {"value": 4.0 * S * S * D / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                        "sample": f"one head, S=2048, D=128, non-causal, the simulation's instruction sequence, {dt:.2f} s"}
    return out


def sharded_attention(torch, pto, dist, world, rank, barrier, iters=20):
    from pto_isa_b200 import shard
    heads, S, D = 32 * 32, 8192, 128
    b, e = shard.unit_range(heads, world, rank)
    mine = e - b
    # at one GPU the whole configuration (12.9 GB of Q, K, V, O) is run in four passes over a quarter of the heads
    passes = 4 if world == 1 else 1
    chunk = mine // passes
    g = torch.Generator(device="cuda").manual_seed(900 + rank)
    q = (torch.randn(chunk, S, D, device="cuda", generator=g) / D ** 0.5).half()
    k = torch.randn(chunk, S, D, device="cuda", generator=g).half()
    v = torch.randn(chunk, S, D, device="cuda", generator=g).half()
    o = torch.empty_like(q)
    for _ in range(3):
        pto.flash_attn_fwd(q, k, v, causal=True, scale=1.0, out=o)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(iters):
        pto.flash_attn_fwd(q, k, v, causal=True, scale=1.0, out=o)
    s1.record()
    barrier()
    t = torch.tensor([s0.elapsed_time(s1) / iters * passes], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops = 4.0 * heads * D * S * (S + 1) / 2
    res = {"workload": "flash_attn_fwd f16 batch 32 x 32 heads, S=8192, D=128, causal, fp16 O; heads sharded",
           "value": flops / ms / 1e9, "unit": "TFLOP/s", "ms": ms, "scaling": "strong", "heads_per_gpu": mine,
           "n_gpus": world, "gpu_launches": iters, "timed_launches": iters,
           "note": "one GPU: the time of four passes over 256 heads each" if passes > 1 else None}
    if dist is not None:
        gathers = []
        for i in range(6):  # the first one is the warm-up
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            full = shard.all_gather_units(o, heads)
            g1.record()
            barrier()
            tg = torch.tensor([g0.elapsed_time(g1)], device="cuda", dtype=torch.float64)
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
            if i > 0:
                gathers.append(float(tg.item()))
            nbytes = int(full.numel() * 2)
            del full
        ag = statistics.median(gathers)
        res["allgather_ms"] = ag
        res["allgather_ms_all"] = gathers
        res["bytes_gathered_per_gpu"] = nbytes
        res["allgather_recv_gbs_per_gpu"] = nbytes * (world - 1) / world / ag / 1e6
        res["value_with_allgather"] = flops / (ms + ag) / 1e9
        # overlapped: the rank's heads go in four launches and each quarter's output is gathered on a second stream while
        # the next quarter is computed (quarter-major result: every gather writes one contiguous block)
        parts = 4
        if mine % parts == 0 and mine >= parts:
            qh = mine // parts
            full_q = torch.empty(parts, world, qh, S, D, dtype=torch.float16, device="cuda")
            comm = torch.cuda.Stream()
            times = []
            for it in range(4):
                barrier()
                o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                o0.record()
                works = []
                for c in range(parts):
                    sl = slice(c * qh, (c + 1) * qh)
                    pto.flash_attn_fwd(q[sl], k[sl], v[sl], causal=True, scale=1.0, out=o[sl])
                    done = torch.cuda.Event()
                    done.record()
                    comm.wait_event(done)
                    with torch.cuda.stream(comm):
                        works.append(dist.all_gather_into_tensor(full_q[c], o[sl], async_op=True))
                for w in works:
                    w.wait()
                torch.cuda.current_stream().wait_stream(comm)
                o1.record()
                barrier()
                to = torch.tensor([o0.elapsed_time(o1)], device="cuda", dtype=torch.float64)
                dist.all_reduce(to, op=dist.ReduceOp.MAX)
                if it > 0:
                    times.append(float(to.item()))
            ov = statistics.median(times)
            res["overlapped_ms"] = ov
            res["overlapped_ms_all"] = times
            res["value_overlapped"] = flops / ov / 1e9
            res["overlapped_note"] = f"{parts} launches of {qh} heads per GPU, each quarter gathered while the next is computed"
            del full_q
    del q, k, v, o
    torch.cuda.empty_cache()
    return res


def gemm_size_sweep(torch, pto, peaks):
    """Throughput of the other square sizes of the configurations (1536, 3072, 7680), operand sets rotated so that
    they come from HBM; 20 launches each after 5 warm-up launches."""
    out = []
    g = torch.Generator(device="cuda").manual_seed(7)
    for size, sets in ((1536, 10), (3072, 4), (7680, 2)):
        a = [(torch.rand(size, size, device="cuda", generator=g) * 2 - 1).half() for _ in range(sets)]
        b = [(torch.rand(size, size, device="cuda", generator=g) * 2 - 1).half() for _ in range(sets)]
        c = [torch.empty(size, size, device="cuda") for _ in range(sets)]
        i = [0]

        def fn():
            j = i[0] % sets
            i[0] += 1
            pto.gemm(a[j], b[j], 1, out=c[j])

        ms = bench_loop(torch, fn, 5, 20)
        note = f"{sets} rotating operand sets, 20 launches"
        eager_ms = None
        if ms < 0.04:
            # the launch is shorter than the host's time for one call through the Python layer (about 17 us): the same
            # 20 launches replayed from one CUDA graph time the kernel, the eager figure is kept beside it
            eager_ms = ms
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(20):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            graph.replay()
            s1.record()
            torch.cuda.synchronize()
            ms = s0.elapsed_time(s1) / 20
            note += " replayed from one CUDA graph"
            del graph
        tf = 2.0 * size ** 3 / ms / 1e9
        out.append({"workload": f"gemm_f16f32 m=n=k={size}, B stored n x k", "value": tf, "unit": "TFLOP/s", "ms": ms,
                    "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                 "frac": tf / peaks["bf16_tflops"], "frac_of_nominal_2250": tf / 2250.0,
                                 "note": note}})
        if eager_ms is not None:
            out[-1]["eager_ms_per_call"] = eager_ms
        del a, b, c
    return out


def extras(torch, pto, peaks, peak_kind):
    """Attention and vector tile ops, rank 0 only, short.  Buffers are rotated so inputs come from HBM."""
    out = []
    bench = lambda fn, warm, iters: bench_loop(torch, fn, warm, iters)

    g = torch.Generator(device="cuda").manual_seed(5)
    B, H, S, D = 4, 32, 4096, 128
    q = (torch.randn(B * H, S, D, device="cuda", generator=g) / D ** 0.5).half()
    k = torch.randn(B * H, S, D, device="cuda", generator=g).half()
    v = torch.randn(B * H, S, D, device="cuda", generator=g).half()
    o = torch.empty_like(q)
    q4, k4, v4 = (t.view(B, H, S, D) for t in (q, k, v))
    stamps = torch.zeros(4096, 4, dtype=torch.int64, device="cuda")
    for causal in (False, True):
        ms = bench(lambda: pto.flash_attn_fwd(q, k, v, causal=causal, scale=1.0, out=o), 3, 10)
        flops = 4.0 * B * H * S * S * D if not causal else 4.0 * B * H * D * S * (S + 1) / 2
        tf = flops / ms / 1e9
        # sustained: launches back to back for about a second
        n_long = max(20, int(1000.0 / ms))
        ms_long = bench(lambda: pto.flash_attn_fwd(q, k, v, causal=causal, scale=1.0, out=o), 0, n_long)
        pto.set_profile_buffer(stamps)
        pto.flash_attn_fwd(q, k, v, causal=causal, scale=1.0, out=o)
        torch.cuda.synchronize()
        pto.set_profile_buffer(None)
        prof = stamps_summary(torch, stamps, B * H * (S // 256))
        row = {"workload": f"flash_attn_fwd f16 B=4 H=32 S=4096 D=128 causal={causal}", "value": tf,
               "unit": "TFLOP/s", "ms": ms, "sustained_tflops": flops / ms_long / 1e9, "sustained_launches": n_long,
               "block_stamps": prof,
               "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                            "frac": tf / peaks["bf16_tflops"], "peak_kind": peak_kind + " burst",
                            "frac_of_nominal_2250": tf / 2250.0}}
        # the vendor library's attention on the same box and inputs (torch SDPA): a denominator measured live
        try:
            import torch.nn.functional as F
            lib_ms = bench(lambda: F.scaled_dot_product_attention(q4, k4, v4, is_causal=causal, scale=1.0), 3, 10)
            row["roofline"]["library_sdpa_tflops"] = flops / lib_ms / 1e9
            row["roofline"]["frac_of_library"] = tf / row["roofline"]["library_sdpa_tflops"]
        except Exception as exc:
            row["roofline"]["library_sdpa_tflops"] = None
            row["roofline"]["library_note"] = str(exc)[:120]
        out.append(row)
    del q, k, v, o, q4, k4, v4
    out.extend(gemm_size_sweep(torch, pto, peaks))
    # MX block-scaled fp8 GEMM at the reference's MxMatmul configuration (6144^3, float8_e5m2 operands, e8m0 scales per
    # 32 k, bfloat16 output); four operand sets in rotation (4 x 75 MB of fp8 > L2); scale packing is inside the timing
    mm = 6144
    sets_mx = 4
    mxa = [torch.randint(0, 256, (mm, mm), device="cuda", dtype=torch.uint8, generator=g) & 0x7b | 0x30 for _ in range(sets_mx)]
    mxb = [torch.randint(0, 256, (mm, mm), device="cuda", dtype=torch.uint8, generator=g) & 0xfb | 0x30 for _ in range(sets_mx)]
    mxsa = [torch.randint(127, 130, (mm, mm // 32), device="cuda", dtype=torch.uint8, generator=g) for _ in range(sets_mx)]
    mxsb = [torch.randint(127, 130, (mm, mm // 32), device="cuda", dtype=torch.uint8, generator=g) for _ in range(sets_mx)]
    mxc = torch.empty(mm, mm, device="cuda", dtype=torch.bfloat16)
    mx_i = [0]

    def mx_step():
        j = mx_i[0] % sets_mx
        mx_i[0] += 1
        pto.mx_gemm(mxa[j], mxb[j], mxsa[j], mxsb[j], torch.bfloat16, out=mxc, fmt=pto.ops.FP8_E5M2)

    ms = bench(mx_step, 4, 20)
    tf = 2.0 * mm ** 3 / ms / 1e9
    out.append({"workload": "MX fp8 GEMM (e5m2 x e5m2, e8m0 scales per 32 k, bf16 out) 6144^3", "value": tf,
                "unit": "TFLOP/s", "ms": ms,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": 4500.0, "unit": "TFLOP/s", "frac": tf / 4500.0,
                             "peak_kind": "nominal dense fp8 (no fp8 peak was measured for this GPU)",
                             "vs_measured_bf16_burst": tf / peaks["bf16_tflops"]}})
    # the vendor library's MXFP8 GEMM on the same box and operand bits (cuBLASLt through torch._scaled_mm, e4m3, unit
    # scales): a denominator measured live, in the role the measured cuBLAS figure plays for the fp16 GEMM
    try:
        ones = torch.full((mm, mm // 32), 127, device="cuda", dtype=torch.uint8).view(torch.float8_e8m0fnu)
        la = [x.view(torch.float8_e4m3fn) for x in mxa]
        lb = [x.view(torch.float8_e4m3fn).t() for x in mxb]

        def lib_step():
            j = mx_i[0] % sets_mx
            mx_i[0] += 1
            torch._scaled_mm(la[j], lb[j], scale_a=ones, scale_b=ones, out_dtype=torch.bfloat16)

        lib_ms = bench(lib_step, 4, 20)
        out[-1]["roofline"]["library_mxfp8_tflops"] = 2.0 * mm ** 3 / lib_ms / 1e9
        out[-1]["roofline"]["frac_of_library"] = tf / out[-1]["roofline"]["library_mxfp8_tflops"]
        del ones, la, lb
    except Exception as exc:  # an older torch or cuBLASLt without block-scaled GEMMs: the comparison is left out
        out[-1]["roofline"]["library_mxfp8_tflops"] = None
        out[-1]["roofline"]["library_note"] = str(exc)[:120]
    # the same with packed fp4 (e2m1) operands: the reference's MXFP4 MxMatmul configuration (6144^3, bf16 output)
    fa = [x[:, : mm // 2].contiguous() for x in mxa]
    fb = [x[:, : mm // 2].contiguous() for x in mxb]

    def mx4_step():
        j = mx_i[0] % sets_mx
        mx_i[0] += 1
        pto.mx_gemm_fp4(fa[j], fb[j], mxsa[j], mxsb[j], torch.bfloat16, out=mxc)

    ms = bench(mx4_step, 4, 20)
    tf = 2.0 * mm ** 3 / ms / 1e9
    out.append({"workload": "MX fp4 GEMM (packed e2m1, e8m0 scales per 32 k, bf16 out) 6144^3", "value": tf,
                "unit": "TFLOP/s", "ms": ms,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": 9000.0, "unit": "TFLOP/s", "frac": tf / 9000.0,
                             "peak_kind": "nominal dense fp4 (no fp4 peak was measured for this GPU)",
                             "vs_measured_bf16_burst": tf / peaks["bf16_tflops"]}})
    # TMATMUL's (int8, int8 -> int32) form at the same size: kind::i8 on the CTA-pair GEMM kernel
    ia = [x.view(torch.int8) for x in mxa]
    ib = [x.view(torch.int8) for x in mxb]
    ic = torch.empty(mm, mm, device="cuda", dtype=torch.int32)

    def i8_step():
        j = mx_i[0] % sets_mx
        mx_i[0] += 1
        pto.gemm_i8(ia[j], ib[j], out=ic)

    ms = bench(i8_step, 4, 20)
    tf = 2.0 * mm ** 3 / ms / 1e9
    out.append({"workload": "int8 GEMM (int32 accumulate and output) 6144^3", "value": tf, "unit": "TOP/s", "ms": ms,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": 4500.0, "unit": "TOP/s", "frac": tf / 4500.0,
                             "peak_kind": "nominal dense int8 (no int8 peak was measured for this GPU)",
                             "vs_measured_bf16_burst": tf / peaks["bf16_tflops"]}})
    del mxa, mxb, mxsa, mxsb, mxc, fa, fb, ia, ib, ic
    n = 1 << 24
    sets = 6
    xs = [torch.randn(n, device="cuda", generator=g) for _ in range(sets)]
    o16 = [torch.empty(n, dtype=torch.float16, device="cuda") for _ in range(sets)]
    ob16 = [torch.empty(n, dtype=torch.bfloat16, device="cuda") for _ in range(sets)]
    idx = [torch.randint(0, n, (n,), device="cuda", dtype=torch.int32, generator=g) for _ in range(sets)]
    for ix in idx:  # >= 10 % duplicates
        pos = torch.randint(0, n, (n // 10,), device="cuda", generator=g)
        ix[pos] = ix[(pos * 2654435761) % n]
    og = [torch.empty(n, device="cuda") for _ in range(sets)]
    ctr = [0]

    def rot(f):
        def g_():
            j = ctr[0] % sets
            ctr[0] += 1
            f(j)
        return g_

    side = 4096  # the same 16 M elements as a 4096 x 4096 tile for the 2-D ops
    x2 = [x.view(side, side) for x in xs]
    o2 = [o.view(side, side) for o in og]
    rowv = [torch.randn(side, device="cuda", generator=g) for _ in range(sets)]
    colv = [torch.empty(side, device="cuda") for _ in range(sets)]
    maskb = [torch.randint(0, 256, (n // 8,), device="cuda", dtype=torch.uint8, generator=g) for _ in range(sets)]
    bitsb = [torch.empty(n // 8, device="cuda", dtype=torch.uint8) for _ in range(sets)]
    col_ws = torch.empty(max(1, pto.lib().pto_b200_tcolreduce_workspace_bytes(side, side) // 4), device="cuda")
    cases = [
        ("TCVT f32->f16 16M elements", 6.0, rot(lambda j: pto.TCVT(xs[j], torch.float16, out=o16[j]))),
        ("TCVT f32->bf16 16M elements", 6.0, rot(lambda j: pto.TCVT(xs[j], torch.bfloat16, out=ob16[j]))),
        ("TGATHER f32 by int32 index, 16M of 16M, 10% duplicates", 12.0,
         rot(lambda j: pto.TGATHER(xs[j], idx[j], out=og[j]))),
        ("TROWEXPANDSUB f32 4096x4096", 8.0, rot(lambda j: pto.TROWEXPANDSUB(x2[j], rowv[j], out=o2[j]))),
        ("TROWMAX f32 4096x4096", 4.0, rot(lambda j: pto.TROWMAX(x2[j], out=colv[j]))),
        ("TCOLSUM f32 4096x4096", 4.0, rot(lambda j: pto.TCOLSUM(x2[j], out=colv[j], workspace=col_ws))),
        ("TTRANS f32 4096x4096", 8.0, rot(lambda j: pto.TTRANS(x2[j], out=o2[j]))),
        ("TSEL f32 16M elements, bit mask", 12.125, rot(lambda j: pto.TSEL(maskb[j], xs[j], xs[(j + 1) % sets], out=og[j]))),
        ("TCMPS f32 16M elements -> bits", 4.125, rot(lambda j: pto.TCMPS(xs[j], 0.0, 4, out=bitsb[j]))),
        ("TFILLPAD f32 4096x4096, valid 3000x3000", 4.0 * (3000 * 3000 / n) + 4.0,
         rot(lambda j: pto.TFILLPAD(x2[j], 3000, 3000, 3, out=o2[j]))),
    ]

    def bench_graph(fn, warm, iters):
        """The same loop captured once in a CUDA graph: these kernels run 13-30 us, less than the host needs for one
        call through the Python layer, so an eager loop would time the host."""
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / iters

    for name, bytes_per_elem, fn in cases:
        ms = bench_graph(fn, 2 * sets, 5 * sets)
        gbs = n * bytes_per_elem / ms / 1e6
        out.append({"workload": name, "value": gbs, "unit": "GB/s", "ms": ms,
                    "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / peaks["hbm_gbs"], "peak_kind": peak_kind,
                                 "note": f"{sets} rotating buffer sets (> L2), {5 * sets} launches replayed from one CUDA graph"}})
    # what bounds TGATHER beside its two streams: this GPU's rate of random 32-byte sectors out of a table of the same
    # size, measured with no index and no output stream (pto_b200_probe_random_reads)
    try:
        probe_ms = bench_graph(lambda: pto.probe_random_reads(xs[0], n), 2, 10)
        gather = next(r for r in out if r["workload"].startswith("TGATHER"))
        gather["roofline"]["random_read_ceiling"] = {
            "reads": n, "table_mib": 64, "us": probe_ms * 1e3, "greads_per_s": n / probe_ms / 1e6,
            "sector_gbs": n * 32 / probe_ms / 1e6,
            "note": "16M random 4-byte reads of the 64 MiB table alone; TGATHER does these plus 128 MB of index and output"}
        gather["roofline"]["frac_of_random_read_ceiling"] = probe_ms / gather["ms"]
        # the same comparison in sectors through L2: TGATHER moves the probe's sectors plus its index and output streams
        gather["roofline"]["l2_sector_gbs"] = n * (32 + 8) / gather["ms"] / 1e6
        gather["roofline"]["frac_of_ceiling_in_l2_sectors"] = (n * (32 + 8) / gather["ms"]) / (n * 32 / probe_ms)
    except Exception as exc:
        out[-1]["roofline"]["probe_note"] = str(exc)[:120]
    out.extend(tile_program_gemm(torch, peaks, peak_kind))
    return out


def tile_program_gemm(torch, peaks, peak_kind):
    """The reference's own GEMM tile program (RunGemmE2E) compiled against this repository's PTO headers, 6144^3: every
    thread executing every instruction, and with the core's pipes on warps of their own (TLOAD by the copy engine,
    TEXTRACT as views).  The libraries are built where the reference tree is available; absent, no rows."""
    import ctypes
    rows = []
    here = os.path.dirname(os.path.abspath(__file__))
    cases = (("libpto_b200_refkernels.so", "pto_refk_gemm_6144", "every thread runs every instruction"),
             ("libpto_b200_refkernels_pw.so", "pto_refk_gemm_pw_6144_k128", "pipes on warps of their own, k step 128"))
    m = n = k = 6144
    g = torch.Generator(device="cuda").manual_seed(11)
    a = (torch.rand(m, k, device="cuda", generator=g) * 2 - 1).half()
    b = (torch.rand(n, k, device="cuda", generator=g) * 2 - 1).half()
    c = torch.empty(m, n, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    for so, name, how in cases:
        path = os.path.join(here, "pto_isa_b200", so)
        if not os.path.exists(path):
            continue
        try:
            fn = getattr(ctypes.CDLL(path), name)
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            ms = bench_loop(torch, lambda: fn(ptr(c), ptr(a), ptr(b), stream, ptr(status)), 3, 10)
            if status.tolist() != [0, 0, 0, 0]:
                raise RuntimeError(f"status record {status.tolist()}")
            tf = 2.0 * m * n * k / ms / 1e9
            rows.append({"workload": f"reference GEMM tile program 6144^3 ({how})", "value": tf, "unit": "TFLOP/s", "ms": ms,
                         "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                      "frac": tf / peaks["bf16_tflops"], "peak_kind": peak_kind + " burst"}})
        except Exception as exc:  # the rows are extras: a missing or failing library must not cost the bench line
            rows.append({"workload": f"reference GEMM tile program 6144^3 ({how})", "value": None, "unit": "TFLOP/s",
                         "note": str(exc)[:160], "roofline": {"frac": None}})
    return rows


def compact_summary(line):
    """The headline figures of all three parts of the metric in a few hundred characters, placed last in the line."""
    r3 = lambda x: None if x is None else round(float(x), 3)
    r0 = lambda x: None if x is None else round(float(x), 1)
    sm = {"gemm6144_tflops": r0(line["roofline"]["achieved"]), "gemm_frac_sustained": r3(line["roofline"]["frac"]),
          "gemm_frac_burst_isolated": r3(line["roofline"].get("isolated_frac_of_burst")),
          "gemm_frac_of_cublas_sustained_same_operands": r3(line["roofline"].get("frac_of_library_sustained")),
          "gemm_best_launch": [r0(line["roofline"].get("best_single_launch_of_10_tflops")),
                               r3(line["roofline"].get("best_single_launch_frac_of_burst")),
                               r3(line["roofline"].get("best_single_launch_frac_of_library"))],
          "e2e_tflops": r0(line["e2e"]["value"])}
    sa = line.get("sharded_attention") or {}
    sm["attn_sharded_tflops"] = r0(sa.get("value"))
    if sa.get("value_with_allgather") is not None:
        sm["attn_sharded_with_allgather"] = r0(sa["value_with_allgather"])
    if sa.get("value_overlapped") is not None:
        sm["attn_overlapped_allgather_tflops"] = r0(sa["value_overlapped"])
    wa = line.get("with_allgather")
    if wa:
        sm["gemm_with_allgather_tflops"] = r0(wa["value"])
        sm["gemm_overlapped_allgather_tflops"] = r0(wa.get("value_overlapped"))
        sm["allgather_ms"] = r3(wa["allgather_ms_per_step"])
    for row in line.get("extras") or []:
        w = row["workload"]
        key = None
        if w.startswith("flash_attn_fwd"):
            key = "fa_causal" if "causal=True" in w else "fa_nc"
        elif w.startswith("TCVT f32->f16"):
            key = "tcvt_f16"
        elif w.startswith("TCVT f32->bf16"):
            key = "tcvt_bf16"
        elif w.startswith("TGATHER"):
            key = "tgather"
        elif w.startswith("gemm_f16f32 m=n=k="):
            key = "gemm" + w.split("=")[3].split(",")[0]
        elif w.startswith("reference GEMM tile program"):
            key = "tile_program_pw" if "pipes on warps" in w else "tile_program"
            if row["value"] is None:
                continue
        if key:
            sm[key] = [r0(row["value"]), r3(row["roofline"]["frac"])]
            if key.startswith("fa_") and row["roofline"].get("frac_of_library") is not None:
                sm[key].append(r3(row["roofline"]["frac_of_library"]))
            if key == "tgather" and row["roofline"].get("frac_of_random_read_ceiling") is not None:
                sm[key].append(r3(row["roofline"]["frac_of_random_read_ceiling"]))
    sm["legend"] = ("[value, frac of measured peak(, frac of vendor library | of random-read ceiling)]; gemm_best_launch: "
                    "best of 10 single launches, the method of the measured burst peak, and the same for cuBLAS at 6144^3")
    return sm


def run_gpu_arm(args):
    import torch

    import pto_isa_b200 as pto

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA kernels are the only implementation")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner (and debug lines) on stdout while the communicator is created; stdout
        # carries the one JSON line, so file descriptor 1 points at stderr until the first collective is through
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    peaks, peak_kind = load_peaks()

    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    P, R = PROBLEMS_PER_RANK, REPEATS
    a = [(torch.rand(M, K, device="cuda", generator=g) * 2 - 1).half() for _ in range(P)]
    b = [(torch.rand(N, K, device="cuda", generator=g) * 2 - 1).half() for _ in range(P)]  # n x k (Layout::DN)
    c = torch.empty(P, M, N, device="cuda")

    def one_pass():
        for i in range(P):
            pto.gemm(a[i], b[i], 1, out=c[i])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- 10 launches timed alone after a pause: the burst regime (against the measured burst peak)
    one_pass()
    barrier()
    time.sleep(1.0)
    iso_ms = bench_loop(torch, lambda: pto.gemm(a[0], b[0], 1, out=c[0]), 0, 10)

    # ---- the burst peak of MEASURED_PEAKS.json is a best of ten single launches: the same method on this kernel, and
    # on the vendor library with the same operands (fp16 output: torch offers no fp32 output for fp16 operands)
    def best_single_launch(fn, n=10):
        best = float("inf")
        for _ in range(n):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e))
        return best

    barrier()
    time.sleep(1.0)
    iso_best_ms = best_single_launch(lambda: pto.gemm(a[0], b[0], 1, out=c[0]))
    lib_best_ms = None
    if world == 1:
        try:
            bt = b[0].t()
            for _ in range(3):
                torch.matmul(a[0], bt)
            torch.cuda.synchronize()
            time.sleep(1.0)
            lib_best_ms = best_single_launch(lambda: torch.matmul(a[0], bt))
        except Exception:
            lib_best_ms = None

    for _ in range(max(args.warmup, 3)):
        for _ in range(R):
            one_pass()
    barrier()
    gpu_uuid = None
    try:
        gpu_uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        pass
    sampler = ClockSampler(local_rank, gpu_uuid) if rank == 0 else None
    if sampler:
        sampler.start()
    stamps = torch.zeros(256, 4, dtype=torch.int64, device="cuda")
    pto.set_profile_buffer(stamps)  # the last launch of the timed region leaves its per-block stamps here
    pass_events = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        for _ in range(R):
            # events around every pass of P launches on the launching stream: the roofline's kernel duration
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            one_pass()
            e.record()
            pass_events.append((s, e))
    ev1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    pto.set_profile_buffer(None)
    elapsed_ms = ev0.elapsed_time(ev1)
    if pto.device_status() != 0:
        raise SystemExit("a kernel reported a device-side wait timeout")
    t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    launches = args.steps * R * P
    total_flops = world * launches * FLOPS_PER_PROBLEM
    value = total_flops / elapsed_ms / 1e9
    per_pass = [s.elapsed_time(e) for s, e in pass_events]
    avg_launch_ms = sum(per_pass) / len(per_pass) / P
    block_stamps = stamps_summary(torch, stamps, 2 * (torch.cuda.get_device_properties(local_rank).multi_processor_count // 2))

    # the vendor library in the same regime, right after the timed region (the GPU is as warm as it was in it): the same
    # passes over the same operands through torch.matmul (cuBLAS; fp16 output, torch offers no fp32 one), as many
    # launches as half a second takes
    lib_sustained = None
    if world == 1:
        try:
            bts = [b[i].t() for i in range(P)]
            outs16 = [torch.empty(M, N, dtype=torch.float16, device="cuda") for _ in range(P)]
            for i in range(P):
                torch.matmul(a[i], bts[i], out=outs16[i])
            torch.cuda.synchronize()
            lib_passes = max(1, int(0.5 / (avg_launch_ms * P / 1e3)))
            l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0.record()
            for _ in range(lib_passes):
                for i in range(P):
                    torch.matmul(a[i], bts[i], out=outs16[i])
            l1.record()
            torch.cuda.synchronize()
            lib_ms = l0.elapsed_time(l1) / (lib_passes * P)
            # like for like: this repository's kernel with the same fp16 output (pto_b200_gemm_f16_out16), same loop
            for i in range(P):
                pto.gemm_out16(a[i], b[i], 1, out=outs16[i])
            torch.cuda.synchronize()
            l0.record()
            for _ in range(lib_passes):
                for i in range(P):
                    pto.gemm_out16(a[i], b[i], 1, out=outs16[i])
            l1.record()
            torch.cuda.synchronize()
            own16_ms = l0.elapsed_time(l1) / (lib_passes * P)
            lib_sustained = {"tflops": FLOPS_PER_PROBLEM / lib_ms / 1e9, "ms_per_launch": lib_ms,
                             "launches": lib_passes * P,
                             "note": "torch.matmul (cuBLAS), same operands, fp16 output, run right after the timed region",
                             "own_fp16_output_tflops": FLOPS_PER_PROBLEM / own16_ms / 1e9,
                             "own_fp16_output_frac_of_library": lib_ms / own16_ms}
            del bts, outs16
        except Exception as exc:
            lib_sustained = {"note": str(exc)[:160]}

    # all-gather of the outputs (every GPU ends up with every C): after the pass, and overlapped with it
    with_allgather = None
    if dist is not None:
        full = torch.empty(world * P, M, N, device="cuda")
        pass_ms = elapsed_ms / (args.steps * R)
        gathers = []
        for i in range(6):  # the first one is the warm-up (communicator set-up)
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            dist.all_gather_into_tensor(full, c)
            g1.record()
            barrier()
            tg = torch.tensor([g0.elapsed_time(g1)], device="cuda", dtype=torch.float64)
            dist.all_reduce(tg, op=dist.ReduceOp.MAX)
            if i > 0:
                gathers.append(float(tg.item()))
        ag_ms = statistics.median(gathers)
        # overlapped: problem i's output is gathered on a second stream as soon as its kernel is done, while the
        # kernels of problems i + 1 .. run; every rank's C of problem i lands at full_v[i, rank] (problem-major, so
        # that each gather writes one contiguous block and needs no staging copy)
        # Two ways to issue a problem's gather, both measured, the faster one reported: into one contiguous block
        # (full_pw[i], problem-major) with all_gather_into_tensor, or into the problem's slices of the rank-major
        # tensor with all_gather on a list (which NCCL runs as grouped broadcasts); which one wins depends on N.
        full_pw = full.view(P, world, M, N)
        full_rm = full.view(world, P, M, N)
        comm = torch.cuda.Stream()

        def overlapped_pass(block):
            works = []
            for i in range(P):
                pto.gemm(a[i], b[i], 1, out=c[i])
                done = torch.cuda.Event()
                done.record()
                comm.wait_event(done)
                with torch.cuda.stream(comm):
                    if block:
                        works.append(dist.all_gather_into_tensor(full_pw[i], c[i], async_op=True))
                    else:
                        works.append(dist.all_gather([full_rm[r, i] for r in range(world)], c[i], async_op=True))
            for w in works:
                w.wait()
            torch.cuda.current_stream().wait_stream(comm)

        overl_by = {}
        for block in (False, True):
            times = []
            for it in range(4):
                barrier()
                o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                o0.record()
                overlapped_pass(block)
                o1.record()
                barrier()
                to = torch.tensor([o0.elapsed_time(o1)], device="cuda", dtype=torch.float64)
                dist.all_reduce(to, op=dist.ReduceOp.MAX)
                if it > 0:
                    times.append(float(to.item()))
            overl_by["one block per problem" if block else "list of slices per problem"] = times
        strategy = min(overl_by, key=lambda k_: statistics.median(overl_by[k_]))
        overl = overl_by[strategy]
        ov_ms = statistics.median(overl)
        nbytes = int(world * P * M * N * 4)
        with_allgather = {"allgather_ms_per_step": ag_ms, "allgather_ms_all": gathers, "bytes_gathered_per_gpu": nbytes,
                          "allgather_recv_gbs_per_gpu": nbytes * (world - 1) / world / ag_ms / 1e6,
                          "nvlink_per_direction_gbs": {"measured_peer_copy": 770.0, "nominal": 900.0},
                          "compute_ms_per_pass": pass_ms,
                          "value": world * P * FLOPS_PER_PROBLEM / (pass_ms + ag_ms) / 1e9,
                          "overlapped_ms_per_pass": ov_ms, "overlapped_ms_all": overl, "overlapped_gather": strategy,
                          "overlapped_ms_by_gather": {k_: statistics.median(v_) for k_, v_ in overl_by.items()},
                          "value_overlapped": world * P * FLOPS_PER_PROBLEM / ov_ms / 1e9, "unit": "TFLOP/s",
                          "limiter": "the gather moves 4 bytes of C per 12288 FLOP; at N GPUs every GPU receives "
                                     "(N-1)/N of N x 1.2 GB over its NVLink receive direction",
                          "note": "a pass = the 8 problems of one GPU once; overlapped = each problem's gather issued "
                                  "on a second stream as soon as its kernel finishes"}
        del full, full_pw, full_rm

    # multi-head attention of the sharding config (batch 32 x 32 heads, S 8192, D 128, causal, fp16 O): the 1024
    # heads are split over the ranks (fixed total work: strong scaling), then every rank gathers all outputs
    sharded_attn = sharded_attention(torch, pto, dist, world, rank, barrier)

    # end to end through the C ABI's host-buffer entry point: a pass's P problems in pinned host memory go through
    # pto_b200_gemm_f16f32_host_batched (copy in, kernel and copy out of consecutive problems overlap)
    e2e_steps = 5
    ha = torch.empty(P, M, K, dtype=torch.float16).pin_memory()
    hb = torch.empty(P, N, K, dtype=torch.float16).pin_memory()
    hc = torch.empty(P, M, N, dtype=torch.float32).pin_memory()
    for i in range(P):
        ha[i].copy_(a[i])
        hb[i].copy_(b[i])
    pto.gemm_host_batched(ha[:2], hb[:2], hc[:2], 1)  # warm-up: staging buffers are allocated on first use
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        pto.gemm_host_batched(ha, hb, hc, 1)
    e2e_s = time.perf_counter() - t0
    te = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te.item())
    e2e_value = world * e2e_steps * P * FLOPS_PER_PROBLEM / e2e_s / 1e12
    e2e_check = bool(torch.equal(hc[P - 1].cuda(), c[P - 1]))  # host path of the last problem equals its device path
    h2d_bytes, d2h_bytes = int(P * (M * K + N * K) * 2), int(P * M * N * 4)
    e2e_host_gbs = world * e2e_steps * (h2d_bytes + d2h_bytes) / e2e_s / 1e9
    del ha, hb, hc

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    achieved = FLOPS_PER_PROBLEM / avg_launch_ms / 1e9
    timed_s = elapsed_ms / 1e3
    # the sustained figure is the denominator of a region that lasts about a second or more; a shorter one is burst
    peak = peaks["bf16_tflops_sustained"] if timed_s >= 0.8 else peaks["bf16_tflops"]
    iso_tf = FLOPS_PER_PROBLEM / iso_ms / 1e9
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                "peak_kind": f"{peak_kind} cuBLAS bf16 8192^3, " + ("sustained loop" if timed_s >= 0.8 else "burst") +
                             f" (the timed region lasts {timed_s:.2f} s)",
                "frac_of_burst": achieved / peaks["bf16_tflops"],
                "frac_of_nominal_2250": achieved / 2250.0, "kernel": "gemm2_f16f32_kernel<1, 256>",
                "avg_launch_ms": avg_launch_ms, "algorithmic_flops_per_launch": FLOPS_PER_PROBLEM,
                "isolated_10_launches_tflops": iso_tf, "isolated_frac_of_burst": iso_tf / peaks["bf16_tflops"],
                "best_single_launch_of_10_tflops": FLOPS_PER_PROBLEM / iso_best_ms / 1e9,
                "best_single_launch_frac_of_burst": FLOPS_PER_PROBLEM / iso_best_ms / 1e9 / peaks["bf16_tflops"],
                "library_best_single_launch_of_10_tflops": (FLOPS_PER_PROBLEM / lib_best_ms / 1e9) if lib_best_ms else None,
                "best_single_launch_frac_of_library": (lib_best_ms / iso_best_ms) if lib_best_ms else None,
                "library_note": "torch.matmul (cuBLAS) on the same fp16 operands with fp16 output, same method, same process",
                "library_sustained": lib_sustained,
                "frac_of_library_sustained": (achieved / lib_sustained["tflops"]) if lib_sustained and lib_sustained.get("tflops") else None,
                "block_stamps_last_launch": block_stamps,
                "tflops_per_ghz": (achieved / (block_stamps["sm_mhz_median"] / 1e3)) if block_stamps else None}
    cpu = None
    extra = None
    if world == 1:
        cpu_tf, info = cpu_gemm_sample(12.0)
        cpu = {"value": cpu_tf, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
               "sample": info["sample"]}
        try:
            cpu["others"] = cpu_vector_and_attention_baselines()
        except Exception as exc:
            cpu["others_note"] = str(exc)[:160]
        extra = extras(torch, pto, peaks, peak_kind)
    line = {
        "metric": "fp16 GEMM TFLOPS (m=n=k=6144, fp32 accumulate and output)", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"gemm_f16f32 m=n=k=6144, {P} independent problems per GPU ({world * P} in total), "
                               f"a step = {R} passes over them ({R * P} launches per GPU), B stored n x k "
                               "(Layout::DN), uniform[-1,1) seeded",
                   "repeats_per_step": R, "timed_region_s": timed_s,
                   "l2": "each pass reads 1.2 GB of distinct operands per GPU (> 126 MB L2)",
                   "parallelism": f"{world} GPU(s), problems sharded, no data-path collective"},
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": d2h_bytes, "steps": e2e_steps, "matches_device_path": e2e_check,
                "host_gbs_both_directions": e2e_host_gbs,
                "limiter": "host <-> device copies: 12 bytes cross PCIe per 12288 FLOP; all ranks share the host's "
                           "memory and PCIe root ports",
                "api": "pto_b200_gemm_f16f32_host_batched (C ABI, pinned host buffers, copies overlapped with kernels); "
                       "an e2e step = one pass over the 8 problems"},
        "gpu_launches": launches, "with_allgather": with_allgather, "sharded_attention": sharded_attn,
        "extras": extra,
    }
    line["summary"] = compact_summary(line)
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
