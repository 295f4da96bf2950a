#!/usr/bin/env python
"""Benchmark of the int8-quantised linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the four CPM-Bee-10B layer linears at M = 4096 tokens (fused QKV 12288x4096, attention-out 4096x4096, FFN-in
10240x4096, FFN-out 4096x10240), fp16 activations N(0,1) and weights N(0,0.02), seeded synthetic data.  One step = one
pass over the four linears; like the reference's bmm, every call quantises BOTH operands (per-row absmax scale + int8
rounding), runs the int8 GEMM and dequantises to fp16: two kernels per linear, eight per step.  ``value`` counts
2*M*N*K operations of the four GEMMs over the whole step time (quantisation passes included), inputs resident in HBM.

N = 1: the public entry point ``cpm_kernels_b200.torch.bmm(x, False, W, True, int8=True)``.
N > 1 (torchrun, one rank per GPU): the same linears column-parallel ("strong" scaling) -- each rank holds N/g rows of
every weight, computes its output columns, and the GEMM's epilogue stores them into every rank's full-width result over
NVLink (``cpm_kernels_b200.sharded``); after the timed region every rank recomputes the unsharded linears and compares
bit for bit (``parity``).

``e2e`` drives the same step from pinned host buffers, copies inside the timed region.  At N > 1 every rank owns M/g
tokens end to end: it uploads its rows, quantises them once (the quantising kernel stores the int8 codes into every
rank's buffer), and downloads its rows of the results.

Beside them in the same line: ``roofline`` (the GEMM kernel alone, CUDA events around its launches), ``cfg5`` (the 48-layer
stack at M = 16384: GEMM-phase rate, end-to-end rate with the exchange, NVLink GB/s), ``sustained`` (the step looped for
two seconds with the clock sampled), ``reference_cuda`` (the reference's own six-launch CUDA pipeline, timed in the same
process on the same tensors), ``cpu_baseline`` (the reference's test formula on the host cores, the whole workload),
``gemv`` (decode GEMV GB/s) and ``other_configs``.

``--impl reference`` times the reference's own arithmetic on the host CPU: the torch expressions its unit tests
hold the kernels to (oracle/test_formula.py), on the same workload, with all host threads.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_TOKENS = 4096
SHAPES = [("qkv", 12288, 4096), ("attn_out", 4096, 4096), ("ffn_in", 10240, 4096), ("ffn_out", 4096, 10240)]  # (name, N, K)
METRIC = "int8_linear_tops"
UNIT = "TOPS"
WORKLOAD = "cpm-bee-10b layer linears (qkv 12288x4096, attn-out 4096x4096, ffn-in 10240x4096, ffn-out 4096x10240), M=4096 tokens, int8"


def total_ops(m_tokens: int | None = None) -> float:
    m_tokens = M_TOKENS if m_tokens is None else m_tokens
    return float(sum(2 * m_tokens * n * k for _, n, k in SHAPES))


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# clocks during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.strip().split(", ") for r in open(self.path).read().strip().splitlines() if r.strip()]
            os.unlink(self.path)
        except Exception:
            return out
        sm, reasons, smax = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax = float(r[2])
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            # the GPU idles between samples of a short run: the clock under load is the upper half of the samples
            sm_sorted = sorted(sm)
            out["sm_mhz"] = statistics.median(sm_sorted[len(sm_sorted) // 2:])
        out["sm_max_mhz"] = smax
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


# ------------------------------------------------------------------------------------------------
# DRAM traffic of the dominant kernel, from the tracked record of the profiler capture it came from
# ------------------------------------------------------------------------------------------------
TRAFFIC_RECORD = os.path.join(ROOT, "profiles", "gemm_i8_tc2_kernel_cpm-bee-linears_M4096.dram_traffic.txt")


def read_dram_traffic() -> dict:
    """``{"bytes_per_launch": mean over the four GEMM launches, "per_shape": {...}, "captured": ..., "source": file}`` from
    the record beside the profile summary; ``None`` values when the record is missing or does not parse (never a
    built-in number)."""
    out = {"bytes_per_launch": None, "per_shape": None, "captured": None, "source": os.path.relpath(TRAFFIC_RECORD, ROOT)}
    try:
        fields = {}
        for line in open(TRAFFIC_RECORD):
            if ":" in line and not line.lstrip().startswith("#"):
                key, val = line.split(":", 1)
                fields[key.strip()] = val.strip()
        per = {}
        for item in fields["dram_bytes_per_launch"].split():
            name, val = item.split("=")
            per[name] = float(val)
        if sorted(per) == sorted(name for name, _, _ in SHAPES):
            out["per_shape"] = per
            out["bytes_per_launch"] = sum(per.values()) / len(per)
            out["captured"] = fields.get("captured")
    except Exception:
        pass
    return out


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's test formula on host cores
# ------------------------------------------------------------------------------------------------
def cpu_baseline(passes: int = 2, tokens: int | None = None) -> dict:
    """The four linears at ``tokens`` (default: the workload's) through the reference's test formula in torch CPU
    fp32 on all host cores; one warm-up pass, then the MEAN of ``passes`` passes (the statistic of the measured arm)."""
    import torch
    from oracle import test_formula
    tokens = M_TOKENS if tokens is None else tokens
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator(device="cpu").manual_seed(0)
    data = []
    for _, n, k in SHAPES:
        x = torch.randn((1, tokens, k), generator=g).half()
        w = (torch.randn((1, n, k), generator=g) * 0.02).half()
        data.append((x, w))
    times = []
    for _ in range(passes + 1):                       # first pass is the warm-up
        t0 = time.perf_counter()
        for x, w in data:
            test_formula.real_bmm(x, False, w, True, True)
        times.append(time.perf_counter() - t0)
    mean = sum(times[1:]) / len(times[1:])
    return {"value": total_ops(tokens) / mean / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "the whole workload: the same four linears at M=%d tokens, reference test formula (tests/test_gemm.py:8-41) "
                      "in torch CPU fp32, mean of %d passes after one warm-up, %.2f s per pass" % (tokens, passes, mean),
            "seconds_per_pass": mean, "tokens": tokens}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(passes=max(1, min(args.steps, 3)), tokens=M_TOKENS)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": base["seconds_per_pass"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(), "tokens": M_TOKENS},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_name() -> str:
    return WORKLOAD if M_TOKENS == 4096 else WORKLOAD + " [REDUCED to %d tokens: profiling case, not a bench value]" % M_TOKENS


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def bind_to_gpu_cpus(gpu_index: int):
    """Run this process on the CPU cores next to its GPU (NVML's CPU affinity of the device, read only), so that the
    pinned host buffers of the end-to-end leg are allocated on that NUMA node and its copies do not cross sockets.
    Returns the number of cores bound to, or None when NVML or the cpuset does not allow it (nothing is changed then)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


class Run:
    """Process-wide state of one benchmark run: device, ranks, streams, timing helpers."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.all_cpus = os.sched_getaffinity(0)
        # (several ranks: for the whole run; one rank: only around its end-to-end leg, its CPU-baseline leg uses every core)
        self.cpu_affinity = bind_to_gpu_cpus(self.local_rank) if self.world > 1 else None
        self.saved_stdout = None
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # libraries print banners on stdout when a communicator is created: keep stdout for the one JSON line
            sys.stdout.flush()
            self.saved_stdout = os.dup(1)
            os.dup2(2, 1)
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream()
        self.peaks = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return float(value)
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, value: int) -> int:
        if self.world == 1:
            return int(value)
        t = self.torch.tensor([value], device=self.dev, dtype=self.torch.int64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return int(t.item())

    def timed(self, fn, iters: int, warm: int = 0) -> float:
        """Milliseconds per call of ``fn`` over ``iters`` calls: CUDA events on the main stream between two rank
        barriers, max over ranks."""
        for _ in range(warm):
            fn()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record(self.stream)
        for _ in range(iters):
            fn()
        e1.record(self.stream)
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1) / iters)

    def emit(self, line: dict):
        if self.saved_stdout is not None:
            sys.stdout.flush()
            os.dup2(self.saved_stdout, 1)
            os.close(self.saved_stdout)
            self.saved_stdout = None
        print(json.dumps(line), flush=True)


SLOTS = 3          # result buffers per linear shape that the sharded steps rotate through


class Lanes:
    """How the sharded steps are issued.  The linears of the synthetic stack are independent, so linear i runs on lane
    (stream) i % n: while one linear's GEMM drains its output over NVLink, the others' quantisation passes and GEMMs run
    beside it (the scattering GEMM's persistent grid leaves `sm_margin` SMs free for that).  The main stream only joins
    the lanes and runs the rank barrier of each step.  Steps are pipelined: step s writes result buffer s % 3, whose
    previous contents (step s-3) every rank has finished with once the barrier of step s-2 has passed, so the lanes of
    step s wait for THAT barrier, not for the latest one -- the link keeps draining step s-1 while step s computes."""

    def __init__(self, run: Run, n_lanes: int, sm_margin: int, arena):
        from cpm_kernels_b200.library import cpmk
        torch = run.torch
        self.run, self.cpmk, self.arena = run, cpmk, arena
        self.sm_margin = sm_margin if n_lanes > 1 else 0
        self.streams = [torch.cuda.Stream() for _ in range(max(1, n_lanes))]
        for s in self.streams:
            s.wait_stream(run.stream)
        self.count = 0                       # steps issued so far
        self.passed = {}                     # step -> event recorded on the main stream after that step's barrier
        self.margin(True)

    def __len__(self):
        return len(self.streams)

    def margin(self, on: bool):
        self.cpmk.set_gemm_sm_margin(self.sm_margin if on and self.sm_margin > 0 else -1)

    def slot(self) -> int:
        return self.count % SLOTS

    def run_step(self, work, barrier: bool = True):
        """work: one callable per linear, called as work[i](slot) under lane i's stream.  Returns their results."""
        torch, main = self.run.torch, self.run.stream
        slot, gate = self.slot(), self.passed.get(self.count - (SLOTS - 1))
        out = [None] * len(work)
        used = set()
        for i, fn in enumerate(work):
            lane = self.streams[i % len(self.streams)]
            with torch.cuda.stream(lane):
                if gate is not None and lane not in used:
                    lane.wait_event(gate)
                used.add(lane)
                out[i] = fn(slot)
        for lane in used:
            main.wait_stream(lane)
        if barrier:
            self.arena.barrier(1)            # every rank's stores of this step have landed
            ev = torch.cuda.Event()
            ev.record(main)
            self.passed[self.count] = ev
            self.passed.pop(self.count - SLOTS, None)
        self.count += 1
        return out

    def run_after_main(self, work):
        """work[i]() under lane i's stream, all lanes ordered after the main stream's work so far; the main stream
        then waits for the lanes (no barrier, no pipelining)."""
        torch, main = self.run.torch, self.run.stream
        out, used = [None] * len(work), set()
        for i, fn in enumerate(work):
            lane = self.streams[i % len(self.streams)]
            with torch.cuda.stream(lane):
                if lane not in used:
                    lane.wait_stream(main)
                used.add(lane)
                out[i] = fn()
        for lane in used:
            main.wait_stream(lane)
        return out

    def drain(self):
        """Order the lanes after everything issued so far on the main stream (used between measurements)."""
        for s in self.streams:
            s.wait_stream(self.run.stream)
        self.passed.clear()


def cfg2_tensors(run: Run, want_full_weights: bool = False):
    """Activations (1, M, K) for the four linears, on every rank, and either this rank's rows of each weight or (for
    the parity check) the full weights: the same device generator sequence in both cases."""
    torch = run.torch
    from cpm_kernels_b200.sharded import shard_bounds
    gen = torch.Generator(device=run.dev).manual_seed(0)
    xs, ws = [], []
    for _, n, k in SHAPES:
        assert n % run.world == 0
        x = torch.randn((1, M_TOKENS, k), generator=gen, device=run.dev).half()
        w_full = (torch.randn((1, n, k), generator=gen, device=run.dev) * 0.02).half()
        if want_full_weights:
            ws.append(w_full)
        else:
            xs.append(x)
            lo, hi = shard_bounds(n, run.world, run.rank)
            ws.append(w_full[:, lo:hi, :].contiguous())
        del w_full
    return xs, ws, gen


def count_mismatches(torch, got, want) -> int:
    return int((got.view(torch.int16) != want.view(torch.int16)).sum().item())


def run_ours(args) -> None:
    run = Run(args)
    torch, dist = run.torch, run.dist
    import cpm_kernels_b200.torch as ct
    import cpm_kernels_b200.kernels as ck
    from cpm_kernels_b200.library import cpmk
    from cpm_kernels_b200.sharded import (ColumnParallelInt8Linear, FusedColumnParallelInt8Linear, SymmetricArena, ExchangeBuffers)
    from cpm_kernels_b200.torch.gemm import quantize, gemm_and_scale

    world, rank, dev, stream, peaks = run.world, run.rank, run.dev, run.stream, run.peaks
    cpmk.check_device()
    xs, ws, gen = cfg2_tensors(run)
    warmup = max(args.warmup, 3)

    # ---- N > 1: peer-mapped buffers and the layers whose GEMM epilogue is the all-gather ----
    arena = layers = lanes = None
    use_multicast = False
    nccl_layers, gathered, comm_stream = None, [], None
    exchange = "none"
    want_cfg5 = not args.kernels_only and not args.no_cfg5 and M_TOKENS == 4096
    if world > 1:
        nbytes = sum(ExchangeBuffers.nbytes(M_TOKENS, k, n, SLOTS) for _, n, k in SHAPES)
        if want_cfg5:
            nbytes += sum(ExchangeBuffers.nbytes(CFG5_TOKENS, k, n, SLOTS) for _, n, k in SHAPES)
        arena = SymmetricArena(nbytes + (1 << 20), dev)
        bufs = [ExchangeBuffers(arena, M_TOKENS, k, n, SLOTS) for _, n, k in SHAPES]
        layers = [FusedColumnParallelInt8Linear(w, buffers=b) for w, b in zip(ws, bufs)]
        n_lanes = int(os.environ.get("CPMK_BENCH_FUSED_STREAMS", "4")) if args.exchange != "fused1" else 1
        lanes = Lanes(run, n_lanes, int(os.environ.get("CPMK_BENCH_FUSED_SM_MARGIN", "32")), arena)
        exchange = ("fused: the GEMM epilogue TMA-stores its output columns into every rank's full-width result over NVLink; activations present "
                    "on every rank; linears on %d streams, scattering GEMM grids leave %d SMs free; one rank barrier per step; results rotate "
                    "through %d buffers, so a step's exchange drains while the next step computes" % (len(lanes), lanes.sm_margin, SLOTS))
        from cpm_kernels_b200.sharded import recommended_forward_sms
        forward_sms = int(os.environ["CPMK_GEMM_FORWARD_SMS"]) if "CPMK_GEMM_FORWARD_SMS" in os.environ else recommended_forward_sms(world)
        cpmk.set_gemm_forward_sms(forward_sms)
        if forward_sms > 0:
            exchange = exchange.replace("the GEMM epilogue TMA-stores its output columns into every rank's full-width result over NVLink",
                                        "the GEMM's computing CTAs store their output columns into this rank's result and %d SMs of the same grid forward "
                                        "each finished tile into every other rank's result over NVLink" % forward_sms)
        use_multicast = args.exchange == "multicast" and arena.multicast_base != 0
        if use_multicast:
            exchange = exchange.replace("fused: the GEMM epilogue TMA-stores its output columns into every rank's full-width result over NVLink",
                                        "multicast: forwarding CTAs of the GEMM's grid send each finished tile once, with multimem stores that the NVLink switch replicates into every rank's result")
        if args.exchange == "nccl":
            nccl_layers = [ColumnParallelInt8Linear(w) for w in ws]
            gathered = [torch.empty((world, M_TOKENS, n // world), dtype=torch.half, device=dev) for _, n, _ in SHAPES]
            comm_stream = torch.cuda.Stream()
            os.environ.setdefault("CPMK_GEMM_SM_MARGIN", "16")       # the collective's kernels run beside the persistent GEMM grid
            exchange = "nccl all_gather_into_tensor on a side stream"

    def step(only_local: bool = False):
        """One pass over the four linears.  N = 1: the public bmm.  N > 1: one library call per linear (quantise both
        operands + scattering GEMM), one rank barrier per step.  only_local: the same without the exchange."""
        if world == 1:
            return [ct.bmm(x, False, w, True, int8=True) for x, w in zip(xs, ws)]
        if nccl_layers is not None:
            out = []
            for i, (x, w) in enumerate(zip(xs, ws)):
                y = ct.bmm(x, False, w, True, int8=True)
                if not only_local:
                    ev = torch.cuda.Event()
                    ev.record(stream)
                    with torch.cuda.stream(comm_stream):
                        comm_stream.wait_event(ev)
                        nccl_layers[i].gather(y, out=gathered[i])
                    y.record_stream(comm_stream)
                out.append(y)
            if not only_local:
                stream.wait_stream(comm_stream)
            return out
        return lanes.run_step([(lambda slot, layer=layer, x=x: layer.launch(x, slot, only_local, multicast=use_multicast)) for layer, x in zip(layers, xs)],
                              barrier=not only_local)

    for _ in range(warmup):
        step()
    run.barrier()
    assert cpmk.last_gemm_path() == 1, "the tensor-core GEMM kernel was not selected"

    # ---- timed region: exactly K steps, device time, max over ranks ----
    sampler = ClockSampler(run.local_rank)
    if rank == 0:
        sampler.start()
    ms_per_step = run.timed(step, args.steps)
    value = total_ops() / (ms_per_step * 1e-3) / 1e12

    # ---- the GEMM kernel alone: events around each GEMM launch of the same step (at N > 1 with the scatter to every rank
    #      active, on one stream, one barrier per step) ----
    gemm_events = []

    def step_recorded():
        slot = 0
        for i, (x, w) in enumerate(zip(xs, ws)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if world == 1 or nccl_layers is not None:
                sa, qa = quantize(x, False)
                sb, qb = quantize(w, False)
                e0.record(stream)
                gemm_and_scale(qa, sa, qb, sb, False, True)
                e1.record(stream)
            else:
                layer, buf = layers[i], layers[i].buffers
                ck.gemm_quantize_rows_pair(1, M_TOKENS, x.data_ptr(), buf.sx[slot].data_ptr(), buf.qx[slot].data_ptr(), 1, layer.n_local,
                                           w.data_ptr(), layer.scale_w.data_ptr(), layer.q_w.data_ptr(), layer.k, stream.cuda_stream)
                e0.record(stream)
                layer.gemm(M_TOKENS, slot)
                e1.record(stream)
            gemm_events.append((i, e0, e1))
        if layers is not None and nccl_layers is None:
            arena.barrier(1)

    if lanes is not None:
        run.barrier()
        lanes.margin(False)
    for _ in range(args.steps):
        step_recorded()
    run.barrier()
    if lanes is not None:
        lanes.drain()
        lanes.margin(True)
    clocks = sampler.stop() if rank == 0 else None

    phases = None
    if world > 1:
        ms_compute = run.timed(lambda: step(only_local=True), args.steps, warm=1)
        gather_bytes = sum(2 * M_TOKENS * n for _, n, _ in SHAPES) * (world - 1) // world
        phases = {"compute_only_ms_per_step": ms_compute, "compute_only_tops": total_ops() / (ms_compute * 1e-3) / 1e12,
                  "allgather_bytes_received_per_rank_per_step": gather_bytes,
                  "nvlink_ingress_GBps_per_rank": gather_bytes / (ms_per_step * 1e-3) / 1e9, "nvlink_nominal_GBps": 900.0,
                  "note": "the all-gather of fp16 outputs moves (g-1)/g * 2*M*N bytes into every rank per linear and bounds the step for g >= 2"}

    per_shape_ms = {}
    for i, a, b in gemm_events:
        per_shape_ms.setdefault(i, []).append(a.elapsed_time(b))
    gemm_ms = sum(statistics.mean(v) for v in per_shape_ms.values())
    gemm_tops = total_ops() / world / (gemm_ms * 1e-3) / 1e12
    peak_tops = 2.0 * peaks["bf16_tflops"]
    traffic = read_dram_traffic()
    roofline = {
        "bound": "tensor", "achieved": gemm_tops, "peak": peak_tops, "unit": "TOPS", "frac": gemm_tops / peak_tops,
        "traffic": traffic["bytes_per_launch"] if (world == 1 and M_TOKENS == 4096) else None,
        "traffic_record": {k: traffic[k] for k in ("source", "captured", "per_shape")},
        "kernel": "gemm_i8_tc2_kernel<dequant> (tcgen05.mma cta_group::2 kind::i8, 256x256 tiles per CTA pair)",
        "timed": "CUDA events around each GEMM launch of the step" + ("" if world == 1 else
                 ("; exchange on: the epilogue stores to all %d ranks, one stream" % world if nccl_layers is None else "; exchange off (NCCL gathers afterwards)")),
        "peak_note": "2 x %s dense bf16 %s TFLOP/s (burst; no int8 figure is measured on this pool); nominal dense int8 is 4500 TOPS: frac_nominal below"
                     % (peaks["source"], peaks["bf16_tflops"]),
        "frac_nominal": gemm_tops / 4500.0,
        "per_shape_tops": {SHAPES[i][0]: 2.0 * M_TOKENS * (SHAPES[i][1] // world) * SHAPES[i][2] / (statistics.mean(v) * 1e-3) / 1e12
                           for i, v in sorted(per_shape_ms.items())},
    }

    # ---- parity of the sharded path, outside the timed region: every rank recomputes the unsharded linears locally and
    #      compares its full-width results (which the peers' epilogues wrote) bit for bit ----
    parity = {"checked": False, "note": "one GPU: nothing is exchanged; parity is the GPU test suite's job"}
    if world > 1 and nccl_layers is None:
        _, w_full, _ = cfg2_tensors(run, want_full_weights=True)
        ys = step()
        run.barrier()
        bad = 0
        for i in range(len(SHAPES)):
            want = ct.bmm(xs[i], False, w_full[i], True, int8=True)
            bad += count_mismatches(torch, ys[i], want)
            del want
        parity = {"checked": True, "mismatches": run.sum_over_ranks(bad), "elements_compared_per_rank": sum(M_TOKENS * n for _, n, _ in SHAPES),
                  "what": "full-width y of the four linears on every rank (activations present in full) against the unsharded bmm computed locally"}

    # ---- e2e: pinned host activations in, fp16 outputs out, every step ----
    e2e = None
    if not args.kernels_only:
        if world == 1 or nccl_layers is not None:
            e2e = measure_e2e_single(run, xs, ws, ct)
        else:
            e2e = measure_e2e_sharded(run, xs, layers, lanes, arena)
            if parity.get("checked"):
                # the e2e path is the other form of the layer (row-sharded activations, codes gathered by the quantiser's stores)
                bad = 0
                lo, hi = rank * (M_TOKENS // world), (rank + 1) * (M_TOKENS // world)
                for i in range(len(SHAPES)):
                    want = ct.bmm(xs[i], False, w_full[i], True, int8=True)[:, lo:hi, :].cpu()
                    bad += count_mismatches(torch, e2e["_host_y"][i], want)
                parity["e2e_mismatches"] = run.sum_over_ranks(bad)
                parity["e2e_what"] = "each rank's downloaded rows of y (row-sharded activations, int8 codes all-gathered by the quantising kernel) against the unsharded bmm"
            e2e.pop("_host_y", None)
    if world > 1 and nccl_layers is None:
        del w_full

    # ---- N = 1 extras: sustained run, the reference's CUDA pipeline, decode GEMV, the other configurations ----
    sustained = reference_cuda = gemv = other = None
    if rank == 0 and world == 1 and not args.kernels_only:
        sustained = measure_sustained(run, step, xs, ws, ms_per_step)
        reference_cuda = measure_reference_cuda(run, xs, ws, ct, ms_per_step, roofline["per_shape_tops"])
    if rank == 0 and not args.kernels_only:
        gemv = measure_gemv(run, gen, ck)
    if rank == 0 and world == 1 and not args.kernels_only:
        other = measure_other_configs(("attention", "prequantised", "transposed", "fp16", "passes"), dev, gen, stream, peaks, xs, ws)

    # ---- configuration 5: the 48-layer stack at M = 16384 ----
    cfg5 = None
    if want_cfg5 and nccl_layers is None:
        del xs, ws
        torch.cuda.empty_cache()
        cfg5 = measure_cfg5(run, arena, lanes, ct)

    status = cpmk.read_status()
    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    os.sched_setaffinity(0, run.all_cpus)            # the CPU arm uses every core the process may use
    base = cpu_baseline() if (world == 1 and not args.kernels_only) else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name(), "tokens": M_TOKENS,
                   "parallelism": "column-parallel x%d; exchange = %s" % (world, exchange) if world > 1 else "single GPU",
                   "l2": "per-step working set (fp16 weights 302 MB + activations 134 MB + outputs 252 MB) exceeds the 126 MB L2; no explicit flush",
                   "weights": "re-quantised on every call, as the reference's bmm does"},
        "roofline": roofline, "e2e": e2e, "gpu_launches": 8 * args.steps, "clocks": clocks, "parity": parity,
        "host": {"cpu_cores_bound_next_to_gpu": run.cpu_affinity},
        "cfg5": cfg5, "sustained": sustained, "reference_cuda": reference_cuda,
        "gemv": gemv, "other_configs": other, "phases": phases, "device_status_word": status,
        "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained", "source")},
    }
    if base is not None:
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    run.emit(line)
    if world > 1:
        dist.destroy_process_group()


def measure_e2e_single(run: Run, xs, ws, ct) -> dict:
    """One GPU (or the NCCL variant): the public bmm from pinned host activations to pinned host results, three-stage
    pipeline upload(i+1) || compute(i) || download(i-1)."""
    torch, stream, args = run.torch, run.stream, run.args
    # one rank: run on the cores next to the GPU while the pinned buffers are allocated (first touch puts them on that
    # NUMA node) and the steps are issued; every core is given back before the CPU-baseline leg (several ranks are
    # bound for the whole run)
    bound_here = run.world == 1 and run.cpu_affinity is None
    if bound_here:
        run.cpu_affinity = bind_to_gpu_cpus(run.local_rank)
    try:
        return _measure_e2e_single(run, xs, ws, ct)
    finally:
        if bound_here:
            os.sched_setaffinity(0, run.all_cpus)


def _measure_e2e_single(run: Run, xs, ws, ct) -> dict:
    torch, stream, args = run.torch, run.stream, run.args
    host_x = [x.cpu().pin_memory() for x in xs]
    host_y = [torch.empty((1, M_TOKENS, w.shape[1]), dtype=torch.half).pin_memory() for w in ws]
    h2d = sum(t.numel() * 2 for t in host_x)
    d2h = sum(t.numel() * 2 for t in host_y)
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    # two sets of device input buffers: the uploads of step s+1 run while step s still computes and downloads
    # (PCIe is full duplex), and wait only for the compute of step s-1, which read the set they overwrite
    dev_x = [[torch.empty_like(x) for x in xs] for _ in range(2)]
    consumed = [None, None]                      # per buffer set: event after the last GEMM that read it
    step_no = [0]

    def e2e_step():
        cur = step_no[0] & 1
        step_no[0] += 1
        ups = []
        with torch.cuda.stream(copy_in):
            if consumed[cur] is not None:
                copy_in.wait_event(consumed[cur])
            for i in range(len(SHAPES)):
                dev_x[cur][i].copy_(host_x[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                ups.append(ev)
        done = None
        for i in range(len(SHAPES)):
            stream.wait_event(ups[i])
            y = ct.bmm(dev_x[cur][i], False, ws[i], True, int8=True)
            done = torch.cuda.Event()
            done.record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                host_y[i].copy_(y, non_blocking=True)
            y.record_stream(copy_out)
        consumed[cur] = done

    for _ in range(2):
        e2e_step()
    run.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(3, min(args.steps, 10))
    a.record(stream)
    copy_in.wait_event(a)                         # nothing of the timed steps starts before the first event
    for _ in range(n_e2e):
        e2e_step()
    stream.wait_stream(copy_out)                  # the last step's results have reached the host
    b.record(stream)
    run.barrier()
    ms_e2e = run.max_over_ranks(a.elapsed_time(b) / n_e2e)
    return {"value": total_ops() / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d * run.world, "d2h_bytes_per_step": d2h * run.world,
            "ms_per_step": ms_e2e, "steps": n_e2e,
            "note": "activations uploaded from pinned host memory and fp16 outputs downloaded every step, copies pipelined against compute on "
                    "separate streams; weights stay resident"}


def measure_e2e_sharded(run: Run, xs, layers, lanes, arena) -> dict:
    """N > 1.  Every rank owns M/g tokens end to end: it uploads only its rows of the activations, quantises them once
    -- the quantising kernel stores codes and scales into every rank's code buffer over NVLink, 1 byte per element --
    runs its columns of the four GEMMs on the gathered codes (epilogue stores into every rank's y), and downloads its
    M/g rows of the full-width results.  Per step: 4 uploads, 4 quantise launches, barrier, 4 GEMM launches, barrier,
    4 downloads; two buffer sets, so upload(s+1) || compute(s) || download(s-1)."""
    torch, stream, args, world, rank = run.torch, run.stream, run.args, run.world, run.rank
    rows = M_TOKENS // world
    lo, hi = rank * rows, (rank + 1) * rows
    host_x = [x[:, lo:hi, :].contiguous().cpu().pin_memory() for x in xs]
    host_y = [torch.empty((1, rows, layer.n_total), dtype=torch.half).pin_memory() for layer in layers]
    h2d = sum(t.numel() * 2 for t in host_x)
    d2h = sum(t.numel() * 2 for t in host_y)
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_x = [[torch.empty((1, rows, x.size(2)), dtype=torch.half, device=run.dev) for x in xs] for _ in range(2)]
    consumed = [None, None]                      # per set: the quantisation that read dev_x[set] has run
    downloaded = [None, None]                    # per set: the download that read y[set] has run
    step_no = [0]

    def e2e_step():
        cur = step_no[0] & 1
        step_no[0] += 1
        ups = []
        with torch.cuda.stream(copy_in):
            if consumed[cur] is not None:
                copy_in.wait_event(consumed[cur])
            for i in range(len(SHAPES)):
                dev_x[cur][i].copy_(host_x[i], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                ups.append(ev)
        for i, layer in enumerate(layers):
            stream.wait_event(ups[i])
            layer.quantize_shard(dev_x[cur][i], cur, M_TOKENS)
        consumed[cur] = torch.cuda.Event()
        consumed[cur].record(stream)
        if downloaded[cur] is not None:
            stream.wait_event(downloaded[cur])    # peers overwrite y[cur] after the next barrier: our download of it must be over
        arena.barrier(0)                          # every rank's codes have landed; every rank is done with y[cur]
        ys = lanes.run_after_main([(lambda layer=layer: layer.gemm(M_TOKENS, cur)) for layer in layers])
        arena.barrier(1)                          # every rank's output columns have landed
        done = torch.cuda.Event()
        done.record(stream)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            for i in range(len(SHAPES)):
                host_y[i].copy_(ys[i][:, lo:hi, :], non_blocking=True)
            downloaded[cur] = torch.cuda.Event()
            downloaded[cur].record(copy_out)

    for _ in range(2):
        e2e_step()
    run.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(3, min(args.steps, 10))
    a.record(stream)
    copy_in.wait_event(a)
    for _ in range(n_e2e):
        e2e_step()
    stream.wait_stream(copy_out)
    b.record(stream)
    run.barrier()
    ms_e2e = run.max_over_ranks(a.elapsed_time(b) / n_e2e)
    codes_in = sum(M_TOKENS * x.size(2) for x in xs) * (world - 1) // world
    return {"value": total_ops() / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
            "h2d_bytes_per_step_per_rank": h2d, "d2h_bytes_per_step_per_rank": d2h, "ms_per_step": ms_e2e, "steps": n_e2e,
            "int8_code_bytes_received_per_rank_per_step": codes_in,
            "note": "every rank uploads its M/g rows of the activations from pinned host memory, quantises them once (the quantising kernel stores "
                    "codes and scales into every rank's buffer over NVLink), computes its columns on the gathered codes (epilogue stores into every "
                    "rank's y) and downloads its M/g rows of the full-width results; byte counts are whole-job totals; weights stay resident",
            "_host_y": host_y}


def measure_sustained(run: Run, step, xs, ws, ms_per_step: float) -> dict:
    """The same step looped for a little over two seconds with the SM clock sampled: what the part settles at under its
    power limit, against the sustained bf16 figure of the peaks file.  Also the GEMM launches alone, operands quantised once."""
    torch, stream, peaks = run.torch, run.stream, run.peaks
    from cpm_kernels_b200.torch.gemm import quantize, gemm_and_scale
    out = {}
    peak = 2.0 * peaks.get("bf16_tflops_sustained", 0.0) if peaks.get("bf16_tflops_sustained") else None

    def loop(fn, ms_guess, name, ops):
        n = max(50, int(2200.0 / max(ms_guess, 1e-3)))
        sampler = ClockSampler(run.local_rank)
        sampler.start()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record(stream)
        for _ in range(n):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = a.elapsed_time(b) / n
        tops = ops / (ms * 1e-3) / 1e12
        out[name] = {"TOPS": tops, "ms_per_step": ms, "steps": n, "seconds": ms * n * 1e-3, "clocks": clocks,
                     "frac_of_sustained_peak": tops / peak if peak else None}

    loop(step, ms_per_step, "step", total_ops())
    quantised = [(quantize(x, False), quantize(w, False)) for x, w in zip(xs, ws)]

    def gemms():
        for (sa, qa), (sb, qb) in quantised:
            gemm_and_scale(qa, sa, qb, sb, False, True)
    loop(gemms, ms_per_step * 0.75, "gemm_only", total_ops())
    out["peak"] = peak
    out["peak_note"] = "2 x %s bf16_tflops_sustained (%s TFLOP/s: a seconds-long cuBLAS bf16 loop under the power cap)" % (peaks["source"], peaks.get("bf16_tflops_sustained"))
    return out


def measure_reference_cuda(run: Run, xs, ws, ct, our_ms_per_step: float, our_gemm_tops: dict) -> dict:
    """The reference's own CUDA pipeline on the same tensors in the same process with the same event loop: its six
    launches per linear (cpm_kernels/torch/gemm.py:86-113: calc_scale, round for both operands, cublasLt int8 GEMM,
    gemm_scale), its kernels compiled unmodified for sm_100 (oracle/_ref), its cublasLt call sequence
    (cpm_kernels/kernels/gemm.py:127-186) replayed by oracle/ref_cuda.py, its allocations per call.  Checker code:
    nothing of it is on the product path."""
    torch, stream = run.torch, run.stream
    try:
        from oracle import ref_cuda
        if not ref_cuda.available():
            return {"unavailable": "oracle/_ref/*.fatbin are not built (no reference checkout where build() ran)"}
        rk, lt = ref_cuda.ReferenceKernels(), ref_cuda.ReferenceCublasLt()
    except Exception as e:                                  # noqa: BLE001
        return {"unavailable": "reference device code could not be loaded: %s" % (e,)}

    def linear(x, w):
        # torch/gemm.py:98-104 with the operand swap of :45-52
        sa = rk.gemm_calc_scale(x)
        qa = rk.gemm_round(x, sa)
        sb = rk.gemm_calc_scale(w)
        qb = rk.gemm_round(w, sb)
        n, k, m = w.size(1), w.size(2), x.size(1)
        acc = torch.empty((1, m, n), dtype=torch.int32, device=x.device)
        lt.gemm_int8(n, k, m, 1, 1, True, False, qb, qa, acc)
        return rk.gemm_scale(acc, sa, sb, True, True), (qa, qb, acc)

    def ref_step():
        for x, w in zip(xs, ws):
            linear(x, w)
    try:
        ms_step = run.timed(ref_step, 5, warm=2)
        gemm_tops, identical = {}, {}
        for (name, n, k), x, w in zip(SHAPES, xs, ws):
            y_ref, (qa, qb, acc) = linear(x, w)
            identical[name] = bool(torch.equal(y_ref.view(torch.int16), ct.bmm(x, False, w, True, int8=True).view(torch.int16)))
            ms = run.timed(lambda: lt.gemm_int8(n, k, x.size(1), 1, 1, True, False, qb, qa, acc), 10, warm=2)
            gemm_tops[name] = 2.0 * x.size(1) * n * k / (ms * 1e-3) / 1e12
            del y_ref, qa, qb, acc
    except Exception as e:                                  # noqa: BLE001
        return {"unavailable": "the reference pipeline failed on this device: %s" % (e,)}
    return {"ms_per_step": ms_step, "TOPS": total_ops() / (ms_step * 1e-3) / 1e12, "launches_per_step": 24,
            "speedup_of_this_repo_whole_step": ms_step / our_ms_per_step,
            "cublaslt_gemm_only_tops": gemm_tops, "this_repo_gemm_only_tops": our_gemm_tops,
            "gemm_only_ratio": {k: our_gemm_tops[k] / gemm_tops[k] for k in gemm_tops},
            "outputs_bit_identical_to_this_repo": identical,
            "what": "reference kernels (cuda/gemm.cu, unmodified, sm_100) + its cublasLt int8 call sequence (int32 result, then cu_gemm_scale), "
                    "same tensors, same process; the GEMM-only figures time the cublasLt call alone (host descriptor churn included, as in the reference)"}


def measure_gemv(run: Run, gen, ck, batches=(1, 4, 16)) -> dict:
    """Decode GEMV HBM GB/s (weight 10240 x 4096 and its transpose; batch 1, 4, 16 with per-batch matrices), inside a
    CUDA graph over rotating weights larger than L2; and, for one matrix, what merely reading it costs (read_floor)."""
    torch, dev, stream, peaks = run.torch, run.dev, run.stream, run.peaks
    from cpm_kernels_b200.library import cpmk
    gemv = {}
    gs = torch.cuda.Stream()                         # capture stream; warmed up first so that the library's
    s = gs.cuda_stream                               # per-stream workspace exists before capture begins

    def graph_time(fn, nbuf, launches):
        """Seconds per launch of fn(j) (j = buffer index), `launches` launches replayed from one CUDA graph."""
        gs.wait_stream(stream)
        with torch.cuda.stream(gs):
            for j in range(nbuf):
                fn(j)
        gs.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=gs):
            for j in range(launches):
                fn(j % nbuf)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e-3 / launches

    for batch in batches:
        nbuf = max(1, 4 // batch)                    # at least 4 x 84 MB of weights rotate: larger than L2
        mats = [(torch.randn((batch, 10240, 4096), generator=gen, device=dev) * 0.02).half() for _ in range(nbuf)]
        vec_in = torch.randn((batch, 4096), generator=gen, device=dev).half()
        y_rows = torch.empty((batch, 10240), dtype=torch.half, device=dev)
        launches = nbuf * max(2, 20 // (nbuf * batch))
        bytes_alg = batch * (2 * 10240 * 4096 + 2 * (10240 + 4096))
        # the transposed weight [4096, 10240] = (dim_in, dim_out): the same buffers, read with the other shape
        for name, fn in (("gemv_fp16", lambda j: ck.gemv_fp16(batch, 10240, 4096, mats[j].data_ptr(), vec_in.data_ptr(), y_rows.data_ptr(), s)),
                         ("gemv_fp16_transpose", lambda j: ck.gemv_fp16_transpose(batch, 10240, 4096, mats[j].data_ptr(), vec_in.data_ptr(), y_rows.data_ptr(), s))):
            sec = graph_time(fn, nbuf, launches)
            gemv["%s_batch%d" % (name, batch)] = {"GBps": bytes_alg / sec / 1e9, "us": sec * 1e6,
                                                 "frac_of_hbm_peak": bytes_alg / sec / 1e9 / peaks["hbm_gbs"]}
        if batch == 1:
            # the same 84 MB matrices merely read, by a plain grid-stride kernel and by the row GEMV's own copy pipeline
            floor = {}
            for mode, name in ((0, "plain_read"), (1, "row_gemv_pipeline_without_arithmetic")):
                sec = graph_time(lambda j: cpmk.call("cpmk_probe_read", mode, 10240, 4096, mats[j].data_ptr(), y_rows.data_ptr(), s), nbuf, launches)
                floor[name] = {"us": sec * 1e6, "GBps": 2 * 10240 * 4096 / sec / 1e9}
            gemv["read_floor_batch1"] = floor
            for name in ("gemv_fp16_batch1", "gemv_fp16_transpose_batch1"):
                gemv[name]["vs_plain_read"] = floor["plain_read"]["us"] / gemv[name]["us"]
        del mats
    return gemv


# ------------------------------------------------------------------------------------------------
# configuration 5: the full 48-layer CPM-Bee-10B linear stack at M = 16384 tokens, weights seeded per layer,
# column-parallel across the ranks
# ------------------------------------------------------------------------------------------------
CFG5_TOKENS = 16384
CFG5_LAYERS = 48
CFG5_BLOCKS = 8          # every weight is generated in 8 row blocks, so that a rank's shard does not depend on how many ranks there are


def cfg5_weight_rows(run: Run, layer: int, shape: int, blocks) -> "torch.Tensor":
    """Rows of weight (layer, shape) made of the given row blocks: fp16 (1, len(blocks) * N / 8, K), N(0, 0.02)."""
    torch = run.torch
    _, n, k = SHAPES[shape]
    parts = []
    for j in blocks:
        g = torch.Generator(device=run.dev).manual_seed(5_000_000 + (layer * len(SHAPES) + shape) * CFG5_BLOCKS + j)
        parts.append((torch.randn((n // CFG5_BLOCKS, k), generator=g, device=run.dev) * 0.02).half())
    return torch.cat(parts).unsqueeze(0).contiguous()


def measure_cfg5(run: Run, arena, lanes, ct) -> dict:
    torch, dev, world, rank, stream = run.torch, run.dev, run.world, run.rank, run.stream
    from cpm_kernels_b200.sharded import FusedColumnParallelInt8Linear, SymmetricArena, ExchangeBuffers
    n_layers = int(os.environ.get("CPMK_BENCH_CFG5_LAYERS", str(CFG5_LAYERS)))
    steps = 2
    if arena is None:
        arena = SymmetricArena(sum(ExchangeBuffers.nbytes(CFG5_TOKENS, k, n, SLOTS) for _, n, k in SHAPES) + (1 << 20), dev)
    if lanes is None:
        lanes = Lanes(run, 1, 0, arena)
    gen = torch.Generator(device=dev).manual_seed(5)
    xs = [torch.randn((1, CFG5_TOKENS, k), generator=gen, device=dev).half() for _, _, k in SHAPES]
    bufs = [ExchangeBuffers(arena, CFG5_TOKENS, k, n, SLOTS) for _, n, k in SHAPES]
    scratch = [(torch.empty((1, n // world, k), dtype=torch.int8, device=dev), torch.empty((1, n // world), dtype=torch.half, device=dev))
               for _, n, k in SHAPES]
    per = CFG5_BLOCKS // world
    my_blocks = range(rank * per, (rank + 1) * per)
    layers = [[FusedColumnParallelInt8Linear(cfg5_weight_rows(run, l, i, my_blocks), buffers=bufs[i], weight_scratch=scratch[i])
               for i in range(len(SHAPES))] for l in range(n_layers)]
    weight_bytes = sum(w.weight.numel() * 2 for row in layers for w in row)

    def stack(only_local: bool):
        # one rank barrier per layer (the layer's outputs are complete on every rank), pipelined as in the main step
        for row in layers:
            lanes.run_step([(lambda slot, layer=layer, x=x: layer.launch(x, slot, only_local)) for layer, x in zip(row, xs)],
                           barrier=not only_local)

    ops = total_ops(CFG5_TOKENS) * n_layers
    ms_e2e = run.timed(lambda: stack(False), steps, warm=1)
    ms_phase = run.timed(lambda: stack(True), steps, warm=1) if world > 1 else ms_e2e
    out = {"workload": "%d-layer CPM-Bee-10B linear stack, M=%d tokens, int8, weights N(0, 0.02) seeded per layer (fp16, %.1f GB resident per rank, "
                       "re-quantised on every call), column-parallel x%d; one step = %d linears" % (n_layers, CFG5_TOKENS, weight_bytes / 1e9, world, n_layers * len(SHAPES)),
           "steps": steps, "end_to_end_with_exchange": {"ms_per_step": ms_e2e, "TOPS": ops / (ms_e2e * 1e-3) / 1e12},
           "gemm_phase": {"ms_per_step": ms_phase, "TOPS": ops / (ms_phase * 1e-3) / 1e12,
                          "what": "the same launches (quantise activations and weight rows, GEMM + dequantisation) with each rank storing into its own result only: no NVLink traffic, no barrier"}}
    if world > 1:
        # one GPU's rate on the unsharded problem, measured here on layer 0's full weights (every rank measures; rank 0's figure is used)
        w_full = [cfg5_weight_rows(run, 0, i, range(CFG5_BLOCKS)) for i in range(len(SHAPES))]

        def single():
            for x, w in zip(xs, w_full):
                ct.bmm(x, False, w, True, int8=True)
        run.barrier()
        lanes.margin(False)
        single()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(3):
            single()
        b.record(stream)
        torch.cuda.synchronize()
        lanes.margin(True)
        single_tops = total_ops(CFG5_TOKENS) / (a.elapsed_time(b) / 3 * 1e-3) / 1e12
        out["gemm_phase"]["one_gpu_unsharded_TOPS"] = single_tops
        out["gemm_phase"]["efficiency"] = out["gemm_phase"]["TOPS"] / (world * single_tops)
        out["end_to_end_with_exchange"]["speedup_over_one_gpu"] = out["end_to_end_with_exchange"]["TOPS"] / single_tops
        ingress = sum(2 * CFG5_TOKENS * n for _, n, _ in SHAPES) * (world - 1) // world * n_layers
        out["nvlink"] = {"bytes_received_per_rank_per_step": ingress, "achieved_GBps_per_rank": ingress / (ms_e2e * 1e-3) / 1e9, "nominal_GBps": 900.0,
                         "frac_of_nominal": ingress / (ms_e2e * 1e-3) / 1e9 / 900.0,
                         "note": "bytes that must enter every GPU ((g-1)/g of the fp16 outputs) over the end-to-end step time"}
        # parity on the first and the last layer: every rank's full-width results against the unsharded bmm computed locally
        bad, compared = 0, 0
        for l in sorted({0, n_layers - 1}):
            if l != 0:
                w_full = [cfg5_weight_rows(run, l, i, range(CFG5_BLOCKS)) for i in range(len(SHAPES))]
            for i, layer in enumerate(layers[l]):
                y = layer.forward(xs[i], sync_before=True, slot=0)
                run.barrier()
                want = ct.bmm(xs[i], False, w_full[i], True, int8=True)
                bad += count_mismatches(torch, y, want)
                compared += want.numel()
                del want
        out["parity"] = {"checked": True, "mismatches": run.sum_over_ranks(bad), "elements_compared_per_rank": compared,
                         "what": "layers 0 and %d, four linears each, every rank's full-width y against the unsharded bmm computed locally" % (n_layers - 1)}
        del w_full
    del layers, xs, bufs, scratch
    torch.cuda.empty_cache()
    return out


def measure_other_configs(cases, dev, gen, stream, peaks, xs=None, ws=None, iters=12):
    """The configurations of the path beside the headline step, each timed with CUDA events over rotating inputs:
    "attention": the batched attention-score bmm (HBM-bound, graded in GB/s); "fp16": the int8=False branch of bmm on
    the four linears; "prequantised": the headline linears with weights quantised once; "transposed": the same linears with weights
    stored (K, N); "passes": quantisation by rows / columns and GELU on
    a 4096 x 10240 operand."""
    import torch
    import cpm_kernels_b200.kernels as ck
    import cpm_kernels_b200.torch as ct
    other = {}

    def timed(fn, nbuf, iters=iters, warm=3):
        for j in range(warm):
            fn(j % nbuf)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for j in range(iters):
            fn(j % nbuf)
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e-3 / iters

    if "attention" in cases:
        # 8 sequences x 32 heads, Q and K (256, 512, 128) -> (256, 512, 512); two input sets rotate
        qs = [torch.randn((256, 512, 128), generator=gen, device=dev).half() for _ in range(2)]
        ks = [torch.randn((256, 512, 128), generator=gen, device=dev).half() for _ in range(2)]
        sec = timed(lambda j: ct.bmm(qs[j], False, ks[j], True, int8=True), 2)
        alg = 2 * 256 * 512 * 128 * 2 + 256 * 512 * 512 * 2
        from cpm_kernels_b200.torch.gemm import quantize, gemm_and_scale
        sq, qq = quantize(qs[0], False)
        sk, qk = quantize(ks[0], False)
        sec_gemm = timed(lambda j: gemm_and_scale(qq, sq, qk, sk, False, True), 1)
        alg_gemm = 2 * 256 * 512 * 128 + 256 * 512 * 512 * 2
        other["attention_scores_bmm_int8"] = {
            "shape": "Q, K (256, 512, 128) fp16 -> (256, 512, 512) fp16", "us": sec * 1e6, "GBps": alg / sec / 1e9,
            "frac_of_hbm_peak": alg / sec / 1e9 / peaks["hbm_gbs"], "algorithmic_bytes": alg,
            "gemm_kernel_only": {"us": sec_gemm * 1e6, "GBps": alg_gemm / sec_gemm / 1e9, "frac_of_hbm_peak": alg_gemm / sec_gemm / 1e9 / peaks["hbm_gbs"]}}
        del qs, ks, sq, qq, sk, qk
    if "prequantised" in cases:
        # the same four linears through the kernel-level API with the weights quantised once (what a serving stack that
        # owns its weights would do; the reference's bmm re-quantises them on every call): per step, per linear, one
        # activation quantisation and one fused GEMM + dequantisation
        from cpm_kernels_b200.torch.gemm import quantize, gemm_and_scale
        wq = [quantize(w, False) for w in ws]                       # (scale, codes) per weight

        def pre_step(j):
            for i in range(len(SHAPES)):
                sa, qa = quantize(xs[i], False)
                gemm_and_scale(qa, sa, wq[i][1], wq[i][0], False, True)
        sec = timed(pre_step, 1, iters=10)
        other["linears_weights_prequantised"] = {"ms_per_step": sec * 1e3, "TOPS": total_ops() / sec / 1e12, "launches_per_step": 8}
        del wq
    if "transposed" in cases:
        # the transposed-weight variant of the configuration: weights stored (K, N), so that bmm(x, False, w, False)
        # quantises them by columns (gemm_calc_scale_transpose / gemm_round_transpose) and the GEMM reads an MN-major operand
        wt = [w.transpose(1, 2).contiguous() for w in ws]

        def t_step(j):
            for i in range(len(SHAPES)):
                ct.bmm(xs[i], False, wt[i], False, int8=True)
        sec = timed(t_step, 1, iters=10)
        other["linears_transposed_weights"] = {"ms_per_step": sec * 1e3, "TOPS": total_ops() / sec / 1e12, "launches_per_step": 16}
        del wt
    if "fp16" in cases:
        # fp16 branch of bmm on the same four linears (tcgen05 kind::f16, fp32 accumulation)
        f16 = {}
        for i, (name, n, k) in enumerate(SHAPES):
            sec = timed(lambda j: ct.bmm(xs[i], False, ws[i], True, int8=False), 1, iters=8)
            f16[name] = 2.0 * M_TOKENS * n * k / sec / 1e12
        other["bmm_fp16_tflops"] = {"per_shape": f16, "peak_bf16_tflops": peaks["bf16_tflops"],
                                    "frac_of_peak": (sum(f16.values()) / len(f16)) / peaks["bf16_tflops"]}
    if "passes" in cases:
        # quantisation passes (3 bytes per element algorithmic), GELU and transpose (4 bytes per element), 4096 x 10240 operands
        big = [torch.randn((1, 4096, 10240), generator=gen, device=dev).half() for _ in range(3)]
        sc_r = torch.empty((1, 4096), dtype=torch.half, device=dev)
        sc_c = torch.empty((1, 10240), dtype=torch.half, device=dev)
        q8 = torch.empty((1, 4096, 10240), dtype=torch.int8, device=dev)
        o16 = torch.empty((1, 4096, 10240), dtype=torch.half, device=dev)
        st = stream.cuda_stream
        nel = 4096 * 10240
        for name, bytes_per, fn in (
                ("quantize_rows", 3, lambda j: ck.gemm_quantize_rows(1, 4096, 10240, big[j].data_ptr(), sc_r.data_ptr(), q8.data_ptr(), st)),
                ("quantize_cols", 3, lambda j: ck.gemm_quantize_cols(1, 4096, 10240, big[j].data_ptr(), sc_c.data_ptr(), q8.data_ptr(), st)),
                ("gelu_forward", 4, lambda j: ck.gelu_forward(1, nel, big[j].data_ptr(), o16.data_ptr(), st)),
                ("transpose", 4, lambda j: ck.transpose(1, 4096, 10240, big[j].data_ptr(), o16.data_ptr(), st))):
            sec = timed(fn, 3)
            other[name] = {"shape": "(1, 4096, 10240) fp16", "us": sec * 1e6, "GBps": bytes_per * nel / sec / 1e9,
                           "frac_of_hbm_peak": bytes_per * nel / sec / 1e9 / peaks["hbm_gbs"]}
        del big, q8, o16
        # layer norm -> affine -> column quantisation of a (batch 8, hidden 4096, seq 512) activation in one call;
        # algorithmic traffic 3 bytes per element (fp16 in, int8 out); the reference's four kernels move 13
        lx = [torch.randn((8, 4096, 512), generator=gen, device=dev).half() for _ in range(4)]
        lw = (torch.randn((4096,), generator=gen, device=dev) * 0.1 + 1.0).half()
        sec = timed(lambda j: ct.layernorm_quantize(lx[j], 1e-6, lw, None, False), 4)
        nel = 8 * 4096 * 512
        other["layernorm_quantize_cols"] = {"shape": "(8, 4096, 512) fp16, RMS form", "us": sec * 1e6, "GBps": 3 * nel / sec / 1e9,
                                            "frac_of_hbm_peak": 3 * nel / sec / 1e9 / peaks["hbm_gbs"]}
        del lx
    return other


def run_case(args):
    """``--case attention|fp16|passes``: only that configuration, a few launches, for profiler captures.  Prints a
    small JSON object of its own (not the benchmark line)."""
    import torch
    from cpm_kernels_b200.library import cpmk
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cpmk.check_device()
    gen = torch.Generator(device=dev).manual_seed(0)
    if args.case == "gemv":
        import cpm_kernels_b200.kernels as ck
        class _R:                                        # the few members measure_gemv uses
            pass
        r = _R()
        r.torch, r.dev, r.stream, r.peaks = torch, dev, torch.cuda.current_stream(), measured_peaks()
        print(json.dumps({"case": "gemv", "result": measure_gemv(r, gen, ck, batches=(1,))}), flush=True)
        return
    xs = ws = None
    if args.case == "fp16":
        xs = [torch.randn((1, M_TOKENS, k), generator=gen, device=dev).half() for _, n, k in SHAPES]
        ws = [(torch.randn((1, n, k), generator=gen, device=dev) * 0.02).half() for _, n, k in SHAPES]
    out = measure_other_configs((args.case,), dev, gen, torch.cuda.current_stream(), measured_peaks(), xs, ws, iters=max(1, args.steps))
    print(json.dumps({"case": args.case, "result": out}), flush=True)


def main():
    global M_TOKENS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="fused", choices=["fused", "fused1", "multicast", "nccl"],
                    help="N > 1: how the output slices reach every rank (fused = stored by the GEMM's own CTAs, linears on several streams; fused1 = the same on one "
                         "stream; multicast = forwarded once per GPU through the NVLink switch's multicast mapping; nccl = all-gather)")
    ap.add_argument("--no-cfg5", action="store_true", help="skip the 48-layer stack at M = 16384 (shorter run)")
    ap.add_argument("--tokens", type=int, default=M_TOKENS,
                    help="tokens per step; anything but the default is a reduced case for profiler captures, not a bench value")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the e2e, GEMV and CPU-baseline legs (profiler captures of the step's kernels)")
    ap.add_argument("--case", default="linears", choices=["linears", "attention", "fp16", "passes", "gemv"],
                    help="anything but 'linears' runs only that secondary configuration (profiler captures; no benchmark line)")
    args = ap.parse_args()
    M_TOKENS = args.tokens
    if args.impl == "reference":
        run_reference(args)
    elif args.case != "linears":
        run_case(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
