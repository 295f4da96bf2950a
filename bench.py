#!/usr/bin/env python
"""Benchmark of the int8-quantised linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the four CPM-Bee-10B layer linears at M = 4096 tokens (fused QKV 12288x4096, attention-out
4096x4096, FFN-in 10240x4096, FFN-out 4096x10240), fp16 activations N(0,1) and weights N(0,0.02), seeded
synthetic data.  One step = one pass over the four linears through the public entry point
``cpm_kernels_b200.torch.bmm(x, False, W, True, int8=True)``, which -- like the reference's bmm -- quantises
BOTH operands on every call (per-row absmax scale + int8 rounding), runs the int8 GEMM and dequantises to fp16:
two kernels per linear (both operands quantised in one launch, then the GEMM), eight per step.  ``value`` counts 2*M*N*K operations of the four GEMMs over the whole
step time (quantisation passes included), inputs resident in HBM.  ``e2e`` is the same step driven from pinned
host buffers: activations copied host->device and fp16 outputs device->host inside the timed region.

N > 1 (torchrun, one rank per GPU): the same linears column-parallel -- each rank holds N/g rows of every weight,
quantises its shard, computes its output slice, and the slices are all-gathered over NCCL ("strong" scaling).

``--impl reference`` times the reference's own arithmetic on the host CPU: the torch expressions its unit tests
hold the kernels to (oracle/test_formula.py), on a bounded sample of the same workload, with all host threads.
"""
from __future__ import annotations

import argparse
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
# CPU baseline: the reference's test formula on host cores (bounded sample)
# ------------------------------------------------------------------------------------------------
CPU_SAMPLE_TOKENS = 1024


def cpu_baseline(repeats: int = 2) -> dict:
    import torch
    from oracle import test_formula
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator(device="cpu").manual_seed(0)
    best = None
    ops = total_ops(CPU_SAMPLE_TOKENS)
    data = []
    for _, n, k in SHAPES:
        x = torch.randn((1, CPU_SAMPLE_TOKENS, k), generator=g).half()
        w = (torch.randn((1, n, k), generator=g) * 0.02).half()
        data.append((x, w))
    for _ in range(repeats + 1):                      # first pass is the warm-up
        t0 = time.perf_counter()
        for x, w in data:
            test_formula.real_bmm(x, False, w, True, True)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": ops / best / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "the same four linears at M=%d tokens (1/%d of the workload), reference test formula "
                      "(tests/test_gemm.py:8-41) in torch CPU fp32, best of %d passes, %.2f s per pass" %
                      (CPU_SAMPLE_TOKENS, M_TOKENS // CPU_SAMPLE_TOKENS, repeats, best),
            "seconds_per_pass": best}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    base = cpu_baseline(repeats=steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": base["seconds_per_pass"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_tokens": CPU_SAMPLE_TOKENS},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    import cpm_kernels_b200.torch as ct
    import cpm_kernels_b200.kernels as ck
    from cpm_kernels_b200.library import cpmk
    from cpm_kernels_b200.sharded import shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    saved_stdout = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # libraries print banners on stdout when a communicator is created: keep stdout for the one JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
    cpmk.check_device()
    peaks = measured_peaks()

    # ---- data: activations replicated, weights sharded along N (rank r holds rows [r*N/g, (r+1)*N/g)) ----
    gen = torch.Generator(device=dev).manual_seed(0)
    xs, ws, outs, gathered = [], [], [], []
    for _, n, k in SHAPES:
        assert n % world == 0
        xs.append(torch.randn((1, M_TOKENS, k), generator=gen, device=dev).half())
        w_full = (torch.randn((1, n, k), generator=gen, device=dev) * 0.02).half()
        lo, hi = shard_bounds(n, world, rank)
        ws.append(w_full[:, lo:hi, :].contiguous())
        del w_full
        if world > 1:
            gathered.append(torch.empty((world, M_TOKENS, n // world), dtype=torch.half, device=dev))
    stream = torch.cuda.current_stream()
    comm_stream = torch.cuda.Stream() if world > 1 else None
    from cpm_kernels_b200.sharded import ColumnParallelInt8Linear, FusedColumnParallelInt8Linear
    layers = [ColumnParallelInt8Linear(w) for w in ws] if world > 1 else None
    # preferred exchange: the GEMM epilogue stores each rank's output slice into every rank's full-width output
    # (peer-mapped symmetric memory); falls back to an NCCL all-gather beside the GEMM if that cannot be set up
    fused_layers, exchange, fused_two_streams = None, "none", False
    fused_margin = os.environ.get("CPMK_BENCH_FUSED_SM_MARGIN", "32")
    n_side = max(1, int(os.environ.get("CPMK_BENCH_FUSED_STREAMS", "4")) - 1)
    side_streams = ([comm_stream] + [torch.cuda.Stream() for _ in range(n_side - 1)]) if world > 1 else []
    if world > 1:
        exchange = "nccl all_gather_into_tensor on a side stream"
        if args.exchange in ("fused", "fused1"):
            try:
                fused_layers = [FusedColumnParallelInt8Linear(w) for w in ws]
                for fl in fused_layers:
                    fl._buffer(M_TOKENS)
                exchange = "fused: GEMM epilogue TMA-stores its slice into every rank's output over NVLink"
            except Exception as e:                       # noqa: BLE001
                sys.stderr.write("fused exchange unavailable (%s); using the NCCL all-gather\n" % (e,))
                fused_layers = None
        if fused_layers is None:
            # the collective's kernels run beside the persistent GEMM grid: leave them a few SMs
            os.environ.setdefault("CPMK_GEMM_SM_MARGIN", "16")
        elif args.exchange == "fused":
            fused_two_streams = True
            exchange += "; the linears run on %d streams, scatter GEMM grids leave %s SMs free" % (n_side + 1, fused_margin)

    gemm_events = []

    def step(record_gemm: bool = False, gather: bool = True):
        """The four linears through the public API.  With record_gemm, CUDA events bracket each GEMM launch."""
        results = []
        if fused_layers is not None and gather and not record_gemm:
            # The linears of the synthetic stack are independent, so they are spread over several streams: while one
            # linear's GEMM drains its output over NVLink, the others' quantisation passes and GEMMs run beside it
            # (the scatter GEMM's persistent grid leaves part of the SMs free for that: CPMK_GEMM_SM_MARGIN).
            if fused_two_streams:
                for s2 in side_streams:
                    s2.wait_stream(stream)
                cpmk.set_gemm_sm_margin(int(fused_margin))
            for i, (fl, x) in enumerate(zip(fused_layers, xs)):
                lane = i % (len(side_streams) + 1) if fused_two_streams else 0
                if lane:
                    with torch.cuda.stream(side_streams[lane - 1]):
                        results.append(fl(x))
                else:
                    results.append(fl(x))
            if fused_two_streams:
                for s2 in side_streams:
                    stream.wait_stream(s2)
                cpmk.set_gemm_sm_margin(-1)
            return results
        for i, (x, w) in enumerate(zip(xs, ws)):
            if record_gemm:
                # same three launches as ct.bmm, spelled out so that events can bracket the GEMM kernel alone
                from cpm_kernels_b200.torch.gemm import quantize, gemm_and_scale
                sa, qa = quantize(x, False)
                sb, qb = quantize(w, False)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                y = gemm_and_scale(qa, sa, qb, sb, False, True)
                e1.record(stream)
                gemm_events.append((i, e0, e1))
            else:
                y = ct.bmm(x, False, w, True, int8=True)
            if world > 1 and gather:
                ev = torch.cuda.Event()
                ev.record(stream)
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ev)
                    layers[i].gather(y, out=gathered[i])
                y.record_stream(comm_stream)
            results.append(y)
        if world > 1 and gather:
            stream.wait_stream(comm_stream)
        return results

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert cpmk.last_gemm_path() == 1, "the tensor-core GEMM kernel was not selected"

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- timed region: exactly K steps, device time, max over ranks ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    # ---- same region again with events around each GEMM launch: per-kernel duration for the roofline
    #      (without the all-gather, whose copy kernels would otherwise share the SMs with the GEMM being timed) ----
    for _ in range(args.steps):
        step(record_gemm=True, gather=False)
    barrier()
    phases = None
    if world > 1:
        # compute phase alone (no exchange), to separate GEMM-phase scaling from the NVLink-bound gather
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        p0.record(stream)
        for _ in range(args.steps):
            step(gather=False)
        p1.record(stream)
        barrier()
        t = torch.tensor([p0.elapsed_time(p1) / args.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_compute = float(t.item())
        gather_bytes = sum(2 * M_TOKENS * n for _, n, _ in SHAPES) * (world - 1) // world
        phases = {"compute_only_ms_per_step": ms_compute, "compute_only_tops": total_ops() / (ms_compute * 1e-3) / 1e12,
                  "allgather_bytes_received_per_rank_per_step": gather_bytes,
                  "note": "the all-gather of fp16 outputs moves (g-1)/g * 2*M*N bytes into every rank per linear and bounds the step for g >= 2"}
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = total_ops() / (ms_per_step * 1e-3) / 1e12

    per_shape_ms = {}
    for i, a, b in gemm_events:
        per_shape_ms.setdefault(i, []).append(a.elapsed_time(b))
    gemm_ms = sum(statistics.mean(v) for v in per_shape_ms.values())
    gemm_ops = total_ops() / world
    gemm_tops = gemm_ops / (gemm_ms * 1e-3) / 1e12
    peak_tops = 2.0 * peaks["bf16_tflops"]
    roofline = {
        "bound": "tensor", "achieved": gemm_tops, "peak": peak_tops, "unit": "TOPS", "frac": gemm_tops / peak_tops,
        # dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of these four launches at N = 1
        # (profiles/gemm_i8_tc2_kernel_cpm-bee-linears_M4096.md): 131.0 / 36.8 / 104.9 / 133.2 MB, mean of the four
        "traffic": 101.5e6 if (world == 1 and M_TOKENS == 4096) else None,
        "kernel": "gemm_i8_tc2_kernel<dequant> (tcgen05.mma cta_group::2 kind::i8, 256x256 tiles per CTA pair)",
        "peak_note": "2 x %s dense bf16 %s TFLOP/s (burst; no int8 figure is measured on this pool); nominal dense int8 is 4500 TOPS: frac_nominal below"
                     % (peaks["source"], peaks["bf16_tflops"]),
        "frac_nominal": gemm_tops / 4500.0,
        "per_shape_tops": {SHAPES[i][0]: 2.0 * M_TOKENS * (SHAPES[i][1] // world) * SHAPES[i][2] / (statistics.mean(v) * 1e-3) / 1e12
                           for i, v in sorted(per_shape_ms.items())},
    }

    # ---- e2e: pinned host activations in, fp16 outputs out, every step ----
    e2e = None
    if not args.kernels_only:
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
            # three-stage pipeline over the four linears: upload(i+1) || compute(i) || download(i-1)
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
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 10))
        a.record(stream)
        copy_in.wait_event(a)                         # nothing of the timed steps starts before the first event
        for _ in range(n_e2e):
            e2e_step()
        stream.wait_stream(copy_out)                  # the last step's results have reached the host
        b.record(stream)
        barrier()
        ms_e2e = a.elapsed_time(b) / n_e2e
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        e2e = {"value": total_ops() / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": ms_e2e,
               "note": "activations uploaded from pinned host memory and this rank's fp16 outputs downloaded every step, "
                       "copies pipelined against compute on separate streams; weights stay resident"}
        del host_x, host_y, dev_x

    # ---- secondary metric of the path: decode GEMV HBM GB/s (weight 10240x4096 and its transpose, batch 1) ----
    gemv = None
    if rank == 0 and not args.kernels_only:
        gemv = {}
        gs = torch.cuda.Stream()                         # capture stream; warmed up first so that the library's
        s = gs.cuda_stream                               # per-stream workspace exists before capture begins
        for batch in (1, 4, 16):
            nbuf = max(1, 4 // batch)                    # at least 4 x 84 MB of weights rotate: larger than L2
            mats = [(torch.randn((batch, 10240, 4096), generator=gen, device=dev) * 0.02).half() for _ in range(nbuf)]
            vec_in = torch.randn((batch, 4096), generator=gen, device=dev).half()
            y_rows = torch.empty((batch, 10240), dtype=torch.half, device=dev)
            # the transposed weight [4096, 10240] = (dim_in, dim_out): the same buffers, read with the other shape
            for name, fn in (("gemv_fp16", lambda j: ck.gemv_fp16(batch, 10240, 4096, mats[j].data_ptr(), vec_in.data_ptr(), y_rows.data_ptr(), s)),
                             ("gemv_fp16_transpose", lambda j: ck.gemv_fp16_transpose(batch, 10240, 4096, mats[j].data_ptr(), vec_in.data_ptr(), y_rows.data_ptr(), s))):
                gs.wait_stream(stream)
                with torch.cuda.stream(gs):
                    for j in range(nbuf):
                        fn(j)
                gs.synchronize()
                reps = max(2, 20 // (nbuf * batch))
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=gs):
                    for j in range(nbuf * reps):
                        fn(j % nbuf)
                graph.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graph.replay()
                b.record()
                torch.cuda.synchronize()
                sec = a.elapsed_time(b) * 1e-3 / (nbuf * reps)
                bytes_alg = batch * (2 * 10240 * 4096 + 2 * (10240 + 4096))
                gemv["%s_batch%d" % (name, batch)] = {"GBps": bytes_alg / sec / 1e9, "us": sec * 1e6,
                                                     "frac_of_hbm_peak": bytes_alg / sec / 1e9 / peaks["hbm_gbs"]}
            del mats
        mats = None
        del mats

    # ---- the other configurations of the path: attention-score bmm, fp16 bmm, quantisation passes, GELU ----
    other = None
    if rank == 0 and world == 1 and not args.kernels_only:
        other = measure_other_configs(("attention", "prequantised", "transposed", "fp16", "passes"), dev, gen, stream, peaks, xs, ws)

    status = cpmk.read_status()
    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    base = cpu_baseline() if (world == 1 and not args.kernels_only) else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD if M_TOKENS == 4096 else WORKLOAD + " [REDUCED to %d tokens: profiling case, not a bench value]" % M_TOKENS, "tokens": M_TOKENS, "parallelism": "column-parallel x%d; exchange = %s" % (world, exchange) if world > 1 else "single GPU",
                   "l2": "per-step working set (fp16 weights 302 MB + activations 134 MB + outputs 252 MB) exceeds the 126 MB L2; no explicit flush",
                   "weights": "re-quantised on every call, as the reference's bmm does"},
        "roofline": roofline, "e2e": e2e, "gpu_launches": 8 * args.steps, "clocks": clocks,
        "gemv": gemv, "other_configs": other, "phases": phases, "device_status_word": status,
        "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained", "source")},
    }
    if base is not None:
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if saved_stdout is not None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--exchange", default="fused", choices=["fused", "fused1", "nccl"],
                    help="N > 1: how the output slices reach every rank (fused = stored by the GEMM epilogue, linears on two alternating streams; fused1 = the same on one stream; nccl = all-gather)")
    ap.add_argument("--tokens", type=int, default=M_TOKENS,
                    help="tokens per step; anything but the default is a reduced case for profiler captures, not a bench value")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the e2e, GEMV and CPU-baseline legs (profiler captures of the step's kernels)")
    ap.add_argument("--case", default="linears", choices=["linears", "attention", "fp16", "passes"],
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
