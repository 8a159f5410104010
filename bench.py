#!/usr/bin/env python
"""Benchmark of the decode hot path: Q4_K GEMV over Q8_1 activations.

Workload (N=1): the FFN products of one Gemma-3-4B-shaped decode step, all 34
layers, Q4_K weights: per layer  x[b,2560] -> Q8_1 -> fused gate/up GeGLU
product (two 10240x2560 matrices) -> Q8_1 -> down product (2560x10240).
Each layer has its own weight copy (34 x 44.2 MB = 1.5 GB, far beyond the
126 MB L2), so every launch streams its weights from HBM, the rotation the
reference's own benchmark uses (benchmarks/vecq_bench.cc:119-121).

One step = that whole pass for one batch.  `value` = algorithmic bytes of the
step / device time (GB/s), inputs resident in HBM, the step replayed as one
CUDA graph.  `e2e` = the same step driven through the C ABI from HOST buffers:
pinned x copied in, y copied back, inside the timed region.

N>1 (torchrun): N-column sharding.  Each rank owns 1/N of every matrix's
output rows; the GLU output and the layer output are all-gathered with NCCL.
Total work is fixed ("strong" scaling).

--impl reference: the CPU arm.  GGML's CPU vec_dot is not part of the
reference build, so the arm times the oracle's restatement of the same
products on the host cores (kind "port").
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LAYERS = 34
HIDDEN, INTER = 2560, 10240
SB = 144  # Q4_K super-block bytes
# dram__bytes_read.sum + dram__bytes_write.sum of one fused gate/up launch at batch 1
# (profiles/vecq_rowlane_glu_b1.md): the matrices' 29,491,200 bytes plus activations.
NCU_GLU_DRAM_BYTES_B1 = 29532928
METRIC = "q4k_decode_gemv_hbm_throughput"
UNIT = "GB/s"


def step_bytes(batch: int, layers: int | None = None) -> int:
    """Algorithmic bytes of one step: every operand once."""
    glu = 2 * INTER * (HIDDEN // 256) * SB + batch * (HIDDEN // 32 * 36) + batch * INTER * 4
    down = HIDDEN * (INTER // 256) * SB + batch * (INTER // 32 * 36) + batch * HIDDEN * 4
    return (LAYERS if layers is None else layers) * (glu + down)


def glu_launch_bytes(batch: int, shard: int = 1) -> int:
    return 2 * (INTER // shard) * (HIDDEN // 256) * SB + batch * (HIDDEN // 32 * 36) + \
        batch * (INTER // shard) * 4


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines: list[str] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm
def run_reference(args, rank: int):
    if rank != 0:
        return
    batch = args.batch
    per_step = []
    # A step of the arm = the 34-layer pass; each timed as a bounded sample of
    # `sample_layers` layers scaled to 34 (every layer is the same work).
    sample_layers = 4
    total = args.warmup + args.steps
    gbs_all, threads, text = [], 1, ""
    for i in range(total):
        gbs, per_layer, threads, text = _cpu_step(batch, sample_layers)
        if i >= args.warmup:
            gbs_all.append(gbs)
            per_step.append(per_layer * LAYERS)
    value = statistics.mean(gbs_all)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * statistics.mean(per_step), 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 dp4a -> int32 per block, f32 sums",
        "data": "synthetic",
        "config": {"workload": f"Gemma-3-4B FFN decode products, Q4_K, {LAYERS} layers, batch {batch}",
                   "batch": batch, "timing": "host wall clock; weights beyond the CPU cache"},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": text},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


_CPU_STATE = {}


def _cpu_step(batch: int, layers: int):
    """One bounded CPU sample: `layers` layer passes, weights built once."""
    import numpy as np

    from llmp_b200 import synth
    from oracle import binding as orc

    if "ws" not in _CPU_STATE:
        orc.build()
        rng = np.random.default_rng(0)
        copies = 8  # 8 x 44 MB: beyond the host's last-level cache
        _CPU_STATE["ws"] = [(synth.q4_k_weights(rng, INTER, HIDDEN),
                             synth.q4_k_weights(rng, INTER, HIDDEN),
                             synth.q4_k_weights(rng, HIDDEN, INTER)) for _ in range(copies)]
        _CPU_STATE["x"] = rng.normal(0, 1, size=(batch, HIDDEN)).astype(np.float32)
        _CPU_STATE["at"] = 0
    threads = orc.host_threads()
    x = _CPU_STATE["x"]
    t0 = time.perf_counter()
    for _ in range(layers):
        gate, up, down = _CPU_STATE["ws"][_CPU_STATE["at"] % len(_CPU_STATE["ws"])]
        _CPU_STATE["at"] += 1
        q8 = orc.quantize_q8_1(x)
        h = orc.vecq(orc.Q4_K, up, q8, HIDDEN, INTER, batch, g=gate, glu=orc.GLU_GEGLU,
                     threads=threads)[:, 0, :]
        orc.vecq(orc.Q4_K, down, orc.quantize_q8_1(h), INTER, HIDDEN, batch, threads=threads)
    dt = time.perf_counter() - t0
    per_layer = dt / layers
    text = (f"{layers} of the step's 34 layer passes per step (gate/up GeGLU + down, Q4_K, batch "
            f"{batch}) over 8 distinct layer copies; oracle port, {threads} threads")
    return step_bytes(batch, 1) / per_layer / 1e9, per_layer, threads, text


# --------------------------------------------------------------------------- GPU arm
def make_q4k_device(torch, rows: int, k: int, gen):
    """Random Q4_K blocks made on the device: random nibbles and 6-bit fields,
    FP16 d = |N(0,0.02)|/480 and dmin = |N(0,0.02)|/32."""
    nb = k // 256
    w = torch.randint(0, 256, (rows, nb, SB), dtype=torch.uint8, device="cuda", generator=gen)
    d = (torch.randn((rows, nb), device="cuda", generator=gen).abs() * (0.02 / 480.0)).half()
    dmin = (torch.randn((rows, nb), device="cuda", generator=gen).abs() * (0.02 / 32.0)).half()
    w[:, :, 0:2] = d.view(torch.uint8).view(rows, nb, 2)
    w[:, :, 2:4] = dmin.view(torch.uint8).view(rows, nb, 2)
    return w.view(rows, nb * SB)


class FfnStep:
    """The step's device state and launches, for one rank's shard."""

    def __init__(self, torch, ops, batch: int, world: int, rank: int, dist, fused: bool = False,
                 q8_out: bool = False):
        self.torch, self.ops, self.batch, self.world, self.dist = torch, ops, batch, world, dist
        self.fused = fused
        # Opt-in (one GPU): the gate/up product writes its output's Q8_1 blocks
        # itself (llmp_b200_vecq_q8), so the down product needs no quantize
        # launch.  Bit-identical; measured slower (0.61 against 0.57 ms a step: the
        # count-and-quantize tail costs the product more than the launch it saves).
        self.q8_out = q8_out and world == 1 and not fused
        self.rows_done = ops.vecq_q8_scratch(INTER, batch, "cuda")
        gen = torch.Generator(device="cuda")
        gen.manual_seed(1234 + rank)
        self.n_glu = INTER // world
        self.n_down = HIDDEN // world
        self.layers = []
        for _ in range(LAYERS):
            self.layers.append((make_q4k_device(torch, self.n_glu, HIDDEN, gen),
                                make_q4k_device(torch, self.n_glu, HIDDEN, gen),
                                make_q4k_device(torch, self.n_down, INTER, gen)))
        g2 = torch.Generator(device="cuda")
        g2.manual_seed(99)
        self.x = torch.randn((LAYERS, batch, HIDDEN), device="cuda", generator=g2)
        self.q8x = torch.empty((batch, ops.q8_1_row_blocks(HIDDEN) * 36), dtype=torch.uint8,
                               device="cuda")
        self.q8h = torch.empty((batch, ops.q8_1_row_blocks(INTER) * 36), dtype=torch.uint8,
                               device="cuda")
        # shard-major gather buffers [world, batch, n/world]; the full vector is
        # re-assembled by a strided view when world > 1
        self.h_shard = torch.empty((batch, self.n_glu), device="cuda")
        self.h_full = torch.empty((world, batch, self.n_glu), device="cuda")
        self.h_rows = torch.empty((batch, INTER), device="cuda")
        self.y_shard = torch.empty((batch, self.n_down), device="cuda")
        self.y_full = torch.empty((LAYERS, world, batch, self.n_down), device="cuda")
        self.launches_per_layer = (2 if (world == 1 and fused) else 3 if self.q8_out
                                   else 4 + (1 if world > 1 else 0))
        self.launches_per_step = LAYERS * self.launches_per_layer

    def layer(self, l: int, x):
        ops, T = self.ops, self.ops.TYPE_Q4_K
        gate, up, down = self.layers[l]
        if self.world == 1 and self.fused:
            # Two launches a layer: each product quantizes its F32 input itself
            # (llmp_b200_vecq_f32), with the quantizer's arithmetic.
            ops.vecq_f32(up, T, HIDDEN, self.n_glu, x, gate=gate, glu=ops.GLU_GEGLU,
                         out=self.h_shard)
            ops.vecq_f32(down, T, INTER, self.n_down, self.h_shard, out=self.y_full[l, 0])
            return
        ops.quantize_q8(x, out=self.q8x)
        if self.q8_out:
            ops.vecq_q8(up, T, HIDDEN, self.n_glu, self.q8x, self.batch, rows_done=self.rows_done,
                        gate=gate, glu=ops.GLU_GEGLU, out=self.h_shard, q8_dst=self.q8h)
            ops.vecq(down, T, INTER, self.n_down, self.q8h, self.batch, out=self.y_full[l, 0])
            return
        ops.vecq(up, T, HIDDEN, self.n_glu, self.q8x, self.batch, gate=gate, glu=ops.GLU_GEGLU,
                 out=self.h_shard)
        if self.world > 1:
            self.dist.all_gather_into_tensor(self.h_full, self.h_shard)
            self.h_rows.view(self.batch, self.world, self.n_glu).copy_(self.h_full.transpose(0, 1))
            h = self.h_rows
        else:
            h = self.h_shard
        ops.quantize_q8(h, out=self.q8h)
        if self.world > 1:
            ops.vecq(down, T, INTER, self.n_down, self.q8h, self.batch, out=self.y_shard)
            self.dist.all_gather_into_tensor(self.y_full[l], self.y_shard)
        else:
            ops.vecq(down, T, INTER, self.n_down, self.q8h, self.batch, out=self.y_full[l, 0])

    def step(self, x_all=None):
        x_all = self.x if x_all is None else x_all
        for l in range(LAYERS):
            self.layer(l, x_all[l])

    def glu_only(self):
        """The dominant kernel alone, one launch per layer copy."""
        ops, T = self.ops, self.ops.TYPE_Q4_K
        if self.world == 1 and self.fused:
            for l, (gate, up, _) in enumerate(self.layers):
                ops.vecq_f32(up, T, HIDDEN, self.n_glu, self.x[l], gate=gate, glu=ops.GLU_GEGLU,
                             out=self.h_shard)
            return
        for gate, up, _ in self.layers:
            if self.q8_out:
                ops.vecq_q8(up, T, HIDDEN, self.n_glu, self.q8x, self.batch,
                            rows_done=self.rows_done, gate=gate, glu=ops.GLU_GEGLU,
                            out=self.h_shard, q8_dst=self.q8h)
            else:
                ops.vecq(up, T, HIDDEN, self.n_glu, self.q8x, self.batch, gate=gate,
                         glu=ops.GLU_GEGLU, out=self.h_shard)


def run_gpu(args, rank: int, world: int, local_rank: int):
    import torch

    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        torch.cuda.set_device(0)
    import llmp_b200 as ops
    if not ops.available():
        raise SystemExit("bench.py: no B200 / native library: " + ops._native.last_error())

    batch = args.batch
    # N > 1: by default every rank runs the whole step on its own batch (replicas of
    # the data-parallel decode path: no collective, weak scaling).  --shard columns
    # splits every matrix's rows over the ranks and all-gathers the outputs (strong
    # scaling; at decode sizes the all-gathers' latency dominates).
    sharded = world > 1 and args.shard == "columns"
    parts = world if sharded else 1
    st = FfnStep(torch, ops, batch, parts, rank, dist, fused=args.fused, q8_out=args.q8_out)
    stream = torch.cuda.Stream()
    sync = torch.cuda.synchronize

    def barrier():
        if world > 1:
            dist.barrier()
        sync()

    with torch.cuda.stream(stream):
        st.step()       # warm: module load, attributes
        sync()
        graph = None
        # Graph replay only for steps without NCCL collectives (one GPU, replicas): a
        # sharded step is queued as plain stream launches.
        graph_kw = {"capture_error_mode": "thread_local"} if world > 1 else {}
        if parts == 1 and not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream, **graph_kw):
                    st.step()
            except Exception as e:  # capture refused: time plain launches
                print(f"bench.py: graph capture unavailable ({e}); timing plain launches",
                      file=sys.stderr)
                graph = None
                sync()
        run = graph.replay if graph is not None else st.step
        for _ in range(max(args.warmup, 3)):
            run()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
        # ---- the dominant kernel alone (roofline): one launch per layer copy, replayed
        # as a CUDA graph so the host's launch rate is not what is timed; CUDA events
        # on the launching stream around the replays
        st.glu_only()
        sync()
        glu_graph = None
        if parts == 1 and not args.no_graph:
            try:
                glu_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(glu_graph, stream=stream, **graph_kw):
                    st.glu_only()
            except Exception:
                glu_graph = None
                sync()
        run_glu = glu_graph.replay if glu_graph is not None else st.glu_only
        run_glu()
        sync()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        k0.record(stream)
        for _ in range(reps):
            run_glu()
        k1.record(stream)
        sync()
        glu_us = 1e3 * k0.elapsed_time(k1) / (reps * LAYERS)
        # ---- end to end through the C ABI from host buffers
        hx = torch.randn((LAYERS, batch, HIDDEN)).pin_memory()
        hy = torch.empty((LAYERS, parts, batch, st.n_down)).pin_memory()
        dx = torch.empty_like(st.x)

        def e2e_body():
            dx.copy_(hx, non_blocking=True)
            for l in range(LAYERS):
                st.layer(l, dx[l])
            hy.copy_(st.y_full, non_blocking=True)

        # The step as a caller would queue it: pinned-host input copy, the C-ABI
        # launches, pinned-host output copy, all captured once and replayed (the
        # reference replays captured steps too, src/engine/step_runs.cc:323).
        e2e_graph = None
        if parts == 1 and not args.no_graph:
            try:
                e2e_body()
                sync()
                e2e_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_graph, stream=stream, **graph_kw):
                    e2e_body()
            except Exception as e:
                print(f"bench.py: e2e graph capture unavailable ({e})", file=sys.stderr)
                e2e_graph = None
                sync()

        def e2e_step():
            if e2e_graph is not None:
                e2e_graph.replay()
            else:
                e2e_body()
            stream.synchronize()

        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        e2e_ms = 1e3 * (time.perf_counter() - t0) / args.steps
        clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        t = torch.tensor([ms, e2e_ms, glu_us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, glu_us = (float(v) for v in t.tolist())
    if rank == 0:
        replicas = world if not sharded else 1
        sb = step_bytes(batch) * replicas      # what all ranks streamed in a step
        value = sb / (ms * 1e-3) / 1e9
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        glu_b = glu_launch_bytes(batch, parts)
        achieved = glu_b / (glu_us * 1e-6) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
            "higher_is_better": True, "scaling": "strong" if sharded or world == 1 else "weak",
            "vs_baseline": None,
            "dtype": "int8 dp4a -> int32 per block, f32 sums", "data": "synthetic",
            "config": {
                "workload": f"Gemma-3-4B FFN decode products, Q4_K, {LAYERS} layers, batch {batch}",
                "batch": batch, "layers": LAYERS, "gate_up": [INTER, HIDDEN],
                "down": [HIDDEN, INTER],
                "l2": f"inputs larger than L2: {LAYERS} distinct layer copies, "
                      f"{LAYERS * 44.2e-3:.2f} GB, streamed in order",
                "launch": "cuda graph replay" if graph is not None else "stream launches",
                "launches_per_layer": st.launches_per_layer,
                "parallelism": "single GPU" if world == 1 else
                               (f"N-column shards x{world}, NCCL all-gather of the GLU output and of "
                                "the layer output" if sharded else
                                f"{world} replicas, one batch a GPU, no collective in the step"),
                "step_bytes": sb,
            },
            "e2e": {"value": round(sb / (e2e_ms * 1e-3) / 1e9, 2), "unit": UNIT,
                    "ms_per_step": round(e2e_ms, 4),
                    "how": "host wall clock around pinned H2D of x, the step's C-ABI launches and "
                           "pinned D2H of y, with a stream synchronize per step"
                           + (" (captured once, replayed)" if e2e_graph is not None else ""),
                    "h2d_bytes_per_step": LAYERS * batch * HIDDEN * 4 * replicas,
                    "d2h_bytes_per_step": LAYERS * batch * HIDDEN * 4 * replicas},
            "gpu_launches": st.launches_per_step * args.steps * world,
            "roofline": {"bound": "hbm", "kernel": "VecQRowLaneKernel<P, GLU> (fused gate/up, Q4_K)",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks
                         else "fallback 6650",
                         "us_per_launch": round(glu_us, 3), "bytes_per_launch": glu_b,
                         "frac_of_8tbs_spec": round(achieved / 8000.0, 4),
                         "traffic": args.traffic if args.traffic is not None else
                         (NCU_GLU_DRAM_BYTES_B1 if batch == 1 and world == 1 else None)},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            _cpu_step(batch, 4)  # warm: builds the host weights
            gbs, per_layer, threads, text = _cpu_step(batch, 24)
            line["cpu_baseline"] = {"value": round(gbs, 3), "unit": UNIT, "cores": threads,
                                    "kind": "port",
                                    "ms_per_step": round(per_layer * LAYERS * 1e3, 1),
                                    "sample": text}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- other configs
def run_other(args):
    """The other BASELINE configs' kernels, one JSON line each (not the headline
    bench line; parity cases that also serve as small, committed ncu drivers).
    Operands rotate over two copies so that a launch's inputs are not L2-resident."""
    import torch

    torch.cuda.set_device(0)
    import llmp_b200 as ops
    if not ops.available():
        raise SystemExit("bench.py: no B200 / native library: " + ops._native.last_error())
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    peaks = {"mxf8f6f4": 4466.5, "i8": 4567.3}  # profiles/tcgen05_microbenchmarks.md

    def timed(fns, steps, warmup):
        for i in range(max(warmup, 3)):
            fns[i % len(fns)]()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fns[i % len(fns)]()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    if args.workload == "mxfp8_gemm":
        m, n, k = args.tokens or 2048, 12288, 4096
        x = torch.randn((m, k), device="cuda", generator=gen).bfloat16()
        a, a_s = ops.mxfp8_quantize(x)
        sets = []
        for _ in range(2):
            w = torch.randn((n, k), device="cuda", generator=gen) * 0.02
            b, bs = ops.mxfp8_quantize(w)
            sets.append((b, bs, torch.empty((m, n), dtype=torch.bfloat16, device="cuda")))
        fns = [lambda t=t: ops.mxfp8_gemm(a, a_s, t[0], t[1], bf16=True, out=t[2]) for t in sets]
        ms = timed(fns, args.steps, args.warmup)
        rate = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        line = {"metric": "mxfp8_gemm_throughput", "value": round(rate, 1), "unit": "TFLOP/s",
                "ms_per_step": round(ms, 5),
                "config": {"workload": f"MXFP8 block-scaled GEMM M {m} K {k} N {n}, BF16 out"},
                "roofline": {"bound": "tensor", "achieved": round(rate, 1),
                             "peak": peaks["mxf8f6f4"], "unit": "TFLOP/s",
                             "frac": round(rate / peaks["mxf8f6f4"], 4),
                             "peak_source": "bare tcgen05.mma loop on this pool "
                                            "(profiles/tcgen05_microbenchmarks.md)"}}
    elif args.workload == "q8_0_gemv":
        # BASELINE configs[0]: Q8_0 4096 x 4096, batch 1 (the reference's CPU-runnable case);
        # 16 weight copies (285 MB) walked in order inside one captured graph.
        import numpy as np

        from llmp_b200 import synth
        n = k = 4096
        rng = np.random.default_rng(0)
        ws = [torch.from_numpy(synth.q8_0_weights(rng, n, k)).cuda() for _ in range(16)]
        q8 = ops.quantize_q8(torch.randn((1, k), device="cuda", generator=gen))
        out = torch.empty((1, n), device="cuda")

        def body():
            for w in ws:
                ops.vecq(w, ops.TYPE_Q8_0, k, n, q8, 1, out=out)

        fns = [body]
        if not args.no_graph:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                body()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    body()
            torch.cuda.synchronize()
            fns = [graph.replay]
        ms = timed(fns, args.steps, args.warmup) / len(ws)
        nbytes = 17_825_792 + 4_608 + 16_384
        rate = nbytes / (ms * 1e-3) / 1e9
        peak = 6535.7
        try:
            peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
        except (OSError, KeyError, ValueError):
            pass
        line = {"metric": "q8_0_decode_gemv_hbm_throughput", "value": round(rate, 1), "unit": "GB/s",
                "ms_per_step": round(ms, 6),
                "config": {"workload": "Q8_0 decode GEMV 4096 x 4096, batch 1, 16 rotating copies"},
                "roofline": {"bound": "hbm", "achieved": round(rate, 1), "peak": peak, "unit": "GB/s",
                             "frac": round(rate / peak, 4), "bytes_per_launch": nbytes}}
    elif args.workload == "mmq_q4k":
        m, n, k = args.tokens or 4096, 14336, 4096
        x = torch.randn((m, k), device="cuda", generator=gen).bfloat16()
        yq = ops.mmq_quantize(x)
        sets = [(make_q4k_device(torch, n, k, gen), torch.empty((m, n), device="cuda"))
                for _ in range(2)]
        fns = [lambda t=t: ops.mmq(t[0], yq, k, n, out=t[1]) for t in sets]
        ms = timed(fns, args.steps, args.warmup)
        rate = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        line = {"metric": "mmq_q4k_int8_gemm_throughput", "value": round(rate, 1), "unit": "TOP/s",
                "ms_per_step": round(ms, 5),
                "config": {"workload": f"Q4_K x Q8_1-MMQ int8 GEMM M {m} K {k} N {n}"},
                "roofline": {"bound": "tensor", "achieved": round(rate, 1), "peak": peaks["i8"],
                             "unit": "TOP/s", "frac": round(rate / peaks["i8"], 4),
                             "peak_source": "bare tcgen05.mma loop on this pool "
                                            "(profiles/tcgen05_microbenchmarks.md)"}}
    else:  # moe
        import numpy as np

        from llmp_b200 import synth
        tokens = args.tokens or 4096
        experts, used, hidden, inter = 128, 8, 2048, 768
        gate_up = make_q4k_device(torch, experts * 2 * inter, hidden, gen).view(experts, 2 * inter, -1)
        down = make_q4k_device(torch, experts * hidden, inter, gen).view(experts, hidden, -1)
        ids, w = synth.topk_route(np.random.default_rng(0), tokens, experts, used)
        ids_d, w_d = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
        x = torch.randn((tokens, hidden), device="cuda", generator=gen)
        fns = [lambda: ops.moe_ffn(x, ids_d, w_d, gate_up, down, hidden, inter)]
        if not args.no_graph:
            # The block queues 7 to 40 small launches: replay them as one captured graph so
            # that the host's launch rate is not what is timed.
            try:
                side = torch.cuda.Stream()
                with torch.cuda.stream(side):
                    fns[0]()
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        fns[0]()
                torch.cuda.synchronize()
                fns = [graph.replay]
            except Exception as e:
                print(f"bench.py: graph capture unavailable ({e}); timing plain launches",
                      file=sys.stderr)
                torch.cuda.synchronize()
        ms = timed(fns, args.steps, args.warmup)
        distinct = int(np.unique(ids).size)
        if tokens <= 16:
            nbytes = distinct * 2654208
            line = {"metric": "moe_decode_hbm_throughput", "unit": "GB/s",
                    "value": round(nbytes / (ms * 1e-3) / 1e9, 1)}
        else:
            ops_count = 3 * 2.0 * hidden * inter * tokens * used
            line = {"metric": "moe_grouped_gemm_throughput", "unit": "TOP/s",
                    "value": round(ops_count / (ms * 1e-3) / 1e12, 1)}
        line.update({"ms_per_step": round(ms, 5),
                     "config": {"workload": f"MoE block, 128 experts top-8, hidden 2048, "
                                            f"intermediate 768, Q4_K, {tokens} tokens "
                                            f"({distinct} distinct experts)"}})
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
                 "higher_is_better": True, "data": "synthetic", "vs_baseline": None,
                 "faults": ops.device_faults()})
    print(json.dumps(line), flush=True)


def run_mmq_sharded(args, rank: int, world: int, local_rank: int):
    """The prefill GEMM N-column sharded (BASELINE configs[2]): every rank holds the weight
    rows [rank * n / world, +n / world) and the whole activation batch, computes its slice
    D[:, slice] and the slices are all-gathered over NVLink (NCCL) into [world, m, n / world]
    on every rank.  Strong scaling: the product is the same at every N."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import llmp_b200 as ops
    from llmp_b200 import shard
    m, n, k = args.tokens or 4096, 14336, 4096
    lo, hi = shard.row_shard(n, world, rank, multiple=128)
    width = shard.row_shard(n, world, 0, multiple=128)
    width = width[1] - width[0]                      # the widest slice; others pad to it
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)                               # the same activations on every rank
    x = torch.randn((m, k), device="cuda", generator=gen).bfloat16()
    gen.manual_seed(100 + rank)
    if hi - lo != width:
        raise SystemExit("bench.py: N-column shards of unequal width are not benchmarked")
    sets = [(make_q4k_device(torch, width, k, gen), torch.empty((m, width), device="cuda"),
             torch.empty((world, m, width), device="cuda")) for _ in range(2)]

    def step(i):
        w, mine, full = sets[i % 2]
        yq = ops.mmq_quantize(x)
        ops.mmq(w, yq, k, width, out=mine)
        dist.all_gather_into_tensor(full, mine)
        return full

    for i in range(max(args.warmup, 3)):
        step(i)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        out = step(i)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = torch.tensor([float(torch.isfinite(out).all())], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        ms = float(t.item())
        rate = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "mmq_q4k_int8_gemm_throughput", "value": round(rate, 1), "unit": "TOP/s",
            "ms_per_step": round(ms, 5), "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "strong",
            "data": "synthetic", "vs_baseline": None, "finite": bool(ok.item()),
            "faults": ops.device_faults(),
            "config": {"workload": f"Q4_K x Q8_1-MMQ int8 GEMM M {m} K {k} N {n}",
                       "parallelism": f"N-column shards x{world} (slices of {width} columns), "
                                      "activation quantizer on every rank, NCCL all-gather of "
                                      f"the F32 output ({m * n * 4 / 1e6:.0f} MB)"},
            "roofline": {"bound": "tensor", "achieved": round(rate, 1), "peak": 4567.3 * world,
                         "unit": "TOP/s", "frac": round(rate / (4567.3 * world), 4),
                         "peak_source": "bare tcgen05.mma loop on this pool "
                                        "(profiles/tcgen05_microbenchmarks.md) x N"}}), flush=True)
    dist.destroy_process_group()


def run_moe_ep(args, rank: int, world: int, local_rank: int):
    """Expert-parallel MoE block: each rank owns 128 / world whole experts and `--tokens` tokens
    (weak scaling); rows travel to their experts' owners and back with NCCL all-to-all
    (llmp_b200/shard.py) and are combined on the home rank in slot order."""
    import numpy as np
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import llmp_b200 as ops
    from llmp_b200 import shard, synth
    tokens = args.tokens or 4096
    experts, used, hidden, inter = 128, 8, 2048, 768
    b, e = shard.expert_range(experts, world, rank)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(100 + rank)
    gate_up = make_q4k_device(torch, (e - b) * 2 * inter, hidden, gen).view(e - b, 2 * inter, -1)
    down = make_q4k_device(torch, (e - b) * hidden, inter, gen).view(e - b, hidden, -1)
    ids, w = synth.topk_route(np.random.default_rng(rank), tokens, experts, used)
    ids_d, w_d = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    x = torch.randn((tokens, hidden), device="cuda", generator=gen)

    def local(rows, local_ids):
        ones = torch.ones((rows.shape[0], 1), device=rows.device)
        return ops.moe_ffn(rows, local_ids.view(-1, 1).contiguous(), ones, gate_up, down, hidden,
                           inter)

    def step():
        return shard.ep_moe_ffn(x, ids_d, w_d, experts, local)

    for _ in range(max(args.warmup, 3)):
        out = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ok = torch.tensor([float(torch.isfinite(out).all())], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        ms = float(t.item())
        ops_count = 3 * 2.0 * hidden * inter * tokens * used * world
        print(json.dumps({
            "metric": "moe_grouped_gemm_throughput", "unit": "TOP/s",
            "value": round(ops_count / (ms * 1e-3) / 1e12, 1), "ms_per_step": round(ms, 4),
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "higher_is_better": True, "scaling": "weak", "data": "synthetic", "vs_baseline": None,
            "finite": bool(ok.item()), "faults": ops.device_faults(),
            "config": {"workload": f"MoE block, 128 experts top-8, hidden 2048, intermediate 768, "
                                   f"Q4_K, {tokens} tokens a rank",
                       "parallelism": f"expert parallel x{world}, NCCL all-to-all dispatch and "
                                      "combine, tokens data-parallel"}}), flush=True)
    dist.destroy_process_group()


def main():
    global LAYERS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1, choices=[1, 2, 4, 8])
    ap.add_argument("--impl", default="llmp_b200", choices=["llmp_b200", "reference"])
    ap.add_argument("--layers", type=int, default=34,
                    help="distinct layer copies a step walks (34: the model's; fewer for a small "
                         "ncu capture, keep >= 4 so the weights exceed L2)")
    ap.add_argument("--workload", default="ffn_q4k",
                    choices=["ffn_q4k", "q8_0_gemv", "mxfp8_gemm", "mmq_q4k", "moe"],
                    help="ffn_q4k is the bench line; the others time the other configs' kernels")
    ap.add_argument("--tokens", type=int, default=0,
                    help="tokens / rows of the other workloads")
    ap.add_argument("--q8-out", action="store_true",
                    help="the gate/up product also writes its output's Q8_1 blocks "
                         "(llmp_b200_vecq_q8): one launch fewer a layer, measured slower")
    ap.add_argument("--fused", action="store_true",
                    help="llmp_b200_vecq_f32: each product quantizes its F32 input itself (two "
                         "launches a layer instead of four; measured slower: 2,200 against 2,717 "
                         "GB/s, the per-CTA quantization sits on the critical path)")
    ap.add_argument("--shard", default="replicas", choices=["replicas", "columns"],
                    help="N > 1: replicas (each GPU its own batch, weak scaling) or columns "
                         "(rows of every matrix split, NCCL all-gather, strong scaling)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--traffic", type=float, default=None,
                    help="dram bytes per launch of the dominant kernel from an ncu capture "
                         "(default: the figure in profiles/vecq_rowlane_glu_b1.md at batch 1)")
    args = ap.parse_args()
    LAYERS = args.layers
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "moe" and world > 1:
        run_moe_ep(args, rank, world, local_rank)
        return
    if args.workload == "mmq_q4k" and world > 1:
        run_mmq_sharded(args, rank, world, local_rank)
        return
    if args.workload != "ffn_q4k":
        if rank == 0:
            run_other(args)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
