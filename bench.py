#!/usr/bin/env python
"""Benchmark of the decode hot path: Q4_K GEMV over Q8_1 activations.

Workload: the FFN products of one Gemma-3-4B-shaped decode step, all 34 layers,
Q4_K weights: per layer  x[b,2560] -> Q8_1 -> fused gate/up GeGLU product (two
10240x2560 matrices) -> Q8_1 -> down product (2560x10240).  Each layer has its
own weight copy (34 x 44.2 MB = 1.5 GB, far beyond the 126 MB L2), so every
launch streams its weights from HBM, the rotation the reference's own benchmark
uses (benchmarks/vecq_bench.cc:119-121).

One step = that whole pass for one batch.  `value` = algorithmic bytes of the
step / device time (GB/s), inputs resident in HBM, the step replayed as one CUDA
graph; the timed block of K steps is repeated and the median reported.  `e2e` =
the same step driven through the C ABI from HOST buffers: pinned x copied in, y
copied back, inside the timed region.  `roofline` = the fused gate/up launch
alone; `roofline.others` = the down product and the Q8_0 4096 x 4096 product.

N > 1 (torchrun): every rank runs the whole step on its own batch (replicas of
the data-parallel decode path, no collective in the step: `value`, weak
scaling), and then, in the same run, the sharded forms the path has, each with
its own timing and a parity flag against the unsharded result (`sharded`):
the prefill GEMM N-column sharded with its all-gather pipelined behind the
next chunk's product, the expert-parallel MoE block with all-to-alls of fixed
size, and the decode step N-column sharded.

--impl reference: the CPU arm.  GGML's CPU vec_dot is not part of the
reference build, so the arm times the oracle's restatement of the same
products on the host cores (kind "port"); a step of the arm is a bounded
sample of the 34-layer pass (4 layers, scaled: every layer is the same work).
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
# dram__bytes_read.sum + dram__bytes_write.sum of one fused gate/up launch at batch 1, from an
# ncu capture of this kernel: the matrices' 29,491,200 bytes plus activations.
NCU_GLU_DRAM_BYTES_B1 = 29532928
METRIC = "q4k_decode_gemv_hbm_throughput"
UNIT = "GB/s"


def step_bytes(batch: int, layers: int | None = None) -> int:
    """Algorithmic bytes of one step: every operand once."""
    glu = 2 * INTER * (HIDDEN // 256) * SB + batch * (HIDDEN // 32 * 36) + batch * INTER * 4
    down = HIDDEN * (INTER // 256) * SB + batch * (INTER // 32 * 36) + batch * HIDDEN * 4
    return (LAYERS if layers is None else layers) * (glu + down)


def down_launch_bytes(batch: int) -> int:
    return HIDDEN * (INTER // 256) * SB + batch * (INTER // 32 * 36) + batch * HIDDEN * 4


def workload_config(batch: int) -> dict:
    """What both arms run, key for key."""
    return {"workload": f"Gemma-3-4B FFN decode products, Q4_K, {LAYERS} layers, batch {batch}",
            "batch": batch, "layers": LAYERS, "gate_up": [INTER, HIDDEN], "down": [HIDDEN, INTER],
            "l2": "inputs larger than the last-level cache: distinct layer copies streamed in order",
            "step_bytes": step_bytes(batch)}


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
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 dp4a -> int32 per block, f32 sums",
        "data": "synthetic", "config": workload_config(batch),
        "arm": {"timing": "host wall clock; a step is a bounded sample: "
                          f"{sample_layers} of the {LAYERS} layer passes, scaled to {LAYERS} "
                          "(every layer is the same work); 8 distinct layer copies, beyond the "
                          "host's last-level cache"},
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
        self.launches_per_layer = self.launches_per_layer_of(world, fused, self.q8_out)
        self.launches_per_step = LAYERS * self.launches_per_layer

    @staticmethod
    def launches_per_layer_of(world: int, fused: bool, q8_out: bool) -> int:
        return 2 if (world == 1 and fused) else 3 if q8_out else 4 + (1 if world > 1 else 0)

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

    def down_only(self):
        """The down product alone, one launch per layer copy."""
        ops, T = self.ops, self.ops.TYPE_Q4_K
        for _, _, down in self.layers:
            ops.vecq(down, T, INTER, self.n_down, self.q8h, self.batch, out=self.y_shard)

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


def _median_ms(run, stream, steps, repeats, barrier, torch):
    """The block of `steps` runs, timed `repeats` times with CUDA events on the launching
    stream between barriers; the median per-step time."""
    times = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            run()
        e1.record(stream)
        barrier()
        times.append(e0.elapsed_time(e1) / steps)
    return statistics.median(times)


def _graphed(torch, fn, stream, enabled, **kw):
    """fn captured once as a CUDA graph (None when capture is off or refused)."""
    if not enabled:
        return None
    try:
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream, **kw):
            fn()
        return graph
    except Exception as e:  # capture refused: time plain launches
        print(f"bench.py: graph capture unavailable ({e}); timing plain launches", file=sys.stderr)
        torch.cuda.synchronize()
        return None


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
    # N > 1: every rank runs the whole step on its own batch (replicas of the data-parallel
    # decode path: no collective, weak scaling); the sharded forms are timed after it.
    # --shard columns makes the N-column form the headline instead (strong scaling).
    sharded = world > 1 and args.shard == "columns"
    parts = world if sharded else 1
    st = FfnStep(torch, ops, batch, parts, rank, dist, fused=args.fused, q8_out=args.q8_out)
    stream = torch.cuda.Stream()
    sync = torch.cuda.synchronize
    repeats = max(1, args.repeats)

    def barrier():
        if world > 1:
            dist.barrier()
        sync()

    with torch.cuda.stream(stream):
        st.step()       # warm: module load, attributes
        sync()
        # Graph replay only for steps without NCCL collectives (one GPU, replicas): a
        # sharded step is queued as plain stream launches.
        graph_kw = {"capture_error_mode": "thread_local"} if world > 1 else {}
        use_graph = parts == 1 and not args.no_graph
        graph = _graphed(torch, st.step, stream, use_graph, **graph_kw)
        run = graph.replay if graph is not None else st.step
        for _ in range(max(args.warmup, 3)):
            run()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ms = _median_ms(run, stream, args.steps, repeats, barrier, torch)
        # ---- the dominant kernel alone (roofline): one launch per layer copy, replayed as a
        # CUDA graph so the host's launch rate is not what is timed; CUDA events on the
        # launching stream around the replays.  The down product likewise.
        glu_graph = _graphed(torch, st.glu_only, stream, use_graph, **graph_kw)
        run_glu = glu_graph.replay if glu_graph is not None else st.glu_only
        run_glu()
        glu_us = 1e3 * _median_ms(run_glu, stream, 5, repeats, sync, torch) / LAYERS
        down_graph = _graphed(torch, st.down_only, stream, use_graph, **graph_kw)
        run_down = down_graph.replay if down_graph is not None else st.down_only
        run_down()
        down_us = 1e3 * _median_ms(run_down, stream, 5, repeats, sync, torch) / LAYERS
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
        e2e_graph = _graphed(torch, e2e_body, stream, use_graph, **graph_kw)

        def e2e_step():
            if e2e_graph is not None:
                e2e_graph.replay()
            else:
                e2e_body()
            stream.synchronize()

        for _ in range(3):
            e2e_step()
        e2e_times = []
        for _ in range(repeats):
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                e2e_step()
            barrier()
            e2e_times.append(1e3 * (time.perf_counter() - t0) / args.steps)
        e2e_ms = statistics.median(e2e_times)
        clocks = sampler.stop() if rank == 0 else None
        # ---- the Q8_0 4096 x 4096 product (the reference's CPU-runnable config), one GPU
        q80 = _q8_0_roofline(torch, ops, stream, use_graph, repeats) if world == 1 else None

    if world > 1:
        t = torch.tensor([ms, e2e_ms, glu_us, down_us], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, glu_us, down_us = (float(v) for v in t.tolist())
    launches = st.launches_per_step * (args.steps * repeats + max(args.warmup, 3) + 1) * world
    del graph, glu_graph, down_graph, e2e_graph
    st = None
    torch.cuda.empty_cache()
    # ---- the sharded forms, in the same run, each with its parity flag
    sharded_lines = None
    if world > 1 and args.shard != "columns" and not args.no_sharded:
        sharded_lines = {
            "mmq_q4k": bench_mmq_sharded(torch, dist, ops, rank, world, tokens=4096, steps=10, warmup=3),
            "moe_ep": bench_moe_ep(torch, dist, ops, rank, world, tokens=1024, steps=10, warmup=3),
            "ffn_columns": bench_ffn_columns(torch, dist, ops, rank, world, batch, steps=5, warmup=2),
        }
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
        source = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650"
        glu_b = glu_launch_bytes(batch, parts)
        achieved = glu_b / (glu_us * 1e-6) / 1e9
        down_b = down_launch_bytes(batch) if parts == 1 else None
        others = []
        if down_b is not None:
            rate = down_b / (down_us * 1e-6) / 1e9
            others.append({"kernel": "down product 2560 x 10240, Q4_K", "bound": "hbm",
                           "achieved": round(rate, 1), "peak": peak, "unit": "GB/s",
                           "frac": round(rate / peak, 4), "us_per_launch": round(down_us, 3),
                           "bytes_per_launch": down_b})
        if q80 is not None:
            q80.update({"peak": peak, "frac": round(q80["achieved"] / peak, 4)})
            others.append(q80)
        config = workload_config(batch)
        config["step_bytes"] = sb
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
            "higher_is_better": True, "scaling": "strong" if sharded else "weak",
            "vs_baseline": None,
            "dtype": "int8 dp4a -> int32 per block, f32 sums", "data": "synthetic",
            "config": config,
            "arm": {
                "launch": "cuda graph replay" if use_graph else "stream launches",
                "timing": f"median of {repeats} blocks of {args.steps} steps, CUDA events on the "
                          "launching stream, max over ranks",
                "launches_per_layer": FfnStep.launches_per_layer_of(parts, args.fused, args.q8_out),
                "parallelism": "single GPU" if world == 1 else
                               (f"N-column shards x{world}, NCCL all-gather of the GLU output and of "
                                "the layer output" if sharded else
                                f"{world} replicas, one batch a GPU, no collective in the step"),
            },
            "e2e": {"value": round(sb / (e2e_ms * 1e-3) / 1e9, 2), "unit": UNIT,
                    "ms_per_step": round(e2e_ms, 4),
                    "how": "host wall clock around pinned H2D of x, the step's C-ABI launches and "
                           "pinned D2H of y, with a stream synchronize per step"
                           + (" (captured once, replayed)" if use_graph else ""),
                    "h2d_bytes_per_step": LAYERS * batch * HIDDEN * 4 * replicas,
                    "d2h_bytes_per_step": LAYERS * batch * HIDDEN * 4 * replicas},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "kernel": "fused gate/up GeGLU product 2 x (10240 x 2560), Q4_K",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_source": source,
                         "us_per_launch": round(glu_us, 3), "bytes_per_launch": glu_b,
                         "frac_of_8tbs_spec": round(achieved / 8000.0, 4),
                         "traffic": args.traffic if args.traffic is not None else
                         (NCU_GLU_DRAM_BYTES_B1 if batch == 1 and world == 1 else None),
                         "others": others},
            "clocks": clocks,
        }
        if sharded_lines is not None:
            line["sharded"] = sharded_lines
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


def _q8_0_roofline(torch, ops, stream, use_graph, repeats):
    """the benchmark specification's config 0: Q8_0 4096 x 4096, batch 1; 16 weight copies (285 MB) walked in
    order inside one captured graph."""
    import numpy as np

    from llmp_b200 import synth
    n = k = 4096
    rng = np.random.default_rng(0)
    ws = [torch.from_numpy(synth.q8_0_weights(rng, n, k)).cuda() for _ in range(16)]
    q8 = ops.quantize_q8(torch.randn((1, k), device="cuda"))
    out = torch.empty((1, n), device="cuda")

    def body():
        for w in ws:
            ops.vecq(w, ops.TYPE_Q8_0, k, n, q8, 1, out=out)

    graph = _graphed(torch, body, stream, use_graph)
    run = graph.replay if graph is not None else body
    run()
    us = 1e3 * _median_ms(run, stream, 5, repeats, torch.cuda.synchronize, torch) / len(ws)
    nbytes = 17_825_792 + 4_608 + 16_384
    return {"kernel": "Q8_0 product 4096 x 4096", "bound": "hbm",
            "achieved": round(nbytes / (us * 1e-6) / 1e9, 1), "unit": "GB/s",
            "us_per_launch": round(us, 3), "bytes_per_launch": nbytes}


# --------------------------------------------------------------------------- other configs
def run_other(args):
    """The other benchmark configs' kernels, one JSON line each (not the headline
    bench line; parity cases that also serve as small, committed ncu drivers).
    Operands rotate over two copies so that a launch's inputs are not L2-resident."""
    import torch

    torch.cuda.set_device(0)
    import llmp_b200 as ops
    if not ops.available():
        raise SystemExit("bench.py: no B200 / native library: " + ops._native.last_error())
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0)
    peaks = {"mxf8f6f4": 4466.5, "i8": 4567.3}  # measured with the bare tcgen05.mma loop (make probe)

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
        def of(variant):
            return timed([lambda t=t: ops.mxfp8_gemm(a, a_s, t[0], t[1], bf16=True, out=t[2],
                                                     variant=variant) for t in sets],
                         args.steps, args.warmup)
        ms = of(0)                      # the entry point's own rule (CTA pairs at this shape)
        ms_one, ms_pair = of(1), of(2)
        rate = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        line = {"metric": "mxfp8_gemm_throughput", "value": round(rate, 1), "unit": "TFLOP/s",
                "ms_per_step": round(ms, 5),
                "ms_one_cta_a_tile": round(ms_one, 5), "ms_cta_pairs": round(ms_pair, 5),
                "config": {"workload": f"MXFP8 block-scaled GEMM M {m} K {k} N {n}, BF16 out"},
                "roofline": {"bound": "tensor", "achieved": round(rate, 1),
                             "peak": peaks["mxf8f6f4"], "unit": "TFLOP/s",
                             "frac": round(rate / peaks["mxf8f6f4"], 4),
                             "peak_source": "bare tcgen05.mma loop measured on this pool"}}
    elif args.workload == "q8_0_gemv":
        # the benchmark specification's config 0: Q8_0 4096 x 4096, batch 1 (the reference's CPU-runnable case);
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
    elif args.workload == "decode_vector":
        # The decode module's vector product (F32 activations, the reference's summation
        # order): Q8_0 4096 x 4096, one activation row, 16 weight copies walked in order
        # inside one captured graph.
        import numpy as np

        from llmp_b200 import synth
        n = k = 4096
        rng = np.random.default_rng(0)
        ws = [torch.from_numpy(synth.q8_0_weights(rng, n, k)).cuda() for _ in range(16)]
        x = torch.randn((1, k), device="cuda", generator=gen)
        out = torch.empty((1, n), device="cuda")

        def body():
            for w in ws:
                ops.decode_vector(ops.DECODER_Q8_0, w, x, k, n, out=out)

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
        nbytes = 17_825_792 + 16_384 + 16_384
        rate = nbytes / (ms * 1e-3) / 1e9
        peak = 6535.7
        try:
            peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
        except (OSError, KeyError, ValueError):
            pass
        line = {"metric": "q8_0_decode_vector_hbm_throughput", "value": round(rate, 1), "unit": "GB/s",
                "ms_per_step": round(ms, 6),
                "config": {"workload": "decode-module vector product, Q8_0 4096 x 4096, F32 activations, "
                                       "one row, 16 rotating copies"},
                "roofline": {"bound": "hbm", "achieved": round(rate, 1), "peak": peak, "unit": "GB/s",
                             "frac": round(rate / peak, 4), "bytes_per_launch": nbytes}}
    elif args.workload == "mmq_q4k":
        m, n, k = args.tokens or 4096, 14336, 4096
        x = torch.randn((m, k), device="cuda", generator=gen).bfloat16()
        yq = ops.mmq_quantize(x)
        sets = [(make_q4k_device(torch, n, k, gen), torch.empty((m, n), device="cuda"))
                for _ in range(2)]
        slabs = [ops.q4k_relayout(t[0], k, n) for t in sets]     # load time: outside the timing
        scratch = ops.mmq_scratch(k, n)
        # the weights relaid at load time (the headline), relaid by every call, unpacked in the kernel
        ms = timed([lambda t=t, sl=sl: ops.mmq(None, yq, k, n, out=t[1], slab=sl)
                    for t, sl in zip(sets, slabs)], args.steps, args.warmup)
        ms_call = timed([lambda t=t: ops.mmq(t[0], yq, k, n, out=t[1], scratch=scratch) for t in sets],
                        args.steps, args.warmup)
        ms_raw = timed([lambda t=t: ops.mmq(t[0], yq, k, n, out=t[1]) for t in sets],
                       args.steps, args.warmup)
        rate = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        line = {"metric": "mmq_q4k_int8_gemm_throughput", "value": round(rate, 1), "unit": "TOP/s",
                "ms_per_step": round(ms, 5),
                "ms_relayout_every_call": round(ms_call, 5), "ms_raw_blocks": round(ms_raw, 5),
                "config": {"workload": f"Q4_K x Q8_1-MMQ int8 GEMM M {m} K {k} N {n}",
                           "weights": "slab relaid at load time (llmp_b200_q4k_relayout)"},
                "roofline": {"bound": "tensor", "achieved": round(rate, 1), "peak": peaks["i8"],
                             "unit": "TOP/s", "frac": round(rate / peaks["i8"], 4),
                             "peak_source": "bare tcgen05.mma loop measured on this pool"}}
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
        # load time, outside the timing: the gate | up slab interleaves its rows for the GLU
        # write-back (the third entry says so)
        slabs = (ops.q4k_relayout(gate_up, hidden, 2 * inter, glu=True),
                 ops.q4k_relayout(down, inter, hidden), True) \
            if tokens > ops.ops.DECODE_TOKENS else None
        fns = [lambda: ops.moe_ffn(x, ids_d, w_d, gate_up, down, hidden, inter, slabs=slabs)]
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


def _max_over_ranks(torch, dist, value: float) -> float:
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _all_true(torch, dist, flag: bool) -> bool:
    t = torch.tensor([1.0 if flag else 0.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item() > 0.5)


def bench_mmq_sharded(torch, dist, ops, rank, world, tokens=4096, steps=10, warmup=3, chunks=4):
    """The prefill GEMM N-column sharded (the benchmark specification's config 2).  Every rank holds the weight
    rows [rank * n / world, +n / world) (relaid into its slab at load time) and the whole
    activation batch, which it quantizes itself; the product runs in `chunks` token chunks,
    and each chunk's F32 slice is all-gathered over NVLink (NCCL) while the next chunk's
    product runs.  The gathered layout is [chunk][rank][tokens / chunks][n / world].  Strong
    scaling: the product is the same at every N.  Parity: rank 0 also holds the whole matrix
    and computes the unsharded product once, outside the timed region; the gathered result
    must equal it bit for bit."""
    from llmp_b200 import shard
    m, n, k = tokens, 14336, 4096
    lo, hi = shard.row_shard(n, world, rank, multiple=128)
    width = hi - lo
    if n % (world * 128) != 0 or m % chunks != 0:
        return {"unavailable": "column shards of unequal width are not benchmarked"}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)                               # the same operands on every rank
    x = torch.randn((m, k), device="cuda", generator=gen).bfloat16()
    w_full = make_q4k_device(torch, n, k, gen)
    w_mine = w_full[lo:hi].contiguous()
    slab = ops.q4k_relayout(w_mine, k, width)
    mc = m // chunks
    mine = [torch.empty((mc, width), device="cuda") for _ in range(chunks)]
    full = torch.empty((chunks, world, mc, width), device="cuda")
    if rank != 0:
        w_full = None

    def step():
        works = []
        for c in range(chunks):
            yq = ops.mmq_quantize(x[c * mc:(c + 1) * mc])
            ops.mmq(None, yq, k, width, out=mine[c], slab=slab)
            works.append(dist.all_gather_into_tensor(full[c], mine[c], async_op=True))
        for w in works:
            w.wait()
        return full

    def one_gpu():
        yq = ops.mmq_quantize(x)
        return ops.mmq(w_mine, yq, k, width, slab=slab)

    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, e0.elapsed_time(e1) / steps)
    # the shard's own product alone (no exchange), for the exchange's share of the step
    one_gpu()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        one_gpu()
    e1.record()
    torch.cuda.synchronize()
    compute_ms = _max_over_ranks(torch, dist, e0.elapsed_time(e1) / steps)
    parity = True
    if rank == 0:
        want = ops.mmq(w_full, ops.mmq_quantize(x), k, n, scratch=ops.mmq_scratch(k, n))  # [m, n]
        got = out.permute(0, 2, 1, 3).reshape(m, n)      # [chunk][rank][mc][width] -> [m][n]
        parity = bool(torch.equal(got, want))
    parity = _all_true(torch, dist, parity)
    rate = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    return {"metric": "mmq_q4k_int8_gemm_throughput", "value": round(rate, 1), "unit": "TOP/s",
            "ms_per_step": round(ms, 5), "shard_product_ms": round(compute_ms, 5), "n_gpus": world,
            "steps": steps, "warmup": warmup, "scaling": "strong", "parity": parity,
            "faults": ops.device_faults(),
            "config": {"workload": f"Q4_K x Q8_1-MMQ int8 GEMM M {m} K {k} N {n}",
                       "parallelism": f"N-column shards x{world} (slices of {width} columns), "
                                      f"activation quantizer on every rank, NCCL all-gather of the "
                                      f"F32 output ({m * n * 4 / 1e6:.0f} MB) in {chunks} token chunks "
                                      "behind the next chunk's product"},
            "roofline": {"bound": "tensor", "achieved": round(rate, 1), "peak": 4567.3 * world,
                         "unit": "TOP/s", "frac": round(rate / (4567.3 * world), 4),
                         "peak_source": "bare tcgen05.mma kind::i8 loop measured on this pool x N"}}


def bench_moe_ep(torch, dist, ops, rank, world, tokens=1024, steps=10, warmup=3):
    """Expert-parallel MoE block (the benchmark specification's config 4): each rank owns 128 / world whole experts
    (relaid into slabs at load time) and `tokens` tokens (weak scaling); rows travel to their
    experts' owners and back in NCCL all-to-alls of fixed size (llmp_b200.moe_ep_pack packs
    lanes of a set capacity, so no split size reaches the host) and are combined on the home
    rank in slot order by llmp_b200.moe_combine.  Parity: rank 0 also holds every expert and
    computes its own tokens' block on one GPU; the two results must be equal bit for bit."""
    import numpy as np

    from llmp_b200 import shard, synth
    experts, used, hidden, inter = 128, 8, 2048, 768
    if experts % world != 0:
        return {"unavailable": "experts must divide over the ranks"}
    per = experts // world
    gen = torch.Generator(device="cuda")
    gen.manual_seed(100)                              # the same experts on every rank
    gate_up_all = make_q4k_device(torch, experts * 2 * inter, hidden, gen).view(experts, 2 * inter, -1)
    down_all = make_q4k_device(torch, experts * hidden, inter, gen).view(experts, hidden, -1)
    b = rank * per
    gate_up = gate_up_all[b:b + per].contiguous()
    down = down_all[b:b + per].contiguous()
    slabs = (ops.q4k_relayout(gate_up, hidden, 2 * inter, glu=True),
             ops.q4k_relayout(down, inter, hidden), True)          # GLU in the product's write-back
    if rank != 0:
        gate_up_all = down_all = None
        torch.cuda.empty_cache()
    ids, w = synth.topk_route(np.random.default_rng(rank), tokens, experts, used)
    ids_d, w_d = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    gen.manual_seed(200 + rank)
    x = torch.randn((tokens, hidden), device="cuda", generator=gen)
    capacity = shard.ep_capacity(tokens, used, world)
    dropped = torch.zeros(1, dtype=torch.int32, device="cuda")
    ones = torch.ones((world * capacity, 1), device="cuda")

    def pack(xt, idt):
        return ops.moe_ep_pack(xt, idt, experts, world, capacity, dropped)

    def local(rows, local_ids):
        return ops.moe_ffn(rows, local_ids.view(-1, 1), ones, gate_up, down, hidden, inter,
                           decode_tokens=0, slabs=slabs)

    def combine(back, home, wt):
        return ops.moe_combine(back, home, wt, tokens, used)

    def step():
        return shard.ep_moe_ffn_padded(x, ids_d, w_d, experts, capacity, pack, local, combine)

    def one_gpu():   # the same rows through this rank's experts only: the compute of a step
        return local(torch.zeros((world * capacity, hidden), device="cuda"),
                     torch.arange(world * capacity, dtype=torch.int32, device="cuda") % per)

    for _ in range(warmup):
        out = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, e0.elapsed_time(e1) / steps)
    one_gpu()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        one_gpu()
    e1.record()
    torch.cuda.synchronize()
    compute_ms = _max_over_ranks(torch, dist, e0.elapsed_time(e1) / steps)
    lost = int(dropped.item())
    parity = lost == 0
    if rank == 0:
        want = ops.moe_ffn(x, ids_d, w_d, gate_up_all, down_all, hidden, inter, decode_tokens=0)
        parity = parity and bool(torch.equal(out, want))
    parity = _all_true(torch, dist, parity)
    ops_count = 3 * 2.0 * hidden * inter * tokens * used * world
    return {"metric": "moe_grouped_gemm_throughput", "unit": "TOP/s",
            "value": round(ops_count / (ms * 1e-3) / 1e12, 1), "ms_per_step": round(ms, 4),
            "local_block_ms": round(compute_ms, 4), "n_gpus": world, "steps": steps,
            "warmup": warmup, "scaling": "weak", "parity": parity, "rows_dropped": lost,
            "faults": ops.device_faults(),
            "config": {"workload": f"MoE block, 128 experts top-8, hidden 2048, intermediate 768, "
                                   f"Q4_K, {tokens} tokens a rank",
                       "parallelism": f"expert parallel x{world}: {per} experts a rank, NCCL "
                                      f"all-to-all dispatch and combine in lanes of {capacity} rows "
                                      "a destination, tokens data-parallel"}}


def bench_ffn_columns(torch, dist, ops, rank, world, batch, steps=5, warmup=2):
    """The decode step N-column sharded: every rank owns 1 / world of every matrix's output
    rows; the GLU output and the layer output are all-gathered (NCCL) inside the step.  Strong
    scaling.  Parity: rank 0 also holds whole matrices for two of the layers and computes
    them unsharded; the gathered outputs must equal them bit for bit."""
    if INTER % (world * 16) != 0 or HIDDEN % (world * 16) != 0:
        return {"unavailable": "rows do not divide over the ranks"}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4321)                             # the same matrices on every rank
    n_glu, n_down = INTER // world, HIDDEN // world
    check_layers = (0, LAYERS - 1)
    whole = {}
    layers = []
    for l in range(LAYERS):
        gate = make_q4k_device(torch, INTER, HIDDEN, gen)
        up = make_q4k_device(torch, INTER, HIDDEN, gen)
        down = make_q4k_device(torch, HIDDEN, INTER, gen)
        layers.append((gate[rank * n_glu:(rank + 1) * n_glu].contiguous(),
                       up[rank * n_glu:(rank + 1) * n_glu].contiguous(),
                       down[rank * n_down:(rank + 1) * n_down].contiguous()))
        if rank == 0 and l in check_layers:
            whole[l] = (gate, up, down)
        del gate, up, down
    x = torch.randn((LAYERS, batch, HIDDEN), device="cuda", generator=gen)
    T = ops.TYPE_Q4_K
    q8x = torch.empty((batch, ops.q8_1_row_blocks(HIDDEN) * 36), dtype=torch.uint8, device="cuda")
    q8h = torch.empty((batch, ops.q8_1_row_blocks(INTER) * 36), dtype=torch.uint8, device="cuda")
    h_shard = torch.empty((batch, n_glu), device="cuda")
    h_full = torch.empty((world, batch, n_glu), device="cuda")
    h_rows = torch.empty((batch, INTER), device="cuda")
    y_shard = torch.empty((batch, n_down), device="cuda")
    y_full = torch.empty((LAYERS, world, batch, n_down), device="cuda")
    h_seen = {}

    def step(keep=False):
        for l, (gate, up, down) in enumerate(layers):
            ops.quantize_q8(x[l], out=q8x)
            ops.vecq(up, T, HIDDEN, n_glu, q8x, batch, gate=gate, glu=ops.GLU_GEGLU, out=h_shard)
            dist.all_gather_into_tensor(h_full, h_shard)
            h_rows.view(batch, world, n_glu).copy_(h_full.transpose(0, 1))
            if keep and l in check_layers:
                h_seen[l] = h_rows.clone()
            ops.quantize_q8(h_rows, out=q8h)
            ops.vecq(down, T, INTER, n_down, q8h, batch, out=y_shard)
            dist.all_gather_into_tensor(y_full[l], y_shard)

    for _ in range(warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, e0.elapsed_time(e1) / steps)
    step(keep=True)
    torch.cuda.synchronize()
    # The F32 sums of a decode product are added in an order the launch geometry fixes, and
    # the geometry follows the rows a CTA owns, so a shard's sums agree with the whole
    # matrix's to rounding, not bit for bit: the bar is the path's 1e-5 of the output scale
    # (the down product is checked on the gathered GLU output itself).
    parity, bits, worst = True, True, 0.0
    if rank == 0:
        for l in check_layers:
            gate, up, down = whole[l]
            q = ops.quantize_q8(x[l])
            h = ops.vecq(up, T, HIDDEN, INTER, q, batch, gate=gate, glu=ops.GLU_GEGLU)
            y = ops.vecq(down, T, INTER, HIDDEN, ops.quantize_q8(h_seen[l]), batch)
            got_y = y_full[l].transpose(0, 1).reshape(batch, HIDDEN)
            for got, want in ((h_seen[l], h), (got_y, y)):
                err = float((got - want).abs().max() / want.abs().max())
                worst = max(worst, err)
                parity = parity and err <= 1e-5
                bits = bits and bool(torch.equal(got, want))
    parity = _all_true(torch, dist, parity)
    sb = step_bytes(batch)
    line = {"metric": METRIC, "value": round(sb / (ms * 1e-3) / 1e9, 2), "unit": UNIT,
            "ms_per_step": round(ms, 4), "n_gpus": world, "steps": steps, "warmup": warmup,
            "scaling": "strong", "parity": parity, "parity_bar": "1e-5 of the output scale",
            "max_rel_err": worst, "bit_equal": bits, "faults": ops.device_faults(),
            "config": {"workload": f"Gemma-3-4B FFN decode products, Q4_K, {LAYERS} layers, batch {batch}",
                       "parallelism": f"N-column shards x{world}, NCCL all-gather of the GLU output "
                                      "and of the layer output, plain stream launches"}}
    if batch == 1:
        for key, in_band in (("peer_stores", False), ("peer_words", True)):
            try:
                line[key] = _ffn_columns_peer(torch, dist, ops, rank, world, layers, whole, check_layers,
                                              x, n_glu, n_down, steps=20, warmup=3, in_band=in_band)
            except Exception as e:                   # the NCCL form above stands by itself
                line[key] = {"unavailable": repr(e)[:200]}
    return line


def _ffn_columns_peer(torch, dist, ops, rank, world, layers, whole, check_layers, x, n_glu, n_down,
                      steps, warmup, in_band):
    """The same sharded step with no collective library in it: each shard product's slice is
    stored into every rank's copy of the vector by llmp_b200_peer_publish (plain peer stores
    into CUDA-IPC mapped memory) and the next quantizer starts by waiting, with a bound, for
    every rank's flag.  No NCCL call inside the step, so the step is one replayed CUDA graph.
    The layers' inputs are independent, as in the one-GPU step, but every layer waits for the
    layer before's output exchange: that is what lets one gathered buffer be reused.
    in_band: the product kernels themselves store their rows, as tagged 8-byte words, into every
    rank's vector (llmp_b200_vecq_fan) and the quantizers poll the words they read: no flag
    words, no fence, no publishing step."""
    from llmp_b200 import peer
    T = ops.TYPE_Q4_K
    ex = peer.PeerExchange(world, rank, {"h": INTER, "y": LAYERS * HIDDEN}, sites=2 * LAYERS,
                           words={"hw": INTER, "yw": LAYERS * HIDDEN})
    everyone = [None] * world
    dist.all_gather_object(everyone, ex.handles())
    ex.connect(everyone)
    polls = 1 << 24                                  # about 1.7 s: ranks start a step together
    q8x = torch.empty((1, ops.q8_1_row_blocks(HIDDEN) * 36), dtype=torch.uint8, device="cuda")
    q8h = torch.empty((1, ops.q8_1_row_blocks(INTER) * 36), dtype=torch.uint8, device="cuda")
    h_shard = torch.empty((1, n_glu), device="cuda")
    y_shard = torch.empty((1, n_down), device="cuda")
    h_seen = {}

    def step_words(keep=False):
        # Four launches a layer and nothing between a product's stores and the next rank's
        # reads but NVLink: tags 2l (GLU output) and 2l + 1 (layer output).
        ex.begin_step()
        for l, (gate, up, down) in enumerate(layers):
            if l == 0:
                ops.quantize_q8(x[0], out=q8x)
            else:       # back-pressure: layer l - 1's output has reached this rank from everyone
                ex.quantize_words(q8x, x=x[l], hold=("yw", (l - 1) * HIDDEN, HIDDEN, (2 * l) - 1),
                                  polls=polls)
            ops.vecq(up, T, HIDDEN, n_glu, q8x, 1, gate=gate, glu=ops.GLU_GEGLU, out=h_shard,
                     fan=ex.fan("hw", rank * n_glu, 2 * l))
            ex.quantize_words(q8h, name="hw", first=0, count=INTER, tag=2 * l, polls=polls)
            if keep and l in check_layers:
                h_seen[l] = ex.word_values("hw", 0, INTER)
            ops.vecq(down, T, INTER, n_down, q8h, 1, out=y_shard,
                     fan=ex.fan("yw", (l * HIDDEN) + (rank * n_down), (2 * l) + 1))
        last = LAYERS - 1
        ex.quantize_words(q8x, x=x[0], hold=("yw", last * HIDDEN, HIDDEN, (2 * last) + 1), polls=polls)

    def step_flags(keep=False):
        # Four launches a layer, as on one GPU: each quantizer first stores the product
        # before's slice into every rank's vector, then waits for all of them.
        ex.begin_step()
        for l, (gate, up, down) in enumerate(layers):
            if l == 0:
                ops.quantize_q8(x[0], out=q8x)
            else:       # layer l - 1's output goes out; back-pressure: it is out everywhere
                ex.exchange_quantize_q8("y", 2 * l - 1, y_shard.view(-1),
                                        ((l - 1) * HIDDEN) + (rank * n_down), q8x, polls, x=x[l])
            ops.vecq(up, T, HIDDEN, n_glu, q8x, 1, gate=gate, glu=ops.GLU_GEGLU, out=h_shard)
            ex.exchange_quantize_q8("h", 2 * l, h_shard.view(-1), rank * n_glu, q8h, polls)
            if keep and l in check_layers:
                h_seen[l] = ex.vectors["h"].clone()
            ops.vecq(down, T, INTER, n_down, q8h, 1, out=y_shard)
        last = LAYERS - 1
        ex.publish("y", (2 * last) + 1, y_shard.view(-1), (last * HIDDEN) + (rank * n_down))
        ex.wait("y", (2 * last) + 1, polls)

    step = step_words if in_band else step_flags
    dist.barrier()
    torch.cuda.synchronize()
    step()                                           # plain launches once
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.synchronize()
    dist.barrier()
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = _max_over_ranks(torch, dist, e0.elapsed_time(e1) / steps)
    timed_out = ex.timed_out()
    dist.barrier()
    step(keep=True)
    torch.cuda.synchronize()
    timed_out = timed_out or ex.timed_out()
    parity, worst = True, 0.0
    if rank == 0:
        for l in check_layers:
            gate, up, down = whole[l]
            h = ops.vecq(up, T, HIDDEN, INTER, ops.quantize_q8(x[l]), 1, gate=gate, glu=ops.GLU_GEGLU)
            y = ops.vecq(down, T, INTER, HIDDEN, ops.quantize_q8(h_seen[l].view(1, -1)), 1)
            got_y = (ex.word_values("yw", l * HIDDEN, HIDDEN) if in_band
                     else ex.vectors["y"][l * HIDDEN:(l + 1) * HIDDEN]).view(1, -1)
            for got, want in ((h_seen[l].view(1, -1), h), (got_y, y)):
                err = float((got - want).abs().max() / want.abs().max())
                worst = max(worst, err)
                parity = parity and err <= 1e-5
    parity = _all_true(torch, dist, parity and not timed_out)
    dist.barrier()
    ex.close()
    return {"value": round(step_bytes(1) / (ms * 1e-3) / 1e9, 2), "unit": UNIT,
            "ms_per_step": round(ms, 4), "steps": steps, "warmup": warmup, "parity": parity,
            "parity_bar": "1e-5 of the output scale", "max_rel_err": worst,
            "waits_timed_out": bool(timed_out), "faults": ops.device_faults(),
            "launch": "cuda graph replay, no collective library in the step",
            "parallelism": (f"N-column shards x{world}; the product kernels store their rows as tagged "
                            "8-byte words into every rank's vector (CUDA IPC, plain peer stores); "
                            "readers poll the words with a bound") if in_band else
                           (f"N-column shards x{world}; each slice stored into every rank's vector "
                            "(CUDA IPC, plain peer stores) and flagged; consumers wait with a bound")}


def run_sharded_only(args, rank: int, world: int, local_rank: int, which: str):
    """--workload mmq_q4k | moe under torchrun: that sharded form alone, one JSON line."""
    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import llmp_b200 as ops
    if which == "mmq_q4k":
        line = bench_mmq_sharded(torch, dist, ops, rank, world, tokens=args.tokens or 4096,
                                 steps=args.steps, warmup=max(args.warmup, 3))
    else:
        line = bench_moe_ep(torch, dist, ops, rank, world, tokens=args.tokens or 1024,
                            steps=args.steps, warmup=max(args.warmup, 3))
    if rank == 0:
        line.update({"higher_is_better": True, "data": "synthetic", "vs_baseline": None})
        print(json.dumps(line), flush=True)
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
                    choices=["ffn_q4k", "q8_0_gemv", "decode_vector", "mxfp8_gemm", "mmq_q4k", "moe"],
                    help="ffn_q4k is the bench line; the others time the other configs' kernels")
    ap.add_argument("--tokens", type=int, default=0,
                    help="tokens / rows of the other workloads")
    ap.add_argument("--q8-out", action="store_true",
                    help="the gate/up product also writes its output's Q8_1 blocks "
                         "(llmp_b200_vecq_q8): one launch fewer a layer, measured slower")
    ap.add_argument("--fused", action="store_true",
                    help="llmp_b200_vecq_f32: each product quantizes its F32 input itself (two "
                         "launches a layer instead of four; measured slower: 0.67 ms a step "
                         "against 0.57, the per-CTA quantization sits on the critical path)")
    ap.add_argument("--shard", default="replicas", choices=["replicas", "columns"],
                    help="N > 1: replicas (each GPU its own batch, weak scaling) or columns "
                         "(rows of every matrix split, NCCL all-gather, strong scaling)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--repeats", type=int, default=10,
                    help="the timed block of --steps steps is repeated this often; the median counts")
    ap.add_argument("--no-sharded", action="store_true",
                    help="N > 1: skip the sharded forms (replicas only)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--traffic", type=float, default=None,
                    help="dram bytes per launch of the dominant kernel from an ncu capture "
                         "(default: the captured figure at batch 1)")
    args = ap.parse_args()
    LAYERS = args.layers
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload in ("moe", "mmq_q4k") and world > 1:
        run_sharded_only(args, rank, world, local_rank, args.workload)
        return
    if args.workload != "ffn_q4k":
        if rank == 0:
            run_other(args)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
