#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (metric: Q4_K GEMV HBM GB/s): the decode GEMV of BASELINE.json's first
config — Q4_K weight [4096, 4096] x f32 activation row — run over a ring of 64 distinct
weights (604 MB, larger than the 126 MB L2) so every launch streams from HBM.  One step =
one pass over the ring = 64 GEMV launches replayed from a CUDA graph.  Weights are resident
in HBM before the timed region (the engine uploads weights once at load).

`value` is device-timed with CUDA events on the launching stream; `e2e` is the same pass
through the C ABI with HOST activations and results (pinned host -> device copy of the 64
activation rows, 64 GEMVs, device -> host copy of the 64 result rows, every step).

With --impl reference the reference's own CPU path (the oracle restatement of matvec_kq,
all host threads) is timed on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_ROWS = K_COLS = 4096
RING = 64
Q4K_BYTES = N_ROWS * K_COLS // 256 * 144                      # GGUF bytes of one weight
ALGO_BYTES_PER_LAUNCH = Q4K_BYTES + 4 * K_COLS + 4 * N_ROWS      # weight + x + y (f32)
METRIC = "Q4_K GEMV HBM GB/s"
WORKLOAD = "q4k_gemv_n4096_k4096_m1_ring64"


def measured_peaks() -> tuple[float, float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples nvidia-smi (read-only queries, every 50 ms) from before the warm-up on; `begin()` / `end()` mark the timed
    region and the summary uses the samples that arrived inside it.  A region shorter than a few samples is followed by
    the same load, untimed, until three samples are in (`keep_loaded`), and the summary says so."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        import threading
        self.index = index
        self.rows = []            # (arrival time, fields)
        self.t0 = self.t1 = None
        self.extended = False
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def inside(self):
        t1 = self.t1 if self.t1 is not None else time.time()
        return [line for t, line in self.rows if self.t0 is not None and self.t0 <= t <= t1 + 0.02]

    def keep_loaded(self, run_step, sync, extra_steps: int):
        """The timed region is over; if it was too short for a few samples, the caller keeps the same load running for
        `extra_steps` more steps (the same number on every rank) and the window is extended over them."""
        if extra_steps <= 0:
            return
        for _ in range(extra_steps):
            run_step()
        sync()
        self.t1 = time.time()
        self.extended = True

    def close(self):
        if not self.proc:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.inside():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.summary = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                            "window": "timed region, then the same load untimed until 3 samples" if self.extended else "timed region"}


# ------------------------------------------------------------------------------ inputs
def ring_weights(count: int, seed: int) -> list[np.ndarray]:
    """`count` distinct Q4_K [4096, 4096] weights: N(0, 0.02) quantized with the library's
    test-input encoder (the first from `seed`), the rest row-rotations of a few bases
    so set-up stays short; HBM streaming only needs distinct bytes at distinct addresses."""
    import ojas_engine_b200 as ob
    bases = []
    for b in range(4):
        rng = np.random.default_rng(seed + b)
        w = rng.standard_normal((N_ROWS, K_COLS), dtype=np.float32) * np.float32(0.02)
        bases.append(ob.encode(ob.Q4_K, w).reshape(N_ROWS, -1))
    out = []
    for i in range(count):
        out.append(np.ascontiguousarray(np.roll(bases[i % 4], 97 * (i // 4), axis=0)).reshape(-1))
    return out


# ------------------------------------------------------------------------------ CPU arm
def cpu_reference_pass(weights: list[np.ndarray], x: np.ndarray, seconds: float, threads: int, native: bool):
    """Times the oracle's matvec_kq over a bounded sample; returns (GB/s, matvecs, elapsed)."""
    import oracle
    import ojas_engine_b200 as ob
    oracle.matvec_kq(weights[0], ob.Q4_K, N_ROWS, K_COLS, x[0], threads, native)  # warm-up
    done, t0 = 0, time.perf_counter()
    while True:
        i = done % len(weights)
        oracle.matvec_kq(weights[i], ob.Q4_K, N_ROWS, K_COLS, x[i % x.shape[0]], threads, native)
        done += 1
        el = time.perf_counter() - t0
        if el >= seconds:
            break
    return done * ALGO_BYTES_PER_LAUNCH / el / 1e9, done, el


def oracle_native_ok() -> bool:
    try:
        import oracle
        oracle.lib(native=True)
        return True
    except Exception:
        return False


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    native = oracle_native_ok()
    import oracle
    # This arm runs the CPU code only: its weights are the oracle's own block generator (the CPU time of a block dot
    # does not depend on the values), so the CUDA library is never loaded here.
    base = oracle.synth_blocks(oracle.Q4_K, N_ROWS * K_COLS // 256).reshape(N_ROWS, -1)
    weights = [np.ascontiguousarray(np.roll(base, 97 * i, axis=0)).reshape(-1) for i in range(4)]
    x = np.random.default_rng(1).standard_normal((4, K_COLS), dtype=np.float32)
    per_step = 8  # matvecs per step: a bounded sample of the 64-weight pass
    for _ in range(max(args.warmup, 1)):
        oracle.matvec_kq(weights[0], oracle.Q4_K, N_ROWS, K_COLS, x[0], threads, native)
    t0 = time.perf_counter()
    for s in range(args.steps):
        for j in range(per_step):
            oracle.matvec_kq(weights[j % 4], oracle.Q4_K, N_ROWS, K_COLS, x[j % 4], threads, native)
    el = time.perf_counter() - t0
    gbs = args.steps * per_step * ALGO_BYTES_PER_LAUNCH / el / 1e9
    sample = f"{per_step} of the {RING} ring GEMVs per step, oracle matvec_kq ({'-march=native' if native else 'portable'} build)"
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x u4 block dots, f32 combine", "data": "synthetic",
        "config": {"workload": WORKLOAD, "where": "host CPU"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------ GPU arm
def time_graph(gpu, graph, steps: int, warmup: int) -> float:
    for _ in range(warmup):
        gpu.graph_launch(graph)
    gpu.sync()
    e0, e1 = gpu.event(), gpu.event()
    gpu.record(e0)
    for _ in range(steps):
        gpu.graph_launch(graph)
    gpu.record(e1)
    gpu.sync()
    return gpu.elapsed_ms(e0, e1)


def extra_gemv(gpu, ob, ggml_type: int, n: int, k: int, m: int, peak: float, tag: str) -> dict:
    """One more GEMV shape, ring sized past L2, timed the same way (reported, not the headline)."""
    import oracle
    gguf = ob.raw_bytes(ggml_type, n, k)
    ring = max(2, int(300e6 // gguf) + 1)
    base = oracle.synth_blocks(ggml_type, n * k // (32 if ggml_type == ob.Q8_0 else 256)).reshape(n, -1)
    ws = [gpu.load_weight(np.ascontiguousarray(np.roll(base, 13 * i, axis=0)), ggml_type, n, k) for i in range(ring)]
    x = gpu.upload(np.random.default_rng(7).standard_normal((m, k), dtype=np.float32))
    y = gpu.alloc(m * n)
    gpu.gemv(ws[0], x, y, m)
    gpu.sync()
    gpu.graph_begin()
    for w in ws:
        gpu.gemv(w, x, y, m)
    g = gpu.graph_end()
    reps = max(3, int(2000 // ring))
    ms = time_graph(gpu, g, reps, 3)
    gpu.graph_destroy(g)
    per_launch_us = ms * 1e3 / (reps * ring)
    algo = gguf + 4 * m * (k + n)
    gbs = algo / (per_launch_us * 1e-6) / 1e9
    for w in ws:
        gpu.free(w.buf)
    gpu.free(x)
    gpu.free(y)
    return {"workload": f"{tag}_gemv_n{n}_k{k}_m{m}", "us_per_launch": round(per_launch_us, 3), "GB/s": round(gbs, 1),
            "frac_of_peak": round(gbs / peak, 4), "ring": ring}


def decode_layer_case(gpu, ob, peak: float) -> dict:
    """The matmul chain of one decode step of an 8B-shaped layer (d = 4096, ffn = 14336, 32 / 8 heads): fused Q|K|V GEMV
    (6144 rows) with the RMSNorm in its prologue, O projection, fused gate|up GEMV (28672 rows) with the RMSNorm in its
    prologue, SiLU * up -> Q8_K, down (Q6_K); also timed with the norms as launches of their own (RMSNorm -> Q8_K) and
    with SiLU * up in the down projection's prologue as well (slower: every CTA repeats the exponentials).  Three layers of distinct weights (414 MB > L2) in one
    CUDA graph; attention itself is not on this path (the O projection reads the first 4096 QKV outputs instead)."""
    import oracle
    d, ffn, nq = 4096, 14336, 6144
    nsb_d, nsb_f = d // 256, ffn // 256

    def weight(t, n, k, roll):
        base = oracle.synth_blocks(t, n * k // 256).reshape(n, -1)
        return gpu.load_weight(np.ascontiguousarray(np.roll(base, roll, axis=0)), t, n, k)

    layers = [(weight(ob.Q4_K, nq, d, 7 * i), weight(ob.Q4_K, d, d, 11 * i), weight(ob.Q4_K, 2 * ffn, d, 13 * i), weight(ob.Q6_K, d, ffn, 17 * i))
              for i in range(3)]
    rng = np.random.default_rng(3)
    x = gpu.upload(rng.standard_normal(d, dtype=np.float32))
    nw = gpu.upload(np.ones(d, np.float32))
    q_d, s_d, b_d = gpu.alloc_bytes(d), gpu.alloc(nsb_d), gpu.alloc_bytes(nsb_d * 8 * 4)
    q_f, s_f, b_f = gpu.alloc_bytes(ffn), gpu.alloc(nsb_f), gpu.alloc_bytes(nsb_f * 8 * 4)
    qkv, attn, gu, y = gpu.alloc(nq), gpu.alloc(d), gpu.alloc(2 * ffn), gpu.alloc(d)
    g_view, u_view = ob.Buf(gu.ptr, ffn * 4), ob.Buf(gu.ptr + ffn * 4, ffn * 4)

    def chain():
        for wqkv, wo, wgu, wdn in layers:
            if fused_norm:
                gpu.gemv_rmsnorm(wqkv, x, nw, 1e-5, qkv)
                gpu.gemv(wo, qkv, attn)
                gpu.gemv_rmsnorm(wgu, attn, nw, 1e-5, gu)
            else:
                gpu.rmsnorm_q8k(x, nw, 1e-5, 1, d, q_d, s_d, b_d)
                gpu.gemv_q8k(wqkv, q_d, s_d, b_d, qkv)
                gpu.gemv(wo, qkv, attn)
                gpu.rmsnorm_q8k(attn, nw, 1e-5, 1, d, q_d, s_d, b_d)
                gpu.gemv_q8k(wgu, q_d, s_d, b_d, gu)
            if fused_norm == 2:
                gpu.gemv_silu_mul(wdn, g_view, u_view, y)
            else:
                gpu.silu_mul_q8k(g_view, u_view, 1, ffn, q_f, s_f, b_f)
                gpu.gemv_q8k(wdn, q_f, s_f, b_f, y)

    us = {}
    for fused_norm in (0, 1, 2):        # producers as launches of their own; norms in the GEMV prologues; SwiGLU too
        chain()
        gpu.sync()
        gpu.graph_begin()
        chain()
        g = gpu.graph_end()
        ms = time_graph(gpu, g, 300, 5)
        gpu.graph_destroy(g)
        us[fused_norm] = ms * 1e3 / 300 / len(layers)
    us_layer = us[1]
    gguf = ob.raw_bytes(ob.Q4_K, nq, d) + ob.raw_bytes(ob.Q4_K, d, d) + ob.raw_bytes(ob.Q4_K, 2 * ffn, d) + ob.raw_bytes(ob.Q6_K, d, ffn)
    for lay in layers:
        for w in lay:
            gpu.free(w.buf)
    for b in (x, nw, q_d, s_d, b_d, q_f, s_f, b_f, qkv, attn, gu, y):
        gpu.free(b)
    return {"workload": "decode_layer_d4096_ffn14336_q4k_q6k_m1", "us_per_layer": round(us_layer, 2), "launches_per_layer": 5,
            "us_per_layer_with_separate_producer_launches": round(us[0], 2), "us_per_layer_with_swiglu_fused_too": round(us[2], 2),
            "GB/s": round(gguf / us_layer / 1e3, 1), "frac_of_peak": round(gguf / us_layer / 1e3 / peak, 4), "weight_bytes": gguf}


def run_ours(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist  # plumbing only: barrier, max over ranks, the all-gather
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import ojas_engine_b200 as ob

    hbm_peak, _, peak_kind = measured_peaks()
    gpu = ob.B200Gpu(local)
    if args.no_pdl:
        gpu.set_option("pdl", 0)
    raws = ring_weights(RING, seed=rank * 1000)
    weights = [gpu.load_weight(r, ob.Q4_K, N_ROWS, K_COLS) for r in raws]
    rng = np.random.default_rng(1 + rank)
    x_host = gpu.host_alloc(RING * K_COLS * 4, np.float32)
    x_host[:] = rng.standard_normal(RING * K_COLS, dtype=np.float32)
    y_host = gpu.host_alloc(RING * N_ROWS * 4, np.float32)
    xd = gpu.upload(x_host)
    yd = gpu.alloc(RING * N_ROWS)

    # multi-GPU: each rank owns the row shard [rank*4096, (rank+1)*4096) of a [world*4096, 4096] projection per ring
    # slot (column-parallel).  The step's 64 outputs of a rank are joined by ONE all-gather kernel of this library:
    # it stores them into every rank's receive window (peer stores over NVLink), raises a flag, waits with a limit
    # for the other ranks and copies out y_all [world][64][4096].  No other data-path exchange, no NCCL call inside
    # the timed region; the whole step is one CUDA graph.
    group = y_all = None
    if dist is not None:
        from ojas_engine_b200 import tp as obtp

        def exchange(blob):
            out = [None] * world
            dist.all_gather_object(out, blob)
            return out

        group = obtp.TpGroup(gpu, world, rank, RING * N_ROWS, exchange)
        y_all = gpu.alloc(world * RING * N_ROWS)

    def launch_pass():
        for i, w in enumerate(weights):
            xi = ob.Buf(xd.ptr + i * K_COLS * 4, K_COLS * 4)
            gpu.gemv(w, xi, ob.Buf(yd.ptr + i * N_ROWS * 4, N_ROWS * 4), 1)
        if group is not None:
            group.allgather(yd, RING * N_ROWS, y_all)

    launch_pass()  # outside capture: one-time function attribute set-up
    gpu.sync()
    l0 = gpu.launch_count
    gpu.graph_begin()
    launch_pass()
    graph = gpu.graph_end()
    launches_per_step = gpu.launch_count - l0

    def step():
        gpu.graph_launch(graph)

    clocks = ClockSampler(local)
    for _ in range(args.warmup):
        step()
    gpu.sync()
    if dist is not None:
        import torch
        torch.cuda.synchronize()
        dist.barrier()
    e0, e1 = gpu.event(), gpu.event()
    clocks.begin()
    gpu.record(e0)
    for _ in range(args.steps):
        step()
    gpu.record(e1)
    gpu.sync()
    clocks.end()
    if dist is not None:
        import torch
        torch.cuda.synchronize()
        dist.barrier()
    ms = gpu.elapsed_ms(e0, e1)
    if dist is not None:
        import torch
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # a timed region shorter than 0.3 s gives nvidia-smi (50 ms period) too few samples: the same steps go on, untimed,
    # until 0.3 s of load have passed (the count follows from the reduced time, so it is the same on every rank)
    extra = int(math.ceil((300.0 - ms) / max(ms / args.steps, 1e-3))) if ms < 300.0 else 0
    clocks.keep_loaded(step, gpu.sync, min(extra, 20000))
    clocks.close()
    ms_per_step = ms / args.steps
    bytes_per_step_all = world * RING * ALGO_BYTES_PER_LAUNCH
    value = bytes_per_step_all / (ms_per_step * 1e-3) / 1e9
    us_per_launch = ms_per_step * 1e3 / RING
    achieved = ALGO_BYTES_PER_LAUNCH / (us_per_launch * 1e-6) / 1e9

    # parity spot check of the timed buffers against the oracle (not timed)
    parity = None
    if rank == 0:
        import oracle
        want = oracle.matvec_kq(raws[0], ob.Q4_K, N_ROWS, K_COLS, np.asarray(x_host[:K_COLS]))
        if group is None:
            got = gpu.read(yd, np.float32, N_ROWS)
        else:
            # the JOINED result: this rank's own shard, and the shard the last rank pushed into this rank's window
            got = gpu.read(y_all, np.float32, N_ROWS, byte_offset=rank * RING * N_ROWS * 4)
            peer = world - 1
            praw = ring_weights(1, seed=peer * 1000)[0]
            px = np.random.default_rng(1 + peer).standard_normal(RING * K_COLS, dtype=np.float32)[:K_COLS]
            pwant = oracle.matvec_kq(praw, ob.Q4_K, N_ROWS, K_COLS, px)
            pgot = gpu.read(y_all, np.float32, N_ROWS, byte_offset=peer * RING * N_ROWS * 4)
            want, got = np.concatenate([want, pwant]), np.concatenate([got, pgot])
        parity = float(np.linalg.norm(got - want) / np.linalg.norm(want))

    # end to end through the C ABI with host buffers: H2D of the step's activations, the pass,
    # D2H of the step's results, one synchronisation per step.
    e2e = None
    if rank == 0 or dist is not None:
        gpu.graph_begin()
        gpu._ck(gpu._l.ojas_b200_upload(gpu.ctx, xd.ptr, x_host.ctypes.data, x_host.nbytes))
        launch_pass()
        gpu._ck(gpu._l.ojas_b200_download(gpu.ctx, y_host.ctypes.data, yd.ptr, y_host.nbytes))
        g2 = gpu.graph_end()
        for _ in range(max(3, args.warmup)):
            gpu.graph_launch(g2)
            gpu.sync()
        if dist is not None:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            gpu.graph_launch(g2)
            gpu.sync()
        el = time.perf_counter() - t0
        if dist is not None:
            import torch
            t = torch.tensor([el], dtype=torch.float64, device=f"cuda:{local}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            el = float(t.item())
        e2e = {"value": bytes_per_step_all * args.steps / el / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": int(x_host.nbytes) * world, "d2h_bytes_per_step": int(y_host.nbytes) * world,
               "ms_per_step": el / args.steps * 1e3}
        gpu.graph_destroy(g2)

    tp_rows = None
    if dist is not None and not args.no_extras:
        try:
            tp_rows = tp70b_rows(gpu, dist, rank, world, local, 5)
        except Exception as exc:      # every rank runs the same sequence; a failure is reported, not fatal to the headline
            tp_rows = [{"case": "tp70b", "error": str(exc)}]
    if rank == 0:
        cpu = None
        extras = []
        if tp_rows is not None:
            extras.append({"workload": f"llama70b_projections_sharded_x{world}", "rows": tp_rows})
        if world == 1:
            threads = os.cpu_count() or 1
            native = oracle_native_ok()
            gbs, n_mv, el = cpu_reference_pass(raws[:8], np.asarray(x_host).reshape(RING, K_COLS), 10.0, threads, native)
            cpu = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                   "sample": f"{n_mv} matvec_kq calls over 8 of the ring weights in {el:.1f} s ({'-march=native' if native else 'portable'} oracle build)"}
            if not args.no_extras:
                for (t, n, k, m, tag) in [(ob.Q4_K, 28672, 8192, 1, "q4k"), (ob.Q4_K, 14336, 4096, 1, "q4k"),
                                          (ob.Q6_K, 14336, 4096, 1, "q6k"), (ob.Q6_K, 4096, 14336, 1, "q6k"),
                                          (ob.Q8_0, 14336, 4096, 1, "q80"), (ob.Q8_0, 4096, 14336, 1, "q80"),
                                          (ob.Q4_K, 4096, 4096, 8, "q4k"), (ob.Q6_K, 14336, 4096, 8, "q6k"),
                                          (ob.Q8_0, 14336, 4096, 8, "q80"), (ob.Q8_0, 4096, 14336, 8, "q80")]:
                    try:
                        extras.append(extra_gemv(gpu, ob, t, n, k, m, hbm_peak, tag))
                    except Exception as exc:  # an extra must not take the headline down
                        extras.append({"workload": f"{tag}_gemv_n{n}_k{k}_m{m}", "error": str(exc)})
            if not args.no_extras:
                _, tc_peak, _ = measured_peaks()
                for (tag, m, n, k) in [("q4k", 512, 4096, 4096), ("q4k", 512, 14336, 4096), ("q4k", 512, 4096, 14336),
                                       ("q4k", 2048, 14336, 4096), ("q4k", 128, 4096, 4096), ("q4k", 512, 28672, 8192),
                                       ("q6k", 512, 8192, 28672), ("q6k", 512, 14336, 4096), ("q80", 512, 14336, 4096)]:
                    try:
                        extras.append(gemm_case(gpu, ob, tag, m, n, k, 10, 3, tc_peak))
                    except Exception as exc:
                        extras.append({"workload": f"{tag}_gemm_m{m}_n{n}_k{k}", "error": str(exc)})
                try:
                    extras.append(decode_layer_case(gpu, ob, hbm_peak))
                except Exception as exc:
                    extras.append({"workload": "decode_layer", "error": str(exc)})
                # config 4 as stated; the same with Q6_K experts; a prefill-sized batch in the prefill form
                for tokens, rows, t_exp in ((64, 0, ob.Q4_K), (64, 0, ob.Q6_K), (2048, 32, ob.Q4_K)):
                    try:
                        extras.append(moe_case(gpu, ob, 20, 3, hbm_peak, tc_peak, tokens, rows, t_exp))
                    except Exception as exc:
                        extras.append({"workload": f"moe_m{tokens}", "error": str(exc)})
        traffic = profile_traffic()
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 x u4 block dots (exact int32), f32 combine", "data": "synthetic",
            "config": {"workload": WORKLOAD, "ring_bytes": RING * Q4K_BYTES, "l2": "inputs larger than L2 (ring of 64 weights, 604 MB)",
                       "launch": "CUDA graph of 64 kernel launches per step",
                       "parallelism": "single GPU" if world == 1 else f"column-parallel row shards x{world}; one all-gather kernel per step (peer stores over NVLink + bounded-wait join, no NCCL in the timed region)"},
            "pct_of_8TBps": value / world / 8000.0,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": traffic, "peak_kind": f"of {peak_kind}", "kernel": "gemv_kernel<Q4_K, 1 row, f32 activations>",
                         "algorithmic_bytes_per_launch": ALGO_BYTES_PER_LAUNCH, "us_per_launch": us_per_launch},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks.summary, "parity_rel_l2_vs_oracle": parity, "extras": extras,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    gpu.close()


def run_case(args) -> None:
    """One GEMV shape on one GPU: `--case q4k:4096:4096:1 [--ring R] [--no-graph]`.  The mode the
    ncu captures and the shape sweeps use; prints one JSON line."""
    import ojas_engine_b200 as ob
    import oracle
    if args.case.startswith("gemm:"):
        return run_gemm_case(args)
    if args.case == "tp70b":
        return run_tp70b(args)
    if args.case == "layer":
        hbm_peak, _, _ = measured_peaks()
        gpu = ob.B200Gpu(0)
        print(json.dumps(decode_layer_case(gpu, ob, hbm_peak)))
        gpu.close()
        return
    if args.case == "moe" or args.case.startswith("moe:"):
        import ojas_engine_b200 as ob
        hbm_peak, tc_peak, _ = measured_peaks()
        gpu = ob.B200Gpu(0)
        for kv in args.opt:
            gpu.set_option(kv.split("=")[0], int(kv.split("=")[1]))
        parts = args.case.split(":")          # moe[:TOKENS[:GEMM_ROWS[:q4k|q6k]]]
        print(json.dumps(moe_case(gpu, ob, args.steps, args.warmup, hbm_peak, tc_peak, int(parts[1]) if len(parts) > 1 else 64,
                                  int(parts[2]) if len(parts) > 2 else 0, ob.Q6_K if len(parts) > 3 and parts[3] == "q6k" else ob.Q4_K)))
        gpu.close()
        return
    tag, n, k, m = args.case.split(":")
    n, k, m = int(n), int(k), int(m)
    t = {"q4k": ob.Q4_K, "q5k": ob.Q5_K, "q6k": ob.Q6_K, "q80": ob.Q8_0, "iq4nl": ob.IQ4_NL, "iq4xs": ob.IQ4_XS}[tag]
    hbm_peak, _, peak_kind = measured_peaks()
    gpu = ob.B200Gpu(0)
    if args.no_pdl:
        gpu.set_option("pdl", 0)
    if args.warps:
        gpu.set_option("gemv_warps", args.warps)
    if args.stages:
        gpu.set_option("gemv_stages", args.stages)
    for kv in args.opt:
        gpu.set_option(kv.split("=")[0], int(kv.split("=")[1]))
    gguf = ob.raw_bytes(t, n, k)
    ring = args.ring or max(2, int(300e6 // gguf) + 1)
    base = oracle.synth_blocks(t, n * k // oracle.block_shape(t)[1]).reshape(n, -1)
    ws = [gpu.load_weight(np.ascontiguousarray(np.roll(base, 13 * i, axis=0)), t, n, k) for i in range(ring)]
    x = gpu.upload(np.random.default_rng(7).standard_normal((m, k), dtype=np.float32))
    y = gpu.alloc(m * n)

    def one_pass():
        for w in ws:
            gpu.gemv(w, x, y, m)

    one_pass()
    gpu.sync()
    graph = None
    if not args.no_graph:
        gpu.graph_begin()
        one_pass()
        graph = gpu.graph_end()
    run = (lambda: gpu.graph_launch(graph)) if graph else one_pass
    for _ in range(args.warmup):
        run()
    gpu.sync()
    e0, e1 = gpu.event(), gpu.event()
    gpu.record(e0)
    for _ in range(args.steps):
        run()
    gpu.record(e1)
    gpu.sync()
    us = gpu.elapsed_ms(e0, e1) * 1e3 / (args.steps * ring)
    algo = gguf + 4 * m * (k + n)
    gbs = algo / (us * 1e-6) / 1e9
    print(json.dumps({"case": args.case, "ring": ring, "graph": graph is not None, "pdl": not args.no_pdl, "us_per_launch": us, "GB/s": gbs,
                      "frac": gbs / hbm_peak, "peak_kind": peak_kind, "algorithmic_bytes": algo}))
    gpu.close()


def gemm_case(gpu, ob, tag: str, m: int, n: int, k: int, steps: int, warmup: int, tc_peak: float, ksplit: int = 0, graph: bool = True) -> dict:
    """Times the tensor-core prefill GEMM (activation preparation + MMA kernel per call), by default as replays of a
    CUDA graph over a ring of weights (graph = False: eager launches, for captures under a profiler)."""
    import oracle
    t = {"q4k": ob.Q4_K, "q6k": ob.Q6_K, "q80": ob.Q8_0}[tag]
    base = oracle.synth_blocks(t, n * k // (32 if t == ob.Q8_0 else 256)).reshape(n, -1)
    ring = max(2, int(200e6 // ob.raw_bytes(t, n, k)) + 1)          # distinct weights: more than L2 in total
    ws = [gpu.load_weight(np.ascontiguousarray(np.roll(base, 13 * i, axis=0)), t, n, k) for i in range(ring)]
    x = gpu.upload(np.random.default_rng(7).standard_normal((m, k), dtype=np.float32))
    y = gpu.alloc(m * n)
    work = gpu.alloc_bytes(gpu.gemm_workspace_bytes(m, k))
    if ksplit:
        gpu.set_option("gemm_ksplit", ksplit)
    for i in range(warmup):
        gpu.gemm(ws[i % ring], x, y, m, workspace=work)
    gpu.sync()
    e0, e1 = gpu.event(), gpu.event()
    if graph:
        # one CUDA graph over the ring of weights, replayed: the device time of a call, not the host's launch path
        per = min(ring, 8)
        gpu.graph_begin()
        for i in range(per):
            gpu.gemm(ws[i % ring], x, y, m, workspace=work)
        g = gpu.graph_end()
        reps = max(1, (steps + per - 1) // per)
        gpu.graph_launch(g)
        gpu.sync()
        gpu.record(e0)
        for _ in range(reps):
            gpu.graph_launch(g)
        gpu.record(e1)
        gpu.sync()
        us = gpu.elapsed_ms(e0, e1) * 1e3 / (reps * per)
        gpu.graph_destroy(g)
    else:
        gpu.record(e0)
        for i in range(steps):
            gpu.gemm(ws[i % ring], x, y, m, workspace=work)
        gpu.record(e1)
        gpu.sync()
        us = gpu.elapsed_ms(e0, e1) * 1e3 / steps
    gpu.set_option("gemm_ksplit", 0)
    for w in ws:
        gpu.free(w.buf)
    for b in (x, y, work):
        gpu.free(b)
    tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
    return {"workload": f"{tag}_gemm_m{m}_n{n}_k{k}", "us_per_call": round(us, 2), "TFLOP/s": round(tf, 1),
            "frac_of_peak": round(tf / tc_peak, 4), "ksplit": ksplit or "auto", "launch": "CUDA graph replay" if graph else "eager"}


def moe_case(gpu, ob, steps: int, warmup: int, hbm_peak: float, tc_peak: float, tokens: int = 64, gemm_rows: int = 0, t_exp: int = 12) -> dict:
    """Mixtral-like expert FFN: 8 experts (gate/up 14336 x 4096, down 4096 x 14336; Q4_K, or Q6_K with t_exp = 14),
    `tokens` tokens, top-2.  gemm_rows > 0 turns on the grouped tensor-core GEMM form from that many rows per expert
    (option moe_gemm_rows)."""
    import oracle
    e, d, ffn, m, ksel = 8, 4096, 14336, tokens, 2
    gpu.set_option("moe_gemm_rows", gemm_rows)
    rng = np.random.default_rng(0)
    mk = lambda n, k: oracle.synth_blocks(t_exp, e * n * k // 256)
    wg, wu, wd = (gpu.load_weight(mk(ffn, d), t_exp, e * ffn, d), gpu.load_weight(mk(ffn, d), t_exp, e * ffn, d),
                  gpu.load_weight(mk(d, ffn), t_exp, e * d, ffn))
    h = gpu.upload(rng.standard_normal((m, d), dtype=np.float32) * np.float32(1e-3))
    lg = gpu.upload(rng.standard_normal((m, e), dtype=np.float32))
    idx, wgt, out = gpu.alloc_bytes(m * ksel * 4), gpu.alloc(m * ksel), gpu.alloc(m * d)
    work = gpu.alloc_bytes(gpu.moe_workspace_bytes(m, e, ksel, d, ffn))

    def step():
        gpu.moe_topk(lg, idx, wgt, m, e, ksel)
        gpu.moe_ffn(wg, wu, wd, h, idx, wgt, out, m, e, ksel, workspace=work)

    for _ in range(warmup):
        step()
    gpu.sync()
    e0, e1 = gpu.event(), gpu.event()
    gpu.record(e0)
    for _ in range(steps):
        step()
    gpu.record(e1)
    gpu.sync()
    us = gpu.elapsed_ms(e0, e1) * 1e3 / steps
    gguf = 3 * ob.raw_bytes(t_exp, e * ffn, d)
    flops = 2.0 * m * ksel * 3 * ffn * d
    tag = {ob.Q4_K: "q4k", ob.Q6_K: "q6k"}.get(t_exp, str(t_exp))
    for b in (wg.buf, wu.buf, wd.buf, h, lg, idx, wgt, out, work):
        gpu.free(b)
    gpu.set_option("moe_gemm_rows", 0)
    return {"workload": f"moe_{tag}_e8_top2_m{m}_d4096_ffn14336" + ("_prefill_form" if gemm_rows else ""), "us_per_call": round(us, 1), "GB/s": round(gguf / us / 1e3, 1),
            "frac_of_hbm_peak": round(gguf / us / 1e3 / hbm_peak, 4), "TFLOP/s": round(flops / us / 1e6, 2),
            "frac_of_tensor_peak": round(flops / us / 1e6 / tc_peak, 5), "expert_bytes": gguf}


def tp70b_rows(gpu, dist, rank: int, world: int, local: int, steps: int) -> list[dict]:
    """The Llama-70B-shaped projections row-sharded over the ranks.  QKV 10240x8192, gate/up 28672x8192 (Q4_K) are
    column-parallel; O 8192x8192 (Q4_K) and down 8192x28672 (Q6_K) are row-parallel (K split on super-block
    boundaries).  M = 1: the GEMV stores its shard / partial vector into every rank's window and a bounded-wait join
    kernel forms the result (no library collective).  M = 512: tensor-core GEMM + NCCL all-gather / all-reduce on the
    same stream.  Time = CUDA events, max over ranks; every row carries the rel-L2 of the JOINED result against the
    CPU oracle (rank 0; M = 512: three sampled tokens)."""
    import torch
    import oracle
    import ojas_engine_b200 as ob
    from ojas_engine_b200 import tp
    dev = f"cuda:{local}"
    stream = torch.cuda.ExternalStream(gpu.stream, device=dev)
    projections = [("qkv", ob.Q4_K, 10240, 8192, "col"), ("o", ob.Q4_K, 8192, 8192, "row"),
                   ("gate_up", ob.Q4_K, 28672, 8192, "col"), ("down", ob.Q6_K, 8192, 28672, "row")]

    def exchange(blob):
        out = [None] * world
        dist.all_gather_object(out, blob)
        return out

    group = tp.TpGroup(gpu, world, rank, 28672, exchange if world > 1 else (lambda blob: [blob]))
    rng = np.random.default_rng(321)
    rows_out = []

    def timed(fn, n):
        for _ in range(3):
            fn()
        gpu.sync(); torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = gpu.event(), gpu.event()
        gpu.record(e0)
        for _ in range(n):
            fn()
        gpu.record(e1)
        gpu.sync(); torch.cuda.synchronize()
        tt = torch.tensor([gpu.elapsed_ms(e0, e1) * 1e3 / n], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    for name, t, n, k, mode in projections:
        raw = oracle.synth_blocks(t, n * k // 256)
        sh = tp.ShardedLinear(raw, t, n, k, mode, rank, world)
        n_loc, k_loc = sh.local_shape
        w = gpu.load_weight(sh.raw, t, n_loc, k_loc)
        tag = {ob.Q4_K: "q4k", ob.Q6_K: "q6k"}[t]
        # ---- M = 1
        x1 = (rng.standard_normal((1, k)) * 0.1).astype(np.float32)
        xb, y = gpu.upload(sh.local_x(x1)), gpu.alloc(n)
        jm = group.COL if mode == "col" else group.ROW
        reps = 16
        gpu.graph_begin()
        for _ in range(reps):
            group.gemv(w, xb)
            group.join(jm, y, n)
        g = gpu.graph_end()
        us = timed(lambda: gpu.graph_launch(g), max(steps, 3)) / reps
        gpu.graph_destroy(g)
        err = None
        if rank == 0:
            want = oracle.matvec_kq(raw, t, n, k, x1[0], os.cpu_count() or 1, oracle_native_ok())
            got = gpu.read(y, np.float32, n)
            err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        rows_out.append({"proj": name, "type": tag, "N": n, "K": k, "mode": mode, "M": 1, "us_per_call": round(us, 2),
                         "aggregate_GB/s": round(ob.raw_bytes(t, n, k) / us / 1e3, 1), "join": "peer stores + bounded-wait join kernel",
                         "rel_l2_joined_vs_oracle": err})
        # ---- M = 512
        m = 512
        xm = (rng.standard_normal((m, k)) * 0.1).astype(np.float32)
        xmb = gpu.upload(sh.local_x(xm))
        yl = torch.empty(m, n_loc, device=dev, dtype=torch.float32)
        ylb = ob.Buf(yl.data_ptr(), yl.numel() * 4)
        work = gpu.alloc_bytes(gpu.gemm_workspace_bytes(m, k_loc))
        out = {}

        def call():
            gpu.gemm(w, xmb, ylb, m, workspace=work)
            if world > 1:
                with torch.cuda.stream(stream):
                    out["full"] = sh.join(yl, dist)
            else:
                out["full"] = yl

        us = timed(call, max(steps, 3))
        err = None
        if rank == 0:
            sample = [0, m // 3, m - 1]
            want = oracle.matmul_kq(raw, t, n, k, xm[sample], os.cpu_count() or 1)
            got = out["full"][sample].cpu().numpy()
            err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        rows_out.append({"proj": name, "type": tag, "N": n, "K": k, "mode": mode, "M": m, "us_per_call": round(us, 2),
                         "aggregate_TFLOP/s": round(2.0 * m * n * k / us / 1e6, 1), "join": "NCCL " + ("all-gather" if mode == "col" else "all-reduce"),
                         "rel_l2_joined_vs_oracle": err})
        for b in (w.buf, xb, y, xmb, work):
            gpu.free(b)
    group.close()
    return rows_out


def run_tp70b(args) -> None:
    """`--case tp70b` under torchrun (or alone for 1 GPU): prints the rows of tp70b_rows as one JSON line."""
    import torch
    import ojas_engine_b200 as ob
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    gpu = ob.B200Gpu(local)
    rows = tp70b_rows(gpu, dist, rank, world, local, args.steps)
    if rank == 0:
        print(json.dumps({"case": "tp70b", "n_gpus": world, "steps": args.steps, "rows": rows}))
    if world > 1:
        dist.destroy_process_group()
    gpu.close()


def run_gemm_case(args) -> None:
    """`--case gemm:q4k:M:N:K [--ksplit S]`: one prefill GEMM shape on one GPU."""
    import ojas_engine_b200 as ob
    _, tag, m, n, k = args.case.split(":")
    _, tc_peak, peak_kind = measured_peaks()
    gpu = ob.B200Gpu(0)
    out = gemm_case(gpu, ob, tag, int(m), int(n), int(k), args.steps, args.warmup, tc_peak, args.ksplit, graph=not args.no_graph)
    out["peak_kind"] = peak_kind
    print(json.dumps(out))
    gpu.close()


def _wrap_device_f32(ptr: int, count: int, device: int):
    """A torch view of a device buffer owned by the library (for the NCCL collective)."""
    import torch

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}
    return torch.as_tensor(h, device=f"cuda:{device}")


def profile_traffic():
    """DRAM bytes per launch of the GEMV kernel from the committed ncu summary, if present."""
    path = os.path.join(ROOT, "profiles", "gemv_q4k_4096x4096.json")
    try:
        with open(path) as fh:
            return json.load(fh).get("dram_bytes_per_launch")
    except Exception:
        return None


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the additional GEMV shapes")
    ap.add_argument("--case", default=None, help="time one GEMV shape instead: tag:N:K:M, e.g. q4k:4096:4096:1")
    ap.add_argument("--ring", type=int, default=0, help="--case: number of distinct weights (default: enough to pass L2)")
    ap.add_argument("--no-graph", action="store_true", help="--case: plain launches instead of a CUDA graph")
    ap.add_argument("--ksplit", type=int, default=0, help="--case gemm: force the K split (0 = automatic)")
    ap.add_argument("--warps", type=int, default=0, help="--case: the gemv_warps option (warps per CTA; 0 = chosen per shape)")
    ap.add_argument("--stages", type=int, default=0, help="--case: the gemv_stages option (ring stages per warp; 0 = chosen per shape)")
    ap.add_argument("--opt", action="append", default=[], help="--case: a library option as key=value (repeatable)")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch (default: with)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
