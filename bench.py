#!/usr/bin/env python
"""Benchmark of the NVFP4 decode hot path: the 497-GEMV per-step mix of the 27B hybrid decoder.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass over every linear layer of one decode step at batch 1: 497 NVFP4 GEMVs
over 9 layer shapes (reference: experiments/_bench_gemv_real_shapes.py:28-38), 14.4 GB of packed
weights and scales, each matrix with its own fp16 activation.  The metric is HBM GB/s computed from
ALGORITHMIC bytes (per GEMV: M*K/2 + M*K/16 + 2K + 2M, the reference's own formula,
experiments/_bench_gemv_real_shapes.py:67) divided by device time.

  value    steps are replayed from a CUDA graph with all inputs resident in HBM.
  e2e      the same step through the C ABI with HOST activations and HOST results: every step
           copies the 497 activation vectors (one arena, one copy) from pinned host memory to the
           device, replays the captured GEMV launches and copies the 497 result vectors (one
           arena, one copy) back; copies are inside the timed region.
  roofline the GEMV kernel against the measured HBM copy bandwidth (MEASURED_PEAKS.json).
  cpu_baseline  the CPU oracle (vectorised codec decode + fp32 torch matvec) timed on this host.

Every step streams 14.4 GB, far more than the 126 MB L2, so each weight byte is a cold HBM read.
Synthetic data: random E2M1 bytes, scale bytes uniform in [118, 122] (the range N(0, 0.02^2)
weights produce), activations ~N(0, 1) fp16.

With --gpus N > 1 (launched by torchrun, one process per GPU) the step is tensor-parallel: q/k/v,
gate/up, in_proj and lm_head are split by output rows, o_proj/out_proj/down_proj by K, and every
K-split layer is followed by an all-reduce of its 5120-element fp16 output (128 per step), done by
the library's one-shot peer-memory kernel over NVLink (NCCL only carries the rendezvous).
Total work is fixed, so scaling is "strong".
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, INTER, VOCAB = 5120, 17408, 248320
N_LAYERS, FULL_ATTN_EVERY = 64, 4

# (name, M, K, split) — split "col": output rows are sharded; "row": K is sharded + all-reduce;
# "kv": 4 KV heads of 256 rows, replicated when there are more ranks than heads.
ATTN_LAYER = [("q_proj", 12288, HIDDEN, "col"), ("k_proj", 1024, HIDDEN, "kv"),
              ("v_proj", 1024, HIDDEN, "kv"), ("o_proj", HIDDEN, 6144, "row")]
LINEAR_LAYER = [("in_proj_qkv", 10240, HIDDEN, "col"), ("in_proj_z", 6144, HIDDEN, "col"),
                ("in_proj_b", 48, HIDDEN, "col"), ("in_proj_a", 48, HIDDEN, "col"),
                ("out_proj", HIDDEN, 6144, "row")]
MLP = [("gate_proj", INTER, HIDDEN, "col"), ("up_proj", INTER, HIDDEN, "col"),
       ("down_proj", HIDDEN, INTER, "row")]


def step_gemvs():
    """The 497 GEMVs of one decode step, in execution order."""
    out = []
    for i in range(N_LAYERS):
        mixer = ATTN_LAYER if (i + 1) % FULL_ATTN_EVERY == 0 else LINEAR_LAYER
        out += [(f"L{i}.{n}", M, K, sp) for n, M, K, sp in mixer]
        out += [(f"L{i}.{n}", M, K, sp) for n, M, K, sp in MLP]
    out.append(("lm_head", VOCAB, HIDDEN, "col"))
    return out


def gemv_bytes(M, K):
    return M * K // 2 + M * K // 16 + 2 * K + 2 * M


def shard(M, K, split, world, rank):
    """Shape of this rank's shard of an [M, K] layer."""
    if world == 1:
        return M, K
    if split == "col":
        per = -(-M // world)
        return max(0, min(M, (rank + 1) * per) - rank * per), K
    if split == "kv":
        heads = M // 256
        return (M // world, K) if world <= heads else (256, K)
    if split == "row":
        assert K % (world * 128) == 0
        return M, K // world
    raise ValueError(split)


# ------------------------------------------------------------------------------------------------
def sample_clocks(stop, out):
    """nvidia-smi clock/throttle samples while the timed region runs."""
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    idx = os.environ.get("LOCAL_RANK", "0")
    try:
        p = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                              "-i", idx, "-lms", "100"], stdout=subprocess.PIPE,
                             stderr=subprocess.DEVNULL, text=True)
    except OSError:
        return
    lines = []

    def reader():
        for line in p.stdout:
            lines.append(line)

    th = threading.Thread(target=reader, daemon=True)
    th.start()
    stop.wait()
    p.terminate()
    try:
        p.wait(timeout=2)
    except Exception:
        p.kill()
    th.join(timeout=2)
    out.extend(lines)


def summarise_clocks(lines):
    sm, smax, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for ln in lines:
        f = [x.strip() for x in ln.split(",")]
        if len(f) < 9:
            continue
        try:
            sm.append(float(f[1]))
            smax.append(float(f[2]))
        except ValueError:
            continue
        for name, val in zip(names, f[5:9]):
            if val.lower().startswith("active"):
                reasons.add(name)
    if not sm:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
            "samples": len(sm)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
def cpu_gemv_gbps(shapes, threads, repeats=1):
    """The CPU oracle (vectorised codec decode + fp32 torch matvec) on a list of shapes.
    Returns (GB/s of algorithmic bytes, seconds spent, description)."""
    import torch

    from oracle import nvfp4_codec_oracle as oc

    torch.set_num_threads(threads)
    rng = np.random.default_rng(0)
    total_bytes, total_t = 0, 0.0
    for M, K in shapes:
        packed = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
        scales = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
        act = rng.standard_normal(K).astype(np.float16)
        for _ in range(repeats):
            t0 = time.perf_counter()
            w = oc.decode(packed, scales)                      # codec dequant -> fp16
            y = torch.from_numpy(w.astype(np.float32)) @ torch.from_numpy(act.astype(np.float32))
            _ = y.to(torch.float16)
            total_t += time.perf_counter() - t0
            total_bytes += gemv_bytes(M, K)
    return total_bytes / total_t / 1e9, total_t


CPU_SAMPLE = [(5120, 5120), (1024, 5120), (5120, 6144), (6144, 5120), (17408, 5120), (5120, 17408)]
CPU_SAMPLE_DESC = ("one GEMV each of 5120x5120, 1024x5120, 5120x6144, 6144x5120, 17408x5120, "
                   "5120x17408 (codec decode to fp16 + fp32 torch matvec)")


# one step of the reference arm: a bounded sample (~4 s of CPU work)
REF_STEP_SAMPLE = CPU_SAMPLE[:3]
REF_STEP_DESC = ("one GEMV each of 5120x5120, 1024x5120, 5120x6144 "
                 "(codec decode to fp16 + fp32 torch matvec)")


def run_reference(args):
    """--impl reference: the reference's CPU path for this metric (codec dequant + torch CPU
    matmul), restated by the oracle, on all host threads.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    cores = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_gemv_gbps(CPU_SAMPLE[:2], cores)
    t0 = time.perf_counter()
    vals = []
    for _ in range(args.steps):
        g, _t = cpu_gemv_gbps(REF_STEP_SAMPLE, cores)
        vals.append(g)
    dt = time.perf_counter() - t0
    v = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": "nvfp4_gemv_hbm_gbps", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "gemv_497_mix_27b", "sample": REF_STEP_DESC},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": REF_STEP_DESC},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from nvfp4_v100_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run "
                             "(one process per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.load()
    vp = ctypes.c_void_p

    gemvs = step_gemvs()
    g = torch.Generator(device="cuda")
    g.manual_seed(1234 + rank)
    layers = []
    total_alg = 0
    shapes = [(name, *shard(M, K, split, world, rank), split) for name, M, K, split in gemvs]
    shapes = [s_ for s_ in shapes if s_[1] > 0]
    # every activation and every result lives in one device arena each (256-byte aligned slices),
    # so that the end-to-end pass moves them with ONE copy per direction and step
    pad = lambda n: (n + 127) // 128 * 128
    act_arena = torch.zeros(sum(pad(k) for _, _, k, _ in shapes), dtype=torch.float16, device="cuda")
    out_arena = torch.zeros(sum(pad(m) for _, m, _, _ in shapes), dtype=torch.float16, device="cuda")
    a_off = o_off = 0
    for name, m, k, split in shapes:
        packed = torch.randint(0, 256, (m * k // 2,), dtype=torch.uint8, device="cuda", generator=g)
        scales = torch.randint(118, 123, (m * k // 16,), dtype=torch.uint8, device="cuda",
                               generator=g)
        act = act_arena[a_off:a_off + k]
        act.copy_(torch.randn(k, dtype=torch.float32, device="cuda", generator=g).to(torch.float16))
        out = out_arena[o_off:o_off + m]
        a_off += pad(k)
        o_off += pad(m)
        layers.append((name, m, k, split, packed, scales, act, out))
        total_alg += gemv_bytes(m, k)
    n_launch = len(layers)
    n_allreduce = sum(1 for l in layers if l[3] == "row") if world > 1 else 0
    comm = None
    if world > 1:
        # K-split layers write their partial vector into this rank's peer-visible buffer; the
        # library's one-shot all-reduce kernel sums the ranks' vectors into `resid`
        from nvfp4_v100_b200.comm import PeerComm

        comm = PeerComm(HIDDEN, rank, world)
        resid = torch.zeros(HIDDEN, dtype=torch.float16, device="cuda")
        assert n_allreduce % 2 == 0

    def gemv(name, m, k, split, packed, scales, act, out, st):
        dst = out.data_ptr()
        parity = 0
        if comm is not None and split == "row":
            dst, parity = comm.next_slot()
        rc = lib.launch_nvfp4_gemv_v8(vp(packed.data_ptr()), vp(scales.data_ptr()),
                                      vp(act.data_ptr()), vp(dst), m, k, st)
        if rc != 0:
            raise RuntimeError(f"{name}: launch_nvfp4_gemv_v8 rc={rc}")
        if comm is not None and split == "row":
            comm.allreduce_residual(resid, parity, st)

    def enqueue_step():
        st = vp(torch.cuda.current_stream().cuda_stream)
        for name, m, k, split, packed, scales, act, out in layers:
            gemv(name, m, k, split, packed, scales, act, out, st)

    # warm-up outside the graph (module load, NCCL channels), then capture one step
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        enqueue_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        enqueue_step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        graph.replay()
    barrier()

    stop = threading.Event()
    clock_lines: list[str] = []
    sampler = threading.Thread(target=sample_clocks, args=(stop, clock_lines), daemon=True)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)

    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        graph.replay()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)

    # ---- end to end: host activations in, host results out, every step ----
    # One copy of the activation arena from pinned host memory, the captured step (the same C-ABI
    # launches), one copy of the result arena back (plus the residual vector when K-split layers
    # are all-reduced into it): what a caller with host buffers does per step.
    h_act = torch.empty_like(act_arena, device="cpu").pin_memory()
    h_out = torch.empty_like(out_arena, device="cpu").pin_memory()
    h_act.copy_(act_arena)
    h_res = torch.empty(HIDDEN, dtype=torch.float16).pin_memory() if comm is not None else None
    h2d = sum(l[2] for l in layers) * 2
    d2h = sum(l[1] for l in layers) * 2

    def e2e_step():
        act_arena.copy_(h_act, non_blocking=True)
        graph.replay()
        h_out.copy_(out_arena, non_blocking=True)
        if h_res is not None:
            h_res.copy_(resid, non_blocking=True)

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    if rank == 0:
        time.sleep(0.2)
        stop.set()
        sampler.join(timeout=5)

    # max over ranks
    t = torch.tensor([ms, e2e_ms, float(total_alg)], dtype=torch.float64, device="cuda")
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = t.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms, e2e_ms, job_bytes = float(tmax[0]), float(tmax[1]), float(tsum[2])
    else:
        job_bytes = float(total_alg)

    def finish():
        """Leave without tearing the communicator down: destroying an NCCL process group while a
        captured graph still references its kernels has been seen to block forever at exit."""
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            os._exit(0)

    if rank != 0:
        finish()
        return

    value = job_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e_value = job_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = (float(total_alg) * args.steps / (ms * 1e-3) / 1e9)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = min(os.cpu_count() or 1, torch.get_num_threads())
        v, secs = cpu_gemv_gbps(CPU_SAMPLE, threads, repeats=3)   # about 10 s of host work
        cpu = {"value": v, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": "three passes over " + CPU_SAMPLE_DESC, "seconds": round(secs, 2)}

    line = {
        "metric": "nvfp4_gemv_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "gemv_497_mix_27b", "gemvs_per_step": n_launch,
                   "algorithmic_bytes_per_step": int(job_bytes),
                   "l2": "each step streams 14.4 GB of weights (>> 126 MB L2): reads are cold",
                   "parallelism": f"tp{world}", "allreduce_per_step": n_allreduce,
                   "allreduce": "one-shot peer-memory kernel" if comm is not None else "none",
                   "comm_status": comm.status() if comm is not None else 0,
                   "launch": "cuda_graph"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": (n_launch + n_allreduce) * args.steps,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak, "traffic": TRAFFIC_PER_LAUNCH, "peak_kind": peak_kind,
                     "kernel": "gemv_mma_kernel",
                     "frac_of_nominal_8000": per_gpu / 8000.0},
        "cpu_baseline": cpu,
        "clocks": summarise_clocks(clock_lines),
    }
    print(json.dumps(line), flush=True)
    finish()


SHAPES_27B = [("lm_head", VOCAB, HIDDEN, 1), ("down_proj", HIDDEN, INTER, 64),
              ("gate/up_proj", INTER, HIDDEN, 128), ("q_proj+gate", 12288, HIDDEN, 16),
              ("in_proj_qkv", 10240, HIDDEN, 48), ("in_proj_z", 6144, HIDDEN, 48),
              ("o/out_proj", HIDDEN, 6144, 64), ("k/v_proj", 1024, HIDDEN, 32),
              ("in_proj_b/a", 48, HIDDEN, 96),
              # shapes BASELINE.json lists beside the reference's own table
              ("q_proj 6144", 6144, HIDDEN, 0), ("o_proj 5120", HIDDEN, HIDDEN, 0),
              ("lm_head 151936", 151936, HIDDEN, 0)]


def run_per_shape(args):
    """Each layer shape timed alone, cold L2: launches rotate over enough weight copies that the
    working set is several times the L2 (method of experiments/_bench_gemv_real_shapes.py:68-94)."""
    import torch

    from nvfp4_v100_b200 import _lib

    torch.cuda.set_device(0)
    lib = _lib.load()
    vp = ctypes.c_void_p
    only = None
    if args.only:
        m, k = args.only.lower().split("x")
        only = (int(m), int(k))
    peak, peak_kind = measured_peak()
    rows = []
    for name, M, K, count in SHAPES_27B:
        if only and (M, K) != only:
            continue
        nbytes = gemv_bytes(M, K)
        ncopy = max(2, min(64, -(-(1 << 30) // nbytes)))
        packed = torch.randint(0, 256, (ncopy, M * K // 2), dtype=torch.uint8, device="cuda")
        scales = torch.randint(118, 123, (ncopy, M * K // 16), dtype=torch.uint8, device="cuda")
        act = torch.randn(ncopy, K, device="cuda").to(torch.float16)
        out = torch.zeros(ncopy, M, dtype=torch.float16, device="cuda")
        st = vp(torch.cuda.current_stream().cuda_stream)

        def launch(i):
            c = i % ncopy
            rc = lib.launch_nvfp4_gemv_v8(vp(packed[c].data_ptr()), vp(scales[c].data_ptr()),
                                          vp(act[c].data_ptr()), vp(out[c].data_ptr()), M, K, st)
            assert rc == 0, rc

        reps = args.reps
        for i in range(max(3, ncopy)):
            launch(i)
        torch.cuda.synchronize()
        # replay the launches from a CUDA graph so that host launch cost (about 9 us per ctypes
        # call) does not hide the kernel time of the small shapes
        graph = None
        if not args.eager:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                st = vp(side.cuda_stream)
                launch(0)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                st = vp(torch.cuda.current_stream().cuda_stream)
                for i in range(reps):
                    launch(i)
            graph.replay()
            torch.cuda.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if graph is not None:
                graph.replay()
            else:
                for i in range(reps):
                    launch(i)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            best = us if best is None else min(best, us)
        gbps = nbytes / (best * 1e-6) / 1e9
        rows.append({"shape": f"{M}x{K}", "name": name, "count_per_step": count, "us": best,
                     "gbps": gbps, "frac_of_" + peak_kind: gbps / peak, "copies": ncopy})
        print(f"{name:16s} {M:7d}x{K:<6d} {best:9.2f} us {gbps:8.1f} GB/s "
              f"{100 * gbps / peak:5.1f}% of {peak_kind} {peak:.0f}", file=sys.stderr, flush=True)
        del packed, scales, act, out
    mix_us = sum(r["us"] * r["count_per_step"] for r in rows)
    mix_bytes = sum(gemv_bytes(*map(int, r["shape"].split("x"))) * r["count_per_step"] for r in rows)
    line = {"metric": "nvfp4_gemv_hbm_gbps_per_shape", "unit": "GB/s", "n_gpus": 1,
            "timing": "cuda events over back-to-back launches (CUDA graph replay unless --eager), best of 3, cold L2 by rotation over weight copies",
            "per_shape": rows,
            "mix_497": {"ms_per_step": mix_us / 1e3,
                        "gbps": (mix_bytes / (mix_us * 1e-6) / 1e9) if mix_us else None}}
    print(json.dumps(line), flush=True)


def run_gemm(args):
    """Dense GEMM through launch_nvfp4_gemmtc_v5 at the 27B layer shapes (BASELINE config 5):
    tokens = 32 (batched decode, weight-bandwidth bound) and 8192 (prefill, tensor bound)."""
    import torch

    from nvfp4_v100_b200 import _lib

    torch.cuda.set_device(0)
    lib = _lib.load()
    vp = ctypes.c_void_p
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        tf_peak, tf_kind = float(peaks["bf16_tflops"]), "measured bf16 burst"
    except Exception:
        tf_peak, tf_kind = 1590.0, "fallback"
    hbm_peak, hbm_kind = measured_peak()
    rows = []
    token_counts = (args.tokens,) if args.tokens else (32, 8192)
    shapes = ((6144, HIDDEN), (INTER, HIDDEN), (HIDDEN, HIDDEN), (HIDDEN, INTER))
    if args.only:
        shapes = (tuple(int(v) for v in args.only.lower().split("x")),)
    for tokens in token_counts:
        for M, K in shapes:
            p = torch.randint(0, 256, (M * K // 2,), dtype=torch.uint8, device="cuda")
            s = torch.randint(118, 123, (M * K // 16,), dtype=torch.uint8, device="cuda")
            a = torch.randn(K, tokens, device="cuda").to(torch.float16)
            o = torch.zeros(M, tokens, dtype=torch.float16, device="cuda")
            st = vp(torch.cuda.current_stream().cuda_stream)
            if args.w4a4:       # activations token-major, quantised per block along K on the fly
                a_tm = torch.randn(tokens, K, device="cuda").to(torch.float16)
                work = torch.empty(K * tokens, dtype=torch.float16, device="cuda")

            def launch():
                if args.w4a4:
                    rc = lib.launch_nvfp4_gemm_w4a4(vp(p.data_ptr()), vp(s.data_ptr()),
                                                    vp(a_tm.data_ptr()), vp(o.data_ptr()),
                                                    vp(work.data_ptr()), M, tokens, K, st)
                else:
                    rc = lib.launch_nvfp4_gemmtc_v5(vp(p.data_ptr()), vp(s.data_ptr()),
                                                    vp(a.data_ptr()), vp(o.data_ptr()), M, tokens,
                                                    K, st)
                assert rc == 0, rc

            for _ in range(3):
                launch()
            torch.cuda.synchronize()
            reps = 20 if tokens == 32 else 5
            best = None
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    launch()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / reps
                best = us if best is None else min(best, us)
            flops = 2.0 * M * tokens * K
            nbytes = M * K * 0.5625 + 2.0 * K * tokens + 2.0 * M * tokens
            rows.append({"tokens": tokens, "M": M, "K": K, "us": best,
                         "tflops": flops / best / 1e6, "frac_tensor_" + tf_kind.split()[0]:
                         flops / best / 1e6 / tf_peak, "gbps": nbytes / best / 1e3,
                         "frac_hbm_" + hbm_kind: nbytes / best / 1e3 / hbm_peak})
            print(f"tokens {tokens:5d}  {M:6d}x{K:<6d} {best:9.1f} us {flops / best / 1e6:8.1f} TFLOP/s "
                  f"({100 * flops / best / 1e6 / tf_peak:4.1f}% of {tf_kind} {tf_peak:.0f}) "
                  f"{nbytes / best / 1e3:7.0f} GB/s", file=sys.stderr, flush=True)
    print(json.dumps({"metric": "nvfp4_gemm_tflops", "unit": "TFLOP/s", "n_gpus": 1, "dtype": "f16",
                      "kernel": ("quant_dequant_T_kernel + gemm_w4a16_tcgen05_kernel (W4A4 values, fp16 "
                                 "tensor path, fp32 accumulation in TMEM)" if args.w4a4 else
                                 "gemm_w4a16_tcgen05_kernel (W4A16: fp16 activations, fp32 "
                                 "accumulation in TMEM)"),
                      "status": lib.nvfp4_gemm_status(0), "shapes": rows}), flush=True)


def decode_step_bytes(cfg, context):
    """Algorithmic HBM bytes of one decode step: every weight byte once, DeltaNet state read and
    written, the KV prefix read, embedding row and logits."""
    w = 0
    for i in range(cfg.n_layers):
        for M, K in cfg.layer_shapes(i).values():
            w += gemv_bytes(M, K)
    w += gemv_bytes(cfg.vocab, cfg.hidden)
    n_dn = sum(0 if cfg.is_attn(i) else 1 for i in range(cfg.n_layers))
    state = 2 * cfg.dn_vheads * 128 * 128 * 4 * n_dn
    kv = (cfg.n_layers - n_dn) * cfg.hkv * context * 256 * 2 * 2
    return w + state + kv


def run_decode(args, quiet=False):
    """27B-shape decode: 512-token prompt fed through the step graph, then 63 greedy tokens
    (BASELINE configs 3 and 4).  Random-init NVFP4 weights, random token ids.  Under torchrun the
    model is tensor-parallel over the ranks (one process per GPU, NCCL all-reduce in the graph)."""
    import torch
    import torch.distributed as dist

    from nvfp4_v100_b200.engine import DecodeEngine, ModelConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = ModelConfig(max_len=1024, vocab=args.vocab)
    if args.layers:
        cfg.n_layers = args.layers          # profiling aid: full width, reduced depth
    eng = DecodeEngine(cfg, device=f"cuda:{local}", tp_rank=rank, tp_world=world,
                       allreduce=args.allreduce)
    eng.load_random(seed=0)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab, args.prompt_len)
    eng.reset(int(prompt[0]))
    if args.fake_context > 0:       # profiling aid: pretend the cache already holds this many keys
        eng.pos.fill_(args.fake_context - 1)
        eng.len.fill_(args.fake_context)
    n_launch = eng.capture(n_warmup=1)
    n_coll = eng.n_collective

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    native_prefill_ms = None
    if not args.fake_context and len(prompt) > 1:
        # chunked prefill through the tensor-core GEMM (512-token chunks, the reference's chunk
        # size); one untimed pass first (one-time attribute and tensor-map set-up), then timed
        head = [int(t) for t in prompt[:-1]]
        eng.prefill(head)
        eng.reset(int(prompt[0]))
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        p0.record()
        eng.prefill(head)
        p1.record()
        barrier()
        prefill_s = time.perf_counter() - t0
        native_prefill_ms = p0.elapsed_time(p1)
        eng.tok.fill_(int(prompt[-1]))
    else:
        t0 = time.perf_counter()
        for t in range(1, len(prompt)):
            eng.step()
            eng.tok.fill_(int(prompt[t]))
        barrier()
        prefill_s = time.perf_counter() - t0
    n_gen = args.gen
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(n_gen):
        eng.step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    # end to end: read every token back on the host as the reference loop does (.item() per step)
    snap_pos = int(eng.pos.item())
    t0 = time.perf_counter()
    toks = []
    for _ in range(min(n_gen, cfg.max_len - snap_pos - 1)):
        eng.step()
        toks.append(int(eng.tok.item()))
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        tm = torch.tensor([ms, e2e_s, prefill_s, native_prefill_ms or 0.0], dtype=torch.float64,
                          device="cuda")
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms, e2e_s, prefill_s, npm = (float(x) for x in tm)
        native_prefill_ms = npm if native_prefill_ms else None
    res = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        step_bytes = decode_step_bytes(cfg, args.prompt_len + n_gen // 2)
        per_gpu = step_bytes / world / (ms / n_gen * 1e-3) / 1e9
        res = {
            "metric": "decode_tok_s", "value": n_gen / (ms * 1e-3), "unit": "tok/s",
            "ms_per_step": ms / n_gen, "n_gpus": world, "prompt_len": int(args.prompt_len),
            "gen": n_gen, "kernel_launches_per_step": n_launch, "collectives_per_step": n_coll,
            "scaling": "strong",
            ("prefill_tok_s" if native_prefill_ms else "prefill_by_decode_tok_s"):
                (len(prompt) - 1) / (native_prefill_ms * 1e-3 if native_prefill_ms else prefill_s),
            "prefill": ("chunked, tensor-core GEMM (device time; host wall "
                        f"{prefill_s * 1e3:.1f} ms)" if native_prefill_ms
                        else "token by token through the decode step"),
            "e2e": {"value": len(toks) / e2e_s, "unit": "tok/s", "d2h_bytes_per_step": 8,
                    "h2d_bytes_per_step": 0},
            "roofline": {"bound": "hbm", "algorithmic_bytes_per_step": step_bytes,
                         "achieved": per_gpu, "peak": peak, "unit": "GB/s (per GPU)",
                         "frac": per_gpu / peak, "peak_kind": peak_kind},
            "config": {"workload": "decode_27b_shape", "layers": cfg.n_layers,
                       "hidden": cfg.hidden, "vocab": cfg.vocab, "launch": "cuda_graph",
                       "weights": "seeded N(0, 0.02^2) fp16 quantised on the device", "parallelism": f"tp{world}",
                       "allreduce": eng.allreduce, "comm_status": eng.comm_status()},
            "finite_logits": bool(torch.isfinite(eng.logits.float()).all().item()),
        }
        if not quiet:
            print(json.dumps(res), flush=True)
    if world > 1:
        sys.stdout.flush()
        dist.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    del eng
    torch.cuda.empty_cache()
    return res


# DRAM bytes (read + write) per average GEMV launch of the mix.  The full-set ncu capture was taken
# on the 151936x5120 shape (profiles/gemv_mma_kernel_lm_head_151936x5120.md): 441.69 MB of DRAM
# traffic for 437.89 MB of algorithmic bytes, ratio 1.0087; every weight byte is read once at any
# shape, so the traffic of the mix's average launch (14 427 447 296 B / 497) is scaled by that ratio.
TRAFFIC_PER_LAUNCH = int(14_427_447_296 / 497 * (441.69 / 437.89))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--per-shape", action="store_true",
                    help="time every 27B layer shape alone (cold L2) instead of the step mix")
    ap.add_argument("--only", default="", help="with --per-shape: a single MxK shape")
    ap.add_argument("--reps", type=int, default=200, help="with --per-shape: launches per timing")
    ap.add_argument("--gemm", action="store_true",
                    help="dense GEMM (tokens = 32 and 8192) at the 27B layer shapes")
    ap.add_argument("--decode", action="store_true",
                    help="27B-shape decode tok/s (512-token prompt, 63 tokens) instead of the mix")
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0,
                    help="with --decode: use this many layers (profiling aid; 0 = the full 64)")
    ap.add_argument("--w4a4", action="store_true",
                    help="with --gemm: quantise the activations to NVFP4 on the fly (W4A4 values)")
    ap.add_argument("--tokens", type=int, default=0,
                    help="with --gemm: a single token count instead of 32 and 8192")
    ap.add_argument("--gen", type=int, default=63)
    ap.add_argument("--vocab", type=int, default=VOCAB)
    ap.add_argument("--allreduce", default="peer", choices=["fused", "peer", "nccl"],
                    help="with --decode under torchrun: GEMV+all-reduce in one kernel, a separate "
                         "one-shot peer-memory all-reduce kernel, or NCCL")
    ap.add_argument("--fake-context", type=int, default=0,
                    help="with --decode: start at this cache length (zero-filled cache)")
    ap.add_argument("--eager", action="store_true",
                    help="with --per-shape: launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--stream-config", default="",
                    help="seven integers for nvfp4_b200_gemv_stream_config (consumer warps, shared "
                         "memory KB, stage KB, stages per warp, CTAs per SM, row unit, flags: bit 0 = use the "
                         "ring kernel, bits 4/5 = attribution probes); "
                         "profiling and attribution aid")
    args = ap.parse_args()
    if args.stream_config:
        from nvfp4_v100_b200 import _lib
        vals = [int(v) for v in args.stream_config.split(",")]
        assert len(vals) == 7 and _lib.load().nvfp4_b200_gemv_stream_config(*vals) == 0
    if args.warmup < 3:
        args.warmup = 3
    if args.gemm:
        run_gemm(args)
    elif args.decode:
        run_decode(args)
    elif args.per_shape:
        run_per_shape(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
