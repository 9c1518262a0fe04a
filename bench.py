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
  cpu_baseline  the reference's CPU path (codec decode + fp32 torch matvec) timed on this host.
  decode   the other half of the metric, in the same line: the 27B-shape decoder (64 layers, 512
           prompt tokens through the chunked prefill, 63 greedy tokens from the step graph).

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
def common_config(world):
    """The workload description both arms print (identical dictionaries)."""
    return {"workload": "gemv_497_mix_27b", "gemvs_per_step": 497,
            "algorithmic_bytes_per_step": sum(gemv_bytes(M, K) for _, M, K, _ in step_gemvs()),
            "l2": "each step streams 14.4 GB of weights (>> 126 MB L2): reads are cold",
            "parallelism": f"tp{world}"}


def load_reference_codec():
    """The reference's own CPU codec, byte-compiled into oracle/_ref/ by oracle/Makefile (the
    reference checkout itself is not present where the benchmark runs).  None if absent."""
    import importlib.machinery
    import importlib.util

    path = os.path.join(ROOT, "oracle", "_ref", "nvfp4_codec.bytecode")
    if not os.path.exists(path):
        return None
    try:
        loader = importlib.machinery.SourcelessFileLoader("nvfp4_codec_reference", path)
        spec = importlib.util.spec_from_loader("nvfp4_codec_reference", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        return mod
    except Exception:
        return None


def synthetic_layer(M, K, seed=0):
    rng = np.random.default_rng(seed + M + K)
    packed = rng.integers(0, 256, size=(M, K // 2), dtype=np.uint8)
    scales = rng.integers(118, 123, size=(M, K // 16), dtype=np.uint8)
    act = rng.standard_normal(K).astype(np.float16)
    return packed, scales, act


def cpu_gemv(decode_fn, packed, scales, act):
    """One GEMV on the CPU as the reference does it: decode to fp16, fp32 matvec, fp16 result.
    Returns (seconds for the decode, seconds for the matvec)."""
    import torch

    t0 = time.perf_counter()
    w = decode_fn(packed, scales)
    t1 = time.perf_counter()
    y = torch.from_numpy(w.astype(np.float32)) @ torch.from_numpy(act.astype(np.float32))
    _ = y.to(torch.float16)
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1


# (M, K, launches per decode step): the reference's shape table
CPU_SHAPES = [(5120, 5120, 0), (1024, 5120, 32), (5120, 6144, 64), (6144, 5120, 48),
              (10240, 5120, 48), (12288, 5120, 16), (17408, 5120, 128), (5120, 17408, 64),
              (48, 5120, 96), (VOCAB, 5120, 1)]


def cpu_protocol(threads, full):
    """The CPU baseline, laid out as the reference's own measurements are: the loop decoder
    (codec/nvfp4_codec.py decode_nvfp4_to_fp16, the reference's own code when its byte-compiled
    copy is present) once at 5120x5120; the vectorised decoder (the table look-up + exp2 recipe of
    pipeline/_qwen38_infer.py:117-128, restated by the oracle) and the fp32 matvec separately for
    every layer shape; their sum over the 497-GEMV mix as a lower bound on a CPU decode step
    (norms, attention and the recurrence excluded).  full: best of 5 and the lm_head at full
    size, in row chunks (about a minute); otherwise best of 2 and a 16384-row sample of the
    lm_head, scaled (about 20 s)."""
    import torch

    from oracle import nvfp4_codec_oracle as oc

    torch.set_num_threads(threads)
    ref = load_reference_codec()
    out = {"cores": threads, "os_cpu_count": os.cpu_count(), "rows": []}
    p, s, a = synthetic_layer(5120, 5120)
    if ref is not None:
        d, m = cpu_gemv(ref.decode_nvfp4_to_fp16, p, s, a)
        out["loop_decode_5120x5120"] = {"decode_s": d, "matvec_s": m, "kind": "reference",
                                        "gbps": gemv_bytes(5120, 5120) / (d + m) / 1e9}
    reps = 5 if full else 2
    mix_s = 0.0
    for M, K, cnt in CPU_SHAPES:
        rows = M
        if M == VOCAB and not full:
            rows = 16384
        # at most 16384 rows at a time: the decoder's float64 intermediate stays below 1 GB
        chunk = 16384
        best_d = best_m = 0.0
        for r0 in range(0, rows, chunk):
            p, s, a = synthetic_layer(min(chunk, rows - r0), K, seed=r0)
            bd = bm = None
            for _ in range(1 if rows > chunk else reps):
                d, m = cpu_gemv(oc.decode, p, s, a)
                bd = d if bd is None else min(bd, d)
                bm = m if bm is None else min(bm, m)
            best_d += bd
            best_m += bm
        scale = M / rows
        row = {"shape": f"{M}x{K}", "decode_s": best_d * scale, "matvec_s": best_m * scale,
               "sampled_rows": rows, "count_per_step": cnt,
               "gbps": gemv_bytes(M, K) / ((best_d + best_m) * scale) / 1e9}
        out["rows"].append(row)
        mix_s += cnt * (best_d + best_m) * scale
        del p, s, a
    out["mix_497_lower_bound_s"] = mix_s
    out["mix_497_gbps"] = common_config(1)["algorithmic_bytes_per_step"] / mix_s / 1e9
    return out


# one timed step of the reference arm: a bounded sample of the mix
REF_STEP_SHAPE = (1024, 5120)
REF_STEP_DESC_REFERENCE = ("one k/v_proj GEMV (1024x5120): the reference's decode_nvfp4_to_fp16 "
                           "(its own byte-compiled codec) + fp32 torch matvec")
REF_STEP_DESC_PORT = ("one GEMV each of 5120x5120, 1024x5120, 5120x6144 (vectorised codec decode "
                      "restated by the oracle + fp32 torch matvec)")


def run_reference(args):
    """--impl reference: the reference's CPU path for this metric (codec decode + torch CPU
    matvec) on the host cores, all threads torch will use.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    from oracle import nvfp4_codec_oracle as oc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ref = load_reference_codec()
    if ref is not None:
        shapes, decode_fn, kind, desc = [REF_STEP_SHAPE], ref.decode_nvfp4_to_fp16, "reference", \
            REF_STEP_DESC_REFERENCE
    else:
        shapes, decode_fn, kind, desc = [(5120, 5120), (1024, 5120), (5120, 6144)], oc.decode, \
            "port", REF_STEP_DESC_PORT
    data = [synthetic_layer(M, K) for M, K in shapes]
    step_bytes = sum(gemv_bytes(M, K) for M, K in shapes)

    def step():
        for p, s, a in data:
            cpu_gemv(decode_fn, p, s, a)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    v = step_bytes * args.steps / dt / 1e9
    protocol = None
    if args.cpu_protocol != "none":
        protocol = cpu_protocol(torch.get_num_threads(), full=(args.cpu_protocol == "full"))
    line = {
        "impl": "reference", "metric": "nvfp4_gemv_hbm_gbps", "value": v, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": common_config(args.gpus),
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": kind, "sample": desc},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "cpu_protocol": protocol,
    }
    print(json.dumps(line), flush=True)


def shutdown(world):
    """Leave a multi-rank run: every object that referenced a captured graph or a peer mapping
    has been released by the caller; synchronise, then tear the process group down.  The
    teardown runs with a time limit: if it does not come back (seen once while a captured graph
    still held library collectives), the process leaves without it rather than hang the job."""
    import gc

    import torch
    import torch.distributed as dist

    sys.stdout.flush()
    sys.stderr.flush()
    if world <= 1:
        return
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    done = threading.Event()

    def destroy():
        try:
            dist.destroy_process_group()
        finally:
            done.set()

    th = threading.Thread(target=destroy, daemon=True)
    th.start()
    if not done.wait(timeout=30):
        os._exit(0)


# ------------------------------------------------------------------------------------------------
def init_ranks():
    """(world, rank, local rank); under torchrun also the NCCL process group, which carries the
    rendezvous only (peer-buffer handles, the prefill's bandwidth-sized all-reduces)."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        # the data path is this library's kernels over peer memory: keep NCCL's in-switch
        # multicast groups out of the picture
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def tp_parity_check(lib, comm, rank, world):
    """A correctness bit for the multi-GPU record: a K-split layer (5120 x 17408) computed on the
    shards and summed inside the consuming GEMV's prologue, against the same layer unsharded on
    this GPU.  Every rank draws the same seeded matrix.  Returns max |difference| / max |output|
    of the all-reduced vector."""
    import torch

    vp = ctypes.c_void_p
    M, K = HIDDEN, INTER
    g = torch.Generator(device="cuda")
    g.manual_seed(4242)
    packed = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device="cuda", generator=g)
    scales = torch.randint(118, 123, (M, K // 16), dtype=torch.uint8, device="cuda", generator=g)
    act = torch.randn(K, device="cuda", generator=g).to(torch.float16)
    st = vp(torch.cuda.current_stream().cuda_stream)
    full = torch.zeros(M, dtype=torch.float16, device="cuda")
    assert lib.launch_nvfp4_gemv_v8(vp(packed.data_ptr()), vp(scales.data_ptr()), vp(act.data_ptr()),
                                    vp(full.data_ptr()), M, K, st) == 0
    k0, k1 = rank * (K // world), (rank + 1) * (K // world)
    p_l = packed[:, k0 // 2:k1 // 2].contiguous()
    s_l = scales[:, k0 // 16:k1 // 16].contiguous()
    a_l = act[k0:k1].contiguous()
    slot, parity = comm.next_slot()
    assert lib.launch_nvfp4_gemv_v8(vp(p_l.data_ptr()), vp(s_l.data_ptr()), vp(a_l.data_ptr()),
                                    vp(slot), M, k1 - k0, st) == 0
    # consumer: any GEMV over the hidden vector; its prologue completes the all-reduce into h
    cw = torch.randint(0, 256, (64 * HIDDEN // 2,), dtype=torch.uint8, device="cuda", generator=g)
    cs = torch.full((64 * HIDDEN // 16,), 120, dtype=torch.uint8, device="cuda")
    ones = torch.ones(HIDDEN, dtype=torch.float32, device="cuda")
    h = torch.zeros(HIDDEN, dtype=torch.float16, device="cuda")
    out = torch.zeros(64, dtype=torch.float16, device="cuda")
    epoch = torch.full((1,), 1 << 20, dtype=torch.int32, device="cuda")   # ahead of every flag so far
    rc = lib.launch_nvfp4_gemv_fused_ar(vp(cw.data_ptr()), vp(cs.data_ptr()), vp(h.data_ptr()),
                                        vp(out.data_ptr()), 64, HIDDEN, vp(ones.data_ptr()), 1e-6, 0,
                                        comm.ptrs, rank, world, HIDDEN, parity, vp(epoch.data_ptr()),
                                        0, 1, st)
    assert rc == 0, rc
    slot2, parity2 = comm.next_slot()      # keep the number of calls even (slot parity per site)
    torch.cuda.synchronize()
    # each rank's partial vector is rounded to fp16 before the sum (2^-11 of a partial's size, and
    # the partials are as large as the result), so the error is measured against the largest
    # output, not element by element
    ref = full.float()
    return float((h.float() - ref).abs().max() / ref.abs().max())


def run_ours(args):
    import torch
    import torch.distributed as dist

    from nvfp4_v100_b200 import _lib

    world, rank, local = init_ranks()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run "
                         "(one process per GPU)")
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
    inline = args.allreduce == "inline"
    if world > 1:
        # K-split layers write their partial vector into this rank's peer-visible buffer.  As in
        # the decode step, the GEMV that follows such a layer (gate_proj after o_proj / out_proj,
        # the next layer's first projection or the lm_head after down_proj) takes the hidden
        # vector as its activation: with --allreduce inline its prologue does the exchange, the
        # sum, the residual add and the RMSNorm; with --allreduce peer a one-CTA kernel does the
        # all-reduce into `resid` first.
        from nvfp4_v100_b200.comm import PeerComm

        comm = PeerComm(HIDDEN, rank, world)
        resid = torch.zeros(HIDDEN, dtype=torch.float16, device="cuda")
        ones = torch.ones(HIDDEN, dtype=torch.float32, device="cuda")
        epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert n_allreduce % 2 == 0

    def enqueue_step():
        st = vp(torch.cuda.current_stream().cuda_stream)
        pending = None
        site = 0
        for name, m, k, split, packed, scales, act, out in layers:
            dst = out.data_ptr()
            if pending is not None:
                assert k == HIDDEN
                rc = lib.launch_nvfp4_gemv_fused_ar(
                    vp(packed.data_ptr()), vp(scales.data_ptr()), vp(act.data_ptr()), vp(dst), m, k,
                    vp(ones.data_ptr()), 1e-6, 0, comm.ptrs, rank, world, HIDDEN, pending,
                    vp(epoch.data_ptr()), site, n_allreduce, st)
                site += 1
                pending = None
            else:
                parity = 0
                if comm is not None and split == "row":
                    dst, parity = comm.next_slot()
                rc = lib.launch_nvfp4_gemv_v8(vp(packed.data_ptr()), vp(scales.data_ptr()),
                                              vp(act.data_ptr()), vp(dst), m, k, st)
                if comm is not None and split == "row":
                    if inline:
                        pending = parity
                    else:
                        comm.allreduce_residual(resid, parity, st)
            if rc != 0:
                raise RuntimeError(f"{name}: GEMV launch rc={rc}")
        if comm is not None and inline:
            if pending is not None:      # the step's last K-split layer has no consumer in the mix
                raise RuntimeError("the mix must end with a consumer of the last K-split layer")
            epoch.add_(1)

    # warm-up outside the graph (module load, peer mappings), then capture one step
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

    # ---- sustained: the same step replayed for at least two seconds ----
    # (every rank must replay the SAME number of steps: the count comes from the slowest rank's time)
    ms_all = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms_all, op=dist.ReduceOp.MAX)
    sus_steps = max(args.steps, int(2.2e3 / max(float(ms_all) / args.steps, 1e-3)))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    s0.record()
    for _ in range(sus_steps):
        graph.replay()
    s1.record()
    barrier()
    sus_ms = s0.elapsed_time(s1)

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

    comm_status = comm.status() if comm is not None else 0
    parity_err = None
    if comm is not None:
        parity_err = tp_parity_check(lib, comm, rank, world)

    # max over ranks
    t = torch.tensor([ms, e2e_ms, sus_ms, float(parity_err or 0.0), float(comm_status)],
                     dtype=torch.float64, device="cuda")
    tb = torch.tensor([float(total_alg)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
    ms, e2e_ms, sus_ms, parity_max, comm_status = (float(x) for x in t)
    job_bytes = float(tb[0])

    # ---- release the mix before the decoder is built ----
    del graph, layers, act_arena, out_arena, h_act, h_out
    if comm is not None:
        comm.close()
        comm = None
    torch.cuda.empty_cache()

    decode = None
    if not args.no_decode:
        decode = run_decode(args, quiet=True)

    if rank != 0:
        shutdown(world)
        return
    gemm = None
    if world == 1 and not args.no_decode:
        gemm = quick_gemm(lib)

    value = job_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e_value = job_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak()
    per_gpu = (float(total_alg) * args.steps / (ms * 1e-3) / 1e9)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = min(os.cpu_count() or 1, torch.get_num_threads())
        t0 = time.perf_counter()
        proto = cpu_protocol(threads, full=False)
        kind = "reference" if "loop_decode_5120x5120" in proto else "port"
        cpu = {"value": proto["mix_497_gbps"], "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": "every layer shape of the mix once or twice (lm_head: 16384 of its rows, "
                         "scaled): vectorised codec decode + fp32 torch matvec, summed over the "
                         "497-GEMV mix; the reference's own loop decoder once at 5120x5120 beside it",
               "seconds": round(time.perf_counter() - t0, 2), "loop_decoder_kind": kind,
               "protocol": proto}

    run = {"allreduce_per_step": n_allreduce,
           "allreduce": ("none" if world == 1 else
                         "inside the consuming GEMV's prologue" if inline else
                         "one-shot peer-memory kernel"),
           "comm_status": int(comm_status), "launch": "cuda_graph",
           "kernel_launches_per_step": n_launch + (0 if inline else n_allreduce)}
    line = {
        "metric": "nvfp4_gemv_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": common_config(world),
        "run": run,
        "sustained": {"value": job_bytes * sus_steps / (sus_ms * 1e-3) / 1e9, "unit": "GB/s",
                      "steps": sus_steps, "seconds": sus_ms * 1e-3},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": run["kernel_launches_per_step"] * args.steps,
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu / peak, "traffic": TRAFFIC_PER_LAUNCH, "peak_kind": peak_kind,
                     "kernel": "gemv_tc_kernel (matrices of >= 50 M elements: 85 % of the step's bytes) + "
                               "gemv_mma_kernel (the rest)",
                     "frac_of_nominal_8000": per_gpu / 8000.0},
        "cpu_baseline": cpu,
        "clocks": summarise_clocks(clock_lines),
        "decode": decode,
        "gemm": gemm,
    }
    if world > 1:
        line["tp_parity"] = {"max_err_over_max_output": parity_max, "ok": bool(parity_max <= 2e-3),
                             "layer": "5120x17408 split along K, partial vectors summed over NVLink "
                                      "peer memory, against the unsharded GEMV"}
    print(json.dumps(line), flush=True)
    shutdown(world)


SHAPES_27B = [("lm_head", VOCAB, HIDDEN, 1), ("down_proj", HIDDEN, INTER, 64),
              ("gate/up_proj", INTER, HIDDEN, 128), ("q_proj+gate", 12288, HIDDEN, 16),
              ("in_proj_qkv", 10240, HIDDEN, 48), ("in_proj_z", 6144, HIDDEN, 48),
              ("o/out_proj", HIDDEN, 6144, 64), ("k/v_proj", 1024, HIDDEN, 32),
              ("in_proj_b/a", 48, HIDDEN, 96),
              # further shapes of the same decoder: q without its gate, the square o_proj, a 151936-row head
              ("q_proj 6144", 6144, HIDDEN, 0), ("o_proj 5120", HIDDEN, HIDDEN, 0),
              ("lm_head 151936", 151936, HIDDEN, 0), ("gate+up fused", 2 * INTER, HIDDEN, 0),
              # two-GPU shards of the MLP projections
              ("gate/up shard", INTER // 2, HIDDEN, 0), ("down shard", HIDDEN, INTER // 2, 0)]


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
            fn = lib.launch_nvfp4_gemv_tc if args.tc else lib.launch_nvfp4_gemv_v8
            rc = fn(vp(packed[c].data_ptr()), vp(scales[c].data_ptr()),
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


def quick_gemm(lib):
    """The dense GEMM on one prefill-sized problem (17408 x 5120 weights, 8192 tokens), for the
    default line: W4A16 (launch_nvfp4_gemmtc_v5, the reference's semantics) and W4A4
    (launch_nvfp4_gemm_w4a4: activations encoded to NVFP4 inside the timed launches, then the
    block-scaled FP4 tensor-core kernel).  CUDA events, best of 3 x 3 launches."""
    import torch

    vp = ctypes.c_void_p
    M, K, tokens = INTER, HIDDEN, 8192
    try:
        tf_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        kind = "measured"
    except Exception:
        tf_peak, kind = 1590.0, "fallback"
    p = torch.randint(0, 256, (M * K // 2,), dtype=torch.uint8, device="cuda")
    s = torch.randint(118, 123, (M * K // 16,), dtype=torch.uint8, device="cuda")
    a_kn = torch.randn(K, tokens, device="cuda").to(torch.float16)
    a_tm = torch.randn(tokens, K, device="cuda").to(torch.float16)
    o = torch.zeros(M, tokens, dtype=torch.float16, device="cuda")
    work = torch.empty(K * tokens, dtype=torch.float16, device="cuda")
    st = vp(torch.cuda.current_stream().cuda_stream)

    def w4a16():
        assert lib.launch_nvfp4_gemmtc_v5(vp(p.data_ptr()), vp(s.data_ptr()), vp(a_kn.data_ptr()),
                                          vp(o.data_ptr()), M, tokens, K, st) == 0

    def w4a4():
        assert lib.launch_nvfp4_gemm_w4a4(vp(p.data_ptr()), vp(s.data_ptr()), vp(a_tm.data_ptr()),
                                          vp(o.data_ptr()), vp(work.data_ptr()), M, tokens, K, st) == 0

    out = {"workload": f"{M}x{K} weights, {tokens} tokens", "flop": 2.0 * M * K * tokens}
    for name, fn in (("w4a16", w4a16), ("w4a4", w4a4)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 3
            best = us if best is None else min(best, us)
        tf = out["flop"] / best / 1e6
        # W4A4 against 4 x the bf16 figure: the FP4 tensor rate is four times the bf16 rate
        peak = tf_peak * (4.0 if name == "w4a4" else 1.0)
        out[name] = {"us": best, "tflops": tf, "peak_tflops": peak, "frac": tf / peak,
                     "peak_kind": kind + (" bf16 burst x 4" if name == "w4a4" else " bf16 burst")}
    out["status"] = lib.nvfp4_gemm_status(0)
    del p, s, a_kn, a_tm, o, work
    torch.cuda.empty_cache()
    return out


def run_gemm(args):
    """Dense GEMM through launch_nvfp4_gemmtc_v5 at the 27B layer shapes:
    tokens = 32 (batched decode, weight-bandwidth bound, weights cold by rotation) and 8192
    (prefill, tensor bound)."""
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
    if args.gemm_rows128:
        lib.nvfp4_b200_gemm_config(0)
    if args.gemm_pair:
        lib.nvfp4_b200_gemm_config(7)
    if args.gemm_config >= 0:
        lib.nvfp4_b200_gemm_config(args.gemm_config)
    if args.fp4_no_split:
        lib.nvfp4_b200_gemm_fp4_config(2)
    if args.fp4_config >= 0:
        lib.nvfp4_b200_gemm_fp4_config(args.fp4_config)
    rows = []
    token_counts = (args.tokens,) if args.tokens else (32, 8192)
    shapes = ((6144, HIDDEN), (INTER, HIDDEN), (HIDDEN, HIDDEN), (HIDDEN, INTER))
    if args.only:
        shapes = (tuple(int(v) for v in args.only.lower().split("x")),)
    for tokens in token_counts:
        for M, K in shapes:
            # few tokens = the weight stream from HBM is the bound: rotate over enough copies of
            # the weights that none is still in L2 when its turn comes again
            copies = 1 if tokens > 64 else max(2, int(np.ceil(300e6 / (M * K * 0.5625))))
            ps = [torch.randint(0, 256, (M * K // 2,), dtype=torch.uint8, device="cuda")
                  for _ in range(copies)]
            ss = [torch.randint(118, 123, (M * K // 16,), dtype=torch.uint8, device="cuda")
                  for _ in range(copies)]
            turn = [0]
            a = torch.randn(K, tokens, device="cuda").to(torch.float16)
            o = torch.zeros(M, tokens, dtype=torch.float16, device="cuda")
            a_tok = a.t().contiguous() if args.gemm_flags >= 0 else None
            st = vp(torch.cuda.current_stream().cuda_stream)
            if args.w4a4 or args.fp4_only:   # activations token-major, NVFP4 per block along K
                a_tm = torch.randn(tokens, K, device="cuda").to(torch.float16)
                work = torch.empty(K * tokens, dtype=torch.float16, device="cuda")
                if args.fp4_only:   # activations encoded once, outside the timed launches
                    a_p = torch.empty(tokens * K // 2, dtype=torch.uint8, device="cuda")
                    a_s = torch.empty(tokens * K // 16, dtype=torch.uint8, device="cuda")
                    assert lib.launch_nvfp4_encode(vp(a_tm.data_ptr()), vp(a_p.data_ptr()),
                                                   vp(a_s.data_ptr()), tokens, K, st) == 0

            def launch():
                p, s = ps[turn[0] % copies], ss[turn[0] % copies]
                turn[0] += 1
                if args.fp4_only:
                    rc = lib.launch_nvfp4_gemm_fp4(vp(p.data_ptr()), vp(s.data_ptr()),
                                                   vp(a_p.data_ptr()), vp(a_s.data_ptr()),
                                                   vp(o.data_ptr()), M, tokens, K, tokens, st)
                elif args.w4a4:
                    rc = lib.launch_nvfp4_gemm_w4a4(vp(p.data_ptr()), vp(s.data_ptr()),
                                                    vp(a_tm.data_ptr()), vp(o.data_ptr()),
                                                    vp(work.data_ptr()), M, tokens, K, st)
                elif args.gemm_flags >= 0:   # token-major sides: bit 0 input, bit 1 output, bit 2 += output
                    f = args.gemm_flags
                    rc = lib.launch_nvfp4_gemm_w4a16_ex(
                        vp(p.data_ptr()), vp(s.data_ptr()), vp((a_tok if f & 1 else a).data_ptr()),
                        K if f & 1 else tokens, vp(o.data_ptr()), M if f & 2 else tokens, M, tokens, K,
                        f, st)
                else:
                    rc = lib.launch_nvfp4_gemmtc_v5(vp(p.data_ptr()), vp(s.data_ptr()),
                                                    vp(a.data_ptr()), vp(o.data_ptr()), M, tokens,
                                                    K, st)
                assert rc == 0, rc

            for _ in range(3):
                launch()
            torch.cuda.synchronize()
            reps = max(20, 2 * copies) if tokens <= 64 else 5
            graph = None
            if tokens <= 64:    # launches of ~10 us: replay a captured graph, or the host's issue rate is what gets timed
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    st = vp(torch.cuda.current_stream().cuda_stream)
                    for _ in range(reps):
                        launch()
                st = vp(torch.cuda.current_stream().cuda_stream)
                graph.replay()
                torch.cuda.synchronize()
            best = None
            for _ in range(3):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                if graph is not None:
                    graph.replay()
                else:
                    for _ in range(reps):
                        launch()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / reps
                best = us if best is None else min(best, us)
            flops = 2.0 * M * tokens * K
            nbytes = M * K * 0.5625 + 2.0 * K * tokens + 2.0 * M * tokens
            if args.fp4_only:
                nbytes = (M + tokens) * K * 0.5625 + 2.0 * M * tokens
            rows.append({"tokens": tokens, "M": M, "K": K, "us": best, "weight_copies": copies,
                         "tflops": flops / best / 1e6, "frac_tensor_" + tf_kind.split()[0]:
                         flops / best / 1e6 / tf_peak, "gbps": nbytes / best / 1e3,
                         "frac_hbm_" + hbm_kind: nbytes / best / 1e3 / hbm_peak})
            print(f"tokens {tokens:5d}  {M:6d}x{K:<6d} {best:9.1f} us {flops / best / 1e6:8.1f} TFLOP/s "
                  f"({100 * flops / best / 1e6 / tf_peak:4.1f}% of {tf_kind} {tf_peak:.0f}) "
                  f"{nbytes / best / 1e3:7.0f} GB/s", file=sys.stderr, flush=True)
    print(json.dumps({"metric": "nvfp4_gemm_tflops", "unit": "TFLOP/s", "n_gpus": 1, "dtype": "f16",
                      "kernel": ("gemm_fp4_block_scaled_kernel (tcgen05.mma kind::mxf4nvf4, block-16 "
                                 "E8M0 scales in TMEM; activations pre-encoded)" if args.fp4_only else
                                 "encode_kernel + gemm_fp4_block_scaled_kernel (fp16 activations "
                                 "encoded to NVFP4 inside the timed launches)" if args.w4a4 else
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
    """27B-shape decode: 64 layers, hidden 5120, a 512-token prompt through the chunked prefill,
    then 63 greedy tokens from the captured step graph.  Random-init NVFP4 weights, random token
    ids.  Under torchrun the model is tensor-parallel over the ranks (one process per GPU; the
    all-reduces run inside the consuming GEMVs over NVLink peer memory).  quiet: return the result
    dictionary (rank 0; None elsewhere) instead of printing it, and leave the process group up."""
    import torch
    import torch.distributed as dist

    from nvfp4_v100_b200.engine import DecodeEngine, ModelConfig

    world, rank, local = init_ranks()
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
    eng.close()
    del eng
    torch.cuda.empty_cache()
    if not quiet:
        shutdown(world)
    return res


# DRAM bytes (read + write) per average GEMV launch of the mix, from two full-set ncu captures on the
# 151936x5120 shape: the tensor-core kernel, which runs 85 % of the step's bytes, moved 452.1 MB for
# 437.6 MB of algorithmic bytes (profiles/gemv_tc_kernel_lm_head_151936x5120.md: ratio 1.033, reads
# 1.024 + partial-sum slots), the register-streaming kernel 441.69 MB for 437.89 MB
# (profiles/gemv_mma_kernel_lm_head_151936x5120.md: 1.0087).  Every weight byte is read once at any
# shape, so the traffic of the mix's average launch (14 427 447 296 B / 497) is scaled by the
# byte-weighted ratio.
TRAFFIC_PER_LAUNCH = int(14_427_447_296 / 497 * (0.85 * 1.033 + 0.15 * 1.0087))


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
    ap.add_argument("--tc-ring", type=int, default=0, help="tensor-core GEMV weight-ring depth (3 or 5)")
    ap.add_argument("--tc-ctas", type=int, default=0, help="tensor-core GEMV CTAs per SM (1 or 2)")
    ap.add_argument("--tc-pre", type=int, default=0, help="tensor-core GEMV weight stages requested at entry")
    ap.add_argument("--tc-min", type=int, default=-1,
                    help="route GEMVs with M*K >= this many 2^20 elements to the tensor-core kernel "
                         "(nvfp4_b200_gemv_tc_config; 0 = never; default: the library's)")
    ap.add_argument("--tc", action="store_true",
                    help="with --per-shape: the FP4 tensor-core GEMV (launch_nvfp4_gemv_tc)")
    ap.add_argument("--gemm-rows128", action="store_true",
                    help="with --gemm: 128-row CTA tiles only (nvfp4_b200_gemm_config(0))")
    ap.add_argument("--gemm-pair", action="store_true",
                    help="with --gemm: the CTA-pair kernel (cta_group::2) for every shape of more than 128 tokens")
    ap.add_argument("--gemm-config", type=int, default=-1,
                    help="with --gemm: nvfp4_b200_gemm_config flags (1 = single-CTA kernels only, 3 = default)")
    ap.add_argument("--gemm-flags", type=int, default=-1,
                    help="with --gemm: time launch_nvfp4_gemm_w4a16_ex with these layout flags "
                         "(bit 0 token-major activations, bit 1 token-major output, bit 2 add into it)")
    ap.add_argument("--fp4-config", type=int, default=-1,
                    help="with --gemm: nvfp4_b200_gemm_fp4_config flags (bit 0 K split, bit 1 CTA-pair kernel)")
    ap.add_argument("--fp4-no-split", action="store_true",
                    help="with --gemm: FP4 GEMM without the K split of few-tile shapes")
    ap.add_argument("--fp4-only", action="store_true",
                    help="with --gemm: time launch_nvfp4_gemm_fp4 alone on pre-encoded activations")
    ap.add_argument("--tokens", type=int, default=0,
                    help="with --gemm: a single token count instead of 32 and 8192")
    ap.add_argument("--gen", type=int, default=63)
    ap.add_argument("--vocab", type=int, default=VOCAB)
    ap.add_argument("--allreduce", default="peer", choices=["inline", "fused", "peer", "nccl"],
                    help="under torchrun: the all-reduce inside the consuming GEMV's prologue, "
                         "GEMV+all-reduce in one kernel (decode only), a separate one-shot "
                         "peer-memory all-reduce kernel, or NCCL (decode only)")
    ap.add_argument("--cpu-protocol", default="full", choices=["full", "quick", "none"],
                    help="with --impl reference: how much of the per-shape CPU protocol to run "
                         "beside the timed steps")
    ap.add_argument("--no-decode", action="store_true",
                    help="default mode: skip the 27B-shape decode section of the line")
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
    if args.tc_min >= 0 and args.impl == "ours":
        from nvfp4_v100_b200 import _lib
        _lib.load().nvfp4_b200_gemv_tc_config(args.tc_min)
        _lib.load().nvfp4_b200_gemv_tc_config_plain(args.tc_min)
    if args.tc_pre and args.impl == "ours":
        from nvfp4_v100_b200 import _lib
        _lib.load().nvfp4_b200_gemv_tc_prefetch(args.tc_pre)
    if args.tc_ctas and args.impl == "ours":
        from nvfp4_v100_b200 import _lib
        _lib.load().nvfp4_b200_gemv_tc_ctas(args.tc_ctas)
    if args.tc_ring and args.impl == "ours":
        from nvfp4_v100_b200 import _lib
        _lib.load().nvfp4_b200_gemv_tc_ring(args.tc_ring)
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
