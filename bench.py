#!/usr/bin/env python
"""Benchmark of the MXFP8 quantise + AllGather-Matmul path on N B200 GPUs of one node.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                      (the CPU golden path on the host cores)
    python bench.py --kernel gemm|quant --m M --n N --k K     (one kernel alone; the profiling commands use it)

A step is one fused call (quantise, allgather over NVLink, flag-gated tcgen05 GEMM) on the TP prefill
workload: per rank A bf16 [1024, 7168] quantised on the fly, weight shard MXFP8 [7168, 2304], output bf16
[N * 1024, 2304].  Per-rank shapes are fixed as N grows (weak scaling).  After the timed regions the
step's output and the stand-alone quantise + allgather output are compared with the CPU oracle on sampled
rows of every source rank; a mismatch ends the run with a non-zero exit code.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from catccos_b200 import workloads  # noqa: E402

CFG = workloads.CONFIGS["c3_prefill"]
QCFG = workloads.CONFIGS["c2_quant_ag"]
METRIC = "mxfp8_allgather_matmul_tflops"
UNIT = "TFLOP/s"
FP8_NOMINAL_TFLOPS = 4500.0
NVLINK_NOMINAL_GBS = 900.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel at N = 1 (the split-K GEMM
# on 1024 x 2304 x 7168), from an ncu capture of `bench.py --kernel gemm --m 1024 --n 2304 --k 7168`
GEMM_DRAM_TRAFFIC_BYTES_N1 = 24.69e6
PARITY_ROWS_PER_RANK = 32


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def workload_config(world: int) -> dict:
    return {
        "workload": "c3_prefill MXFP8 AllGather-Matmul (TP prefill shape)",
        "m_local": CFG.m_local, "k": CFG.k, "n_local": CFG.n_local, "world": world,
        "a": "bf16 N(0,1), quantised on the fly to E4M3 + E8M0 per 32 along K",
        "b": "E4M3 [K, N_local] + E8M0 [K/64, N_local, 2], from bf16 N(0,0.02)",
        "c": "bf16 [world*m_local, n_local], fp32 accumulate",
        "l2": "flushed between timed steps (256 MiB written, then read back so that no dirty lines remain)",
        "rank_alignment": "one-word all-reduce on the stream before each timed step's start event (not timed)",
    }


def stats(ms: np.ndarray) -> dict:
    s = np.sort(np.asarray(ms, dtype=np.float64))
    return {"mean": float(s.mean()), "p50": float(s[len(s) // 2]), "min": float(s[0]), "max": float(s[-1]),
            "p10": float(s[len(s) // 10]), "p90": float(s[(len(s) * 9) // 10]), "samples": int(len(s))}


# ------------------------------------------------------------------------------------------------
# CPU legs (oracle port of the reference's golden path; with the parity checks below the only parts of
# this file that touch oracle/)
# ------------------------------------------------------------------------------------------------
def cpu_golden_step(world: int, rows_per_rank: int, a_f32, b_deq, torch):
    from oracle import mx_oracle

    return mx_oracle.golden_allgather_matmul_torch([a[:rows_per_rank] for a in a_f32[:world]], b_deq)


def cpu_problem(world: int, torch):
    from oracle import mx_oracle

    a_f32 = [torch.from_numpy(workloads.bf16_bits_to_f32(workloads.activation_bits(CFG, r, seed=0)).copy())
             for r in range(world)]
    bc, bs = mx_oracle.quantize_weight(workloads.weight_bits(CFG, 0, seed=0))
    b_deq = torch.from_numpy(mx_oracle.dequant_weight(bc, bs))
    return a_f32, b_deq


def run_cpu_baseline(world: int, budget_s: float = 12.0) -> dict:
    """Times the torch-CPU port of the reference golden (quantise every rank's A, dequantise, fp32
    matmul) for one rank's problem on all host cores."""
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    a_f32, b_deq = cpu_problem(world, torch)
    cpu_golden_step(world, CFG.m_local, a_f32, b_deq, torch)  # warm-up
    reps, t0 = 0, time.perf_counter()
    while reps < 5 and (time.perf_counter() - t0) < budget_s:
        cpu_golden_step(world, CFG.m_local, a_f32, b_deq, torch)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    flops = workloads.gemm_flops(CFG, world)
    return {
        "value": flops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"one rank's full problem at world {world} ({world}x quantise [1024,7168] + fp32 matmul "
                  f"[{world * CFG.m_local},7168]x[7168,2304]), {reps} repetitions, {dt * 1e3:.1f} ms each",
    }


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    world = args.gpus
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    a_f32, b_deq = cpu_problem(world, torch)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_golden_step(world, CFG.m_local, a_f32, b_deq, torch)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_golden_step(world, CFG.m_local, a_f32, b_deq, torch)
    dt = (time.perf_counter() - t0) / args.steps
    val = workloads.gemm_flops(CFG, world) / dt / 1e12
    sample = (f"every step is one rank's full problem at world {world}: quantise {world} x [1024,7168], "
              f"dequantise, fp32 torch.matmul [{world * CFG.m_local},7168]x[7168,2304] on {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (dequantised E4M3 x E8M0)", "data": "synthetic", "config": workload_config(world),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def sample_rows(m_local: int, world: int, seed: int) -> np.ndarray:
    """PARITY_ROWS_PER_RANK gathered-row indices under every source rank: the shard's first and last rows
    (chunk and tile edges) and seeded rows in between."""
    rng = np.random.default_rng(seed)
    rows = []
    for r in range(world):
        n = min(PARITY_ROWS_PER_RANK, m_local)
        pick = {0, m_local - 1, m_local // 2, min(m_local - 1, 127), min(m_local - 1, 128)}
        while len(pick) < n:
            pick.add(int(rng.integers(0, m_local)))
        rows.extend(r * m_local + i for i in sorted(pick))
    return np.asarray(rows, dtype=np.int64)


def check_c_parity(cfg, world, rows, c_rows_f32, b_codes, b_scales, seed=0) -> dict:
    """The step's output rows against the oracle: quantise the sampled rows of every rank's A, dequantise,
    fp32 GEMM with the dequantised weight; |out - gold| <= 1e-3 + 1e-2 |gold| (the benchmark's tolerance)."""
    from oracle import mx_oracle

    bits = {r: workloads.activation_bits(cfg, r, seed=seed) for r in sorted({int(i) // cfg.m_local for i in rows})}
    a_bits = np.stack([bits[int(i) // cfg.m_local][int(i) % cfg.m_local] for i in rows])
    ac, asc = mx_oracle.quantize_rows(a_bits)
    gold = mx_oracle.gemm_f32(mx_oracle.dequant_rows(ac, asc), mx_oracle.dequant_weight(b_codes, b_scales))
    bad, maxdiff = mx_oracle.check_close(c_rows_f32, gold, 1e-2, 1e-3)
    return {"c_bad": int(bad), "c_max_abs_diff": float(maxdiff), "rows_checked": int(len(rows))}


def check_quant_parity(cfg, world, rows, codes_rows, scales_rows, seed=0) -> dict:
    from oracle import mx_oracle

    bits = {r: workloads.activation_bits(cfg, r, seed=seed) for r in sorted({int(i) // cfg.m_local for i in rows})}
    a_bits = np.stack([bits[int(i) // cfg.m_local][int(i) % cfg.m_local] for i in rows])
    ac, asc = mx_oracle.quantize_rows(a_bits)
    return {"codes_bad": int((ac != codes_rows).sum()), "scales_bad": int((asc != scales_rows).sum()),
            "quant_rows_checked": int(len(rows))}


# ------------------------------------------------------------------------------------------------
# clocks, placement
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str):
        self.uuid, self.proc, self.path = uuid, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx = float(parts[1])
                except ValueError:
                    continue
                for nm, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


def bind_to_gpu_numa_node(torch, local_rank: int) -> str:
    """Runs this process on the CPUs next to its GPU, so that the pinned host buffers it allocates afterwards
    (first touch) sit on that NUMA node and the PCIe copies do not cross the socket link."""
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        bdf = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            if "-" in part:
                lo, hi = part.split("-")
                cpus.update(range(int(lo), int(hi) + 1))
            elif part:
                cpus.add(int(part))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"cpus {spec} (next to GPU {bdf})"
    except (OSError, AttributeError, ValueError):
        pass
    return "unchanged"


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def quantise_weight_on_gpu(capi, torch, cfg, rank, dev):
    """The weight shard quantised by the library's own kernel on the transposed weight (blocks of 32 run along
    K): B^T [N, K] rows -> codes [N, K], scales [N, K/32]; stored as [K, N] / [K/64, N, 2]."""
    w_bits = workloads.weight_bits(cfg, rank, seed=0)
    wt = torch.from_numpy(np.ascontiguousarray(w_bits.T).view(np.int16).copy()).to(dev).view(torch.bfloat16)
    wc, ws = capi.mx_quant(wt)
    b_codes = wc.t().contiguous()
    b_scales = ws.t().contiguous().view(cfg.k // 64, 2, cfg.n_local).permute(0, 2, 1).contiguous()
    return b_codes, b_scales


def run_gpu(args) -> None:
    import torch
    import torch.distributed as dist

    from catccos_b200 import build, capi

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the GPU arm")
    torch.cuda.set_device(local_rank)
    placement = bind_to_gpu_numa_node(torch, local_rank)
    if rank == 0:
        build.build()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist.barrier()
        port = int(os.environ.get("MASTER_PORT", "29500")) + 211
        capi.init(rank, world, local_rank, f"tcp://127.0.0.1:{port}")
    else:
        capi.init(0, 1, local_rank, None)
    dev = torch.device("cuda", local_rank)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- data (seeded, resident in HBM before the timed region) ----
    a_bits = workloads.activation_bits(CFG, rank, seed=0)
    n_buf = 2  # host and device buffers of the end-to-end pipeline
    a_host = [torch.from_numpy(a_bits.view(np.int16).copy()).view(torch.bfloat16).pin_memory() for _ in range(n_buf)]
    a_dev = a_host[0].to(dev, non_blocking=False)
    b_codes, b_scales = quantise_weight_on_gpu(capi, torch, CFG, rank, dev)
    c_dev = torch.empty((world * CFG.m_local, CFG.n_local), dtype=torch.bfloat16, device=dev)
    tiling = capi.make_tiling(CFG.m_local, CFG.k, CFG.n_local, world)
    symm = capi.symm_alloc(capi.symm_bytes_needed(tiling, False))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    flush_sink = torch.zeros((), dtype=torch.int64, device=dev)

    def step():
        capi.mx_quant_allgather_matmul(a_dev, b_codes, b_scales, c_dev, symm, world)

    align_word = torch.zeros(1, dtype=torch.float32, device=dev)

    def timed(fn, steps, warmup, flush_l2=True):
        barrier()
        for _ in range(warmup):
            fn()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for e0, e1 in evs:
            if flush_l2:
                flush.fill_(1)  # evict everything ...
                flush_sink.copy_(flush.view(torch.int32).sum())  # ... and read it back: no dirty lines remain
            if world > 1:
                # a one-word all-reduce on the stream, outside the timed region: the ranks' streams reach the
                # step within microseconds of each other instead of carrying the flush kernels' jitter into it
                dist.all_reduce(align_word)
            e0.record()
            fn()
            e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) for e0, e1 in evs], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)  # per step: the slowest rank
        return ms.cpu().numpy()

    warmup = max(args.warmup, 3)
    barrier()  # the ranks' set-up times differ by more than a device-side wait's limit: start the first call together
    uuid = str(torch.cuda.get_device_properties(local_rank).uuid)
    sampler = ClockSampler("GPU-" + uuid if not uuid.startswith("GPU-") else uuid)
    if rank == 0:
        sampler.start()
    # the timed region lasts a few milliseconds, far below nvidia-smi's sampling period: hold the GPU under
    # the same load for about 1.5 s first (same step count on every rank) so that the clock record means something
    calib = timed(step, 20, warmup, flush_l2=False)
    n_load = int(min(40000, max(0, 1.5e3 / max(float(calib.mean()), 1e-3))))
    for _ in range(n_load):
        step()
    barrier()
    launches0 = capi.launch_count()
    ms = timed(step, args.steps, warmup)
    launches = capi.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    code, st = capi.last_status()
    if code != 0:
        raise SystemExit(f"device-side wait ran out: {st}")
    ms_per_step = float(ms.mean())
    flops_per_gpu = workloads.gemm_flops(CFG, world)
    value = world * flops_per_gpu / (ms_per_step * 1e-3) / 1e12

    # ---- parity of the step that was timed: sampled rows of every source rank against the oracle ----
    rows = sample_rows(CFG.m_local, world, seed=1234 + rank)
    c_dev.zero_()
    step()
    torch.cuda.synchronize()
    rows_t = torch.from_numpy(rows).to(dev)
    parity = check_c_parity(CFG, world, rows, c_dev[rows_t].float().cpu().numpy(), b_codes.cpu().numpy(),
                            b_scales.cpu().numpy())

    # ---- the dominant kernel alone.  With one rank the step is the quantise kernel followed by the GEMM kernel
    # on one stream; the GEMM kernel is timed by itself on the same quantised operands (same flush, same events).
    # With several ranks the quantise-and-push warps ride inside the GEMM kernel, which then spans the step. ----
    gemm_ms = ms_per_step
    if world == 1:
        qa_codes, qa_scales = capi.mx_quant(a_dev)
        lib = capi.load()
        stream = torch.cuda.current_stream().cuda_stream

        def gemm_only():
            rc = lib.catccos_b200_mx_gemm(stream, qa_codes.data_ptr(), qa_scales.data_ptr(), b_codes.data_ptr(),
                                          b_scales.data_ptr(), c_dev.data_ptr(), CFG.m_local, CFG.n_local, CFG.k)
            if rc != 0:
                raise SystemExit(f"catccos_b200_mx_gemm: {rc}")

        gemm_ms = float(timed(gemm_only, args.steps, warmup).mean())
    gemm_tflops = flops_per_gpu / (gemm_ms * 1e-3) / 1e12

    # ---- end to end through the C ABI with HOST buffers.  Every step copies A from pinned host memory, runs
    # the fused call and copies C back to pinned host memory; the three run on three streams chained by events,
    # two buffers deep, so that step i's copy-out, step i+1's call and step i+2's copy-in overlap (both PCIe
    # directions busy).  Timed as one region over all steps. ----
    c_host = [torch.empty((world * CFG.m_local, CFG.n_local), dtype=torch.bfloat16).pin_memory() for _ in range(n_buf)]
    a_devs = [a_dev, torch.empty_like(a_dev)]
    c_devs = [c_dev, torch.empty_like(c_dev)]
    s_in, s_out, s_main = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]
    ev_done = [torch.cuda.Event() for _ in range(n_buf)]
    ev_out = [torch.cuda.Event() for _ in range(n_buf)]

    def e2e_steps(n):
        for i in range(n):
            b = i % n_buf
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[b])  # the call that last read this A buffer has finished
                a_devs[b].copy_(a_host[b], non_blocking=True)
                ev_in[b].record(s_in)
            s_main.wait_event(ev_in[b])
            s_main.wait_event(ev_out[b])  # the copy that last read this C buffer has finished
            capi.mx_quant_allgather_matmul(a_devs[b], b_codes, b_scales, c_devs[b], symm, world)
            ev_done[b].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                c_host[b].copy_(c_devs[b], non_blocking=True)
                ev_out[b].record(s_out)
        s_main.wait_stream(s_out)

    e2e_n = max(4, min(args.steps, 20))
    e2e_steps(4)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_steps(e2e_n)
    e1.record()
    barrier()
    e2e_ms_t = torch.tensor([e0.elapsed_time(e1) / e2e_n], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms_t, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms_t.item())
    e2e_value = world * flops_per_gpu / (e2e_ms * 1e-3) / 1e12
    e2e_ok = bool(torch.equal(c_host[0].to(dev), c_devs[0]))
    del c_devs, a_devs

    # ---- extras, each on its own: a broken leg reports its own error and takes nothing else with it ----
    extras = {}

    def leg(name, fn):
        try:
            extras[name] = fn()
        except Exception as exc:  # noqa: BLE001 - reported, not swallowed: the key carries the error
            extras[name] = {"error": repr(exc)}
            barrier()

    def quant_allgather_leg():
        qa_bits = workloads.activation_bits(QCFG, rank, seed=0)
        qa = torch.from_numpy(qa_bits.view(np.int16).copy()).to(dev).view(torch.bfloat16)
        qt = capi.make_tiling(QCFG.m_local, 1, QCFG.k, world)
        qsymm = capi.symm_alloc(capi.symm_bytes_needed(qt, True)) if world > 1 else 0
        nc, ns = world * QCFG.m_local * QCFG.k, world * QCFG.m_local * (QCFG.k // 32)
        if world > 1:
            # outputs in symmetric memory (what the operator class allocates): the peers' shards land in them directly
            ns_off = (nc + 1023) // 1024 * 1024
            qout = capi.symm_alloc(ns_off + ns)
            qc = capi.symm_tensor(qout, nc).view(world * QCFG.m_local, QCFG.k)
            qs = capi.symm_tensor(qout, ns, ns_off).view(world * QCFG.m_local, QCFG.k // 32)
        else:
            qc = torch.empty((world * QCFG.m_local, QCFG.k), dtype=torch.uint8, device=dev)
            qs = torch.empty((world * QCFG.m_local, QCFG.k // 32), dtype=torch.uint8, device=dev)
        q_ms = timed(lambda: capi.mx_quant_allgather(qa, qc, qs, qsymm, world), 20, 3)
        q_us = float(np.median(q_ms)) * 1e3
        qrows = sample_rows(QCFG.m_local, world, seed=99 + rank)
        qrows_t = torch.from_numpy(qrows).to(dev)
        parity.update(check_quant_parity(QCFG, world, qrows, qc[qrows_t].cpu().numpy(), qs[qrows_t].cpu().numpy()))
        del qc, qs
        if world > 1:
            capi.symm_free(qout)
            capi.symm_free(qsymm)
        return {
            "workload": f"c2 per rank bf16 [{QCFG.m_local},{QCFG.k}] at world {world}", "us": q_us,
            "us_stats": stats(q_ms * 1e3),
            "hbm_gbs": workloads.quant_ag_hbm_bytes(QCFG, world) / q_us / 1e3,
            "nvlink_ingress_gbs": workloads.quant_ag_ingress_bytes(QCFG, world) / q_us / 1e3,
            "frac_of_bound": (max(workloads.quant_ag_ingress_bytes(QCFG, world) / NVLINK_NOMINAL_GBS,
                                  workloads.quant_ag_hbm_bytes(QCFG, world) / read_peaks()["hbm_gbs"]) / 1e3) / q_us,
        }

    def unfused_leg():
        # quantise, NCCL all-gather of codes and scales, then the same GEMM kernel on gathered data
        g_codes = torch.empty((world * CFG.m_local, CFG.k), dtype=torch.uint8, device=dev)
        g_scales = torch.empty((world * CFG.m_local, CFG.k // 32), dtype=torch.uint8, device=dev)

        def unfused():
            codes, scales = capi.mx_quant(a_dev)
            if world > 1:
                dist.all_gather_into_tensor(g_codes, codes)
                dist.all_gather_into_tensor(g_scales, scales)
                capi.mx_gemm(g_codes, g_scales, b_codes, b_scales, out=c_dev)
            else:
                capi.mx_gemm(codes, scales, b_codes, b_scales, out=c_dev)

        u_ms = timed(unfused, 20, 3)
        return {"what": "quantise kernel, ncclAllGather of codes and of scales, GEMM kernel on local memory",
                "ms_per_step": float(u_ms.mean()), "ms_stats": stats(u_ms),
                "tflops_per_gpu": flops_per_gpu / (float(u_ms.mean()) * 1e-3) / 1e12}

    def decode_leg():
        # decode shape (C5): per-call latency over 1000 calls, no L2 flush (weights stay hot, as in a decode loop)
        dcfg = workloads.CONFIGS["c5_decode"]
        d_a = torch.from_numpy(workloads.activation_bits(dcfg, rank, seed=0).view(np.int16).copy()).to(dev).view(torch.bfloat16)
        d_b, d_bs = quantise_weight_on_gpu(capi, torch, dcfg, rank, dev)
        d_c = torch.empty((world * dcfg.m_local, dcfg.n_local), dtype=torch.bfloat16, device=dev)
        d_symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(dcfg.m_local, dcfg.k, dcfg.n_local, world), False))
        d_ms = timed(lambda: capi.mx_quant_allgather_matmul(d_a, d_b, d_bs, d_c, d_symm, world), 1000, 20, flush_l2=False)
        d_us = np.sort(d_ms) * 1e3
        d_flops = workloads.gemm_flops(dcfg, world)
        drows = np.arange(world * dcfg.m_local)
        dpar = check_c_parity(dcfg, world, drows, d_c.float().cpu().numpy(), d_b.cpu().numpy(), d_bs.cpu().numpy())
        parity["decode_c_bad"] = dpar["c_bad"]
        capi.symm_free(d_symm)
        return {
            "workload": f"c5 per rank A bf16 [16,7168], B MXFP8 [7168,4096], C bf16 [{world * 16},4096], 1000 calls",
            "p50_us": float(d_us[500]), "p99_us": float(d_us[990]),
            "tflops_per_gpu_at_p50": d_flops / float(d_us[500]) / 1e6,
            "weight_stream_floor_us": (dcfg.k * dcfg.n_local * 33 / 32) / read_peaks()["hbm_gbs"] / 1e3,
        }

    def fp4_gemm_leg():
        # the FP4 operator's GEMM (packed E2M1 operands, E8M0 scales per 32 along K) on the headline shape, kernel
        # alone: the per-call copy of the weight into K-major order and the GEMM.  Random codes; parity of this
        # path is the tests' business (tests/test_gemm_gpu.py), nothing is checked here.
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        mg, kk, nn = world * CFG.m_local, CFG.k, CFG.n_local
        fa = torch.randint(0, 256, (mg, kk // 2), dtype=torch.uint8, device=dev, generator=gen)
        fas = torch.randint(122, 128, (mg, kk // 32), dtype=torch.uint8, device=dev, generator=gen)
        fb = torch.randint(0, 256, (kk, nn // 2), dtype=torch.uint8, device=dev, generator=gen)
        fbs = torch.randint(122, 128, (kk // 64, nn, 2), dtype=torch.uint8, device=dev, generator=gen)
        capi.set_option("a_dtype", 2)
        capi.set_option("b_dtype", 2)
        try:
            fc = torch.empty((mg, nn), dtype=torch.bfloat16, device=dev)
            lib, stream = capi.load(), torch.cuda.current_stream().cuda_stream

            def fp4_call():
                rc = lib.catccos_b200_mx_gemm(stream, fa.data_ptr(), fas.data_ptr(), fb.data_ptr(), fbs.data_ptr(),
                                              fc.data_ptr(), mg, nn, kk)
                if rc != 0:
                    raise RuntimeError(f"catccos_b200_mx_gemm (fp4) returned {rc}")

            f_ms = timed(fp4_call, 20, 3)
        finally:
            capi.set_option("a_dtype", 0)
            capi.set_option("b_dtype", 0)
        return {"what": f"mx_gemm on packed E2M1 operands [{mg},{kk}] x [{kk},{nn}] (kind::mxf8f6f4: the FP8 issue rate), "
                        "weight copied to K-major order inside every call",
                "ms_per_call": float(f_ms.mean()), "ms_stats": stats(f_ms),
                "tflops_per_gpu": flops_per_gpu / (float(f_ms.mean()) * 1e-3) / 1e12}

    if not args.lean:
        leg("quant_allgather", quant_allgather_leg)
        leg("decode_c5", decode_leg)
        leg("unfused_baseline", unfused_leg)
        leg("fp4_gemm", fp4_gemm_leg)
    code, st = capi.last_status()
    if code != 0:
        raise SystemExit(f"device-side wait ran out in an extra leg: {st}")

    # every rank checked its own output; the line carries the sum over ranks
    keys = sorted(k for k in parity if k.endswith("_bad"))
    if world > 1:
        agg = torch.tensor([parity[k] for k in keys], dtype=torch.int64, device=dev)
        dist.all_reduce(agg)
        for k, v in zip(keys, agg.cpu().tolist()):
            parity[k] = int(v)
        parity["ranks_checked"] = world
    parity["e2e_host_copy_equals_device"] = e2e_ok
    parity_failed = any(parity[k] != 0 for k in keys) or not e2e_ok

    peaks = read_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    per_gpu = flops_per_gpu / (ms_per_step * 1e-3) / 1e12
    t_compute = flops_per_gpu / (FP8_NOMINAL_TFLOPS * 1e12)
    t_link = (world - 1) * CFG.m_local * (CFG.k + CFG.k // 32) / (NVLINK_NOMINAL_GBS * 1e9)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "ms_per_step_stats": stats(ms), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8 e4m3 x e8m0 block scales, fp32 accumulate, bf16 out", "data": "synthetic",
        "config": workload_config(world),
        "per_gpu_tflops": per_gpu,
        "frac_of_nominal_roofline": max(t_compute, t_link) / (ms_per_step * 1e-3),
        "roofline": {
            "bound": "tensor", "achieved": gemm_tflops, "peak": fp8_peak, "unit": UNIT, "frac": gemm_tflops / fp8_peak,
            "traffic": GEMM_DRAM_TRAFFIC_BYTES_N1 if world == 1 else None,
            "kernel": "mx_gemm_kernel (tcgen05.mma kind::mxf8f6f4.block_scale)",
            "kernel_ms": gemm_ms,
            "peak_source": f"2 x cuBLAS bf16 burst of {peaks['source']} ({peaks['bf16_tflops']} TFLOP/s); "
                           "the peaks file holds no fp8 figure, fp8 issues at twice the bf16 rate",
            "achieved_from": "2*(world*m_local)*k*n_local FLOP per launch / CUDA-event time of the GEMM kernel: "
                             + ("timed alone on the step's quantised operands (the step is quantise kernel, then GEMM kernel)"
                                if world == 1 else
                                "the step time: the flag-gated kernel's span depends on when its rows arrive"),
        },
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(a_host[0].numel() * 2), "d2h_bytes_per_step": int(c_host[0].numel() * 2),
                "how": f"{e2e_n} steps as one timed region; copy-in, call and copy-out on three streams, two buffers deep",
                "host_placement": placement},
        "gpu_launches": int(launches),
        "parity": parity,
        "clocks": clocks,
        **extras,
    }
    if rank == 0:
        if world == 1 and not args.lean:
            line["cpu_baseline"] = run_cpu_baseline(1)
        print(json.dumps(line))
    barrier()
    capi.finalize()
    if world > 1:
        dist.destroy_process_group()
    if parity_failed:
        raise SystemExit(f"parity check failed: {parity}")


# ------------------------------------------------------------------------------------------------
# one kernel alone (what the committed profiling commands run under ncu; also a quick timing by CUDA events)
# ------------------------------------------------------------------------------------------------
def run_kernel(args) -> None:
    import torch

    from catccos_b200 import build, capi

    torch.cuda.set_device(0)
    build.build()
    L = capi.load()
    capi.init(0, 1, 0, None)
    m, n, k = args.m, args.n, args.k
    st = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    if args.kernel == "quant":
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        codes = torch.empty(m, k, dtype=torch.uint8, device="cuda")
        sc = torch.empty(m, k // 32, dtype=torch.uint8, device="cuda")
        fn = lambda: L.catccos_b200_mx_quant(st, x.data_ptr(), m, k, codes.data_ptr(), sc.data_ptr())  # noqa: E731
        work, unit = (m * k * 2 + m * k + m * k // 32) / 1e3, "GB/s"
    else:
        a = torch.randint(0x20, 0x58, (m, k), dtype=torch.uint8, device="cuda", generator=g)
        asc = torch.randint(120, 130, (m, k // 32), dtype=torch.uint8, device="cuda", generator=g)
        b = torch.randint(0x20, 0x58, (k, n), dtype=torch.uint8, device="cuda", generator=g)
        bsc = torch.randint(120, 130, (k // 64, n, 2), dtype=torch.uint8, device="cuda", generator=g)
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        fn = lambda: L.catccos_b200_mx_gemm(st, a.data_ptr(), asc.data_ptr(), b.data_ptr(), bsc.data_ptr(),  # noqa: E731
                                            c.data_ptr(), m, n, k)
        work, unit = 2.0 * m * n * k / 1e6, "TFLOP/s"
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for e0, e1 in evs:
        flush.fill_(1)
        flush.view(torch.int32).sum()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    us = np.array([e0.elapsed_time(e1) * 1e3 for e0, e1 in evs])
    code, status = capi.last_status()
    print(json.dumps({"kernel": args.kernel, "m": m, "n": n, "k": k, "us": stats(us), "rate_at_p50": work / float(np.median(us)),
                      "unit": unit, "l2": "flushed before every launch", "status": code}))
    capi.finalize()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--lean", action="store_true",
                    help="headline step, end-to-end and parity only (no extra legs, no CPU baseline): the launch-list capture")
    ap.add_argument("--kernel", choices=["gemm", "quant"], default=None,
                    help="time one kernel alone on one GPU instead of the benchmark (shape: --m --n --k)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=7168)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.kernel is not None:
        run_kernel(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
