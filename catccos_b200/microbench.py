"""Times the single-GPU building blocks of the library with CUDA events.

    python -m catccos_b200.microbench gemm  --m 8192 --n 2304 --k 7168 [--cta-pair 0|1|2] [--block-n 0|128|256]
    python -m catccos_b200.microbench quant --m 4096 --k 7168
    python -m catccos_b200.microbench fused --m 1024 --n 2304 --k 7168

Options --iters / --warmup choose the loop lengths, --seconds S repeats the kernel for about S seconds
while sampling nvidia-smi clocks (what the SM clock is under this kernel's load), --flush flushes L2
between timed launches.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import time

import torch

from . import capi


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for e0, e1 in evs:
        if flush is not None:
            flush.fill_(1)
            flush.view(torch.int32).sum()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    ts = sorted(e0.elapsed_time(e1) * 1e3 for e0, e1 in evs)
    return ts[len(ts) // 2], ts[0]


def _clocks_under_load(fn, seconds):
    q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.sw_power_cap,clocks_event_reasons.hw_slowdown"
    proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100"],
                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    t0 = time.time()
    n = 0
    while time.time() - t0 < seconds:
        for _ in range(200):
            fn()
        torch.cuda.synchronize()
        n += 200
    dt = time.time() - t0
    proc.terminate()
    out = proc.communicate()[0].strip().splitlines()
    rows = [[c.strip() for c in line.split(",")] for line in out if line.count(",") >= 4]
    sm = sorted(float(r[0]) for r in rows[len(rows) // 3:]) if rows else []
    return {"launches": n, "us_per_launch_wall": dt / n * 1e6, "sm_mhz_median": sm[len(sm) // 2] if sm else None,
            "sm_mhz_min": sm[0] if sm else None, "power_w_max": max((float(r[2]) for r in rows), default=None),
            "sw_power_cap_seen": any(r[3].lower().startswith("active") for r in rows), "samples": len(rows)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "quant", "fused"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--seconds", type=float, default=0.0)
    ap.add_argument("--flush", action="store_true")
    ap.add_argument("--cta-pair", type=int, default=0)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--b-layout", type=int, default=0)
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE", help="library option, e.g. split_k=1")
    args = ap.parse_args()

    torch.cuda.set_device(0)
    L = capi.load()
    capi.set_option("cta_pair", args.cta_pair)
    capi.set_option("block_n", args.block_n)
    capi.set_option("b_layout", args.b_layout)
    for kv in args.opt:
        key, value = kv.split("=")
        capi.set_option(key, int(value))
    m, n, k = args.m, args.n, args.k
    st = torch.cuda.current_stream().cuda_stream
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if args.flush else None
    g = torch.Generator(device="cuda").manual_seed(0)
    res = {"what": args.what, "m": m, "n": n, "k": k}
    if args.what == "quant":
        x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
        codes = torch.empty(m, k, dtype=torch.uint8, device="cuda")
        sc = torch.empty(m, k // 32, dtype=torch.uint8, device="cuda")
        fn = lambda: L.catccos_b200_mx_quant(st, x.data_ptr(), m, k, codes.data_ptr(), sc.data_ptr())  # noqa: E731
        med, mn = _time(fn, args.iters, args.warmup, flush)
        byt = m * k * 2 + m * k + m * k // 32
        res.update(us_median=med, us_min=mn, algorithmic_bytes=byt, gbs=byt / med / 1e3)
    else:
        a = torch.randint(0x20, 0x58, (m, k), dtype=torch.uint8, device="cuda", generator=g)
        asc = torch.randint(120, 130, (m, k // 32), dtype=torch.uint8, device="cuda", generator=g)
        b = torch.randint(0x20, 0x58, (k, n), dtype=torch.uint8, device="cuda", generator=g)
        bsc = torch.randint(120, 130, (k // 64, n, 2), dtype=torch.uint8, device="cuda", generator=g)
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        if args.what == "gemm":
            bb = capi.transpose_weight(b) if args.b_layout else b
            fn = lambda: L.catccos_b200_mx_gemm(st, a.data_ptr(), asc.data_ptr(), bb.data_ptr(), bsc.data_ptr(),  # noqa: E731
                                                c.data_ptr(), m, n, k)
        else:
            x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
            symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(m, k, n, 1), False))
            fn = lambda: capi.mx_quant_allgather_matmul(x, b, bsc, c, symm, 1)  # noqa: E731
        med, mn = _time(fn, args.iters, args.warmup, flush)
        res.update(us_median=med, us_min=mn, tflops=2.0 * m * n * k / med / 1e6)
    if args.seconds > 0:
        res["under_load"] = _clocks_under_load(fn, args.seconds)
    code, status = capi.last_status()
    res["status"] = code
    print(json.dumps(res))


if __name__ == "__main__":
    main()
