"""Device-side timeline of one fused quantise + AllGather-Matmul step (the trace build of the library).

    python -m catccos_b200.build --trace
    CATCCOS_B200_TRACE=1 python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29533 -m catccos_b200.timeline --gpus N [--m 1024 --k 7168 --n 2304] [--opt key=value ...]

Every rank warms the step up, arms the timeline for one launch (L2 flushed, ranks aligned by a one-word
all-reduce, as in bench.py), reads the per-CTA stamps back and reduces them; rank 0 prints one table per rank.
Times are microseconds since the first CTA of that rank started (each GPU has its own %globaltimer; ranks are
not compared with each other).  "min / med / max" run over the CTAs (or pushers) that wrote the slot.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from . import workloads

# slot layout: csrc/trace.cuh
STAMPS = [
    ("setup done", 1), ("first TMA load issued", 2), ("last TMA load issued", 3), ("first MMA", 6), ("last tile committed", 7),
    ("epilogue: last tile written", 10), ("quantise: first item published", 12), ("quantise: last item published", 13),
    ("CTA end", 72),
]
WAITS = [
    ("TMA producer waiting for ready flags", 4), ("TMA producer waiting for a free stage", 5),
    ("MMA issuer waiting for full stages", 8), ("MMA issuer waiting for an accumulator", 9),
    ("epilogue waiting for accumulators", 11), ("quantise thread 0 in barrier + fence + flags", 14),
]
PUSH_FIRST, PUSH_LAST, PUSH_FLAGWAIT, PUSH_FENCE, PUSH_ITEMS = 16, 22, 28, 34, 40
TILE_START, TILE_END, TILES = 46, 55, 9
SF_GATE, SF_EMPTY = 64, 68


def _mmm(v):
    v = np.asarray(v, dtype=np.float64)
    if v.size == 0:
        return None
    return [round(float(v.min()), 2), round(float(np.median(v)), 2), round(float(v.max()), 2)]


def summarise(tr: np.ndarray) -> dict:
    """tr: [CTAs, slots] uint64 -> a dict of [min, median, max] in microseconds."""
    t0 = tr[:, 0][tr[:, 0] > 0].min()
    out = {"ctas": int(tr.shape[0])}

    def rel(col):
        v = tr[:, col]
        return (v[v > 0].astype(np.float64) - float(t0)) / 1e3

    out["CTA start"] = _mmm(rel(0))
    qs, qe = int(tr[0, 73]), int(tr[0, 74])
    if qe > 0 and qs != 0xFFFFFFFFFFFFFFFF:
        out["quantise kernel: first CTA starts / last CTA ends"] = [round((qs - float(t0)) / 1e3, 2), round((qe - float(t0)) / 1e3, 2)]
    for name, col in STAMPS:
        out[name] = _mmm(rel(col))
    for name, col in WAITS:
        v = tr[:, col]
        out[name + " (total per CTA)"] = _mmm(v[v > 0].astype(np.float64) / 1e3)
    q = tr[:, 15]
    out["quantise items per CTA"] = _mmm(q[q > 0])
    first = np.concatenate([rel(PUSH_FIRST + i) for i in range(6)])
    last = np.concatenate([rel(PUSH_LAST + i) for i in range(6)])
    out["pusher: first item's local flag seen"] = _mmm(first)
    out["pusher: last item's peer flags stored"] = _mmm(last)
    for name, base in (("pusher waiting for local flags (total per pusher)", PUSH_FLAGWAIT),
                       ("pusher in system fences (total per pusher)", PUSH_FENCE)):
        v = tr[:, base:base + 6].reshape(-1)
        out[name] = _mmm(v[v > 0].astype(np.float64) / 1e3)
    it = tr[:, PUSH_ITEMS:PUSH_ITEMS + 6].reshape(-1)
    out["pusher items (per working pusher)"] = _mmm(it[it > 0])
    for i in range(TILES):
        s, e = rel(TILE_START + i), rel(TILE_END + i)
        if s.size:
            out[f"tile {i}: producer starts"] = _mmm(s)
        if e.size:
            out[f"tile {i}: issuer commits"] = _mmm(e)
        both = (tr[:, TILE_START + i] > 0) & (tr[:, TILE_END + i] > 0)
        if both.any():
            out[f"tile {i}: duration"] = _mmm((tr[both, TILE_END + i].astype(np.float64) - tr[both, TILE_START + i].astype(np.float64)) / 1e3)
    for name, base in (("scale loader waiting for ready flags (total per warp)", SF_GATE),
                       ("scale loader waiting for a free stage (total per warp)", SF_EMPTY)):
        v = tr[:, base:base + 4].reshape(-1)
        out[name] = _mmm(v[v > 0].astype(np.float64) / 1e3)
    return out


def main():
    import torch
    import torch.distributed as dist

    from . import capi

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--m", type=int, default=1024)
    ap.add_argument("--k", type=int, default=7168)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE", help="library option (test hooks included)")
    ap.add_argument("--label", default="")
    ap.add_argument("--raw", default="", help="also save every rank's raw [CTAs, slots] array to this .npz")
    ap.add_argument("--sweep", action="append", default=[], metavar="KEY=V1,V2,...",
                    help="no timeline: time the step (20 launches, slowest rank per launch) under every value of one "
                         "option, in one process; given more than once, under every combination; works with the "
                         "product build too")
    ap.add_argument("--also-shape", action="append", default=[], metavar="M,K,N",
                    help="with --sweep: one more per-rank shape to run the same sweep on (may be repeated)")
    args = ap.parse_args()
    if not capi.TRACE and not args.sweep:
        raise SystemExit("set CATCCOS_B200_TRACE=1: the timeline needs the trace build of the library")

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus

    def progress(what):
        print(f"[timeline rank {rank}] {what}", file=sys.stderr, flush=True)

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        dist.barrier()
        capi.init(rank, world, local_rank, f"tcp://127.0.0.1:{int(os.environ.get('MASTER_PORT', '29500')) + 223}")
    else:
        capi.init(0, 1, local_rank, None)
    for kv in args.opt:
        key, val = kv.split("=", 1)
        capi.set_option(key, int(val))
    progress("library initialised")

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    word = torch.zeros(1, device=dev)

    def make_step(m, k, n):
        """Buffers of one shape and the function that runs (and times) one step on them."""
        cfg = workloads.Config("timeline", m, k, n, (world,), "normal", "")
        a = torch.from_numpy(workloads.activation_bits(cfg, rank, seed=0).view(np.int16).copy()).to(dev).view(torch.bfloat16)
        wt = torch.from_numpy(np.ascontiguousarray(workloads.weight_bits(cfg, rank, seed=0).T).view(np.int16).copy()).to(dev).view(torch.bfloat16)
        wc, ws = capi.mx_quant(wt)
        b = wc.t().contiguous()
        bs = ws.t().contiguous().view(cfg.k // 64, 2, cfg.n_local).permute(0, 2, 1).contiguous()
        c = torch.empty((world * m, n), dtype=torch.bfloat16, device=dev)
        symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(m, k, n, world), False))

        def one():
            flush.fill_(1)
            flush.view(torch.int32).sum()
            if world > 1:
                dist.all_reduce(word)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            capi.mx_quant_allgather_matmul(a, b, bs, c, symm, world)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3

        return one

    if args.sweep:
        import itertools

        keys = [sw.split("=", 1)[0] for sw in args.sweep]
        points = list(itertools.product(*[sw.split("=", 1)[1].split(",") for sw in args.sweep]))
        shapes = [(args.m, args.k, args.n)] + [tuple(int(x) for x in sh.split(",")) for sh in args.also_shape]
        res = {}
        for (m, k, n) in shapes:
            one = make_step(m, k, n)
            progress(f"buffers ready for {m}x{k}x{n}")
            for point in points:
                for key, val in zip(keys, point):
                    capi.set_option(key, int(val))
                for _ in range(args.warmup):
                    one()
                t = torch.tensor([one() for _ in range(20)], dtype=torch.float64, device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ts = sorted(t.cpu().tolist())
                code, st = capi.last_status()
                name = f"{m}x{k}x{n} " + " ".join(f"{key}={val}" for key, val in zip(keys, point))
                res[name] = {"p50_us": round(ts[10], 2), "min_us": round(ts[0], 2), "max_us": round(ts[-1], 2), "status": code}
                progress(f"{name}: {res[name]}")
        if rank == 0:
            print(json.dumps({"sweep": res, "world": world, "trace_build": capi.TRACE}))
        if world > 1:
            dist.barrier()
        capi.finalize()
        if world > 1:
            dist.destroy_process_group()
        return
    one = make_step(args.m, args.k, args.n)
    progress("buffers ready")
    for i in range(args.warmup):
        us = one()
        if i == 0:
            progress(f"first step done in {us:.1f} us, status {capi.last_status()}")
    plain = sorted(one() for _ in range(10))
    progress(f"untraced steps done, p50 {plain[5]:.1f} us")
    if world > 1:
        dist.barrier()
    capi.trace_arm()
    us = one()
    tr = capi.trace_read()
    code, st = capi.last_status()
    summary = {"rank": rank, "label": args.label, "options": args.opt, "shape": [args.m, args.k, args.n], "world": world,
               "status": code, "step_us_by_events": round(us, 2), "untraced_step_us_p50": round(plain[5], 2),
               **summarise(tr)}
    gathered = [summary]
    raws = [tr]
    if world > 1:
        gathered = [None] * world
        dist.all_gather_object(gathered, summary)
        raws = [None] * world
        dist.all_gather_object(raws, tr)
    if rank == 0:
        keys = [k for k in gathered[0] if isinstance(gathered[0][k], list) and k not in ("options", "shape")]
        print(f"== timeline {args.label} world {world} shape {args.m}x{args.k}x{args.n} options {args.opt}")
        print("   step us by CUDA events (traced launch): " + " ".join(f"r{g['rank']}={g['step_us_by_events']}" for g in gathered))
        print("   step us p50 of 10 untraced launches:    " + " ".join(f"r{g['rank']}={g['untraced_step_us_p50']}" for g in gathered))
        for k in keys:
            cells = ["/".join(str(x) for x in g[k]) if g.get(k) else "-" for g in gathered]
            print(f"   {k:62s} " + "  ".join(f"r{i}:{cell}" for i, cell in enumerate(cells)))
        print(json.dumps({"timeline": gathered}))
        if args.raw:
            np.savez_compressed(args.raw, **{f"rank{i}": r for i, r in enumerate(raws)})
    if world > 1:
        dist.barrier()
    capi.finalize()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
