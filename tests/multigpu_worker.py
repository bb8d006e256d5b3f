"""Worker of tests/test_multigpu.py: one process per GPU (launched by torch.distributed.run).  Each rank
drives the C ABI in its real multi-process mode (cuMem/VMM peer-mapped symmetric buffers, flags over
NVLink) and checks its results against the oracle: gathered codes and scales bit for bit, GEMM output
within rtol 1e-2 / atol 1e-3.  The benchmark configurations run at their full per-rank sizes; the oracle
is evaluated on sampled rows of every source rank there (shard and tile edges plus seeded rows)."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from catccos_b200 import capi, workloads  # noqa: E402
from oracle import mx_oracle  # noqa: E402


def dev_bf16(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).cuda().view(torch.bfloat16)


def sample_rows(m, world, rng, per_rank=24):
    rows = []
    for s in range(world):
        pick = {0, m - 1, m // 2, min(m - 1, 127), min(m - 1, 128), min(m - 1, 255), min(m - 1, 256)}
        while len(pick) < min(per_rank, m):
            pick.add(int(rng.integers(0, m)))
        rows.extend(s * m + i for i in sorted(pick))
    return np.asarray(rows, dtype=np.int64)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    torch.distributed.init_process_group("gloo")  # host-side barrier only: the ranks enter each call together
    port = int(os.environ.get("MASTER_PORT", "29500")) + 97
    capi.init(rank, world, local, f"tcp://127.0.0.1:{port}")

    # sections to run, e.g. "mmrs,fp4" as the first argument (default: all)
    only = set(sys.argv[1].split(",")) if len(sys.argv) > 1 else {"quant_ag", "agmm", "mmrs", "fp4"}

    def status_ok(tag):
        code, st = capi.last_status()
        assert code == 0, (tag, rank, st)

    # ---- quantise + allgather: gathered outputs identical on every rank, bit-exact.  C2 and the reference's
    # ragged M = 8190 at full size (sampled rows), small shapes in full; outputs in plain device memory
    # (through the stage) and in symmetric memory (written by the peers directly) ----
    for (m, k, dist_name) in [(256, 1024, "normal"), (190, 512, "normal"), (4096, 7168, "normal"), (8190, 1024, "normal"),
                              (512, 5120, "student_t3_outlier")] if "quant_ag" in only else []:
        cfg = workloads.Config("q", m, k, 0, (world,), dist_name, "")
        t = capi.make_tiling(m, 1, k, world)
        symm = capi.symm_alloc(capi.symm_bytes_needed(t, True))
        nc, ns = world * m * k, world * m * (k // 32)
        ns_off = (nc + 1023) // 1024 * 1024
        out_symm = capi.symm_alloc(ns_off + ns)
        for rnd in range(3):
            symmetric = rnd % 2 == 1
            bits = [workloads.activation_bits(cfg, r, seed=rnd) for r in range(world)]
            if symmetric:
                oc = capi.symm_tensor(out_symm, nc).view(world * m, k)
                osc = capi.symm_tensor(out_symm, ns, ns_off).view(world * m, k // 32)
                oc.fill_(0xAA)
                osc.fill_(0xAA)
            else:
                oc = torch.full((world * m, k), 0xAA, dtype=torch.uint8, device="cuda")
                osc = torch.full((world * m, k // 32), 0xAA, dtype=torch.uint8, device="cuda")
            torch.cuda.synchronize()
            torch.distributed.barrier()  # nobody writes a peer's output before the peer has reset it
            capi.mx_quant_allgather(dev_bf16(bits[rank]), oc, osc, symm, world)
            status_ok(("quant_ag", m, k, rnd))
            rows = sample_rows(m, world, np.random.default_rng(rnd), per_rank=64) if m * k > (1 << 20) else np.arange(world * m)
            want_c, want_s = mx_oracle.quantize_rows(np.stack([bits[i // m][i % m] for i in rows]))
            rows_t = torch.from_numpy(rows).cuda()
            assert np.array_equal(oc[rows_t].cpu().numpy(), want_c), ("codes", m, k, rnd, rank)
            assert np.array_equal(osc[rows_t].cpu().numpy(), want_s), ("scales", m, k, rnd, rank)
            torch.distributed.barrier()
        capi.symm_free(out_symm)
        capi.symm_free(symm)

    # ---- fused allgather-matmul at the benchmark's per-rank sizes: C1, C3, C4, C5; every transfer mode ----
    shapes = [("c1", 256, 1024, 1024, "normal"), ("c3", 1024, 7168, 2304, "normal"),
              ("c4", 4096, 5120, 3456, "student_t3_outlier"), ("c5", 16, 7168, 4096, "normal")]
    for (name, m, k, n, dist_name) in shapes if "agmm" in only else []:
        cfg = workloads.Config(name, m, k, n, (world,), dist_name, "")
        t = capi.make_tiling(m, k, n, world)
        symm = capi.symm_alloc(capi.symm_bytes_needed(t, False))
        bc, bs = mx_oracle.quantize_weight(workloads.weight_bits(cfg, rank, seed=0))
        b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda()
        b_deq = mx_oracle.dequant_weight(bc, bs)
        for rnd, fuse_mode in enumerate((-1, 0, 5, 4, 6, 7)):  # the default, then every multi-rank variant by name
            capi.set_option("fuse_mode", fuse_mode)
            bits = [workloads.activation_bits(cfg, r, seed=rnd) for r in range(world)]
            c = torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda")
            torch.distributed.barrier()
            capi.mx_quant_allgather_matmul(dev_bf16(bits[rank]), b_d, bs_d, c, symm, world)
            status_ok((name, rnd))
            rows = sample_rows(m, world, np.random.default_rng(100 + rnd)) if m > 256 else np.arange(world * m)
            ac, asc = mx_oracle.quantize_rows(np.stack([bits[i // m][i % m] for i in rows]))
            gold = mx_oracle.gemm_f32(mx_oracle.dequant_rows(ac, asc), b_deq)
            bad, maxdiff = mx_oracle.check_close(c[torch.from_numpy(rows).cuda()].float().cpu().numpy(), gold, 1e-2, 1e-3)
            assert bad == 0, (name, rnd, fuse_mode, rank, bad, maxdiff)
            if rnd == 0 and name == "c1":
                # the reference operator's own signature: A arrives quantised
                aq = mx_oracle.quantize_rows(bits[rank])
                c2 = torch.zeros_like(c)
                torch.distributed.barrier()
                capi.fp8_mx_allgather_matmul(torch.from_numpy(aq[0]).cuda(), torch.from_numpy(aq[1]).cuda(),
                                             b_d, bs_d, c2, symm, world)
                status_ok((name, "prequant"))
                assert torch.equal(c2, c), "pre-quantised and fused paths must agree bit for bit"
        capi.set_option("fuse_mode", -1)
        capi.symm_free(symm)
    # ---- MXFP8 Matmul + ReduceScatter: rank r keeps row chunk r of the sum of all ranks' products.  Every rank
    # draws all ranks' operands from one seed, so each can compute the whole golden sum ----
    for (m, k, n) in [(256, 512, 512), (1024, 1024, 2304)] if "mmrs" in only else []:
        t = capi.make_tiling(m, k, n, world)
        symm = capi.symm_alloc(capi.symm_bytes_needed(t, 2))
        for rnd in range(3):  # both stages, and the first one again
            rng = np.random.default_rng(7000 + rnd)
            gold = np.zeros((m, n), np.float32)
            mine = None
            for r in range(world):
                aq = mx_oracle.quantize_rows(workloads.f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)))
                bq = mx_oracle.quantize_weight(workloads.f32_to_bf16_bits(rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05)))
                gold += mx_oracle.gemm_f32(mx_oracle.dequant_rows(*aq), mx_oracle.dequant_weight(*bq))
                if r == rank:
                    mine = [torch.from_numpy(x).cuda() for x in (aq[0], aq[1], bq[0], bq[1])]
            d = torch.zeros((m // world, n), dtype=torch.bfloat16, device="cuda")
            torch.distributed.barrier()
            capi.mxfp8_matmul_reduce_scatter(mine[0], mine[1], mine[2], mine[3], d, symm, world)
            status_ok(("mmrs", m, rnd))
            rows = m // world
            bad, maxdiff = mx_oracle.check_close(d.float().cpu().numpy(), gold[rank * rows:(rank + 1) * rows], 1e-2, 1e-3)
            assert bad == 0, ("mmrs", m, rnd, rank, bad, maxdiff)
        torch.distributed.barrier()
        capi.symm_free(symm)

    # ---- FP4 AllGather-Matmul: packed E2M1 operands, A gathered in packed form ----
    for (m, k, n) in [(256, 1024, 512)] if "fp4" in only else []:
        t = capi.make_tiling(m, k, n, world)
        symm = capi.symm_alloc(capi.symm_bytes_needed(t, False))
        for rnd in range(2):
            rng = np.random.default_rng(8000 + rnd)
            aq = [mx_oracle.quantize_rows_e2m1(workloads.f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)))
                  for _ in range(world)]
            a_deq = np.concatenate([mx_oracle.dequant_rows_e2m1(pk, sc) for pk, sc in aq])
            bw = None
            for r in range(world):
                b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05)
                if r != rank:
                    continue
                pt, st = mx_oracle.quantize_rows_e2m1(workloads.f32_to_bf16_bits(np.ascontiguousarray(b.T)))  # [N, K/2], [N, K/32]
                nib = np.empty((n, k), np.uint8)
                nib[:, 0::2] = pt & 0x0F
                nib[:, 1::2] = pt >> 4
                nib = np.ascontiguousarray(nib.T)  # [K, N] one code per byte, then packed along N
                bw = ((nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8),
                      np.ascontiguousarray(st.T.reshape(k // 64, 2, n).transpose(0, 2, 1)),
                      mx_oracle.dequant_rows_e2m1(pt, st).T.copy())
            a_p, a_s = torch.from_numpy(aq[rank][0]).cuda(), torch.from_numpy(aq[rank][1]).cuda()
            b_p, b_s = torch.from_numpy(bw[0]).cuda(), torch.from_numpy(bw[1]).cuda()
            c = torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda")
            torch.distributed.barrier()
            capi.fp4_mx_allgather_matmul(a_p, a_s, b_p, b_s, c, symm, world)
            status_ok(("fp4", m, rnd))
            bad, maxdiff = mx_oracle.check_close(c.float().cpu().numpy(), mx_oracle.gemm_f32(a_deq, bw[2]), 1e-2, 1e-3)
            assert bad == 0, ("fp4", m, rnd, rank, bad, maxdiff)
        torch.distributed.barrier()
        capi.symm_free(symm)
    capi.finalize()
    torch.distributed.destroy_process_group()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    main()
