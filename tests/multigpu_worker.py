"""Worker of tests/test_multigpu.py: one process per GPU (launched by torch.distributed.run).  Each rank
drives the C ABI in its real multi-process mode (cuMem/VMM peer-mapped symmetric buffers, flags over
NVLink) and checks its results against the oracle: gathered codes and scales bit for bit, GEMM output
within rtol 1e-2 / atol 1e-3."""
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


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    port = int(os.environ.get("MASTER_PORT", "29500")) + 97
    capi.init(rank, world, local, f"tcp://127.0.0.1:{port}")

    def status_ok(tag):
        code, st = capi.last_status()
        assert code == 0, (tag, rank, st)

    # ---- quantise + allgather: gathered outputs identical on every rank, bit-exact ----
    for (m, k, dist) in [(256, 1024, "normal"), (190, 512, "normal"), (512, 7168, "normal"), (128, 5120, "student_t3_outlier")]:
        cfg = workloads.Config("q", m, k, 0, (world,), dist, "")
        t = capi.make_tiling(m, 1, k, world)
        symm = capi.symm_alloc(capi.symm_bytes_needed(t, True))
        for rnd in range(3):
            bits = [workloads.activation_bits(cfg, r, seed=rnd) for r in range(world)]
            oc = torch.full((world * m, k), 0xAA, dtype=torch.uint8, device="cuda")
            osc = torch.full((world * m, k // 32), 0xAA, dtype=torch.uint8, device="cuda")
            capi.mx_quant_allgather(dev_bf16(bits[rank]), oc, osc, symm, world)
            status_ok(("quant_ag", m, k, rnd))
            want = [mx_oracle.quantize_rows(b) for b in bits]
            assert np.array_equal(oc.cpu().numpy(), np.concatenate([w[0] for w in want])), ("codes", m, k, rnd, rank)
            assert np.array_equal(osc.cpu().numpy(), np.concatenate([w[1] for w in want])), ("scales", m, k, rnd, rank)
        capi.symm_free(symm)

    # ---- fused allgather-matmul: C1 in full, C3/C4 with fewer rows per rank, C5 in full ----
    rows = 256 if world <= 2 else 128  # the CPU oracle's GEMM is the slow part: fewer rows per rank at larger worlds
    shapes = [("c1", 256, 1024, 1024, "normal"), ("c3", rows, 7168, 2304, "normal"),
              ("c4", rows, 5120, 3456, "student_t3_outlier"), ("c5", 16, 7168, 4096, "normal")]
    for (name, m, k, n, dist) in shapes:
        cfg = workloads.Config(name, m, k, n, (world,), dist, "")
        t = capi.make_tiling(m, k, n, world)
        symm = capi.symm_alloc(capi.symm_bytes_needed(t, False))
        bc, bs = mx_oracle.quantize_weight(workloads.weight_bits(cfg, rank, seed=0))
        b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda()
        b_deq = mx_oracle.dequant_weight(bc, bs)
        for rnd, fuse_mode in enumerate((-1, 0, 4)):  # the default, then every multi-rank variant by name
            capi.set_option("fuse_mode", fuse_mode)
            bits = [workloads.activation_bits(cfg, r, seed=rnd) for r in range(world)]
            c = torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda")
            capi.mx_quant_allgather_matmul(dev_bf16(bits[rank]), b_d, bs_d, c, symm, world)
            status_ok((name, rnd))
            aq = [mx_oracle.quantize_rows(b) for b in bits]
            a_deq = mx_oracle.dequant_rows(np.concatenate([q[0] for q in aq]), np.concatenate([q[1] for q in aq]))
            gold = mx_oracle.gemm_f32(a_deq, b_deq)
            bad, maxdiff = mx_oracle.check_close(c.float().cpu().numpy(), gold, 1e-2, 1e-3)
            assert bad == 0, (name, rnd, rank, bad, maxdiff)
            if rnd == 0 and name == "c1":
                # the reference operator's own signature: A arrives quantised
                c2 = torch.zeros_like(c)
                capi.fp8_mx_allgather_matmul(torch.from_numpy(aq[rank][0]).cuda(), torch.from_numpy(aq[rank][1]).cuda(),
                                             b_d, bs_d, c2, symm, world)
                status_ok((name, "prequant"))
                assert torch.equal(c2, c), "pre-quantised and fused paths must agree bit for bit"
        capi.set_option("fuse_mode", -1)
        capi.symm_free(symm)
    capi.finalize()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    main()
