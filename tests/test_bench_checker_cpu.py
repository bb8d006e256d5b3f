"""CPU tests of bench.py's parity checker (the block that makes a benchmark run fail when the CUDA path's output
differs from the oracle's): it accepts the oracle's own result, and it sees a single flipped code, a single
changed scale byte and a single output element outside the tolerance."""
import importlib.util
import os

import numpy as np

from catccos_b200 import workloads
from oracle import mx_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bench)

CFG = workloads.Config("checker", 160, 256, 64, (2,), "normal", "")


def test_sample_rows_cover_every_rank_and_the_edges():
    rows = bench.sample_rows(1024, 4, seed=3)
    assert len(rows) == 4 * bench.PARITY_ROWS_PER_RANK and len(set(rows.tolist())) == len(rows)
    for r in range(4):
        mine = rows[(rows >= r * 1024) & (rows < (r + 1) * 1024)] - r * 1024
        assert len(mine) == bench.PARITY_ROWS_PER_RANK
        assert {0, 127, 128, 512, 1023} <= set(mine.tolist())
    small = bench.sample_rows(16, 2, seed=0)  # a decode shard: every row
    assert sorted(small.tolist()) == list(range(32))


def test_quant_checker_sees_one_wrong_byte():
    world = 2
    rows = bench.sample_rows(CFG.m_local, world, seed=1)
    bits = [workloads.activation_bits(CFG, r, seed=0) for r in range(world)]
    a = np.stack([bits[i // CFG.m_local][i % CFG.m_local] for i in rows])
    codes, scales = mx_oracle.quantize_rows(a)
    ok = bench.check_quant_parity(CFG, world, rows, codes, scales)
    assert ok["codes_bad"] == 0 and ok["scales_bad"] == 0 and ok["quant_rows_checked"] == len(rows)
    c2 = codes.copy()
    c2[5, 17] ^= 1
    assert bench.check_quant_parity(CFG, world, rows, c2, scales)["codes_bad"] == 1
    s2 = scales.copy()
    s2[7, 3] += 1
    assert bench.check_quant_parity(CFG, world, rows, codes, s2)["scales_bad"] == 1


def test_output_checker_sees_one_element_out_of_tolerance():
    world = 2
    rows = bench.sample_rows(CFG.m_local, world, seed=2)
    bits = [workloads.activation_bits(CFG, r, seed=0) for r in range(world)]
    a = np.stack([bits[i // CFG.m_local][i % CFG.m_local] for i in rows])
    bc, bs = mx_oracle.quantize_weight(workloads.weight_bits(CFG, 0, seed=0))
    gold = mx_oracle.gemm_f32(mx_oracle.dequant_rows(*mx_oracle.quantize_rows(a)), mx_oracle.dequant_weight(bc, bs))
    ok = bench.check_c_parity(CFG, world, rows, gold.copy(), bc, bs)
    assert ok["c_bad"] == 0 and ok["rows_checked"] == len(rows)
    off = gold.copy()
    off[3, 9] += 2e-3 + 2e-2 * abs(off[3, 9])  # just outside |d| <= 1e-3 + 1e-2 |gold|
    assert bench.check_c_parity(CFG, world, rows, off, bc, bs)["c_bad"] == 1
    near = gold.copy()
    near[3, 9] += 0.5e-3  # inside
    assert bench.check_c_parity(CFG, world, rows, near, bc, bs)["c_bad"] == 0


def test_stats():
    s = bench.stats(np.array([3.0, 1.0, 2.0, 10.0]))
    assert s["min"] == 1.0 and s["max"] == 10.0 and s["p50"] == 3.0 and s["samples"] == 4 and s["mean"] == 4.0
