"""CPU tests of the multi-rank host logic: the rendezvous layer (TCP star + descriptor passing) as
forked processes, and the rank-order gather semantics with two gloo ranks."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def selftest_bin(tmp_path_factory):
    out = tmp_path_factory.mktemp("host") / "bootstrap_selftest"
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-o", str(out),
                           os.path.join(ROOT, "tests", "host", "bootstrap_selftest.cpp")])
    return str(out)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_bootstrap_rendezvous_and_fd_exchange(selftest_bin, world):
    port = 30000 + (os.getpid() % 2000) + world
    r = subprocess.run([selftest_bin, str(world), str(port)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


_GLOO_WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from catccos_b200 import workloads
from oracle import mx_oracle

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
cfg = workloads.Config("t", 24, 256, 64, (world,), "normal", "")
bits = workloads.activation_bits(cfg, rank, seed=3)
codes, scales = mx_oracle.quantize_rows(bits)
g_codes = [torch.empty(codes.shape, dtype=torch.uint8) for _ in range(world)]
g_scales = [torch.empty(scales.shape, dtype=torch.uint8) for _ in range(world)]
dist.all_gather(g_codes, torch.from_numpy(codes))
dist.all_gather(g_scales, torch.from_numpy(scales))
# what every rank must end with: the rank-order concatenation (mx_quant_allgather.hpp:46-48)
want = [mx_oracle.quantize_rows(workloads.activation_bits(cfg, r, seed=3)) for r in range(world)]
assert np.array_equal(torch.cat(g_codes).numpy(), np.concatenate([w[0] for w in want]))
assert np.array_equal(torch.cat(g_scales).numpy(), np.concatenate([w[1] for w in want]))
# the benchmark's timing rule: per step the slowest rank counts
ms = torch.tensor([1.0 + rank, 5.0 - rank], dtype=torch.float64)
dist.all_reduce(ms, op=dist.ReduceOp.MAX)
assert ms.tolist() == [float(world), 5.0]
dist.destroy_process_group()
print("ok", rank)
"""


def test_rank_order_gather_two_gloo_ranks(tmp_path, oracle):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    port = 31000 + (os.getpid() % 2000)
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", str(port), str(script), ROOT],
        capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("ok") == 2


def test_reference_arm_other_ranks_do_no_work():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_tile_and_item_visiting_order(tmp_path):
    """The order in which CTAs visit output tiles (own shard, then the peers in ring order, slice by slice) and
    in which quantise / pusher workers visit (chunk, K segment) items, checked on the host against its contract
    (tests/host/schedule_selftest.cu; compiled with nvcc, runs without a GPU)."""
    out = tmp_path / "schedule_selftest"
    subprocess.check_call(["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(out),
                           os.path.join(ROOT, "tests", "host", "schedule_selftest.cu")])
    r = subprocess.run([str(out)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
