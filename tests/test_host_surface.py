"""The C++ operator surface (catccos_b200/host): host-only self test on CPU, and on a GPU the two
drivers run with the reference's command lines and file names, checked against the oracle."""
import os
import subprocess

import numpy as np
import pytest

from catccos_b200 import workloads
from conftest import ROOT

HOST = os.path.join(ROOT, "catccos_b200", "host")


@pytest.fixture(scope="module")
def host_bins(capi):
    subprocess.check_call(["make", "-C", HOST], stdout=subprocess.DEVNULL)
    return os.path.join(HOST, "bin")


def test_host_selftest(host_bins):
    r = subprocess.run([os.path.join(host_bins, "host_selftest")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr


def test_drivers_reject_bad_arguments(host_bins):
    r = subprocess.run([os.path.join(host_bins, "mx_quant_allgather"), "1", "0", "tcp://127.0.0.1:8789", "64", "100", "1"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 1 and "divisible by 32" in r.stderr
    r = subprocess.run([os.path.join(host_bins, "fp8_mx_allgather_matmul"), "1", "0"], capture_output=True, text=True,
                       timeout=60)
    assert r.returncode == 1 and "Invalid arguments" in r.stderr


def test_batch_driver_rejects_bad_arguments(host_bins, tmp_path):
    exe = os.path.join(host_bins, "dynamic_tiling")
    r = subprocess.run([exe, "a5fp8mxagmm", "1", "1", "0"], capture_output=True, text=True, timeout=60)
    assert r.returncode != 0 and "Invalid command line options" in r.stderr
    csv = tmp_path / "shapes.csv"
    csv.write_text("M,K,N,Transpose A,Transpose B\n256,1024,1024,0,0\n")
    r = subprocess.run([exe, "no_such_kernel", "1", "1", "0", "tcp://127.0.0.1:8791", "0", "0", "0", "0", "1", str(tmp_path),
                        str(csv), "1", "1"], capture_output=True, text=True, timeout=60)
    assert r.returncode != 0 and "not part of this library" in r.stderr


@pytest.mark.gpu
def test_batch_driver_single_rank(host_bins, oracle, cuda, tmp_path):
    # the reference's batch driver command line (tests/dynamic_tiling): a CSV of shapes, warm-up and timed launches
    # through KernelDispatcher, one line per shape in output/tiling/tilingData_<time>.csv
    exe = os.path.join(host_bins, "dynamic_tiling")
    m, k, n = 256, 1024, 1024
    cfg = workloads.Config("t", m, k, n, (1,), "normal", "")
    ac, asc = oracle.quantize_rows(workloads.activation_bits(cfg, 0, seed=4))
    bc, bsc = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=4))
    data = tmp_path / "data"
    data.mkdir()
    ac.tofile(data / "input_a_0.bin")
    asc.tofile(data / "input_a_scale_0.bin")
    bc.tofile(data / "input_b_0.bin")
    bsc.tofile(data / "input_b_scale_0.bin")
    csv = tmp_path / "shapes.csv"
    csv.write_text("M,K,N,Transpose A,Transpose B\n8,8,8,0,0\n%d,%d,%d,0,0\n" % (m, k, n))
    r = subprocess.run([exe, "a5fp8mxagmm", "1", "1", "0", "tcp://127.0.0.1:8792", "0", "0", "0", "1", "1", str(tmp_path),
                        str(csv), "2", "5", "0", str(data)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "[ERROR]" not in r.stdout and "cudaError:" not in r.stderr, r.stdout + r.stderr
    out = workloads.bf16_bits_to_f32(np.fromfile(data / "output_0.bin", dtype=np.uint16).reshape(m, n))
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    bad, maxdiff = oracle.check_close(out, gold, 1e-2, 1e-3)
    assert bad == 0, (bad, maxdiff)
    files = os.listdir(tmp_path / "output" / "tiling")
    assert len(files) == 1
    rows = (tmp_path / "output" / "tiling" / files[0]).read_text().strip().splitlines()
    assert len(rows) == 2 and rows[1].startswith("Ascend950Fp8MxAllGatherMatmul,%d,%d,%d,0,0," % (m, k, n))
    assert float(rows[1].split(",")[-1]) > 0.0
    # the quantiser over several shapes, timing only (no data directory: the operator fills its input itself)
    csv.write_text("M,K,N,Transpose A,Transpose B\n190,1,1024,0,0\n1024,1,7168,0,0\n")
    r = subprocess.run([exe, "mxqtag", "36", "1", "0", "tcp://127.0.0.1:8793", "0", "0", "0", "0", "2", str(tmp_path),
                        str(csv), "2", "5"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.count("cudaStreamSynchronize success") == 2, r.stdout + r.stderr


@pytest.mark.gpu
def test_quant_driver_files_single_rank(host_bins, oracle, cuda, tmp_path):
    m, n = 190, 1024  # ragged M, as in the reference's test_shapes.csv (8190 = 63 * 128 + 126)
    bits = workloads.f32_to_bf16_bits(np.random.default_rng(11).standard_normal((m, n), dtype=np.float32))
    bits.tofile(tmp_path / "rank_0_input.bin")
    r = subprocess.run([os.path.join(host_bins, "mx_quant_allgather"), "1", "0", "tcp://127.0.0.1:8789", str(m), str(n),
                        "1", str(tmp_path), "0"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "[ERROR]" not in r.stdout and "cudaError:" not in r.stderr, r.stdout + r.stderr
    want_c, want_s = oracle.quantize_rows(bits)
    got_c = np.fromfile(tmp_path / "rank_0_output.bin", dtype=np.uint8).reshape(m, n)
    got_s = np.fromfile(tmp_path / "rank_0_mxscale.bin", dtype=np.uint8).reshape(m, n // 32)
    assert np.array_equal(got_c, want_c) and np.array_equal(got_s, want_s)


@pytest.mark.gpu
def test_matmul_driver_files_single_rank(host_bins, oracle, cuda, tmp_path):
    m, n, k = 256, 1024, 512  # a shape of the reference's test_shapes.csv
    cfg = workloads.Config("t", m, k, n, (1,), "normal", "")
    ac, asc = oracle.quantize_rows(workloads.activation_bits(cfg, 0, seed=2))
    bc, bsc = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=2))
    ac.tofile(tmp_path / "input_a_0.bin")
    asc.tofile(tmp_path / "input_a_scale_0.bin")
    bc.tofile(tmp_path / "input_b_0.bin")
    bsc.tofile(tmp_path / "input_b_scale_0.bin")
    r = subprocess.run([os.path.join(host_bins, "fp8_mx_allgather_matmul"), "1", "0", "tcp://127.0.0.1:8789", str(m),
                        str(n), str(k), str(tmp_path), "0"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "[ERROR]" not in r.stdout and "cudaError:" not in r.stderr, r.stdout + r.stderr
    out_bits = np.fromfile(tmp_path / "output_0.bin", dtype=np.uint16).reshape(m, n)
    out = workloads.bf16_bits_to_f32(out_bits)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    bad, maxdiff = oracle.check_close(out, gold, 1e-2, 1e-3)
    assert bad == 0, (bad, maxdiff)
