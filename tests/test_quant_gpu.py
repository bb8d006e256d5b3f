"""GPU parity of the MX quantise kernel against the oracle and the reference-generated fixtures.
Codes and scales are compared bit for bit.  All calls go through the C ABI."""
import numpy as np
import pytest

from catccos_b200 import workloads
from conftest import to_dev_bf16

pytestmark = pytest.mark.gpu


def _quant_gpu(capi, torch, bits):
    codes, scales = capi.mx_quant(to_dev_bf16(torch, np.ascontiguousarray(bits)))
    torch.cuda.synchronize()
    return codes.cpu().numpy(), scales.cpu().numpy()


def _assert_bit_exact(got, want, what):
    if not np.array_equal(got, want):
        idx = np.argwhere(got != want)
        lines = [f"{tuple(i)}: got {got[tuple(i)]:#04x} want {want[tuple(i)]:#04x}" for i in idx[:20]]
        raise AssertionError(f"{what}: {len(idx)} mismatches, first 20:\n" + "\n".join(lines))


@pytest.mark.parametrize("name", ["quant_normal", "quant_outlier", "quant_edges"])
def test_fixture_parity(capi, cuda, golden, name):
    d = golden(name)
    codes, scales = _quant_gpu(capi, cuda, d["x"])
    _assert_bit_exact(codes, d["codes"], "codes")
    _assert_bit_exact(scales, d["scales"], "scales")


def test_all_bf16_values_under_every_scale_position(capi, cuda, oracle):
    # every finite bf16 bit pattern, each in a block whose maximum sits 0..12 binades above it
    vals = np.arange(0x10000, dtype=np.uint32)
    finite = vals[((vals >> 7) & 0xFF) != 0xFF].astype(np.uint16)
    rows = []
    for shift in (0, 1, 2, 5, 9, 12):
        blk = np.zeros((finite.size, 32), np.uint16)
        blk[:, 0] = finite
        e = (finite >> 7) & 0xFF
        top = np.minimum(e.astype(np.int32) + shift, 254).astype(np.uint16) << 7
        blk[:, 1] = top
        rows.append(blk)
    x = np.concatenate(rows).reshape(-1, 32 * 8)
    want_c, want_s = oracle.quantize_rows(x)
    got_c, got_s = _quant_gpu(capi, cuda, x)
    _assert_bit_exact(got_s, want_s, "scales")
    _assert_bit_exact(got_c, want_c, "codes")


@pytest.mark.parametrize("rows,k", [(1, 32), (16, 96), (17, 160), (127, 512), (129, 1056), (5, 7168), (130, 5120)])
def test_ragged_shapes(capi, cuda, oracle, rows, k):
    rng = np.random.default_rng(rows * 100003 + k)
    x = workloads.f32_to_bf16_bits(rng.standard_normal((rows, k), dtype=np.float32) * np.float32(3.0))
    want_c, want_s = oracle.quantize_rows(x)
    got_c, got_s = _quant_gpu(capi, cuda, x)
    _assert_bit_exact(got_s, want_s, "scales")
    _assert_bit_exact(got_c, want_c, "codes")


@pytest.mark.parametrize("cfg_name", ["c1_golden", "c2_quant_ag", "c3_prefill", "c4_outlier", "c5_decode"])
def test_config_inputs(capi, cuda, oracle, cfg_name):
    cfg = workloads.CONFIGS[cfg_name]
    x = workloads.activation_bits(cfg, rank=1, seed=0, rows=min(cfg.m_local, 512))
    want_c, want_s = oracle.quantize_rows(x)
    got_c, got_s = _quant_gpu(capi, cuda, x)
    _assert_bit_exact(got_s, want_s, "scales")
    _assert_bit_exact(got_c, want_c, "codes")
    if cfg.dist == "student_t3_outlier":
        assert ((want_c & 0x7F) == 0x7E).any()


def test_device_tiny_block_rule(capi, cuda, oracle, golden):
    d = golden("quant_edges")
    capi.set_option("tiny_block_rule", 1)
    try:
        got_c, got_s = _quant_gpu(capi, cuda, d["x"])
    finally:
        capi.set_option("tiny_block_rule", 0)
    want_c, want_s = oracle.quantize_rows(d["x"], oracle.MODE_DEVICE)
    _assert_bit_exact(got_s, want_s, "scales")
    _assert_bit_exact(got_c, want_c, "codes")


def test_nonfinite_blocks(capi, cuda, oracle):
    x = workloads.f32_to_bf16_bits(np.random.default_rng(5).standard_normal((4, 128), dtype=np.float32))
    x[0, 3] = 0x7F80   # +inf
    x[1, 40] = 0xFF80  # -inf
    x[2, 100] = 0x7FC0  # nan
    want_c, want_s = oracle.quantize_rows(x)
    got_c, got_s = _quant_gpu(capi, cuda, x)
    _assert_bit_exact(got_s, want_s, "scales")
    _assert_bit_exact(got_c, want_c, "codes")
    assert got_s[0, 0] == 0xFF and (got_c[0, :32] == 0x7F).all()


def test_idempotent_on_dequantised_input(capi, cuda, oracle):
    cfg = workloads.CONFIGS["c3_prefill"]
    x = workloads.activation_bits(cfg, 0, seed=1, rows=64)
    c1, s1 = _quant_gpu(capi, cuda, x)
    deq = workloads.f32_to_bf16_bits(oracle.dequant_rows(c1, s1))
    c2, s2 = _quant_gpu(capi, cuda, deq)
    _assert_bit_exact(c2, c1, "codes")
    _assert_bit_exact(s2, s1, "scales")


def test_full_size_checksum_properties(capi, cuda, oracle):
    # full benchmark shape (4096 x 7168): scales equal the per-block exponent rule computed with torch
    # integer ops on the device, and a sampled slab equals the oracle
    torch = cuda
    cfg = workloads.CONFIGS["c2_quant_ag"]
    x = workloads.activation_bits(cfg, 0, seed=0)
    xd = to_dev_bf16(torch, x)
    codes, scales = capi.mx_quant(xd)
    bits = xd.view(torch.int16).to(torch.int32) & 0x7FFF
    amax = bits.view(cfg.m_local, cfg.k // 32, 32).amax(-1)
    assert torch.equal(scales.to(torch.int32), (amax >> 7) - 8)
    rows = np.r_[0:64, 2000:2064, 4032:4096]
    want_c, want_s = oracle.quantize_rows(x[rows])
    _assert_bit_exact(codes.cpu().numpy()[rows], want_c, "codes")
    _assert_bit_exact(scales.cpu().numpy()[rows], want_s, "scales")


# ---- E5M2 output type (option "a_dtype" = 1) ----

@pytest.mark.parametrize("tag", ["normal", "outlier", "edges"])
def test_e5m2_fixture_parity(capi, cuda, golden, tag):
    d = golden("quant_e5m2")
    capi.set_option("a_dtype", 1)
    try:
        codes, scales = _quant_gpu(capi, cuda, d["x_" + tag])
    finally:
        capi.set_option("a_dtype", 0)
    _assert_bit_exact(scales, d["scales_" + tag], "scales")
    _assert_bit_exact(codes, d["codes_" + tag], "codes")


def test_e5m2_all_bf16_values(capi, cuda, oracle):
    # every finite bf16 bit pattern alone in its block, and three binades below the block maximum
    vals = np.arange(0x10000, dtype=np.uint32)
    finite = vals[((vals >> 7) & 0xFF) != 0xFF].astype(np.uint16)
    rows = []
    for shift in (0, 3):
        blk = np.zeros((finite.size, 32), np.uint16)
        blk[:, 0] = finite
        e = (finite >> 7) & 0xFF
        blk[:, 1] = np.minimum(e.astype(np.int32) + shift, 254).astype(np.uint16) << 7
        rows.append(blk)
    x = np.concatenate(rows).reshape(-1, 32 * 8)
    want_c, want_s = oracle.quantize_rows(x, fmt=oracle.FMT_E5M2)
    capi.set_option("a_dtype", 1)
    try:
        got_c, got_s = _quant_gpu(capi, cuda, x)
    finally:
        capi.set_option("a_dtype", 0)
    _assert_bit_exact(got_s, want_s, "scales")
    _assert_bit_exact(got_c, want_c, "codes")


# ---- FP4 E2M1 output type (catccos_b200_mx_quant_fp4): round to nearest even, as the reference's device cast ----

def _quant_fp4_gpu(capi, torch, bits):
    packed, scales = capi.mx_quant_fp4(to_dev_bf16(torch, np.ascontiguousarray(bits)))
    torch.cuda.synchronize()
    return packed.cpu().numpy(), scales.cpu().numpy()


def test_fp4_matches_reference_golden_on_dequantised_input(capi, cuda, golden):
    # the reference feeds its kernel the dequantised tensor (gen_mx_quant_allgather_data.py:529-534): there the
    # device's rounding and the golden's table rounding agree, and the golden fixture is the expected output
    d = golden("quant_e2m1")
    for tag in ("normal", "outlier"):
        bits = workloads.f32_to_bf16_bits(d["dequant_" + tag])
        packed, scales = _quant_fp4_gpu(capi, cuda, bits)
        _assert_bit_exact(scales, d["scales_" + tag], "scales " + tag)
        _assert_bit_exact(packed, d["packed_" + tag], "codes " + tag)


@pytest.mark.parametrize("rows,k", [(1, 32), (17, 160), (130, 1056), (5, 7168)])
def test_fp4_matches_oracle_device_rule(capi, cuda, oracle, golden, rows, k):
    rng = np.random.default_rng(rows * 7919 + k)
    x = workloads.f32_to_bf16_bits(rng.standard_normal((rows, k), dtype=np.float32) * np.float32(2.0))
    capi.set_option("tiny_block_rule", 1)
    try:
        want_c, want_s = oracle.quantize_rows_e2m1(x, oracle.MODE_DEVICE)
        got_c, got_s = _quant_fp4_gpu(capi, cuda, x)
        _assert_bit_exact(got_s, want_s, "scales")
        _assert_bit_exact(got_c, want_c, "codes")
        e = golden("quant_e2m1")["x_edges"]  # zeros, subnormals, tiny blocks, ties, Inf/NaN blocks
        want_c, want_s = oracle.quantize_rows_e2m1(e, oracle.MODE_DEVICE)
        got_c, got_s = _quant_fp4_gpu(capi, cuda, e)
        _assert_bit_exact(got_s, want_s, "edge scales")
        _assert_bit_exact(got_c, want_c, "edge codes")
    finally:
        capi.set_option("tiny_block_rule", 0)
