"""CPU tests: the oracle against the reference-generated golden fixtures, and the three
restatements (C, numpy, torch port) against one another."""
import numpy as np
import pytest

from catccos_b200 import workloads


@pytest.mark.parametrize("name", ["quant_normal", "quant_outlier", "quant_edges"])
def test_quantise_matches_reference_golden(oracle, golden, name):
    d = golden(name)
    codes, scales = oracle.quantize_rows(d["x"])
    assert np.array_equal(codes, d["codes"])
    assert np.array_equal(scales, d["scales"])
    codes_np, scales_np = oracle.quantize_rows_np(d["x"])
    assert np.array_equal(codes_np, d["codes"])
    assert np.array_equal(scales_np, d["scales"])


def test_outlier_fixture_saturates(golden):
    d = golden("quant_outlier")
    assert ((d["codes"] & 0x7F) == 0x7E).sum() > 0
    assert d["scales"].max() - d["scales"].min() >= 5


def test_allgather_matmul_matches_reference_golden(oracle, golden):
    d = golden("agmm_small")
    for r in range(2):
        c, s = oracle.quantize_rows(d["a_bits"][r])
        assert np.array_equal(c, d["a_codes"][r]) and np.array_equal(s, d["a_scales"][r])
    bc, bs = oracle.quantize_weight(d["b_bits"])
    assert np.array_equal(bc, d["b_codes"]) and np.array_equal(bs, d["b_scales"])
    c = oracle.allgather_matmul(list(d["a_codes"]), list(d["a_scales"]), d["b_codes"], d["b_scales"])
    bad, _ = oracle.check_close(c, d["golden"], rtol=1e-5, atol=1e-6)
    assert bad == 0


def test_torch_port_matches_c_oracle(oracle):
    import torch

    cfg = workloads.CONFIGS["c4_outlier"]
    bits = workloads.activation_bits(cfg, rank=1, seed=3, rows=64)
    codes, scales = oracle.quantize_rows(bits)
    tc, ts, deq = oracle.golden_quantize_torch(torch.from_numpy(workloads.bf16_bits_to_f32(bits).copy()))
    assert np.array_equal(tc.numpy(), codes)
    assert np.array_equal(ts.numpy(), scales)
    assert np.array_equal(deq.numpy(), oracle.dequant_rows(codes, scales))
    assert ((codes & 0x7F) == 0x7E).any(), "the outlier workload must reach saturation"


def test_device_rule_differs_only_for_tiny_blocks(oracle, golden):
    d = golden("quant_edges")
    cg, sg = oracle.quantize_rows(d["x"], oracle.MODE_GOLDEN)
    cd, sd = oracle.quantize_rows(d["x"], oracle.MODE_DEVICE)
    amax = (d["x"].reshape(d["x"].shape[0], -1, 32) & 0x7FFF).max(-1)
    tiny = amax <= 0x2B8C
    assert np.array_equal(sg[~tiny], sd[~tiny])
    assert (sg[tiny] == 0x7F).all()
    same_codes = (cg == cd).reshape(cg.shape[0], -1, 32).all(-1)
    assert same_codes[~tiny].all()


def test_quantise_is_idempotent_on_dequantised_input(oracle):
    # the reference feeds its kernel the dequantised tensor (gen_mx_quant_allgather_data.py:529-534)
    cfg = workloads.CONFIGS["c1_golden"]
    bits = workloads.activation_bits(cfg, 0, seed=0, rows=32)
    c1, s1 = oracle.quantize_rows(bits)
    deq_bits = workloads.f32_to_bf16_bits(oracle.dequant_rows(c1, s1))
    c2, s2 = oracle.quantize_rows(deq_bits)
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2)


def test_e4m3_codec_round_trip(oracle):
    L = oracle.lib()
    for code in range(256):
        if code & 0x7F == 0x7F:
            continue
        v = L.mxo_e4m3_to_f32(code)
        assert L.mxo_e4m3_from_f32(v) == code
    # ties go to the even code: 1.0625 is halfway between 1.0 (0x38) and 1.125 (0x39)
    assert L.mxo_e4m3_from_f32(1.0625) == 0x38
    assert L.mxo_e4m3_from_f32(1.1875) == 0x3A
    assert L.mxo_e4m3_from_f32(-1e-9) == 0x80
    assert L.mxo_e4m3_from_f32(1000.0) == 0x7E


# ---- E5M2 output type (MX_QUANT_DTYPE = 1 in the reference: emax 15, max 57344) ----

@pytest.mark.parametrize("tag", ["normal", "outlier", "edges"])
def test_e5m2_quantise_matches_reference_golden(oracle, golden, tag):
    d = golden("quant_e5m2")
    codes, scales = oracle.quantize_rows(d["x_" + tag], fmt=oracle.FMT_E5M2)
    assert np.array_equal(scales, d["scales_" + tag])
    assert np.array_equal(codes, d["codes_" + tag])


def test_e5m2_allgather_matmul_matches_reference_golden(oracle, golden):
    d, g = golden("quant_e5m2"), golden("agmm_small")
    for r in range(2):  # the generator's own quantiser call (axis 1) agrees with the row quantiser
        c, s = oracle.quantize_rows(g["a_bits"][r], fmt=oracle.FMT_E5M2)
        assert np.array_equal(c, d["agmm_a_codes"][r]) and np.array_equal(s, d["agmm_a_scales"][r])
    out = oracle.allgather_matmul(list(d["agmm_a_codes"]), list(d["agmm_a_scales"]), g["b_codes"], g["b_scales"],
                                  a_fmt=oracle.FMT_E5M2)
    assert np.abs(out - d["agmm_golden"]).max() <= 1e-5 * np.abs(d["agmm_golden"]).max()


def test_e5m2_codec_round_trip(oracle):
    L = oracle.lib()
    for code in range(256):
        if code & 0x7F >= 0x7C:  # infinities and NaNs
            continue
        assert L.mxo_e5m2_from_f32(L.mxo_e5m2_to_f32(code)) == code
    assert L.mxo_e5m2_from_f32(1.125) == 0x3C   # halfway between 1.0 (0x3C) and 1.25 (0x3D): even code
    assert L.mxo_e5m2_from_f32(1.375) == 0x3E   # halfway between 1.25 (0x3D) and 1.5 (0x3E)
    assert L.mxo_e5m2_from_f32(1e9) == 0x7B     # saturates at 57344, never infinity
    assert L.mxo_e5m2_from_f32(-1e-9) == 0x80


# ---- FP4 E2M1 output type: oracle and fixtures only (no CUDA kernel reads them yet) ----

@pytest.mark.parametrize("tag", ["normal", "outlier", "edges"])
def test_e2m1_quantise_matches_reference_golden(oracle, golden, tag):
    d = golden("quant_e2m1")
    packed, scales = oracle.quantize_rows_e2m1(d["x_" + tag])
    assert np.array_equal(scales, d["scales_" + tag])
    assert np.array_equal(packed, d["packed_" + tag])
    deq = oracle.dequant_rows_e2m1(packed, scales)
    assert np.array_equal(deq, d["dequant_" + tag])


def test_e2m1_rounding_rules_agree_on_dequantised_input(oracle, golden):
    # the golden breaks ties toward zero, the device rounds to nearest even; the reference feeds its kernel the
    # dequantised tensor (gen_mx_quant_allgather_data.py:529-534), on which both rules give the same codes
    d = golden("quant_e2m1")
    deq_bits = workloads.f32_to_bf16_bits(d["dequant_normal"])
    g_c, g_s = oracle.quantize_rows_e2m1(deq_bits, oracle.MODE_GOLDEN)
    d_c, d_s = oracle.quantize_rows_e2m1(deq_bits, oracle.MODE_DEVICE)
    assert np.array_equal(g_s, d["scales_normal"]) and np.array_equal(d_s, g_s)
    # the golden writes +0 for every zero, the device keeps the sign: compare magnitudes
    assert np.array_equal(g_c & 0x77, d_c & 0x77)
    assert np.array_equal(g_c, d["packed_normal"])
    # on the raw input the two rules differ on ties only
    r_g, _ = oracle.quantize_rows_e2m1(d["x_normal"], oracle.MODE_GOLDEN)
    r_d, _ = oracle.quantize_rows_e2m1(d["x_normal"], oracle.MODE_DEVICE)
    assert 0 < np.count_nonzero((r_g & 0x77) != (r_d & 0x77)) < r_g.size // 4


def test_e2m1_codec(oracle):
    L = oracle.lib()
    values = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for code in range(16):
        v = L.mxo_e2m1_to_f32(code)
        assert abs(v) == values[code & 7] and (v <= 0 if code & 8 else v >= 0)
        if code != 8:  # -0 is never written by the golden
            assert L.mxo_e2m1_from_f32(v, 1) == code
        assert L.mxo_e2m1_from_f32(v, 0) == code
    # ties: golden toward zero, device to the even code
    for x, toward_zero, even in ((0.75, 1, 2), (1.75, 3, 4), (3.5, 5, 6), (0.25, 0, 0), (1.25, 2, 2), (2.5, 4, 4), (5.0, 6, 6)):
        assert L.mxo_e2m1_from_f32(x, 1) == toward_zero and L.mxo_e2m1_from_f32(x, 0) == even
        assert L.mxo_e2m1_from_f32(-x, 0) == even | 8
    assert L.mxo_e2m1_from_f32(100.0, 0) == 7 and L.mxo_e2m1_from_f32(-100.0, 1) == 15
    assert L.mxo_e2m1_from_f32(-0.1, 1) == 0 and L.mxo_e2m1_from_f32(-0.1, 0) == 8


@pytest.mark.parametrize("tag", ["normal", "edges"])
def test_e1m2_quantise_matches_reference_golden(oracle, golden, tag):
    # the other FP4 type of the reference generator (emax 0, max 1.75): oracle only.  The edge fixture holds a block
    # whose maximum has exponent 254, which this format divides by 2^127 (a subnormal multiplier)
    d = golden("quant_e1m2")
    packed, scales = oracle.quantize_rows_e1m2(d["x_" + tag])
    assert np.array_equal(scales, d["scales_" + tag])
    assert np.array_equal(packed, d["packed_" + tag])
    assert np.array_equal(oracle.dequant_rows_e1m2(packed, scales), d["dequant_" + tag])


def test_workload_shapes_and_determinism():
    cfg = workloads.CONFIGS["c4_outlier"]
    a = workloads.activation_bits(cfg, 2, seed=0, rows=8)
    b = workloads.activation_bits(cfg, 2, seed=0, rows=8)
    assert np.array_equal(a, b) and a.shape == (8, 5120)
    assert len(workloads.outlier_channels(cfg.k, 0)) == 6
    assert workloads.gemm_flops(workloads.CONFIGS["c3_prefill"], 8) == pytest.approx(270.6e9, rel=1e-3)
    assert workloads.quant_ag_ingress_bytes(workloads.CONFIGS["c2_quant_ag"], 8) == pytest.approx(211.94e6, rel=1e-3)


def test_reference_tolerance_rule(oracle):
    g = np.array([0.5, 2.0, -100.0], np.float32)
    assert oracle.check_reference_rule(g + np.array([0.01, 0.03, 1.5], np.float32), g, k=4096)[0] == 0
    assert oracle.check_reference_rule(g + np.array([0.02, 0.0, 0.0], np.float32), g, k=4096)[0] == 1
