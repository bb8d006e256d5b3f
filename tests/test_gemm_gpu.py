"""GPU parity of the tcgen05 MXFP8 block-scaled GEMM against the oracle's fp32 golden.
Tolerance (stated by the benchmark definition): |out - gold| <= 1e-3 + 1e-2 * |gold| for bf16 output;
the reference's own rule (rtol 2^-6 of max(1, |gold|) for K >= 2048) is checked beside it."""
import numpy as np
import pytest

from catccos_b200 import workloads

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-2, 1e-3


def _rand_problem(oracle, m, n, k, seed, a_scale=1.0, dist="normal"):
    rng = np.random.default_rng(seed)
    if dist == "normal":
        a = rng.standard_normal((m, k), dtype=np.float32) * np.float32(a_scale)
    else:
        a = rng.standard_t(3.0, size=(m, k)).astype(np.float32)
        a[:, rng.choice(k, max(1, k // 1000), replace=False)] *= np.float32(100.0)
    b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)
    ac, asc = oracle.quantize_rows(workloads.f32_to_bf16_bits(a))
    bc, bsc = oracle.quantize_weight(workloads.f32_to_bf16_bits(b))
    return ac, asc, bc, bsc


def _run(capi, torch, ac, asc, bc, bsc, block_n=0, f16=False, cta_pair=2):
    capi.set_option("cta_pair", cta_pair)
    capi.set_option("block_n", block_n)
    capi.set_option("c_dtype", 1 if f16 else 0)
    try:
        a_d, as_d = torch.from_numpy(ac).cuda(), torch.from_numpy(asc).cuda()
        b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bsc).cuda()
        out = capi.mx_gemm(a_d, as_d, b_d, bs_d, out_dtype=torch.float16 if f16 else torch.bfloat16)
        code, st = capi.last_status()
        assert code == 0, st
        return out.float().cpu().numpy()
    finally:
        capi.set_option("cta_pair", 0)
        capi.set_option("block_n", 0)
        capi.set_option("c_dtype", 0)


def _check(oracle, out, gold, k):
    bad, maxdiff = oracle.check_close(out, gold, RTOL, ATOL)
    assert bad == 0, f"{bad} of {gold.size} elements outside rtol {RTOL} / atol {ATOL}; max |diff| {maxdiff}"
    bad_ref, eb = oracle.check_reference_rule(out, gold, k, bf16=True)
    assert bad_ref == 0 and eb < 2.0 ** -7


@pytest.mark.parametrize("block_n", [128, 256])
def test_single_tile_unit_scales(capi, cuda, oracle, block_n):
    # one output tile, one K tile, all scales 1.0: isolates the operand descriptors from the scale path
    rng = np.random.default_rng(1)
    m, n, k = 128, 256, 128
    ac = rng.integers(0x30, 0x48, (m, k)).astype(np.uint8) | (rng.integers(0, 2, (m, k)).astype(np.uint8) << 7)
    bc = rng.integers(0x30, 0x48, (k, n)).astype(np.uint8) | (rng.integers(0, 2, (k, n)).astype(np.uint8) << 7)
    asc = np.full((m, k // 32), 0x7F, np.uint8)
    bsc = np.full((k // 64, n, 2), 0x7F, np.uint8)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc, block_n)
    _check(oracle, out, gold, k)


@pytest.mark.parametrize("block_n", [128, 256])
def test_scale_factor_routing(capi, cuda, oracle, block_n):
    # every (row, k-block) and (column, k-block) gets its own power of two: a wrong scale-factor
    # layout shows up as errors of a factor of two or more
    rng = np.random.default_rng(2)
    m, n, k = 256, 512, 512
    ac = rng.integers(0x30, 0x48, (m, k)).astype(np.uint8)
    bc = rng.integers(0x30, 0x48, (k, n)).astype(np.uint8)
    asc = (120 + (np.arange(m)[:, None] * 7 + np.arange(k // 32)[None, :] * 3) % 13).astype(np.uint8)
    bs_kn = (118 + (np.arange(k // 32)[:, None] * 5 + np.arange(n)[None, :]) % 11).astype(np.uint8)
    bsc = np.ascontiguousarray(bs_kn.reshape(k // 64, 2, n).transpose(0, 2, 1))
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc, block_n)
    _check(oracle, out, gold, k)


def test_reference_golden_fixture(capi, cuda, oracle, golden):
    d = golden("agmm_small")
    ac = np.concatenate(list(d["a_codes"]))
    asc = np.concatenate(list(d["a_scales"]))
    # K = 256, N = 64: a partial tile in both N and M
    out = _run(capi, cuda, ac, asc, d["b_codes"], d["b_scales"])
    _check(oracle, out, d["golden"], 256)


@pytest.mark.parametrize(
    "m,n,k",
    [(512, 1024, 1024), (100, 272, 384), (1, 16, 128), (385, 2304, 7168), (200, 3456, 5120), (128, 4096, 7168)],
)
def test_shapes(capi, cuda, oracle, m, n, k):
    ac, asc, bc, bsc = _rand_problem(oracle, m, n, k, seed=m + n + k)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc)
    _check(oracle, out, gold, k)


def test_many_tiles_per_cta_and_fp16_output(capi, cuda, oracle):
    # more tiles than SMs: exercises the accumulator double buffering and stage ring wrap-around
    m, n, k = 3072, 2048, 256
    ac, asc, bc, bsc = _rand_problem(oracle, m, n, k, seed=9)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    for block_n in (128, 256):
        out = _run(capi, cuda, ac, asc, bc, bsc, block_n=block_n)
        _check(oracle, out, gold, k)
    out16 = _run(capi, cuda, ac, asc, bc, bsc, f16=True)
    bad, _ = oracle.check_reference_rule(out16, gold, k, bf16=False)
    assert bad == 0


def test_outlier_inputs(capi, cuda, oracle):
    m, n, k = 256, 512, 5120
    ac, asc, bc, bsc = _rand_problem(oracle, m, n, k, seed=4, dist="student")
    assert ((ac & 0x7F) == 0x7E).any()
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc)
    _check(oracle, out, gold, k)


def test_linearity_in_scales_at_full_size(capi, cuda, oracle):
    # size-independent property at the benchmark shape: adding 1 to every A scale byte doubles C exactly
    torch = cuda
    cfg = workloads.CONFIGS["c3_prefill"]
    m, n, k = cfg.m_local, cfg.n_local, cfg.k
    ac, asc = oracle.quantize_rows(workloads.activation_bits(cfg, 0, seed=0))
    bc, bsc = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=0))
    a_d, b_d, bs_d = torch.from_numpy(ac).cuda(), torch.from_numpy(bc).cuda(), torch.from_numpy(bsc).cuda()
    c1 = capi.mx_gemm(a_d, torch.from_numpy(asc).cuda(), b_d, bs_d)
    c2 = capi.mx_gemm(a_d, torch.from_numpy(asc + 1).cuda(), b_d, bs_d)
    assert torch.equal(c2.float(), c1.float() * 2)
    rows = np.r_[0:32, 500:532, 992:1024]
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc, rows=rows)
    _check(oracle, c1.float().cpu().numpy()[rows], gold, k)


# ---- split K (few output tiles: each (tile, K part) on its own SM, partial tiles added in part order) ----

@pytest.mark.parametrize("split_k", [1, 2, 4, 8])
@pytest.mark.parametrize("block_n", [0, 128])
def test_split_k_parts(capi, cuda, oracle, split_k, block_n):
    m, n, k = 200, 528, 4096  # 2 x 3 tiles of 256 columns (one partial in M and in N), 32 K tiles
    ac, asc, bc, bsc = _rand_problem(oracle, m, n, k, seed=77)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    capi.set_option("split_k", split_k)
    try:
        for _ in range(2):  # the second call meets the first call's partial tiles and flags
            out = _run(capi, cuda, ac, asc, bc, bsc, block_n=block_n)
            _check(oracle, out, gold, k)
        out16 = _run(capi, cuda, ac, asc, bc, bsc, block_n=block_n, f16=True)
        assert oracle.check_reference_rule(out16, gold, k, bf16=False)[0] == 0
    finally:
        capi.set_option("split_k", 0)


def test_split_k_uneven_k_falls_back(capi, cuda, oracle):
    # 7 K tiles: no even split with four or more tiles per part exists, the GEMM runs unsplit
    m, n, k = 128, 256, 896
    ac, asc, bc, bsc = _rand_problem(oracle, m, n, k, seed=78)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc)
    _check(oracle, out, gold, k)


# ---- E5M2 activations (option "a_dtype" = 1; weights stay E4M3) ----

@pytest.mark.parametrize("cta_pair", [2, 1])
def test_e5m2_activations(capi, cuda, oracle, golden, cta_pair):
    d, g = golden("quant_e5m2"), golden("agmm_small")
    capi.set_option("a_dtype", 1)
    try:
        # the reference-generated 2-rank problem
        out = _run(capi, cuda, np.concatenate(list(d["agmm_a_codes"])), np.concatenate(list(d["agmm_a_scales"])),
                   g["b_codes"], g["b_scales"], cta_pair=cta_pair)
        _check(oracle, out, d["agmm_golden"], 256)
        # a larger seeded problem against the oracle
        rng = np.random.default_rng(55)
        m, n, k = 300, 528, 2048
        a = rng.standard_normal((m, k), dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)
        ac, asc = oracle.quantize_rows(workloads.f32_to_bf16_bits(a), fmt=oracle.FMT_E5M2)
        bc, bsc = oracle.quantize_weight(workloads.f32_to_bf16_bits(b))
        gold = oracle.allgather_matmul([ac], [asc], bc, bsc, a_fmt=oracle.FMT_E5M2)
        out = _run(capi, cuda, ac, asc, bc, bsc, cta_pair=cta_pair)
        _check(oracle, out, gold, k)
    finally:
        capi.set_option("a_dtype", 0)


# ---- CTA pairs (256 x 256 tiles, tcgen05 cta_group::2) ----------------------------------------------

def test_pair_single_tile_unit_scales(capi, cuda, oracle):
    rng = np.random.default_rng(21)
    m, n, k = 256, 256, 128
    ac = rng.integers(0x30, 0x48, (m, k)).astype(np.uint8) | (rng.integers(0, 2, (m, k)).astype(np.uint8) << 7)
    bc = rng.integers(0x30, 0x48, (k, n)).astype(np.uint8) | (rng.integers(0, 2, (k, n)).astype(np.uint8) << 7)
    asc = np.full((m, k // 32), 0x7F, np.uint8)
    bsc = np.full((k // 64, n, 2), 0x7F, np.uint8)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc, cta_pair=1)
    _check(oracle, out, gold, k)


def test_pair_scale_factor_routing(capi, cuda, oracle):
    rng = np.random.default_rng(22)
    m, n, k = 512, 512, 512
    ac = rng.integers(0x30, 0x48, (m, k)).astype(np.uint8)
    bc = rng.integers(0x30, 0x48, (k, n)).astype(np.uint8)
    asc = (120 + (np.arange(m)[:, None] * 7 + np.arange(k // 32)[None, :] * 3) % 13).astype(np.uint8)
    bs_kn = (118 + (np.arange(k // 32)[:, None] * 5 + np.arange(n)[None, :]) % 11).astype(np.uint8)
    bsc = np.ascontiguousarray(bs_kn.reshape(k // 64, 2, n).transpose(0, 2, 1))
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc, cta_pair=1)
    _check(oracle, out, gold, k)


@pytest.mark.parametrize("m,n,k", [(512, 1024, 1024), (100, 272, 384), (385, 2304, 7168), (3072, 2048, 256), (130, 3456, 5120)])
def test_pair_shapes(capi, cuda, oracle, m, n, k):
    ac, asc, bc, bsc = _rand_problem(oracle, m, n, k, seed=m + n + k + 1)
    gold = oracle.allgather_matmul([ac], [asc], bc, bsc)
    out = _run(capi, cuda, ac, asc, bc, bsc, cta_pair=1)
    _check(oracle, out, gold, k)
    out16 = _run(capi, cuda, ac, asc, bc, bsc, cta_pair=1, f16=True)
    assert oracle.check_reference_rule(out16, gold, k, bf16=False)[0] == 0


# ---- FP4 (E2M1) operands, packed two per byte: the reference's float4_e2m1x2_t operator variant
# (examples/ascend950_fp4_mx_allgather_matmul/ascend950_fp4_mx_allgather_matmul_device.h:42-49) ----

def _fp4_weight(oracle, b_f32):
    """B [K, N] -> packed E2M1 [K, N/2] (low nibble = even column, as gen_data_fp4_mx_allgather_matmul.py:521-544
    packs it), scales [K/64, N, 2] (32 along K), and the dequantised fp32 matrix."""
    k, n = b_f32.shape
    pt, st = oracle.quantize_rows_e2m1(workloads.f32_to_bf16_bits(np.ascontiguousarray(b_f32.T)))  # [N, K/2], [N, K/32]
    deq = oracle.dequant_rows_e2m1(pt, st).T.copy()
    nib = np.empty((n, k), np.uint8)
    nib[:, 0::2] = pt & 0x0F
    nib[:, 1::2] = pt >> 4
    nib = np.ascontiguousarray(nib.T)  # [K, N]
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    scales = np.ascontiguousarray(st.T.reshape(k // 64, 2, n).transpose(0, 2, 1))
    return packed, scales, deq


@pytest.mark.parametrize("cta_pair", [2, 1])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (300, 512, 2048), (1024, 2304, 7168)])
def test_fp4_operands(capi, cuda, oracle, m, n, k, cta_pair):
    torch = cuda
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)
    ap, asc = oracle.quantize_rows_e2m1(workloads.f32_to_bf16_bits(a))
    bp, bsc, b_deq = _fp4_weight(oracle, b)
    gold = oracle.gemm_f32(oracle.dequant_rows_e2m1(ap, asc), b_deq)
    capi.set_option("a_dtype", 2)
    capi.set_option("b_dtype", 2)
    capi.set_option("cta_pair", cta_pair)
    try:
        c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        dev = [torch.from_numpy(x).cuda() for x in (ap, asc, bp, bsc)]  # kept alive until the kernel has run
        rc = capi.load().catccos_b200_mx_gemm(torch.cuda.current_stream().cuda_stream, dev[0].data_ptr(), dev[1].data_ptr(),
                                               dev[2].data_ptr(), dev[3].data_ptr(), c.data_ptr(), m, n, k)
        assert rc == 0
        code, st = capi.last_status()
        assert code == 0, st
        _check(oracle, c.float().cpu().numpy(), gold, k)
    finally:
        capi.set_option("a_dtype", 0)
        capi.set_option("b_dtype", 0)
        capi.set_option("cta_pair", 0)
