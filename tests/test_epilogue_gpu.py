"""GPU tests of the producers that quantise where the data is made: the GEMM whose epilogue MX-quantises its own
output (the reference's QuantFromUb / QuantFromUb2D, include/catccos/comm/block/comm_block_mx_quant.hpp:209-310)
and the routing-side quantise-and-scatter into packed rows (QuantScatterPacked, :312-368).  Both are bit-exact
against the oracle's quantiser."""
import numpy as np
import pytest

from catccos_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cta_pair", [2, 1])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (300, 544, 1024), (1024, 2304, 2048), (16, 4096, 7168)])
def test_gemm_with_quantised_output(capi, cuda, oracle, m, n, k, cta_pair):
    # The epilogue quantises the bf16 rounding of what the plain GEMM would store, so its codes and scales must be
    # exactly the oracle's quantisation of the plain GEMM's bf16 output (same kernel, same accumulators); the plain
    # output itself is checked against the fp32 golden in test_gemm_gpu.py.
    torch = cuda
    rng = np.random.default_rng(m * 7 + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)
    ac, asc = oracle.quantize_rows(workloads.f32_to_bf16_bits(a))
    bc, bsc = oracle.quantize_weight(workloads.f32_to_bf16_bits(b))
    a_d, as_d = torch.from_numpy(ac).cuda(), torch.from_numpy(asc).cuda()
    b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bsc).cuda()
    capi.set_option("cta_pair", cta_pair)
    try:
        plain = capi.mx_gemm(a_d, as_d, b_d, bs_d)
        codes, scales = capi.mx_gemm_quant_out(a_d, as_d, b_d, bs_d)
        code, st = capi.last_status()
        assert code == 0, st
    finally:
        capi.set_option("cta_pair", 0)
    bits = plain.view(torch.int16).cpu().numpy().view(np.uint16)
    want_c, want_s = oracle.quantize_rows(bits)
    assert np.array_equal(scales.cpu().numpy(), want_s)
    assert np.array_equal(codes.cpu().numpy(), want_c)


@pytest.mark.parametrize("tokens,n,top_k", [(64, 7168, 8), (37, 160, 2), (1, 32, 1), (300, 2048, 4)])
def test_quant_scatter_packed(capi, cuda, oracle, tokens, n, top_k):
    torch = cuda
    rng = np.random.default_rng(tokens + n)
    x_bits = workloads.f32_to_bf16_bits(rng.standard_normal((tokens, n), dtype=np.float32) * np.float32(3.0))
    rows_out = tokens * top_k + 5
    idx = rng.permutation(rows_out)[: tokens * top_k].astype(np.int32).reshape(tokens, top_k)
    idx[rng.random((tokens, top_k)) < 0.1] = -1  # dropped routes
    row_bytes = capi.packed_row_bytes(n)
    assert row_bytes % 32 == 0 and row_bytes >= n + n // 32
    out = torch.full((rows_out, row_bytes), 0xAA, dtype=torch.uint8, device="cuda")
    x_d = torch.from_numpy(x_bits.view(np.int16).copy()).cuda().view(torch.bfloat16)
    capi.mx_quant_scatter_packed(x_d, torch.from_numpy(idx).cuda(), out, top_k)
    got = out.cpu().numpy()
    want = np.full((rows_out, row_bytes), 0xAA, np.uint8)
    wc, ws = oracle.quantize_rows(x_bits)
    for t in range(tokens):
        for r in range(top_k):
            if idx[t, r] >= 0:
                want[idx[t, r], :n] = wc[t]
                want[idx[t, r], n:n + n // 32] = ws[t]
                want[idx[t, r], n + n // 32:] = 0
    assert np.array_equal(got, want)
