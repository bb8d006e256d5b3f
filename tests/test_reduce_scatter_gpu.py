"""GPU tests of MXFP8 Matmul + ReduceScatter (the reference's Ascend950MxFp8MatmulReduceScatter operator,
include/catccos/dgemm/kernel/matmul_reduce_scatter_mx_tla.hpp, golden
examples/ascend950_mxfp8_matmul_reduce_scatter/scripts/gen_data_mxfp8_mmrs.py:374-392: the ranks' products are
summed and rank r keeps row chunk r).  All ranks are hosted on one GPU: every rank's GEMM-and-scatter half runs
first, the reducing halves afterwards.  Tolerance as for the GEMM: |out - gold| <= 1e-3 + 1e-2 |gold|."""
import numpy as np
import pytest

from catccos_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture()
def local_world(capi, cuda):
    def _make(world):
        capi.finalize()
        capi.init_local(world, [0] * world)
        return world

    yield _make
    capi.set_option("phase_mask", 3)
    capi.set_option("cta_pair", 0)
    capi.set_option("a_dtype", 0)
    capi.set_option("b_dtype", 0)
    capi.finalize()


@pytest.mark.parametrize("cta_pair", [2, 1])
@pytest.mark.parametrize("world,m,k,n,e5m2", [(2, 256, 512, 512, False), (4, 512, 256, 272, False), (8, 2048, 1024, 2304, False),
                                              (2, 64, 1024, 1024, True), (1, 128, 256, 256, False)])
def test_matmul_reduce_scatter_emulated(capi, cuda, oracle, local_world, world, m, k, n, e5m2, cta_pair):
    torch = cuda
    local_world(world)
    capi.set_option("cta_pair", cta_pair)
    fmt = oracle.FMT_E5M2 if e5m2 else oracle.FMT_E4M3
    if e5m2:  # the reference's example feeds E5M2 operands (ascend950_mxfp8_matmul_reduce_scatter_host.h:40-41)
        capi.set_option("a_dtype", 1)
        capi.set_option("b_dtype", 1)
    t = capi.make_tiling(m, k, n, world)
    symm = []
    for r in range(world):
        capi.set_rank(r)
        symm.append(capi.symm_alloc(capi.symm_bytes_needed(t, 2)))
    rng = np.random.default_rng(world * 100 + m)
    for rnd in range(2):  # both stages
        a = [rng.standard_normal((m, k), dtype=np.float32) for _ in range(world)]
        b = [rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05) for _ in range(world)]
        aq = [oracle.quantize_rows(workloads.f32_to_bf16_bits(x), fmt=fmt) for x in a]
        # weights: blocks of 32 along K, scales in the [K/64, N, 2] file layout
        bq = []
        for x in b:
            ct, st = oracle.quantize_rows(workloads.f32_to_bf16_bits(np.ascontiguousarray(x.T)), fmt=fmt)  # [N, K], [N, K/32]
            bq.append((np.ascontiguousarray(ct.T), np.ascontiguousarray(st.T.reshape(k // 64, 2, n).transpose(0, 2, 1)),
                       oracle.dequant_rows(ct, st, fmt=fmt).T.copy()))
        gold = sum(oracle.gemm_f32(oracle.dequant_rows(aq[r][0], aq[r][1], fmt=fmt), bq[r][2]) for r in range(world))
        dev = [[torch.from_numpy(x).cuda() for x in (aq[r][0], aq[r][1], bq[r][0], bq[r][1])] for r in range(world)]
        d = [torch.zeros((m // world, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for phase in (1, 2):
            capi.set_option("phase_mask", phase)
            for r in range(world):
                capi.set_rank(r)
                capi.mxfp8_matmul_reduce_scatter(dev[r][0], dev[r][1], dev[r][2], dev[r][3], d[r], symm[r], world)
        torch.cuda.synchronize()
        capi.set_option("phase_mask", 3)
        rows = m // world
        for r in range(world):
            capi.set_rank(r)
            code, st = capi.last_status()
            assert code == 0, (r, st)
            bad, maxdiff = oracle.check_close(d[r].float().cpu().numpy(), gold[r * rows:(r + 1) * rows], 1e-2, 1e-3)
            assert bad == 0, (rnd, r, bad, maxdiff)
