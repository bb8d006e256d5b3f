"""GPU tests of the multi-rank protocol on ONE device: the single-process harness hosts all ranks,
runs every rank's producer half first (for the fused operator: the quantise and pusher warps of the fused
kernel, its GEMM warps idle) and the consumers afterwards (kernels of different ranks never wait on one
another while sharing a GPU).  Results are compared with the oracle: gathered codes and scales bit for
bit, GEMM output within rtol 1e-2 / atol 1e-3."""
import numpy as np
import pytest

from catccos_b200 import workloads
from conftest import to_dev_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture()
def local_world(capi, cuda):
    made = {}

    def _make(world):
        capi.finalize()
        capi.init_local(world, [0] * world)
        made["w"] = world
        return world

    yield _make
    capi.set_option("phase_mask", 3)
    capi.set_option("timeout_ms", 2000)
    capi.set_option("cta_pair", 0)
    capi.set_option("fuse_mode", -1)
    capi.finalize()


def _alloc_symm(capi, world, nbytes):
    ptrs = []
    for r in range(world):
        capi.set_rank(r)
        ptrs.append(capi.symm_alloc(nbytes))
    return ptrs


def _quant_allgather_round(capi, torch, xs, outs, symm, world):
    for phase in (1, 2):
        capi.set_option("phase_mask", phase)
        for r in range(world):
            capi.set_rank(r)
            capi.mx_quant_allgather(xs[r], outs[r][0], outs[r][1], symm[r], world)
    torch.cuda.synchronize()
    capi.set_option("phase_mask", 3)
    for r in range(world):
        capi.set_rank(r)
        code, st = capi.last_status()
        assert code == 0, (r, st)


@pytest.mark.parametrize("symmetric_out", [False, True])
@pytest.mark.parametrize("world,m,k", [(2, 64, 1024), (4, 126, 512), (3, 37, 160), (8, 16, 7168), (2, 8190, 512)])
def test_quant_allgather_emulated(capi, cuda, oracle, local_world, world, m, k, symmetric_out):
    # (2, 8190, 512): the reference's ragged row count (scripts/test_shapes.csv: 8190 = 63 * 128 + 126)
    torch = cuda
    local_world(world)
    t = capi.make_tiling(m, 1, k, world)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(t, True))
    nc, ns = world * m * k, world * m * (k // 32)
    ns_off = (nc + 1023) // 1024 * 1024
    out_symm = _alloc_symm(capi, world, ns_off + ns) if symmetric_out else None
    rng = np.random.default_rng(world * 1000 + m)
    for rnd in range(3):  # three rounds: both stages and the reuse of the first
        bits = [workloads.f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)) for _ in range(world)]
        xs = [to_dev_bf16(torch, b) for b in bits]
        if symmetric_out:
            # outputs inside symmetric memory at the same offset on every rank: the peers write them directly
            outs = [(capi.symm_tensor(out_symm[r], nc).view(world * m, k),
                     capi.symm_tensor(out_symm[r], ns, ns_off).view(world * m, k // 32)) for r in range(world)]
            for oc, osc in outs:
                oc.fill_(0xAA)
                osc.fill_(0xAA)
        else:
            outs = [(torch.full((world * m, k), 0xAA, dtype=torch.uint8, device="cuda"),
                     torch.full((world * m, k // 32), 0xAA, dtype=torch.uint8, device="cuda")) for _ in range(world)]
        _quant_allgather_round(capi, torch, xs, outs, symm, world)
        want = [oracle.quantize_rows(b) for b in bits]
        want_c = np.concatenate([w[0] for w in want])
        want_s = np.concatenate([w[1] for w in want])
        for r in range(world):
            assert np.array_equal(outs[r][0].cpu().numpy(), want_c), (rnd, r)
            assert np.array_equal(outs[r][1].cpu().numpy(), want_s), (rnd, r)


def _agmm_round(capi, torch, call, world):
    for phase in (1, 2):
        capi.set_option("phase_mask", phase)
        for r in range(world):
            capi.set_rank(r)
            call(r)
    torch.cuda.synchronize()
    capi.set_option("phase_mask", 3)
    for r in range(world):
        capi.set_rank(r)
        code, st = capi.last_status()
        assert code == 0, (r, st)


@pytest.mark.parametrize("fuse_mode", [0, 5, 6, 7])  # pusher warps of the fused kernel / copy engines / quantise kernel stores to all
@pytest.mark.parametrize("cta_pair", [2, 1])
@pytest.mark.parametrize("world,m,k,n", [(2, 256, 1024, 1024), (4, 128, 512, 256), (8, 16, 1024, 512), (2, 100, 256, 272),
                                         (2, 16, 7168, 512), (4, 48, 4096, 272)])  # the last two: K split in 8 and 4 parts
def test_quant_allgather_matmul_emulated(capi, cuda, oracle, local_world, world, m, k, n, cta_pair, fuse_mode):
    torch = cuda
    local_world(world)
    capi.set_option("cta_pair", cta_pair)
    capi.set_option("fuse_mode", fuse_mode)
    t = capi.make_tiling(m, k, n, world)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(t, False))
    cfg = workloads.Config("t", m, k, n, (world,), "normal", "")
    for rnd in range(2):
        a_bits = [workloads.activation_bits(cfg, r, seed=rnd) for r in range(world)]
        w = [oracle.quantize_weight(workloads.weight_bits(cfg, r, seed=rnd)) for r in range(world)]
        a_d = [to_dev_bf16(torch, b) for b in a_bits]
        b_d = [(torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda()) for bc, bs in w]
        c_d = [torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        _agmm_round(capi, torch,
                    lambda r: capi.mx_quant_allgather_matmul(a_d[r], b_d[r][0], b_d[r][1], c_d[r], symm[r], world),
                    world)
        aq = [oracle.quantize_rows(b) for b in a_bits]
        for r in range(world):
            gold = oracle.allgather_matmul([q[0] for q in aq], [q[1] for q in aq], w[r][0], w[r][1])
            bad, maxdiff = oracle.check_close(c_d[r].float().cpu().numpy(), gold, 1e-2, 1e-3)
            assert bad == 0, (rnd, r, bad, maxdiff)


def test_prequantised_allgather_matmul_emulated(capi, cuda, oracle, local_world, golden):
    # the reference's operator signature: A arrives quantised, in the reference's file layouts
    torch = cuda
    d = golden("agmm_small")
    world, m, k = d["a_codes"].shape
    n = d["b_codes"].shape[1]
    local_world(world)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(capi.make_tiling(m, k, n, world), False))
    a_d = [(torch.from_numpy(d["a_codes"][r]).cuda(), torch.from_numpy(d["a_scales"][r]).cuda()) for r in range(world)]
    b_d, bs_d = torch.from_numpy(d["b_codes"]).cuda(), torch.from_numpy(d["b_scales"]).cuda()
    c_d = [torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    _agmm_round(capi, torch,
                lambda r: capi.fp8_mx_allgather_matmul(a_d[r][0], a_d[r][1], b_d, bs_d, c_d[r], symm[r], world), world)
    for r in range(world):
        bad, maxdiff = oracle.check_close(c_d[r].float().cpu().numpy(), d["golden"], 1e-2, 1e-3)
        assert bad == 0, (r, bad, maxdiff)


@pytest.mark.parametrize("fuse_mode", [0, 3, 4])
@pytest.mark.parametrize("m,k,n", [(16, 7168, 1024), (200, 3584, 528)])
def test_fused_single_rank_split_k(capi, cuda, oracle, fuse_mode, m, k, n):
    # few output tiles: K is split over the idle SMs and the quantiser feeds the K parts round-robin
    torch = cuda
    capi.finalize()
    capi.set_option("fuse_mode", fuse_mode)
    cfg = workloads.Config("t", m, k, n, (1,), "normal", "")
    bc, bs = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=11))
    symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(m, k, n, 1), False))
    b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda()
    try:
        for call in range(3):
            a_bits = workloads.activation_bits(cfg, 0, seed=20 + call)
            a_d = to_dev_bf16(torch, a_bits)
            c_d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
            capi.mx_quant_allgather_matmul(a_d, b_d, bs_d, c_d, symm, 1)
            code, st = capi.last_status()
            assert code == 0, st
            ac, asc = oracle.quantize_rows(a_bits)
            gold = oracle.allgather_matmul([ac], [asc], bc, bs)
            bad, maxdiff = oracle.check_close(c_d.float().cpu().numpy(), gold, 1e-2, 1e-3)
            assert bad == 0, (call, bad, maxdiff)
    finally:
        capi.symm_free(symm)
        capi.set_option("fuse_mode", -1)


@pytest.mark.parametrize("fuse_mode", [0, 3])
def test_fused_single_rank_e5m2(capi, cuda, oracle, fuse_mode):
    # bf16 in, E5M2 codes quantised on the fly and consumed by the GEMM in the same call
    torch = cuda
    capi.finalize()
    capi.set_option("fuse_mode", fuse_mode)
    capi.set_option("a_dtype", 1)
    cfg = workloads.Config("t", 272, 2048, 528, (1,), "normal", "")
    a_bits = workloads.activation_bits(cfg, 0, seed=3)
    bc, bs = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=3))
    symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(cfg.m_local, cfg.k, cfg.n_local, 1), False))
    try:
        c_d = torch.zeros((cfg.m_local, cfg.n_local), dtype=torch.bfloat16, device="cuda")
        capi.mx_quant_allgather_matmul(to_dev_bf16(torch, a_bits), torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda(),
                                       c_d, symm, 1)
        code, st = capi.last_status()
        assert code == 0, st
        ac, asc = oracle.quantize_rows(a_bits, fmt=oracle.FMT_E5M2)
        gold = oracle.allgather_matmul([ac], [asc], bc, bs, a_fmt=oracle.FMT_E5M2)
        bad, maxdiff = oracle.check_close(c_d.float().cpu().numpy(), gold, 1e-2, 1e-3)
        assert bad == 0, (bad, maxdiff)
    finally:
        capi.symm_free(symm)
        capi.set_option("fuse_mode", -1)
        capi.set_option("a_dtype", 0)


@pytest.mark.parametrize("cta_pair", [2, 1])
@pytest.mark.parametrize("fuse_mode", [0, 3, 4])
def test_fused_single_rank(capi, cuda, oracle, fuse_mode, cta_pair):
    # world 1 through every path: quantise warps inside the GEMM kernel (0), or one kernel after the other on
    # one stream, the GEMM free of flags (3, the default) or gated on them (4)
    torch = cuda
    capi.finalize()
    capi.set_option("fuse_mode", fuse_mode)
    capi.set_option("cta_pair", cta_pair)
    cfg = workloads.Config("t", 640, 1024, 768, (1,), "normal", "")
    a_bits = workloads.activation_bits(cfg, 0, seed=7)
    bc, bs = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=7))
    symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(cfg.m_local, cfg.k, cfg.n_local, 1), False))
    a_d = to_dev_bf16(torch, a_bits)
    b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda()
    c_d = torch.zeros((cfg.m_local, cfg.n_local), dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        capi.mx_quant_allgather_matmul(a_d, b_d, bs_d, c_d, symm, 1)
    code, st = capi.last_status()
    assert code == 0, st
    ac, asc = oracle.quantize_rows(a_bits)
    gold = oracle.allgather_matmul([ac], [asc], bc, bs)
    bad, maxdiff = oracle.check_close(c_d.float().cpu().numpy(), gold, 1e-2, 1e-3)
    assert bad == 0, (bad, maxdiff)
    capi.symm_free(symm)
    capi.set_option("fuse_mode", -1)
    capi.set_option("cta_pair", 0)


def test_missing_peer_is_reported_not_hung(capi, cuda, local_world):
    # failure detection without a GPU fault: rank 1 never launches its producer, so rank 0's
    # consumer waits on flags that nothing sets; the bounded wait runs out, the kernel ends and the
    # status names the rank and chunk it was waiting for
    torch = cuda
    world, m, k = 2, 32, 256
    local_world(world)
    capi.set_option("timeout_ms", 100)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(capi.make_tiling(m, 1, k, world), True))
    x = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    oc = torch.zeros((world * m, k), dtype=torch.uint8, device="cuda")
    osc = torch.zeros((world * m, k // 32), dtype=torch.uint8, device="cuda")
    capi.set_rank(0)
    capi.mx_quant_allgather(x, oc, osc, symm[0], world)  # producer and consumer of rank 0 only
    code, st = capi.last_status()
    assert code == -7 and st[0] == 1 and st[1] == 1 and st[3] == 1, (code, st)
    # the context is still usable and the record was cleared
    assert torch.zeros(4, device="cuda").sum().item() == 0
    assert capi.last_status()[0] == 0


@pytest.mark.parametrize("cta_pair", [2, 1])
def test_missing_peer_ends_the_gemm_kernel_quickly(capi, cuda, local_world, cta_pair):
    # the same failure on the AllGather-Matmul path: rank 0 makes its call and rank 1 never does, so rank 0's
    # GEMM warps wait for rank 1's rows on flags that nothing sets.  The first wait that runs out must end the
    # whole kernel (every other wait gives up as soon as it looks), not one limit per wait: with 8 K segments
    # and several tiles per CTA a kernel that paid the limit per wait would run for seconds.
    import time

    torch = cuda
    world, m, k, n = 2, 512, 4096, 1024
    local_world(world)
    capi.set_option("cta_pair", cta_pair)
    capi.set_option("timeout_ms", 100)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(capi.make_tiling(m, k, n, world), False))
    a = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((k, n), dtype=torch.uint8, device="cuda")
    bs = torch.full((k // 64, n, 2), 0x7F, dtype=torch.uint8, device="cuda")
    c = torch.full((world * m, n), 7.0, dtype=torch.bfloat16, device="cuda")
    capi.set_rank(0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    capi.mx_quant_allgather_matmul(a, b, bs, c, symm[0], world)
    code, st = capi.last_status()
    dt = time.perf_counter() - t0
    assert code == -7 and st[0] == 1 and st[1] == 1 and st[3] == 1, (code, st)
    assert dt < 1.0, f"the kernel took {dt:.2f} s to end after a 0.1 s limit"
    # rank 0's own rows were computed (all zeros here); nothing was written from accumulators that never filled
    assert torch.all(c[m:] == 7.0)
    assert capi.last_status()[0] == 0


@pytest.mark.parametrize("world,cfg_name,ranks_checked", [(8, "c3_prefill", (0, 5)), (4, "c3_prefill", (3,))])
def test_prefill_shape_at_full_size_emulated(capi, cuda, oracle, local_world, world, cfg_name, ranks_checked):
    # The benchmark's own shape (per rank A [1024, 7168], B [7168, 2304]) with all ranks hosted on one GPU:
    # several waves of 256 x 256 tiles per CTA pair, 256-row send groups, seven K segments per chunk.
    # Sampled rows of every source rank are compared with the oracle.
    torch = cuda
    cfg = workloads.CONFIGS[cfg_name]
    m, k, n = cfg.m_local, cfg.k, cfg.n_local
    local_world(world)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(capi.make_tiling(m, k, n, world), False))
    a_bits = [workloads.activation_bits(cfg, r, seed=0) for r in range(world)]
    a_d = [to_dev_bf16(torch, b) for b in a_bits]
    w = {r: oracle.quantize_weight(workloads.weight_bits(cfg, r, seed=0)) for r in ranks_checked}
    b_d = {r: (torch.from_numpy(w[r][0]).cuda(), torch.from_numpy(w[r][1]).cuda()) for r in ranks_checked}
    c_d = [torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for rnd in range(2):  # both stages of the symmetric buffer
        for c in c_d:
            c.zero_()
        _agmm_round(capi, torch,
                    lambda r: capi.mx_quant_allgather_matmul(a_d[r], b_d[ranks_checked[0] if r not in b_d else r][0],
                                                             b_d[ranks_checked[0] if r not in b_d else r][1], c_d[r],
                                                             symm[r], world), world)
        rng = np.random.default_rng(rnd)
        rows = np.sort(np.concatenate([s * m + np.r_[0, 127, 128, 255, 256, m - 1, rng.integers(0, m, 10)] for s in range(world)]))
        a_rows = np.stack([a_bits[i // m][i % m] for i in rows])
        ac, asc = oracle.quantize_rows(a_rows)
        for r in ranks_checked:
            gold = oracle.gemm_f32(oracle.dequant_rows(ac, asc), oracle.dequant_weight(w[r][0], w[r][1]))
            out = c_d[r][torch.from_numpy(rows).cuda()].float().cpu().numpy()
            bad, maxdiff = oracle.check_close(out, gold, 1e-2, 1e-3)
            assert bad == 0, (rnd, r, bad, maxdiff)


@pytest.mark.parametrize("world,m,k,n", [(1, 256, 512, 256), (2, 128, 1024, 512), (4, 272, 2048, 384)])
def test_fp4_allgather_matmul_emulated(capi, cuda, oracle, local_world, world, m, k, n):
    # the reference's FP4 operator: both operands packed E2M1 (two per byte), E8M0 scales per 32 along K
    torch = cuda
    local_world(world)
    symm = _alloc_symm(capi, world, capi.symm_bytes_needed(capi.make_tiling(m, k, n, world), False))
    rng = np.random.default_rng(world + m + k)
    for rnd in range(2):
        aq = [oracle.quantize_rows_e2m1(workloads.f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)))
              for _ in range(world)]
        a_deq = np.concatenate([oracle.dequant_rows_e2m1(p, s) for p, s in aq])
        bw = []
        for _ in range(world):
            b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.05)
            pt, st = oracle.quantize_rows_e2m1(workloads.f32_to_bf16_bits(np.ascontiguousarray(b.T)))  # [N, K/2], [N, K/32]
            nib = np.empty((n, k), np.uint8)
            nib[:, 0::2] = pt & 0x0F
            nib[:, 1::2] = pt >> 4
            nib = np.ascontiguousarray(nib.T)
            bw.append(((nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8),
                       np.ascontiguousarray(st.T.reshape(k // 64, 2, n).transpose(0, 2, 1)),
                       oracle.dequant_rows_e2m1(pt, st).T.copy()))
        a_d = [(torch.from_numpy(p).cuda(), torch.from_numpy(s).cuda()) for p, s in aq]
        b_d = [(torch.from_numpy(x[0]).cuda(), torch.from_numpy(x[1]).cuda()) for x in bw]
        c_d = [torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        _agmm_round(capi, torch,
                    lambda r: capi.fp4_mx_allgather_matmul(a_d[r][0], a_d[r][1], b_d[r][0], b_d[r][1], c_d[r], symm[r], world),
                    world)
        for r in range(world):
            gold = oracle.gemm_f32(a_deq, bw[r][2])
            bad, maxdiff = oracle.check_close(c_d[r].float().cpu().numpy(), gold, 1e-2, 1e-3)
            assert bad == 0, (rnd, r, bad, maxdiff)
