"""The allocation-free entry point, catccos_b200_mx_quant_matmul_static.

Some callers cannot allocate device memory at the point where they call the library: a server that
handed all of HBM to its own pools at start-up, or a latency-critical loop that cannot afford the
device-wide pause of an allocation.  For them the library carries its scratch (the quantised copy of
A and the ready flags) in a built-in device array.  This test calls that entry point through the C ABI
twice in a row and checks each result against the regular entry point, which takes its scratch from
catccos_b200_symm_alloc; with K splitting switched off (the allocation-free path has no scratch for partial
tiles) both run the same kernels, so the outputs must agree exactly (the file sorts
last so that a run that stops at the first failure has already seen every other test)."""
import numpy as np
import pytest

from catccos_b200 import workloads
from conftest import to_dev_bf16

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_regular_entry_point_twice(capi, cuda, oracle):
    torch = cuda
    capi.finalize()  # a fresh, single-rank library state whatever ran before
    m, k, n = 384, 1024, 512
    cfg = workloads.Config("noalloc", m, k, n, (1,), "normal", "")
    bc, bs = oracle.quantize_weight(workloads.weight_bits(cfg, 0, seed=5))
    b_d, bs_d = torch.from_numpy(bc).cuda(), torch.from_numpy(bs).cuda()
    symm = capi.symm_alloc(capi.symm_bytes_needed(capi.make_tiling(m, k, n, 1), False))
    capi.set_option("split_k", 1)
    for call in range(2):
        a_bits = workloads.activation_bits(cfg, 0, seed=100 + call)  # new data each call: stale scratch would show
        a_d = to_dev_bf16(torch, a_bits)
        want = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        capi.mx_quant_allgather_matmul(a_d, b_d, bs_d, want, symm, 1)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        if call == 0:
            # the first call on a device looks the array's address up and configures the kernels: not measured
            capi.mx_quant_matmul_static(a_d, b_d, bs_d, got)
            torch.cuda.synchronize()
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # the driver's count: sees any allocation, also one made inside the library
        capi.mx_quant_matmul_static(a_d, b_d, bs_d, got)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the call"
        code, st = capi.static_status()  # the record of this path, kept in the built-in array
        assert code == 0, st
        # same kernels, same inputs: bit-identical; and within the stated tolerance of the oracle
        assert torch.equal(got, want), f"call {call}: outputs differ"
        ac, asc = oracle.quantize_rows(a_bits)
        gold = oracle.allgather_matmul([ac], [asc], bc, bs)
        bad, maxdiff = oracle.check_close(got.float().cpu().numpy(), gold, 1e-2, 1e-3)
        assert bad == 0, (call, bad, maxdiff)
    capi.set_option("split_k", 0)
    capi.symm_free(symm)


def test_static_scratch_rejects_oversize(capi, cuda):
    torch = cuda
    a = torch.zeros((8, 128), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((128, 16), dtype=torch.uint8, device="cuda")
    bs = torch.zeros((2, 16, 2), dtype=torch.uint8, device="cuda")
    c = torch.zeros((8, 16), dtype=torch.bfloat16, device="cuda")
    L = capi.load()
    st = torch.cuda.current_stream().cuda_stream
    # m * k beyond the built-in 8 Mi elements: refused before anything is launched
    assert L.catccos_b200_mx_quant_matmul_static(st, a.data_ptr(), b.data_ptr(), bs.data_ptr(), c.data_ptr(),
                                                 1 << 17, 16, 128) == -4
    assert L.catccos_b200_mx_quant_matmul_static(st, a.data_ptr(), b.data_ptr(), bs.data_ptr(), c.data_ptr(),
                                                 8, 16, 100) == -1
