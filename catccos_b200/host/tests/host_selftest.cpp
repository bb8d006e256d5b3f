// Host-only checks of the operator surface (no GPU work): registry behaviour, tiling validation,
// size arithmetic and error behaviour, the launcher table, file helpers.  Exit code 0 = pass.
#include <cstdio>

#include "../examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_device.h"
#include "../examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_host.h"
#include "../examples/ascend950_fp4_mx_allgather_matmul/ascend950_fp4_mx_allgather_matmul_host.h"
#include "../examples/ascend950_mx_quant_allgather/mx_quant_allgather_host.h"
#include "../examples/ascend950_mxfp8_matmul_reduce_scatter/ascend950_mxfp8_matmul_reduce_scatter_host.h"
#include "dynamic_tiling/launch_map.h"

#define EXPECT(cond)                                                     \
    do {                                                                 \
        if (!(cond)) {                                                   \
            std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond);   \
            return 1;                                                    \
        }                                                                \
    } while (0)

// The reference driver's type lines (examples/ascend950_fp8_mx_allgather_matmul/main.cpp:16-31) with half output:
// they must keep compiling against this tree's headers.
namespace compat {
using Config = Ascend950Fp8MxAllGatherMatmulConfig_M0_128<float8_e4m3_t, Catlass::layout::RowMajor, float8_e4m3_t,
                                                         Catlass::layout::RowMajor, float8_e8m0_t, Catlass::layout::RowMajor,
                                                         float8_e8m0_t, Catlass::layout::RowMajor, half,
                                                         Catlass::layout::RowMajor>;
using DeviceOp = Config::Device;
}  // namespace compat

static int device_op_checks()
{
    // the reference's call sequence (main.cpp:150-183) on a shape the kernels cannot take: it must be refused
    // by Initialize / Run through Catlass::Status, without touching a GPU
    Catlass::GemmCoord problemShape{256, 1000, 100};
    Catlass::MatrixCoord commCoreSplit{16, 2};
    Catlass::MatrixCoord commBlockShape{64, 0x7FFFFFFFu};
    Catlass::MatrixCoord commTileShape{32, 256};
    uint8_t dummy = 0;
    compat::DeviceOp::Arguments args{problemShape, 0u, 1u, 3u, &dummy, &dummy, &dummy, &dummy, &dummy, &dummy,
                                     commCoreSplit, commBlockShape, commTileShape};
    compat::DeviceOp deviceOp;
    EXPECT(compat::DeviceOp::GetWorkspaceSize(args) == 0);
    EXPECT(deviceOp.Initialize(args) == Catlass::Status::kErrorInvalidProblem);  // k % 128 != 0
    EXPECT(deviceOp.Run(nullptr, 1, 0) == Catlass::Status::kErrorInvalidProblem);
    EXPECT(deviceOp.params().tiling.m == 256 && deviceOp.params().tiling.rankSize == 1);
    args.problemShape = Catlass::GemmCoord{256, 1024, 512};
    EXPECT(deviceOp.Initialize(args) == Catlass::Status::kSuccess);
    EXPECT((std::is_same<compat::DeviceOp::Kernel::ElementC, half>::value));
    return 0;
}

int main()
{
    if (device_op_checks() != 0) {
        return 1;
    }
    auto& reg = OperatorRegistry::Instance();
    auto q = reg.CreateOperator("MxQuantAllGather");
    auto g = reg.CreateOperator("Ascend950Fp8MxAllGatherMatmul");
    EXPECT(q != nullptr && g != nullptr);
    {
        // the FP4 variant and the row-parallel partner: registry names, enum ids and short names of the reference
        auto f4 = reg.CreateOperator("Ascend950Fp4MxAllGatherMatmul");
        auto rs = reg.CreateOperator("Ascend950MxFp8MatmulReduceScatter");
        EXPECT(f4 != nullptr && rs != nullptr);
        CocTilingParams s;
        s.m = 1024;
        s.k = 7168;
        s.n = 2304;
        s.rankSize = 8;
        EXPECT(f4->GetActualKernelType(s) == 23 && GetCommType("a5fp4mxagmm") == ASCEND950_FP4_MX_ALLGATHER_MATMUL);
        EXPECT(rs->GetActualKernelType(s) == 18 && GetCommType("a5mxfp8mmrs") == ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER);
        EXPECT(f4->CheckCocTilingParams(8, s) && rs->CheckCocTilingParams(8, s));
        s.n = 2320;  // a multiple of 16 but not of 128: fine for the reduce-scatter, not for packed FP4 rows
        EXPECT(!f4->CheckCocTilingParams(8, s) && rs->CheckCocTilingParams(8, s));
        s.m = 1000;  // 125 rows per rank
        EXPECT(!rs->CheckCocTilingParams(8, s));
        EXPECT(rs->GetSymmetricSize(s) > 2ull * 1000 * 2320 * 4);
    }
    EXPECT(reg.CreateOperator("NoSuchOperator") == nullptr);
    EXPECT(!reg.RegisterOperator("MxQuantAllGather", [] { return std::unique_ptr<CatccosOperator>(); }));

    CocTilingParams t;
    t.m = 4096;
    t.n = 7168;
    t.k = 1;
    t.m0 = 32;
    t.n0 = 256;
    t.k0 = 256;
    t.rankSize = 8;
    EXPECT(q->ValidateCocTilingParams(8, t));
    EXPECT(!q->ValidateCocTilingParams(4, t));  // rank count disagrees with the tiling
    t.n = 7170;
    EXPECT(!q->ValidateCocTilingParams(8, t));  // not a multiple of 32
    t.n = 7168;
    t.m = 1u << 20;
    EXPECT(!q->ValidateCocTilingParams(8, t));  // does not fit the reference's buffer bound
    t.m = 4096;
    EXPECT(q->GetActualKernelType(t) == MX_QUANT_ALLGATHER && q->GetWorkspaceSize(t) == 0);
    EXPECT(q->GetSymmetricSize(t) > 2ull * 8 * 4096 * 7168 && q->GetSymmetricSize(t) < (size_t)SHMEM_BUFF_BYTES);
    auto sz = MxQuantAllGatherOperator::BufferSizes(t);
    EXPECT(sz.input == 4096ull * 7168 * 2 && sz.codes == 8ull * 4096 * 7168 && sz.scales == 8ull * 4096 * 224);

    CocTilingParams mm;
    mm.m = 1024;
    mm.k = 7168;
    mm.n = 2304;
    mm.m0 = 128;
    mm.n0 = 256;
    mm.k0 = 256;
    mm.commInterval = 3;
    mm.rankSize = 8;
    EXPECT(g->ValidateCocTilingParams(8, mm));
    mm.k = 7200;
    EXPECT(!g->ValidateCocTilingParams(8, mm));
    EXPECT(g->GetActualKernelType(mm) == ASCEND950_FP8_MX_ALLGATHER_MATMUL);

    bool threw = false;
    try {
        CheckedBufferSize({size_t(1) << 40, size_t(1) << 40});
    } catch (const std::overflow_error&) {
        threw = true;
    }
    EXPECT(threw);
    threw = false;
    try {
        CheckQuantBlockCount(100, 0);
    } catch (const std::invalid_argument&) {
        threw = true;
    }
    EXPECT(threw);

    EXPECT(GetCommType("mxqtag") == MX_QUANT_ALLGATHER && GetCommType("a5fp8mxagmm") == ASCEND950_FP8_MX_ALLGATHER_MATMUL);
    EXPECT(GetCommType("nope") == UNKNOWN);
    EXPECT(KernelDispatcher::GetKernelFunc(MX_QUANT_ALLGATHER, FP8E4M3FN) == &LaunchAscend950BF16QuantAllGatherFP8E4M3FN);
    EXPECT(KernelDispatcher::GetKernelFunc(ASCEND950_FP8_MX_ALLGATHER_MATMUL, FP16) ==
           &LaunchAscend950Fp8MxAllGatherMatmulFP16);
    EXPECT(KernelDispatcher::GetKernelFunc(MX_QUANT_ALLGATHER, INT8) == nullptr);

    const std::string path = "/tmp/catccos_b200_host_selftest.bin";
    const char payload[8] = {1, 2, 3, 4, 5, 6, 7, 8};
    EXPECT(WriteFile(path, payload, sizeof(payload)));
    char back[8] = {};
    EXPECT(ReadFile(path, back, sizeof(back)) && memcmp(back, payload, 8) == 0);
    EXPECT(!ReadFile(path, back, 4));  // size mismatch is an error, as in the reference
    threw = false;
    try {
        ReadFileOrThrow(path + ".missing", back, 8);
    } catch (const std::runtime_error&) {
        threw = true;
    }
    EXPECT(threw);
    unlink(path.c_str());
    std::printf("PASS\n");
    return 0;
}
