// Driver of the Ascend950Fp8MxAllGatherMatmul operator, one process per rank, with the reference's
// command line (examples/ascend950_fp8_mx_allgather_matmul/main.cpp:35-87):
//   allgather_matmul rank_size rank_id ip_port m n k data_path [device_id_list]
#include <cstdio>
#include <sstream>

#include <climits>

#include "ascend950_fp8_mx_allgather_matmul_device.h"
#include "ascend950_fp8_mx_allgather_matmul_host.h"

using namespace Catccos;

using LayoutA = Catlass::layout::RowMajor;
using LayoutB = Catlass::layout::RowMajor;
using LayoutMxScaleA = Catlass::layout::RowMajor;
using LayoutMxScaleB = Catlass::layout::RowMajor;
using LayoutC = Catlass::layout::RowMajor;

using ElementA = float8_e4m3_t;
using ElementB = float8_e4m3_t;
using ElementMxScaleA = float8_e8m0_t;
using ElementMxScaleB = float8_e8m0_t;
using ElementC = bfloat16_t;  // the reference's driver writes half (main.cpp:28); the benchmark's C is bf16

using Config = Ascend950Fp8MxAllGatherMatmulConfig_M0_128<ElementA, LayoutA, ElementB, LayoutB, ElementMxScaleA, LayoutMxScaleA,
                                                         ElementMxScaleB, LayoutMxScaleB, ElementC, LayoutC>;
using DeviceOp = Config::Device;

int main(int argc, char** argv)
{
    if (argc < 8 || argc > 9) {
        printf("Usage: allgather_matmul rank_size rank_id ip_port m n k data_path [device_id_list]\n");
        std::cerr << "Invalid arguments\n";
        return 1;
    }
    const int rankSize = atoi(argv[1]);
    const int rankId = atoi(argv[2]);
    const std::string ipPort = argv[3];
    const uint32_t m = static_cast<uint32_t>(atoll(argv[4]));
    const uint32_t n = static_cast<uint32_t>(atoll(argv[5]));
    const uint32_t k = static_cast<uint32_t>(atoll(argv[6]));
    const std::string dataPath = argv[7];
    std::vector<int> devices;
    if (argc > 8) {
        std::stringstream ss(argv[8]);
        std::string tok;
        while (std::getline(ss, tok, ',')) {
            devices.push_back(atoi(tok.c_str()));
        }
    }
    for (int r = static_cast<int>(devices.size()); r < rankSize; ++r) {
        devices.push_back(r);
    }
    if (rankSize < 1 || rankId < 0 || rankId >= rankSize) {
        std::cerr << "Invalid arguments\n";
        return 1;
    }

    CocTilingParams tiling;
    tiling.m = m;
    tiling.n = n;
    tiling.k = k;
    tiling.m0 = 128;
    tiling.n0 = 256;
    tiling.k0 = 256;
    tiling.commTileM = 64;
    tiling.commInterval = 3;
    tiling.commNpuSplit = rankSize >= 2 ? 2 : 1;
    tiling.commDataSplit = 16;
    tiling.commBlockM = 64;
    tiling.rankSize = rankSize;

    std::cout << "[TEST] input rank_size: " << rankSize << " rank_id:" << rankId << " input_ip: " << ipPort << std::endl;
    if (set_attr(rankId, rankSize, 0, ipPort.c_str(), devices[rankId]) != CATCCOS_SHMEM_SUCCESS) {
        ERROR_LOG("rendezvous failed");
        return -1;
    }
    cudaStream_t stream = nullptr;
    CUDA_CHECK(cudaStreamCreate(&stream));

    auto op = OperatorRegistry::Instance().CreateOperator("Ascend950Fp8MxAllGatherMatmul");
    if (!op) {
        std::cout << "Operator Ascend950Fp8MxAllGatherMatmul not found!" << std::endl;
        return -1;
    }
    if (!op->ValidateCocTilingParams(rankSize, tiling)) {
        ERROR_LOG("tiling rejected: m=%u n=%u k=%u (k must be a multiple of 128, n of 16)", m, n, k);
        return -1;
    }
    KernelParams params;
    op->AllocateDeviceSpace(params, tiling, rankId, dataPath);
    uint8_t* symm = static_cast<uint8_t*>(shmem_calloc(1, op->GetSymmetricSize(tiling)));

    Catlass::GemmCoord problemShape{m, n, k};
    Catlass::MatrixCoord commCoreSplit{tiling.commDataSplit, tiling.commNpuSplit};
    Catlass::MatrixCoord commBlockShape{tiling.commBlockM, UINT_MAX / 2};
    Catlass::MatrixCoord commTileShape{tiling.commTileM / 2, tiling.n0};
    DeviceOp::Arguments args{problemShape,
                             static_cast<uint32_t>(rankId),
                             static_cast<uint32_t>(rankSize),
                             tiling.commInterval,
                             params.ptrA,
                             params.ptrB,
                             params.customPtrs[0],
                             params.customPtrs[1],
                             params.ptrC,
                             symm,
                             commCoreSplit,
                             commBlockShape,
                             commTileShape};

    DeviceOp deviceOp;
    int rc = 0;
    const uint32_t blockNum = 1;  // accepted and ignored: the kernels size their own grids
    const uint64_t fftsAddr = 0;
    if (deviceOp.Initialize(args) != Catlass::Status::kSuccess ||
        deviceOp.Run(stream, blockNum, fftsAddr) != Catlass::Status::kSuccess) {
        ERROR_LOG("device op failed");
        rc = -1;
    }
    uint32_t st[4];
    if (catccos_b200_last_status(st) != 0) {
        rc = -1;
    }
    if (rc == 0) {
        op->WriteResultFile(params, tiling, rankId, dataPath);
        std::printf("rankId %d test finished\n", rankId);
    }
    shmem_free(symm);
    FreeDeviceSpace(params);
    CUDA_CHECK(cudaStreamDestroy(stream));
    shmem_finalize();
    std::cout << "[TEST] exit rankId: " << rankId << std::endl;
    return rc;
}
