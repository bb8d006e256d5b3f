// Host side of the Ascend950Fp4MxAllGatherMatmul operator on B200: the FP4 (E2M1, two values per byte) variant of
// the AllGather-Matmul.  File names, pointer roles (ptrA / ptrB packed codes, ptrC output, customPtrs[0] / [1] the
// A / B scales), buffer sizes (m * k / 2, k * n / 2) and the registry name follow the reference
// (examples/ascend950_fp4_mx_allgather_matmul/ascend950_fp4_mx_allgather_matmul_host.h:18-139).
// Launch: catccos_b200_fp4_mx_allgather_matmul(stream, ptrA, ptrB, customPtrs[0], customPtrs[1], ptrC, symm, &tiling, 0).
#ifndef ASCEND950_FP4_MX_ALLGATHER_MATMUL_HOST_H
#define ASCEND950_FP4_MX_ALLGATHER_MATMUL_HOST_H

#include "../../utils/operator_registry.h"

class Ascend950Fp4MxAllGatherMatmulOperator : public CatccosOperator {
public:
    static constexpr uint32_t MX_SCALE_GROUP_NUM = 32;

    void AllocateDeviceSpace(KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                             std::string dataFile) override
    {
        const size_t m = cocTiling.m, n = cocTiling.n, k = cocTiling.k;
        const size_t scaleK = (k + MX_SCALE_GROUP_NUM - 1) / MX_SCALE_GROUP_NUM;
        const std::string r = std::to_string(rankId);
        uint8_t* a = LoadOrFill(m * k / 2, dataFile, "/input_a_" + r + ".bin");
        uint8_t* b = LoadOrFill(k * n / 2, dataFile, "/input_b_" + r + ".bin");
        uint8_t* aScale = LoadOrFill(m * scaleK, dataFile, "/input_a_scale_" + r + ".bin");
        uint8_t* bScale = LoadOrFill(scaleK * n, dataFile, "/input_b_scale_" + r + ".bin");
        uint8_t* c = nullptr;
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&c), m * n * cocTiling.rankSize * sizeof(uint16_t)));
        params.SetKernelParams(a, b, c, aScale, bScale);
    }

    void WriteResultFile(const KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                         std::string dataFile) override
    {
        const size_t bytes = static_cast<size_t>(cocTiling.m) * cocTiling.rankSize * cocTiling.n * sizeof(uint16_t);
        std::vector<uint8_t> host(bytes);
        CUDA_CHECK(cudaMemcpy(host.data(), params.ptrC, bytes, cudaMemcpyDeviceToHost));
        WriteFile(dataFile + "/output_" + std::to_string(rankId) + ".bin", host.data(), bytes);
    }

    size_t GetWorkspaceSize(const CocTilingParams&) override { return 0; }

    CocCommType GetActualKernelType(const CocTilingParams&) override
    {
        return CocCommType::ASCEND950_FP4_MX_ALLGATHER_MATMUL;
    }

    size_t GetSymmetricSize(const CocTilingParams& cocTiling) override
    {
        return catccos_b200_symm_bytes_needed(reinterpret_cast<const catccos_b200_tiling_t*>(&cocTiling), 0);
    }

    bool CheckCocTilingParams(uint32_t, const CocTilingParams& cocTiling) override
    {
        // what the CUDA kernels need: whole 128-value rows for the packed TMA loads
        return cocTiling.m > 0 && cocTiling.k % 128 == 0 && cocTiling.n % 128 == 0;
    }

private:
    static uint8_t* LoadOrFill(size_t bytes, const std::string& dir, const std::string& name)
    {
        uint8_t* dev = nullptr;
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&dev), bytes));
        std::vector<uint8_t> host(bytes, 1);  // without a data directory every byte is 1, as in the reference
        if (!dir.empty()) {
            ReadFileOrThrow(dir + name, host.data(), bytes);
        }
        CUDA_CHECK(cudaMemcpy(dev, host.data(), bytes, cudaMemcpyHostToDevice));
        return dev;
    }
};

REGISTER_OPERATOR("Ascend950Fp4MxAllGatherMatmul", Ascend950Fp4MxAllGatherMatmulOperator);

#endif  // ASCEND950_FP4_MX_ALLGATHER_MATMUL_HOST_H
