// Host side of the Ascend950Fp8MxAllGatherMatmul operator on B200: loads the reference's input files
// (input_a_<r>.bin, input_a_scale_<r>.bin, input_b_<r>.bin, input_b_scale_<r>.bin), allocates the output
// and writes output_<r>.bin.  Class name, registry name, pointer roles (ptrA/ptrB codes, ptrC output,
// customPtrs[0]/[1] the A/B scales) and the tiling check follow the reference
// (examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_host.h:18-139).
// The output element is 16 bits wide: bf16 by default, fp16 when the library option "c_dtype" is 1.
#ifndef ASCEND950_FP8_MX_ALLGATHER_MATMUL_HOST_H
#define ASCEND950_FP8_MX_ALLGATHER_MATMUL_HOST_H

#include "../../utils/operator_registry.h"

class Ascend950Fp8MxAllGatherMatmulOperator : public CatccosOperator {
public:
    static constexpr uint32_t MX_SCALE_GROUP_NUM = 32;

    void AllocateDeviceSpace(KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                             std::string dataFile) override
    {
        const size_t m = cocTiling.m, n = cocTiling.n, k = cocTiling.k;
        const size_t scaleK = (k + MX_SCALE_GROUP_NUM - 1) / MX_SCALE_GROUP_NUM;
        const std::string r = std::to_string(rankId);
        // without a data directory every byte is 1, as in the reference
        uint8_t* a = LoadOrFill(m * k, dataFile, "/input_a_" + r + ".bin");
        uint8_t* b = LoadOrFill(k * n, dataFile, "/input_b_" + r + ".bin");
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
        return CocCommType::ASCEND950_FP8_MX_ALLGATHER_MATMUL;
    }

    size_t GetSymmetricSize(const CocTilingParams& cocTiling) override
    {
        return catccos_b200_symm_bytes_needed(reinterpret_cast<const catccos_b200_tiling_t*>(&cocTiling), 0);
    }

    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams& cocTiling) override
    {
        // the reference's bound on one communication step, kept so that the same tilings are accepted
        const uint32_t kLoops = CeilDev(cocTiling.k, cocTiling.k0);
        const int32_t perRank = SHMEM_BUFF_BYTES / static_cast<int32_t>(rankSize) / static_cast<int32_t>(MAX_BLOCK_COUNT);
        const uint64_t stepBytes = static_cast<uint64_t>(cocTiling.commInterval) * cocTiling.m0 * cocTiling.k0 * kLoops;
        if (stepBytes >= static_cast<uint64_t>(perRank)) {
            return false;
        }
        // what the CUDA kernels need
        return cocTiling.k % 128 == 0 && cocTiling.n % 16 == 0;
    }

private:
    static uint8_t* LoadOrFill(size_t bytes, const std::string& dir, const std::string& name)
    {
        uint8_t* dev = nullptr;
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&dev), bytes));
        std::vector<uint8_t> host(bytes, 1);
        if (!dir.empty()) {
            ReadFileOrThrow(dir + name, host.data(), bytes);
        }
        CUDA_CHECK(cudaMemcpy(dev, host.data(), bytes, cudaMemcpyHostToDevice));
        return dev;
    }
};

REGISTER_OPERATOR("Ascend950Fp8MxAllGatherMatmul", Ascend950Fp8MxAllGatherMatmulOperator);

#endif  // ASCEND950_FP8_MX_ALLGATHER_MATMUL_HOST_H
