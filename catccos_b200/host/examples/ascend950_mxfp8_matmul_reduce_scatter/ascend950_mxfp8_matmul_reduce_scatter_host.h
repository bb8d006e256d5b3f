// Host side of the Ascend950MxFp8MatmulReduceScatter operator on B200: the row-parallel partner of the
// AllGather-Matmul.  Every rank holds its K slice: rank_<r>_a.bin [m, k], rank_<r>_b.bin [k, n],
// rank_<r>_a_scale.bin [m, k/32], rank_<r>_b_scale.bin [k/64, n, 2]; the summed product is scattered by rows and
// every rank writes its [m / rankSize, n] chunk at its offset of one shared output.bin.  File names, pointer
// roles and the registry name follow the reference
// (examples/ascend950_mxfp8_matmul_reduce_scatter/ascend950_mxfp8_matmul_reduce_scatter_host.h:29-145); the
// operand element type is what the library options say (the reference's example feeds E5M2: "a_dtype" = "b_dtype" = 1).
// Launch: catccos_b200_mxfp8_matmul_reduce_scatter(stream, ptrA, ptrB, customPtrs[0], customPtrs[1], ptrC, symm, &tiling, 0).
#ifndef ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER_HOST_H
#define ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER_HOST_H

#include "../../utils/operator_registry.h"

class Ascend950MxFp8MatmulReduceScatterOperator : public CatccosOperator {
public:
    static constexpr uint32_t MX_SCALE_GROUP_NUM = 32;

    void AllocateDeviceSpace(KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                             std::string dataFile) override
    {
        const size_t m = cocTiling.m, n = cocTiling.n, k = cocTiling.k;
        const size_t scaleK = (k + MX_SCALE_GROUP_NUM - 1) / MX_SCALE_GROUP_NUM;
        const std::string prefix = "/rank_" + std::to_string(rankId);
        uint8_t* a = LoadOrFill(m * k, dataFile, prefix + "_a.bin");
        uint8_t* b = LoadOrFill(k * n, dataFile, prefix + "_b.bin");
        uint8_t* aScale = LoadOrFill(m * scaleK, dataFile, prefix + "_a_scale.bin");
        uint8_t* bScale = LoadOrFill(scaleK * n, dataFile, prefix + "_b_scale.bin");
        uint8_t* d = nullptr;
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&d), ChunkBytes(cocTiling)));
        params.SetKernelParams(a, b, d, aScale, bScale);
    }

    void WriteResultFile(const KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                         std::string dataFile) override
    {
        const size_t bytes = ChunkBytes(cocTiling);
        std::vector<uint8_t> host(bytes);
        CUDA_CHECK(cudaMemcpy(host.data(), params.ptrC, bytes, cudaMemcpyDeviceToHost));
        WriteFile(dataFile + "/output.bin", host.data(), bytes, rankId * bytes);  // every rank its own row chunk
    }

    size_t GetWorkspaceSize(const CocTilingParams&) override { return 0; }

    CocCommType GetActualKernelType(const CocTilingParams&) override
    {
        return CocCommType::ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER;
    }

    size_t GetSymmetricSize(const CocTilingParams& cocTiling) override
    {
        return catccos_b200_symm_bytes_needed(reinterpret_cast<const catccos_b200_tiling_t*>(&cocTiling), 2);
    }

    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams& cocTiling) override
    {
        // m is the whole M; every rank keeps m / rankSize rows of the sum
        return rankSize > 0 && cocTiling.m % rankSize == 0 && (cocTiling.m / rankSize) % 32 == 0 && cocTiling.k % 128 == 0 &&
               cocTiling.n % 16 == 0;
    }

private:
    static size_t ChunkBytes(const CocTilingParams& t)
    {
        return static_cast<size_t>(t.m) / t.rankSize * t.n * sizeof(uint16_t);
    }

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

REGISTER_OPERATOR("Ascend950MxFp8MatmulReduceScatter", Ascend950MxFp8MatmulReduceScatterOperator);

#endif  // ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER_HOST_H
