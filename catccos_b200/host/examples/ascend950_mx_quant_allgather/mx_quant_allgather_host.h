// Host side of the MxQuantAllGather operator: allocates the per-rank bf16 input and the gathered
// outputs, loads / stores the reference's file names, and checks that a problem fits the symmetric buffer.
// Same class name, registry name, pointer roles (ptrA input, ptrB scales, ptrC codes) and file names as
// the reference (examples/ascend950_mx_quant_allgather/mx_quant_allgather_host.h:10-132).
#ifndef MX_QUANT_ALLGATHER_HOST_H
#define MX_QUANT_ALLGATHER_HOST_H

#include <cuda_bf16.h>

#include "../../utils/operator_registry.h"
#include "../../utils/quant_size_utils.h"

class MxQuantAllGatherOperator : public CatccosOperator {
public:
    static constexpr uint32_t MX_BLOCK_SIZE = 32;  // elements per E8M0 scale
    static constexpr uint32_t PACK_RATIO = 1;      // one byte per E4M3 code

    // the quantised axis is cocTiling.n; k is unused by this operator
    static bool CheckProblemShape(uint32_t rankSize, const CocTilingParams& t)
    {
        const bool ranksOk = rankSize > 0 && rankSize <= static_cast<uint32_t>(MAX_RANK_SIZE);
        return ranksOk && t.m > 0 && t.n > 0 && t.n % MX_BLOCK_SIZE == 0;
    }

    struct Sizes {
        size_t input, codes, scales;
    };

    static Sizes BufferSizes(const CocTilingParams& t)
    {
        Sizes s;
        s.input = CheckedBufferSize({t.m, t.n, sizeof(uint16_t)});
        s.codes = CheckedBufferSize({t.m, t.n / PACK_RATIO, t.rankSize});
        s.scales = static_cast<size_t>(t.m) * (t.n / MX_BLOCK_SIZE) * t.rankSize;  // bounded by s.codes
        return s;
    }

    void AllocateDeviceSpace(KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                             std::string dataFile) override
    {
        const Sizes sz = BufferSizes(cocTiling);
        uint8_t *input = nullptr, *codes = nullptr, *scales = nullptr;
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&input), sz.input));
        // The gathered outputs live in symmetric memory (every rank makes these two calls in the same order):
        // the peers' shards are then written into them directly instead of passing through a stage and one more
        // local copy.  FreeDeviceSpace knows both kinds of buffer.
        void *codesSymm = nullptr, *scalesSymm = nullptr;
        if (catccos_b200_symm_alloc(sz.codes, &codesSymm) != 0 || catccos_b200_symm_alloc(sz.scales, &scalesSymm) != 0) {
            ERROR_LOG("MxQuantAllGather: symmetric allocation of the outputs failed");
        }
        codes = static_cast<uint8_t*>(codesSymm);
        scales = static_cast<uint8_t*>(scalesSymm);
        std::vector<uint16_t> host(sz.input / sizeof(uint16_t));
        if (!dataFile.empty()) {
            ReadFileOrThrow(dataFile + "/rank_" + std::to_string(rankId) + "_input.bin", host.data(), sz.input);
        } else {
            // no data directory: every element is rank + 1, as the reference fills it
            const __nv_bfloat16 v = __float2bfloat16(static_cast<float>(rankId + 1));
            uint16_t bits;
            memcpy(&bits, &v, sizeof(bits));
            std::fill(host.begin(), host.end(), bits);
        }
        CUDA_CHECK(cudaMemcpy(input, host.data(), sz.input, cudaMemcpyHostToDevice));
        params.SetKernelParams(input, scales, codes);
    }

    void WriteResultFile(const KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                         std::string dataFile) override
    {
        const Sizes sz = BufferSizes(cocTiling);
        const std::string prefix = dataFile + "/rank_" + std::to_string(rankId);
        DumpDeviceBuffer(params.ptrC, sz.codes, prefix + "_output.bin");
        DumpDeviceBuffer(params.ptrB, sz.scales, prefix + "_mxscale.bin");
    }

    size_t GetWorkspaceSize(const CocTilingParams&) override { return 0; }

    CocCommType GetActualKernelType(const CocTilingParams&) override { return CocCommType::MX_QUANT_ALLGATHER; }

    // header + two stages of the gathered codes and scales
    size_t GetSymmetricSize(const CocTilingParams& cocTiling) override
    {
        return catccos_b200_symm_bytes_needed(reinterpret_cast<const catccos_b200_tiling_t*>(&cocTiling), 1);
    }

    bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams& cocTiling) override
    {
        if (!CheckProblemShape(rankSize, cocTiling)) {
            return false;
        }
        // the reference's bound: one rank's codes + scales must fit its slice of one stage of the default buffer
        const int32_t perRank = SHMEM_BUFF_BYTES / static_cast<int32_t>(rankSize) / static_cast<int32_t>(MAX_BLOCK_COUNT);
        const size_t shard = CheckedBufferSize(
            {cocTiling.m, static_cast<size_t>(cocTiling.n) + cocTiling.n / MX_BLOCK_SIZE});
        return shard < static_cast<size_t>(perRank);
    }

private:
    static void DumpDeviceBuffer(const uint8_t* device, size_t bytes, const std::string& path)
    {
        std::vector<uint8_t> host(bytes);
        CUDA_CHECK(cudaMemcpy(host.data(), device, bytes, cudaMemcpyDeviceToHost));
        WriteFile(path, host.data(), bytes);
    }
};

REGISTER_OPERATOR("MxQuantAllGather", MxQuantAllGatherOperator);

#endif  // MX_QUANT_ALLGATHER_HOST_H
