// Tiling / argument structs and operator ids of the host surface, layout-compatible with the
// reference (utils/info.h): CocTilingParams is the same 17 x uint32 POD (:97-115), KernelParams the
// same move-only pointer bundle (:134-193), FreeDeviceSpace the same free function (:195-214), and the
// two operators of this path keep their enumerator values (22, 24), short names and registry names
// (:68,70,237,239).  Device memory is CUDA memory; the pointer array lives in pinned host memory.
#ifndef CATCCOS_B200_HOST_INFO_H
#define CATCCOS_B200_HOST_INFO_H

#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <string>

#include "../../../include/catccos_b200.h"
#include "utils.h"

constexpr uint32_t M0 = 128;
constexpr uint32_t N0 = 256;
constexpr uint32_t K0 = 256;
constexpr uint32_t WORKSPACE_STAGES = 2;
constexpr uint32_t MAX_BLOCK_COUNT = 2;
constexpr uint32_t WARM_UP_TIMES = 10;
constexpr uint32_t PERF_TEST_CYCLE_TIMES = 3;
constexpr int32_t SHMEM_BUFF_BYTES = 1004 * 1024 * 1024;  // the reference's default symmetric buffer
constexpr uint32_t SYNC_UNIT_SIZE = 4 * sizeof(int64_t);
constexpr int32_t MAX_RANK_SIZE = 128;  // accepted by the shape checks; this build runs at most 8 ranks

// Only the operators of the MX quantise + AllGather-Matmul path and its row-parallel partner exist here; the
// numeric values of the reference enum are kept so that ids stored by callers stay valid.
enum CocCommType {
    ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER = 18,
    ASCEND950_FP8_MX_ALLGATHER_MATMUL = 22,
    ASCEND950_FP4_MX_ALLGATHER_MATMUL = 23,
    MX_QUANT_ALLGATHER = 24,
    TYPE_NUM = 45,
    UNKNOWN
};

enum CocDataType { FP16 = 1, INT8 = 2, BF16 = 27, FP8E4M3FN = 36 };

struct CocTilingParams {
    uint32_t m = 0;
    uint32_t k = 0;
    uint32_t n = 0;
    uint32_t transA = 0;
    uint32_t transB = 0;
    uint32_t m0 = 0;
    uint32_t k0 = 0;
    uint32_t n0 = 0;
    uint32_t commTileM = 0;
    uint32_t commInterval = 0;
    uint32_t commNpuSplit = 0;
    uint32_t commDataSplit = 0;
    uint32_t commBlockM = 0;
    uint32_t rankSize = 0;
    uint32_t epSize = 0;
    uint32_t expertNum = 0;
    uint32_t topK = 1;
};
static_assert(sizeof(CocTilingParams) == 17 * sizeof(uint32_t), "passed by pointer through the C ABI");

inline bool CheckCommonCocTilingParams(uint32_t rankSize, const CocTilingParams& t)
{
    const bool ranksAgree = rankSize > 0 && t.rankSize == rankSize;
    const bool shapeSet = t.m > 0 && t.k > 0 && t.n > 0;
    const bool tileSet = t.m0 > 0 && t.k0 > 0 && t.n0 > 0;
    return ranksAgree && shapeSet && tileSet;
}

struct COCMatMulInfo {
    int64_t m;
    int64_t k;
    int64_t n;
};

// Device pointers of one operator call.  Move-only: the pinned array of extra pointers belongs to it.
struct KernelParams {
    uint8_t* ptrA = nullptr;
    uint8_t* ptrB = nullptr;
    uint8_t* ptrC = nullptr;
    uint8_t** customPtrs = nullptr;
    uint32_t customCount = 0;

    KernelParams() = default;
    KernelParams(const KernelParams&) = delete;
    KernelParams& operator=(const KernelParams&) = delete;
    KernelParams& operator=(KernelParams&&) = delete;

    KernelParams(KernelParams&& o) noexcept
        : ptrA(o.ptrA), ptrB(o.ptrB), ptrC(o.ptrC), customPtrs(o.customPtrs), customCount(o.customCount)
    {
        o.ptrA = o.ptrB = o.ptrC = nullptr;
        o.customPtrs = nullptr;
        o.customCount = 0;
    }

    template <typename... Extra>
    void SetKernelParams(uint8_t* a, uint8_t* b, uint8_t* c, Extra... extra)
    {
        ptrA = a;
        ptrB = b;
        ptrC = c;
        ReleaseCustom();
        constexpr uint32_t count = sizeof...(extra);
        customCount = count;
        if constexpr (count > 0) {
            CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&customPtrs), count * sizeof(uint8_t*)));
            uint8_t* list[] = {extra...};
            for (uint32_t i = 0; i < count; ++i) {
                customPtrs[i] = list[i];
            }
        }
    }

    ~KernelParams() { ReleaseCustom(); }

private:
    void ReleaseCustom()
    {
        if (customPtrs != nullptr) {
            CUDA_CHECK(cudaFreeHost(customPtrs));
            customPtrs = nullptr;
        }
    }
};

// A buffer an operator allocated: from the symmetric heap (outputs the peers write into) or from cudaMalloc.
inline void FreeDeviceBuffer(uint8_t* p)
{
    if (p != nullptr && catccos_b200_symm_free(p) != 0) {
        CUDA_CHECK(cudaFree(p));
    }
}

inline void FreeDeviceSpace(KernelParams& params)
{
    uint8_t** main3[] = {&params.ptrA, &params.ptrB, &params.ptrC};
    for (uint8_t** p : main3) {
        FreeDeviceBuffer(*p);
        *p = nullptr;
    }
    for (uint32_t i = 0; i < params.customCount; ++i) {
        FreeDeviceBuffer(params.customPtrs[i]);
    }
}

const std::map<std::string, CocCommType> CommTypeMap = {
    {"a5mxfp8mmrs", CocCommType::ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER},
    {"a5fp8mxagmm", CocCommType::ASCEND950_FP8_MX_ALLGATHER_MATMUL},
    {"a5fp4mxagmm", CocCommType::ASCEND950_FP4_MX_ALLGATHER_MATMUL},
    {"mxqtag", CocCommType::MX_QUANT_ALLGATHER},
};

inline CocCommType GetCommType(const std::string& kernelName)
{
    auto it = CommTypeMap.find(kernelName);
    return it == CommTypeMap.end() ? CocCommType::UNKNOWN : it->second;
}

const std::map<CocCommType, std::string> CommTypeOpNameMap = {
    {ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER, "Ascend950MxFp8MatmulReduceScatter"},
    {ASCEND950_FP8_MX_ALLGATHER_MATMUL, "Ascend950Fp8MxAllGatherMatmul"},
    {ASCEND950_FP4_MX_ALLGATHER_MATMUL, "Ascend950Fp4MxAllGatherMatmul"},
    {MX_QUANT_ALLGATHER, "MxQuantAllGather"},
};

inline int32_t CeilDev(int32_t num, int32_t div) { return div == 0 ? 0 : (num + div - 1) / div; }

#endif  // CATCCOS_B200_HOST_INFO_H
