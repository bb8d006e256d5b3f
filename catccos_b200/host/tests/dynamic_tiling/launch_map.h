// Function-pointer launcher table of the batch driver, as in the reference
// (tests/dynamic_tiling/include/launch_map.h:16-56): KernelFuncPtr, KernelDispatcher keyed by
// (CocCommType, CocDataType), REGISTER_KERNEL_FUNC, and the two launchers of this path
// (tests/dynamic_tiling/impl/kernel_mxfp_ascend950.cpp:20-27, impl/kernel_fp16_ascend950.cpp:261-275).
// blockNum, fftsAddr, workSpace, transA and transB are accepted and ignored.
#ifndef CATCCOS_B200_HOST_LAUNCH_MAP_H
#define CATCCOS_B200_HOST_LAUNCH_MAP_H

#include <unordered_map>

#include "../../utils/info.h"
#include "../../../../include/catccos_b200.h"

using KernelFuncPtr =
    void (*)(void*, uint32_t, uint64_t, KernelParams&, uint8_t*, uint8_t*, CocTilingParams&, uint32_t, uint32_t);

class KernelDispatcher {
public:
    static KernelFuncPtr GetKernelFunc(CocCommType commType, CocDataType dataType)
    {
        auto& table = Table();
        auto it = table.find(Key(commType, dataType));
        return it == table.end() ? nullptr : it->second;
    }

    static void RegisterKernelFunc(CocCommType commType, CocDataType dataType, KernelFuncPtr func)
    {
        Table().emplace(Key(commType, dataType), func);
    }

private:
    static int Key(CocCommType commType, CocDataType dataType) { return (static_cast<int>(commType) << 8) | dataType; }
    static std::unordered_map<int, KernelFuncPtr>& Table()
    {
        static std::unordered_map<int, KernelFuncPtr> table;
        return table;
    }
};

#define REGISTER_KERNEL_FUNC(kernelName, commType, dataType)                                                 \
    void Launch##kernelName##dataType(                                                                       \
        void*, uint32_t, uint64_t, KernelParams&, uint8_t*, uint8_t*, CocTilingParams&, uint32_t, uint32_t); \
    namespace {                                                                                              \
    struct AutoRegister##kernelName##dataType {                                                              \
        AutoRegister##kernelName##dataType()                                                                 \
        {                                                                                                    \
            KernelDispatcher::RegisterKernelFunc(commType, dataType, &Launch##kernelName##dataType);         \
        }                                                                                                    \
    } s_autoRegister##kernelName##dataType;                                                                  \
    }

REGISTER_KERNEL_FUNC(Ascend950BF16QuantAllGather, MX_QUANT_ALLGATHER, FP8E4M3FN);
REGISTER_KERNEL_FUNC(Ascend950Fp8MxAllGatherMatmul, ASCEND950_FP8_MX_ALLGATHER_MATMUL, FP16);

inline void LaunchAscend950BF16QuantAllGatherFP8E4M3FN(void* stream, uint32_t, uint64_t, KernelParams& kernelParams,
                                                      uint8_t*, uint8_t* symmetricPtr, CocTilingParams& cocTiling,
                                                      uint32_t, uint32_t)
{
    CATCCOS_CHECK(catccos_b200_mx_quant_allgather(stream, kernelParams.ptrA, kernelParams.ptrC, kernelParams.ptrB,
                                                  symmetricPtr,
                                                  reinterpret_cast<const catccos_b200_tiling_t*>(&cocTiling), 10));
}

inline void LaunchAscend950Fp8MxAllGatherMatmulFP16(void* stream, uint32_t, uint64_t, KernelParams& kernelParams,
                                                   uint8_t*, uint8_t* symmetricPtr, CocTilingParams& cocTiling, uint32_t,
                                                   uint32_t)
{
    CATCCOS_CHECK(catccos_b200_fp8_mx_allgather_matmul(
        stream, kernelParams.ptrA, kernelParams.ptrB, kernelParams.customPtrs[0], kernelParams.customPtrs[1],
        kernelParams.ptrC, symmetricPtr, reinterpret_cast<const catccos_b200_tiling_t*>(&cocTiling), 0));
}

#endif  // CATCCOS_B200_HOST_LAUNCH_MAP_H
