// Type composition of the AllGather-Matmul operator under the reference's names
// (examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_device.h:42-104): a driver's
// `using Config = Ascend950Fp8MxAllGatherMatmulConfig_M0_128<ElementA, LayoutA, ...>; using DeviceOp =
// Config::Device;` lines (main.cpp:16-31) keep compiling.  The reference composes CATLASS tile shapes, a block
// scheduler and remote-copy tiles here; on B200 the kernels choose their own tiling, so only the element types
// carry information: A, B E4M3 (or E5M2 through the library options), scales E8M0, C half or bf16.
#ifndef CATCCOS_B200_HOST_FP8_MX_ALLGATHER_MATMUL_DEVICE_H
#define CATCCOS_B200_HOST_FP8_MX_ALLGATHER_MATMUL_DEVICE_H

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../dgemm/device/device_dgemm.hpp"

// element tags a driver names for the 8-bit operands (one byte each in memory)
struct float8_e4m3_t {
    uint8_t bits;
};
struct float8_e5m2_t {
    uint8_t bits;
};
struct float8_e8m0_t {
    uint8_t bits;
};
using bfloat16_t = __nv_bfloat16;

template <uint32_t M0, uint32_t N0, class ElementA, class LayoutA, class ElementB, class LayoutB, class ElementMxScaleA,
          class LayoutMxScaleA, class ElementMxScaleB, class LayoutMxScaleB, class ElementC, class LayoutC>
struct Ascend950Fp8MxAllGatherMatmulConfig {
    static_assert(sizeof(ElementA) == 1 && sizeof(ElementB) == 1 && sizeof(ElementMxScaleA) == 1 && sizeof(ElementMxScaleB) == 1,
                  "A, B and their MX scales are 8-bit types");
    static_assert(sizeof(ElementC) == 2, "C is half or bf16");
    static constexpr uint32_t WORKSPACE_STAGES = 2;  // the symmetric buffer holds two stages here as well
    using Kernel = Catccos::DGemm::Kernel::MxAllGatherMatmulTla<ElementC>;
    using Device = Catccos::DGemm::Device::DeviceDGemm<Kernel>;
};

template <class ElementA, class LayoutA, class ElementB, class LayoutB, class ElementMxScaleA, class LayoutMxScaleA,
          class ElementMxScaleB, class LayoutMxScaleB, class ElementC, class LayoutC>
using Ascend950Fp8MxAllGatherMatmulConfig_M0_128 =
    Ascend950Fp8MxAllGatherMatmulConfig<128, 256, ElementA, LayoutA, ElementB, LayoutB, ElementMxScaleA, LayoutMxScaleA,
                                        ElementMxScaleB, LayoutMxScaleB, ElementC, LayoutC>;

template <class ElementA, class LayoutA, class ElementB, class LayoutB, class ElementMxScaleA, class LayoutMxScaleA,
          class ElementMxScaleB, class LayoutMxScaleB, class ElementC, class LayoutC>
using Ascend950Fp8MxAllGatherMatmulConfig_M0_256 =
    Ascend950Fp8MxAllGatherMatmulConfig<256, 128, ElementA, LayoutA, ElementB, LayoutB, ElementMxScaleA, LayoutMxScaleA,
                                        ElementMxScaleB, LayoutMxScaleB, ElementC, LayoutC>;

#endif  // CATCCOS_B200_HOST_FP8_MX_ALLGATHER_MATMUL_DEVICE_H
