// Device launcher with the spelling of the reference's DeviceDGemm<Kernel>
// (include/catccos/dgemm/device/device_dgemm.hpp:25-153), so that a driver written against the reference keeps
// its `using DeviceOp = ...::DeviceDGemm<Kernel>; DeviceOp::Arguments args{...}; deviceOp.Initialize(args);
// deviceOp.Run(stream, blockNum, fftsAddr);` lines (examples/ascend950_fp8_mx_allgather_matmul/main.cpp:150-183)
// with only its include lines changed.
//
//   Catlass::Status / GemmCoord / MatrixCoord        the three CATLASS types those lines name
//   Catccos::DGemm::Kernel::MxAllGatherMatmulTla<C>  the kernel tag: Arguments in the reference's field order
//                                                    (include/catccos/dgemm/kernel/mx_allgather_matmul.hpp:121-135),
//                                                    Params, ToUnderlyingArguments, GetWorkspaceSize; C is the
//                                                    output element type (half or bf16)
//   Catccos::DGemm::Device::DeviceDGemm<Kernel>      Initialize / Run / operator() / GetWorkspaceSize / params()
//
// Run forwards to the C ABI (catccos_b200_fp8_mx_allgather_matmul) and synchronises the stream, as the reference's
// Run does (:141); blockDim and fftsAddr are accepted and ignored, the communication tile fields likewise.
#ifndef CATCCOS_B200_HOST_DEVICE_DGEMM_HPP
#define CATCCOS_B200_HOST_DEVICE_DGEMM_HPP

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <type_traits>

#include "../../../../include/catccos_b200.h"

namespace Catlass {

enum class Status { kSuccess = 0, kErrorInvalidProblem, kErrorInternal };

struct GemmCoord {
    uint32_t coord[3];
    GemmCoord(uint32_t m_ = 0, uint32_t n_ = 0, uint32_t k_ = 0) : coord{m_, n_, k_} {}
    uint32_t m() const { return coord[0]; }
    uint32_t n() const { return coord[1]; }
    uint32_t k() const { return coord[2]; }
};

struct MatrixCoord {
    uint32_t coord[2];
    MatrixCoord(uint32_t row_ = 0, uint32_t column_ = 0) : coord{row_, column_} {}
    uint32_t row() const { return coord[0]; }
    uint32_t column() const { return coord[1]; }
};

namespace layout {
struct RowMajor {};
}  // namespace layout

}  // namespace Catlass

namespace Catccos::DGemm::Kernel {

template <class ElementC_ = half>
struct MxAllGatherMatmulTla {
    using ElementC = ElementC_;

    struct Arguments {
        Catlass::GemmCoord problemShape;  // per rank: m = M_local, n = N_local, k = K
        uint32_t rankIdx;
        uint32_t rankSize;
        uint32_t commInterval;
        uint8_t* ptrA;          // E4M3 [m, k]
        uint8_t* ptrB;          // E4M3 [k, n]
        uint8_t* ptrMxScaleA;   // E8M0 [m, k/32]
        uint8_t* ptrMxScaleB;   // E8M0 [k/64, n, 2]
        uint8_t* ptrC;          // ElementC [rankSize * m, n]
        uint8_t* ptrSymmetric;  // from catccos_b200_symm_alloc (shmem_calloc in utils/shmem_init.h)
        Catlass::MatrixCoord commCoreSplit;
        Catlass::MatrixCoord commBlockShape;
        Catlass::MatrixCoord commTileShape;
    };

    struct Params {
        Arguments args{};
        catccos_b200_tiling_t tiling{};
        bool valid = false;
    };

    static bool CanImplement(const Arguments& a)
    {
        return a.rankSize >= 1 && a.problemShape.m() > 0 && a.problemShape.k() % 128 == 0 && a.problemShape.n() % 16 == 0 &&
               a.ptrSymmetric != nullptr;
    }

    static size_t GetWorkspaceSize(const Arguments&) { return 0; }

    static Params ToUnderlyingArguments(const Arguments& a, uint8_t* /*workspace*/)
    {
        Params p;
        p.args = a;
        p.tiling.m = a.problemShape.m();
        p.tiling.n = a.problemShape.n();
        p.tiling.k = a.problemShape.k();
        p.tiling.m0 = 128;
        p.tiling.n0 = 256;
        p.tiling.k0 = 256;
        p.tiling.commInterval = a.commInterval;
        p.tiling.rankSize = a.rankSize;
        p.tiling.topK = 1;
        p.valid = CanImplement(a);
        return p;
    }

    // What the reference's KernelAdapter launch stands for here: one call of the C ABI on the stream.
    static int Launch(const Params& p, cudaStream_t stream)
    {
        if (!p.valid) {
            return CATCCOS_B200_EINVAL;
        }
        int rc = catccos_b200_set_option("c_dtype", std::is_same<ElementC, half>::value ? 1 : 0);
        if (rc != 0) {
            return rc;
        }
        return catccos_b200_fp8_mx_allgather_matmul(stream, p.args.ptrA, p.args.ptrB, p.args.ptrMxScaleA, p.args.ptrMxScaleB,
                                                    p.args.ptrC, p.args.ptrSymmetric, &p.tiling, 0);
    }
};

}  // namespace Catccos::DGemm::Kernel

namespace Catccos::DGemm::Device {

template <class DGemmKernel>
class DeviceDGemm {
public:
    using Kernel = DGemmKernel;
    using Arguments = typename DGemmKernel::Arguments;
    using Params = typename DGemmKernel::Params;

    DeviceDGemm() = default;
    DeviceDGemm(const DeviceDGemm&) = delete;
    DeviceDGemm& operator=(const DeviceDGemm&) = delete;
    DeviceDGemm(DeviceDGemm&&) = default;
    DeviceDGemm& operator=(DeviceDGemm&&) = default;

    Params const& params() const { return params_; }

    static size_t GetWorkspaceSize(Arguments const& args) { return DGemmKernel::GetWorkspaceSize(args); }

    Catlass::Status Initialize(Arguments const& args, uint8_t* workspace = nullptr)
    {
        params_ = DGemmKernel::ToUnderlyingArguments(args, workspace);
        return params_.valid ? Catlass::Status::kSuccess : Catlass::Status::kErrorInvalidProblem;
    }

    Catlass::Status Run(cudaStream_t stream, uint32_t /*blockDim*/ = 0, uint64_t /*fftsAddr*/ = 0)
    {
        const int rc = DGemmKernel::Launch(params_, stream);
        if (rc != 0 || cudaStreamSynchronize(stream) != cudaSuccess) {
            return rc == CATCCOS_B200_EINVAL ? Catlass::Status::kErrorInvalidProblem : Catlass::Status::kErrorInternal;
        }
        return Catlass::Status::kSuccess;
    }

    Catlass::Status operator()(cudaStream_t stream, uint32_t blockDim = 0, uint64_t fftsAddr = 0)
    {
        return Run(stream, blockDim, fftsAddr);
    }

private:
    Params params_{};
};

}  // namespace Catccos::DGemm::Device

#endif  // CATCCOS_B200_HOST_DEVICE_DGEMM_HPP
