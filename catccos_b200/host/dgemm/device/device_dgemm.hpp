// Device launcher with the shape of the reference's DeviceDGemm<Kernel>
// (include/catccos/dgemm/device/device_dgemm.hpp:26-153): an Arguments struct, Initialize(args, workspace),
// Run(stream, blockDim, fftsAddr) returning a status and synchronising the stream, as the reference does
// (:141).  The argument names follow MxAllGatherMatmulTla::Arguments
// (include/catccos/dgemm/kernel/mx_allgather_matmul.hpp:121-135); the communication tile fields are
// accepted and ignored, blockDim and fftsAddr likewise.
#ifndef CATCCOS_B200_HOST_DEVICE_DGEMM_HPP
#define CATCCOS_B200_HOST_DEVICE_DGEMM_HPP

#include <cuda_runtime.h>

#include <cstdint>

#include "../../../../include/catccos_b200.h"

namespace Catccos::DGemm::Device {

enum class Status { kSuccess = 0, kInvalid, kErrorInternal };

struct GemmCoord {
    uint32_t m, n, k;
};

struct MatrixCoord {
    uint32_t row, column;
};

class MxAllGatherMatmulDevice {
public:
    struct Arguments {
        GemmCoord problemShape;  // per rank: m = M_local, n = N_local, k = K
        uint32_t rankIdx;
        uint32_t rankSize;
        uint32_t commInterval;
        uint8_t* ptrA;          // E4M3 [m, k]
        uint8_t* ptrB;          // E4M3 [k, n]
        uint8_t* ptrMxScaleA;   // E8M0 [m, k/32]
        uint8_t* ptrMxScaleB;   // E8M0 [k/64, n, 2]
        uint8_t* ptrC;          // 16-bit [rankSize * m, n]
        uint8_t* ptrSymmetric;  // from catccos_b200_symm_alloc
        MatrixCoord commCoreSplit{16, 2};
        MatrixCoord commBlockShape{64, 0xFFFFFFFFu};
        MatrixCoord commTileShape{32, 256};
    };

    static bool CanImplement(const Arguments& a)
    {
        return a.rankSize >= 1 && a.problemShape.m > 0 && a.problemShape.k % 128 == 0 && a.problemShape.n % 16 == 0 &&
               a.ptrSymmetric != nullptr;
    }

    Status Initialize(const Arguments& args, uint8_t* /*workspace*/ = nullptr)
    {
        if (!CanImplement(args)) {
            return Status::kInvalid;
        }
        args_ = args;
        tiling_ = {};
        tiling_.m = args.problemShape.m;
        tiling_.n = args.problemShape.n;
        tiling_.k = args.problemShape.k;
        tiling_.m0 = 128;
        tiling_.n0 = 256;
        tiling_.k0 = 256;
        tiling_.commInterval = args.commInterval;
        tiling_.rankSize = args.rankSize;
        tiling_.topK = 1;
        ready_ = true;
        return Status::kSuccess;
    }

    Status Run(cudaStream_t stream, uint32_t /*blockDim*/ = 0, uint64_t /*fftsAddr*/ = 0)
    {
        if (!ready_) {
            return Status::kInvalid;
        }
        int rc = catccos_b200_fp8_mx_allgather_matmul(stream, args_.ptrA, args_.ptrB, args_.ptrMxScaleA,
                                                      args_.ptrMxScaleB, args_.ptrC, args_.ptrSymmetric, &tiling_, 0);
        if (rc != 0 || cudaStreamSynchronize(stream) != cudaSuccess) {
            return Status::kErrorInternal;
        }
        return Status::kSuccess;
    }

private:
    Arguments args_{};
    catccos_b200_tiling_t tiling_{};
    bool ready_ = false;
};

}  // namespace Catccos::DGemm::Device

#endif  // CATCCOS_B200_HOST_DEVICE_DGEMM_HPP
