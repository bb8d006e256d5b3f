// Driver of the MxQuantAllGather operator, one process per rank, with the reference's command line
// (examples/ascend950_mx_quant_allgather/main.cpp:43-44,125-228):
//   mx_quant_allgather rank_size rank_id ip_port m n k [data_path] [device_id_list] [-p]
// -p times 5 warm-up + 50 launches and prints "[PERF] Avg latency".
#include <chrono>
#include <cstdio>
#include <sstream>

#include "mx_quant_allgather_host.h"

namespace {

struct Options {
    int rankSize = 1, rankId = 0;
    std::string ipPort, dataPath;
    uint32_t m = 0, n = 0, k = 1;
    std::vector<int> devices;
    bool perf = false;

    bool Parse(int argc, char** argv)
    {
        std::vector<std::string> pos;
        for (int i = 1; i < argc; ++i) {
            std::string a = argv[i];
            if (a == "-p") {
                perf = true;
            } else {
                pos.push_back(a);
            }
        }
        if (pos.size() < 6) {
            std::cerr << "usage: rank_size rank_id ip_port m n k [data_path] [device_id_list] [-p]\n";
            return false;
        }
        rankSize = atoi(pos[0].c_str());
        rankId = atoi(pos[1].c_str());
        ipPort = pos[2];
        m = static_cast<uint32_t>(atoll(pos[3].c_str()));
        n = static_cast<uint32_t>(atoll(pos[4].c_str()));
        k = static_cast<uint32_t>(atoll(pos[5].c_str()));
        if (pos.size() > 6) {
            dataPath = pos[6];
        }
        if (pos.size() > 7) {
            std::stringstream ss(pos[7]);
            std::string tok;
            while (std::getline(ss, tok, ',')) {
                devices.push_back(atoi(tok.c_str()));
            }
        }
        for (int r = static_cast<int>(devices.size()); r < rankSize; ++r) {
            devices.push_back(r);
        }
        return rankSize > 0 && rankId >= 0 && rankId < rankSize;
    }
};

CocTilingParams SetupTilingParams(uint32_t m, uint32_t n, uint32_t k)
{
    CocTilingParams t;
    t.m = m;
    t.n = n;
    t.k = k;
    // the communication tile fields are carried for compatibility; the CUDA kernels pick their own split
    t.m0 = 32;
    t.n0 = 256;
    t.k0 = 256;
    t.commTileM = 64;
    t.commInterval = 3;
    t.commNpuSplit = 1;
    t.commDataSplit = 20;
    t.commBlockM = 32;
    return t;
}

}  // namespace

int main(int argc, char** argv)
{
    Options opt;
    if (!opt.Parse(argc, argv)) {
        std::cerr << "Invalid arguments\n";
        return 1;
    }
    CocTilingParams tiling = SetupTilingParams(opt.m, opt.n, opt.k);
    if (!MxQuantAllGatherOperator::CheckProblemShape(opt.rankSize, tiling)) {
        std::cerr << "[ERROR] M and N must be positive, and N must be divisible by "
                  << MxQuantAllGatherOperator::MX_BLOCK_SIZE << "\n";
        return 1;
    }
    const int device = opt.devices[opt.rankId];
    if (set_attr(opt.rankId, opt.rankSize, 0, opt.ipPort.c_str(), device) != CATCCOS_SHMEM_SUCCESS) {
        ERROR_LOG("rendezvous failed");
        return -1;
    }
    cudaStream_t stream = nullptr;
    CUDA_CHECK(cudaStreamCreate(&stream));
    tiling.rankSize = opt.rankSize;
    if (tiling.k == 0) {
        tiling.k = 1;
    }
    std::cout << "[TEST] MxQuantAllGather rank_size: " << opt.rankSize << " rank_id: " << opt.rankId << " M=" << opt.m
              << " N=" << opt.n << " dtype=fp8_e4m3" << std::endl;

    auto op = OperatorRegistry::Instance().CreateOperator("MxQuantAllGather");
    if (!op) {
        std::cout << "Operator MxQuantAllGather not found!" << std::endl;
        return -1;
    }
    KernelParams params;
    op->AllocateDeviceSpace(params, tiling, opt.rankId, opt.dataPath);
    void* symm = shmem_calloc(1, op->GetSymmetricSize(tiling));
    const auto* ctiling = reinterpret_cast<const catccos_b200_tiling_t*>(&tiling);

    auto launch = [&](uint32_t magic) {
        CATCCOS_CHECK(catccos_b200_mx_quant_allgather(stream, params.ptrA, params.ptrC, params.ptrB, symm, ctiling, magic));
    };
    int rc = 0;
    if (opt.perf) {
        constexpr uint32_t kWarm = 5, kIters = 50;
        for (uint32_t i = 0; i < kWarm; ++i) launch(i);
        CUDA_CHECK(cudaStreamSynchronize(stream));
        auto t0 = std::chrono::high_resolution_clock::now();
        for (uint32_t i = 0; i < kIters; ++i) launch(i);
        CUDA_CHECK(cudaStreamSynchronize(stream));
        double us = std::chrono::duration<double, std::micro>(std::chrono::high_resolution_clock::now() - t0).count();
        if (opt.rankId == 0) {
            std::printf("[PERF] MxQuantAllGather M=%u N=%u rankSize=%d\n", opt.m, opt.n, opt.rankSize);
            std::printf("[PERF]   Avg latency: %.2f us/iter\n", us / kIters);
        }
    } else {
        for (uint32_t i = 0; i < 10; ++i) launch(i);
        CUDA_CHECK(cudaStreamSynchronize(stream));
        op->WriteResultFile(params, tiling, opt.rankId, opt.dataPath);
        std::printf("rankId %d test finished\n", opt.rankId);
    }
    uint32_t st[4];
    if (catccos_b200_last_status(st) != 0) {
        rc = -1;
    }
    shmem_free(symm);
    FreeDeviceSpace(params);
    CUDA_CHECK(cudaStreamDestroy(stream));
    shmem_finalize();
    std::cout << "[TEST] exit rankId: " << opt.rankId << std::endl;
    return rc;
}
