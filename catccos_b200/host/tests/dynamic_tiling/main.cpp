// Batch driver over a CSV of shapes, with the reference's command line
// (tests/dynamic_tiling/main.cpp:14-96,168-384; shape file tests/dynamic_tiling/scripts/test_shapes.csv):
//
//   dynamic_tiling kernel_name data_type rank_size rank_id ip_port m n k start_line collect_rows parent_path
//                  csv_file warm_up_times test_cycle_times [device_id_list] [data_file]
//
// kernel_name is the reference's short name ("mxqtag", "a5fp8mxagmm"), data_type the CocDataType number
// (36 = FP8E4M3FN for the quantiser, 1 = FP16 for the matmul launcher).  For every row "M,K,N,Transpose A,
// Transpose B" of the CSV (rows start_line .. start_line + collect_rows - 1 below the header) the driver
// creates the operator through the registry, validates the tiling, allocates through the operator, launches
// through KernelDispatcher (warm_up_times untimed, test_cycle_times timed) and frees everything again.
// rank 0 appends one line per shape to <parent_path>/output/tiling/tilingData_<time>.csv.
//
// What differs from the reference: the reference searches communication tilings (or asks its NPU cost model)
// and leaves the timing to an external profiler; the CUDA kernels choose their own work split, so there is
// one candidate per shape, and the driver times it itself with CUDA events and writes the average with the
// tiling.  m, n, k on the command line are accepted and unused when a CSV is given, as in the reference.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <fstream>
#include <iomanip>
#include <sstream>
#include <sys/stat.h>

#include "../../examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_host.h"
#include "../../examples/ascend950_mx_quant_allgather/mx_quant_allgather_host.h"
#include "launch_map.h"

namespace {

struct Options {
    std::string kernelName, ipPort, parentPath, csvFile, dataFile;
    CocDataType dataType = FP16;
    int rankSize = 1, rankId = 0;
    uint32_t m = 0, n = 0, k = 0, startLine = 0, collectRows = 0, warmUpTimes = 0, testCycleTimes = 0;
    std::vector<int> deviceIdList;

    // positional arguments 1..14 are required, 15 (device list) and 16 (data directory) optional
    bool Parse(int argc, char** argv)
    {
        if (argc < 15 || argc > 17) {
            return false;
        }
        kernelName = argv[1];
        dataType = static_cast<CocDataType>(std::atoi(argv[2]));
        rankSize = std::atoi(argv[3]);
        rankId = std::atoi(argv[4]);
        ipPort = argv[5];
        m = static_cast<uint32_t>(std::atoll(argv[6]));
        n = static_cast<uint32_t>(std::atoll(argv[7]));
        k = static_cast<uint32_t>(std::atoll(argv[8]));
        startLine = static_cast<uint32_t>(std::atoll(argv[9]));
        collectRows = static_cast<uint32_t>(std::atoll(argv[10]));
        parentPath = argv[11];
        csvFile = argv[12];
        warmUpTimes = static_cast<uint32_t>(std::atoll(argv[13]));
        testCycleTimes = static_cast<uint32_t>(std::atoll(argv[14]));
        if (argc > 15) {
            std::stringstream ss(argv[15]);
            std::string tok;
            while (std::getline(ss, tok, ',')) {
                deviceIdList.push_back(std::atoi(tok.c_str()));
            }
        }
        for (int r = static_cast<int>(deviceIdList.size()); r < rankSize; ++r) {
            deviceIdList.push_back(r);
        }
        if (argc > 16) {
            dataFile = argv[16];
        }
        return rankSize > 0 && rankId >= 0 && rankId < rankSize;
    }
};

struct Shape {
    uint32_t m, k, n, transA, transB;
};

// Rows of the CSV below its header line; a row whose column count differs from the header's is reported and skipped.
std::vector<Shape> ReadShapes(const Options& opt)
{
    std::vector<Shape> shapes;
    std::ifstream file(opt.csvFile);
    if (!file.is_open()) {
        std::cerr << "Unable to open file: " << opt.csvFile << std::endl;
        return shapes;
    }
    std::string line;
    if (!std::getline(file, line)) {
        std::cerr << "The file is empty or the header line fails to be read." << std::endl;
        return shapes;
    }
    const size_t columns = static_cast<size_t>(std::count(line.begin(), line.end(), ',')) + 1;
    uint32_t row = 0;
    while (std::getline(file, line) && shapes.size() < opt.collectRows) {
        if (line.empty()) {
            continue;
        }
        if (row++ < opt.startLine) {
            continue;
        }
        std::vector<uint32_t> cells;
        std::stringstream ss(line);
        std::string cell;
        while (std::getline(ss, cell, ',')) {
            cells.push_back(static_cast<uint32_t>(std::strtoul(cell.c_str(), nullptr, 10)));
        }
        if (cells.size() != columns || cells.size() < 5) {
            std::cerr << "The number of data columns in row " << (row - 1)
                      << " does not match the number of header columns: " << line << std::endl;
            continue;
        }
        shapes.push_back(Shape{cells[0], cells[1], cells[2], cells[3], cells[4]});
    }
    return shapes;
}

std::string TimeStamp()
{
    std::time_t now = std::time(nullptr);
    std::tm tm = *std::localtime(&now);
    std::stringstream ss;
    ss << std::put_time(&tm, "%Y%m%d%H%M%S");
    return ss.str();
}

void MakeDirs(const std::string& path)
{
    for (size_t pos = 1; pos <= path.size(); ++pos) {
        if (pos == path.size() || path[pos] == '/') {
            ::mkdir(path.substr(0, pos).c_str(), 0755);
        }
    }
}

}  // namespace

int main(int argc, char** argv)
{
    Options opt;
    if (!opt.Parse(argc, argv)) {
        std::cerr << "Invalid command line options" << std::endl;
        return -1;
    }
    const CocCommType commType = GetCommType(opt.kernelName);
    if (CommTypeOpNameMap.find(commType) == CommTypeOpNameMap.end()) {
        std::cerr << "[ERROR] kernel " << opt.kernelName << " is not part of this library" << std::endl;
        return -1;
    }
    const std::string opName = CommTypeOpNameMap.at(commType);
    const std::vector<Shape> shapes = ReadShapes(opt);
    std::cout << "[TEST] input rank_size: " << opt.rankSize << " rank_id: " << opt.rankId << " input_ip: " << opt.ipPort
              << "\n";

    if (set_attr(opt.rankId, opt.rankSize, 0, opt.ipPort.c_str(), opt.deviceIdList[opt.rankId]) != CATCCOS_SHMEM_SUCCESS) {
        ERROR_LOG("rendezvous failed");
        return -1;
    }
    cudaStream_t stream = nullptr;
    CUDA_CHECK(cudaStreamCreate(&stream));
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    CUDA_CHECK(cudaEventCreate(&t0));
    CUDA_CHECK(cudaEventCreate(&t1));

    const std::string tilingDir = opt.parentPath + "/output/tiling";
    const std::string tilingFile = tilingDir + "/tilingData_" + TimeStamp() + ".csv";
    if (opt.rankId == 0) {
        MakeDirs(tilingDir);
        std::ofstream out(tilingFile);
        out << "Op,M,K,N,Transpose A,Transpose B,m0,k0,n0,commTileM,commInterval,commNpuSplit,commDataSplit,commBlockM,"
               "rankSize,avg_us\n";
    }

    int rc = 0;
    for (const Shape& shape : shapes) {
        CocTilingParams tiling;
        tiling.m = shape.m;
        tiling.k = shape.k;
        tiling.n = shape.n;
        tiling.transA = shape.transA;
        tiling.transB = shape.transB;
        tiling.m0 = 128;
        tiling.k0 = 256;
        tiling.n0 = 256;
        tiling.commTileM = 64;
        tiling.commInterval = 10;
        tiling.commNpuSplit = 1;
        tiling.commDataSplit = 16;
        tiling.commBlockM = 64;
        tiling.rankSize = static_cast<uint32_t>(opt.rankSize);
        tiling.epSize = static_cast<uint32_t>(opt.rankSize);
        tiling.expertNum = 8;

        auto op = OperatorRegistry::Instance().CreateOperator(opName);
        if (!op) {
            std::cout << "Operator " << opName << " not found!" << std::endl;
            return -1;
        }
        if (!op->ValidateCocTilingParams(opt.rankSize, tiling)) {
            std::printf("M: %d, K: %d, N: %d coc params check failed!\n", tiling.m, tiling.k, tiling.n);
            continue;
        }
        const CocCommType kernelType = op->GetActualKernelType(tiling);
        KernelFuncPtr kernelFunc = KernelDispatcher::GetKernelFunc(kernelType, opt.dataType);
        if (kernelFunc == nullptr) {
            std::cerr << "[ERROR] no launcher registered for (" << opName << ", data type " << opt.dataType << ")\n";
            rc = -1;
            continue;
        }

        KernelParams kernelParams;
        op->AllocateDeviceSpace(kernelParams, tiling, opt.rankId, opt.dataFile);
        uint8_t* symm = static_cast<uint8_t*>(shmem_calloc(1, op->GetSymmetricSize(tiling)));
        if (symm == nullptr) {
            ERROR_LOG("symmetric allocation failed for M %u K %u N %u", tiling.m, tiling.k, tiling.n);
            FreeDeviceSpace(kernelParams);
            rc = -1;
            continue;
        }
        CUDA_CHECK(cudaStreamSynchronize(stream));
        for (uint32_t i = 0; i < opt.warmUpTimes; ++i) {
            kernelFunc(stream, 0, 0, kernelParams, nullptr, symm, tiling, shape.transA, shape.transB);
        }
        CUDA_CHECK(cudaStreamSynchronize(stream));
        CUDA_CHECK(cudaEventRecord(t0, stream));
        for (uint32_t i = 0; i < opt.testCycleTimes; ++i) {
            kernelFunc(stream, 0, 0, kernelParams, nullptr, symm, tiling, shape.transA, shape.transB);
        }
        CUDA_CHECK(cudaEventRecord(t1, stream));
        CUDA_CHECK(cudaStreamSynchronize(stream));
        float ms = 0.0f;
        CUDA_CHECK(cudaEventElapsedTime(&ms, t0, t1));
        const double avgUs = opt.testCycleTimes > 0 ? 1e3 * ms / opt.testCycleTimes : 0.0;
        uint32_t st[4];
        if (catccos_b200_last_status(st) != 0) {
            rc = -1;
        }
        if (!opt.dataFile.empty()) {
            op->WriteResultFile(kernelParams, tiling, opt.rankId, opt.dataFile);
        }
        if (opt.rankId == 0) {
            std::ofstream out(tilingFile, std::ios::app);
            out << opName << ',' << tiling.m << ',' << tiling.k << ',' << tiling.n << ',' << shape.transA << ','
                << shape.transB << ',' << tiling.m0 << ',' << tiling.k0 << ',' << tiling.n0 << ',' << tiling.commTileM
                << ',' << tiling.commInterval << ',' << tiling.commNpuSplit << ',' << tiling.commDataSplit << ','
                << tiling.commBlockM << ',' << tiling.rankSize << ',' << std::fixed << std::setprecision(2) << avgUs
                << '\n';
            std::printf("M: %d, K: %d, N: %d cudaStreamSynchronize success! avg %.2f us over %u launches\n", tiling.m,
                        tiling.k, tiling.n, avgUs, opt.testCycleTimes);
        }
        FreeDeviceSpace(kernelParams);
        shmem_free(symm);
    }

    std::cout << "[TEST] begin to exit...... rankId: " << opt.rankId << std::endl;
    CUDA_CHECK(cudaEventDestroy(t0));
    CUDA_CHECK(cudaEventDestroy(t1));
    CUDA_CHECK(cudaStreamDestroy(stream));
    shmem_finalize();
    return rc;
}
