// C ABI of libcatccos_b200.so (declarations and reference citations: include/catccos_b200.h).
// Host logic only: rank contexts, symmetric buffers (cuMem/VMM, peer mapped), epochs, launches.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/catccos_b200.h"
#include "bootstrap.hpp"
#include "internal_options.h"
#include "common.cuh"
#include "mx_gemm.cuh"
#include "mx_gemm_pair.cuh"
#include "mx_quant.cuh"

using namespace catccos;

static_assert(sizeof(catccos_b200_tiling_t) == 17 * sizeof(uint32_t), "must match CocTilingParams");

#define ERROR_LOG(fmt, ...) fprintf(stdout, "[ERROR] " fmt "\n", ##__VA_ARGS__)

// Same shape as the reference's ACL_CHECK (utils/utils.h:28-34): print and carry the code on.
#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t err__ = (expr);                                                                 \
        if (err__ != cudaSuccess) {                                                                 \
            fprintf(stderr, "%s:%d cudaError:%d (%s)\n", __FILE__, __LINE__, (int)err__,            \
                    cudaGetErrorString(err__));                                                     \
            return CATCCOS_B200_ECUDA;                                                              \
        }                                                                                           \
    } while (0)

#define CU_TRY(expr)                                                                                \
    do {                                                                                            \
        CUresult err__ = (expr);                                                                    \
        if (err__ != CUDA_SUCCESS) {                                                                \
            fprintf(stderr, "%s:%d cudaError:%d (driver)\n", __FILE__, __LINE__, (int)err__);       \
            return CATCCOS_B200_ECUDA;                                                              \
        }                                                                                           \
    } while (0)

namespace {

// ---------------------------------------------------------------------------------------------
// driver entry points (resolved at run time so that the library links against cudart only)
// ---------------------------------------------------------------------------------------------
struct Driver {
    decltype(&cuMemCreate) MemCreate = nullptr;
    decltype(&cuMemRelease) MemRelease = nullptr;
    decltype(&cuMemExportToShareableHandle) MemExport = nullptr;
    decltype(&cuMemImportFromShareableHandle) MemImport = nullptr;
    decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
    decltype(&cuMemAddressFree) MemAddressFree = nullptr;
    decltype(&cuMemMap) MemMap = nullptr;
    decltype(&cuMemUnmap) MemUnmap = nullptr;
    decltype(&cuMemSetAccess) MemSetAccess = nullptr;
    decltype(&cuMemGetAllocationGranularity) MemGetGranularity = nullptr;
    decltype(&cuTensorMapEncodeTiled) TensorMapEncodeTiled = nullptr;
    bool ok = false;

    template <typename F>
    bool Get(const char* name, F& fn)
    {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) {
            ERROR_LOG("driver entry point %s not found", name);
            return false;
        }
        fn = reinterpret_cast<F>(p);
        return true;
    }

    bool Load()
    {
        if (ok) {
            return true;
        }
        ok = Get("cuMemCreate", MemCreate) && Get("cuMemRelease", MemRelease) &&
             Get("cuMemExportToShareableHandle", MemExport) && Get("cuMemImportFromShareableHandle", MemImport) &&
             Get("cuMemAddressReserve", MemAddressReserve) && Get("cuMemAddressFree", MemAddressFree) &&
             Get("cuMemMap", MemMap) && Get("cuMemUnmap", MemUnmap) && Get("cuMemSetAccess", MemSetAccess) &&
             Get("cuMemGetAllocationGranularity", MemGetGranularity) &&
             Get("cuTensorMapEncodeTiled", TensorMapEncodeTiled);
        return ok;
    }
};

// ---------------------------------------------------------------------------------------------
// state
// ---------------------------------------------------------------------------------------------
constexpr size_t kHeaderBytes = 1u << 20;       // counters + flag words at the start of a symmetric buffer
constexpr uint32_t kMaxFlags = 24576;           // flag words per source rank: (16-row chunks) x (K segments)
constexpr size_t kFlagsOff = 256u << 10;        // uint32 [kMaxRanks][kMaxFlags]; the first 256 KiB are reserved
static_assert(kFlagsOff + (size_t)kMaxRanks * kMaxFlags * 4 <= kHeaderBytes, "header layout");

constexpr size_t kSplitKTileBytes = 128u * 256u * 4u;  // one fp32 partial tile of the widest GEMM tile

struct RankCtx {
    int device = 0;
    int num_sms = 0;
    StatusBlock* status = nullptr;  // device memory
    // split-K scratch of this rank's GEMM launches: one fp32 partial tile and four flag words per SM, and the
    // count of split launches so far (the flags are epochs).  Launches of one rank are stream-ordered.
    uint8_t* fp4_bt = nullptr;  // the transposed copy of a packed E2M1 weight, made on every call that gets one
    size_t fp4_bt_bytes = 0;
    float* splitk_ws = nullptr;
    uint32_t* splitk_flags = nullptr;
    uint32_t splitk_epoch = 0;
    // copy-engine allgather: one stream per peer (the transfers to the peers run side by side), an event that
    // marks "this rank's shard is quantised" and one per stream that marks "everything for that peer has left"
    cudaStream_t side = nullptr;  // the quantise-and-push kernel runs here, beside the GEMM on the caller's stream
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaStream_t copy[kMaxRanks] = {};
    cudaEvent_t ev_quant = nullptr;
    cudaEvent_t ev_copy[kMaxRanks] = {};
#ifdef CATCCOS_TRACE
    unsigned long long* trace = nullptr;  // [SMs][kTraceSlots] timeline words of the armed launch
    int trace_grid = 0;
#endif
};

struct SymmAlloc {
    size_t size = 0;                       // bytes per rank
    std::vector<uint8_t*> base;            // base[r]: address of rank r's copy, valid for the acting rank's device
    std::vector<uint32_t> epoch;           // per acting rank: collectives issued on this buffer
    std::vector<bool> released;          // local mode: which ranks have fetched their pointer
    // VMM bookkeeping (one process per rank)
    bool vmm = false;
    CUdeviceptr va = 0;
    size_t va_size = 0;
    std::vector<CUmemGenericAllocationHandle> handles;
};

enum class Mode { kNone, kProcess, kLocal };

struct State {
    std::mutex mu;
    Mode mode = Mode::kNone;
    int world = 1;
    int rank = 0;  // acting rank
    std::vector<RankCtx> ranks;
    std::vector<std::unique_ptr<SymmAlloc>> allocs;
    Bootstrap boot;
    Driver drv;
    // options
    // options a caller may set (include/catccos_b200.h)
    int tiny_block_rule = 0;
    int c_dtype = 0;
    // test and tuning hooks (internal_options.h)
    int block_n = 0;
    int phase_mask = 3;
    int cta_pair = 0;        // 0 = automatic, 1 = always CTA pairs (cta_group::2), 2 = never
    int fuse_mode = -1;      // -1 = automatic, 0 = quantise warps inside the GEMM kernel, 3 = (one rank only) quantise
                             // kernel, then GEMM kernel, 4 = quantise kernel, then GEMM-and-push kernel
    int a_dtype = 0;         // element type of the A codes (what the quantiser writes, what the GEMM reads): 0 = E4M3, 1 = E5M2
    int b_dtype = 0;         // element type of the B codes the caller passes
    int split_k = 0;         // 0 = automatic, 1 = never split K, 2..8 = split K in that many parts when it fits
    int tile_order = -1;     // gated GEMM: -1 = automatic, 1 = own shard first, 0 = slice by slice over all ranks
    uint64_t timeout_ns = 2000ull * 1000000ull;
#ifdef CATCCOS_TRACE
    bool trace_armed = false;  // the next GEMM launch of the acting rank writes its timeline
#endif
    std::vector<uint32_t> local_alloc_cursor;  // local mode: next allocation index per rank
};

State g;
std::atomic<uint64_t> g_launches{0};

int setup_rank_ctx(RankCtx& rc, int device)
{
    rc.device = device;
    CUDA_TRY(cudaSetDevice(device));
    CUDA_TRY(cudaFree(nullptr));
    CUDA_TRY(cudaDeviceGetAttribute(&rc.num_sms, cudaDevAttrMultiProcessorCount, device));
    CUDA_TRY(cudaMalloc(&rc.status, sizeof(StatusBlock)));
    CUDA_TRY(cudaMemset(rc.status, 0, sizeof(StatusBlock)));
    CUDA_TRY(cudaMalloc(&rc.fp4_bt, 1u << 20));
    rc.fp4_bt_bytes = 1u << 20;
    CUDA_TRY(cudaMalloc(&rc.splitk_ws, (size_t)rc.num_sms * kSplitKTileBytes));
    CUDA_TRY(cudaMalloc(&rc.splitk_flags, (size_t)rc.num_sms * 4 * sizeof(uint32_t)));
    CUDA_TRY(cudaMemset(rc.splitk_flags, 0, (size_t)rc.num_sms * 4 * sizeof(uint32_t)));
    rc.splitk_epoch = 0;
    {
        int lo = 0, hi = 0;
        CUDA_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        CUDA_TRY(cudaStreamCreateWithPriority(&rc.side, cudaStreamNonBlocking, hi));
    }
    CUDA_TRY(cudaEventCreateWithFlags(&rc.ev_fork, cudaEventDisableTiming));
    CUDA_TRY(cudaEventCreateWithFlags(&rc.ev_join, cudaEventDisableTiming));
    CUDA_TRY(cudaEventCreateWithFlags(&rc.ev_quant, cudaEventDisableTiming));
    for (int t = 0; t < kMaxRanks; ++t) {
        CUDA_TRY(cudaStreamCreateWithFlags(&rc.copy[t], cudaStreamNonBlocking));
        CUDA_TRY(cudaEventCreateWithFlags(&rc.ev_copy[t], cudaEventDisableTiming));
    }
#ifdef CATCCOS_TRACE
    CUDA_TRY(cudaMalloc(&rc.trace, (size_t)rc.num_sms * kTraceSlots * sizeof(unsigned long long)));
    CUDA_TRY(cudaMemset(rc.trace, 0, (size_t)rc.num_sms * kTraceSlots * sizeof(unsigned long long)));
#endif
    return 0;
}

void destroy_rank_ctx(RankCtx& rc)
{
    cudaSetDevice(rc.device);
    if (rc.status) cudaFree(rc.status);
    if (rc.fp4_bt) cudaFree(rc.fp4_bt);
    if (rc.splitk_ws) cudaFree(rc.splitk_ws);
    if (rc.splitk_flags) cudaFree(rc.splitk_flags);
    if (rc.side) cudaStreamDestroy(rc.side);
    if (rc.ev_fork) cudaEventDestroy(rc.ev_fork);
    if (rc.ev_join) cudaEventDestroy(rc.ev_join);
    if (rc.ev_quant) cudaEventDestroy(rc.ev_quant);
    for (int t = 0; t < kMaxRanks; ++t) {
        if (rc.copy[t]) cudaStreamDestroy(rc.copy[t]);
        if (rc.ev_copy[t]) cudaEventDestroy(rc.ev_copy[t]);
    }
#ifdef CATCCOS_TRACE
    if (rc.trace) cudaFree(rc.trace);
#endif
    rc = RankCtx();
}

// A world of one needs no set-up call: the first operator call adopts the current device.
int ensure_init()
{
    if (g.mode != Mode::kNone) {
        return 0;
    }
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    g.world = 1;
    g.rank = 0;
    g.ranks.resize(1);
    int rc = setup_rank_ctx(g.ranks[0], dev);
    if (rc != 0) {
        return rc;
    }
    g.mode = Mode::kProcess;
    return 0;
}

RankCtx& cur() { return g.ranks[g.mode == Mode::kLocal ? g.rank : 0]; }

SymmAlloc* find_symm(const void* p)
{
    for (auto& a : g.allocs) {
        if (a && a->base[g.rank] == p) {
            return a.get();
        }
    }
    return nullptr;
}

// The symmetric allocation that holds [p, p + bytes) on the acting rank, and p's offset inside it.
SymmAlloc* find_symm_containing(const void* p, size_t bytes, size_t* offset)
{
    const uint8_t* q = static_cast<const uint8_t*>(p);
    for (auto& a : g.allocs) {
        if (a && a->base[g.rank] != nullptr && q >= a->base[g.rank] && q + bytes <= a->base[g.rank] + a->size) {
            *offset = (size_t)(q - a->base[g.rank]);
            return a.get();
        }
    }
    return nullptr;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct StageLayout {
    size_t stage_bytes, codes_off, scales_off;
};

// Two stages after the header; a stage holds the gathered codes [W*M, K] then the scales [W*M, K/32].
bool stage_layout(size_t symm_bytes, uint32_t W, uint32_t M, uint32_t K, StageLayout& L)
{
    if (symm_bytes < kHeaderBytes + 2048) {
        return false;
    }
    L.stage_bytes = ((symm_bytes - kHeaderBytes) / 2) & ~(size_t)1023;
    L.codes_off = 0;
    L.scales_off = align_up((size_t)W * M * K, 1024);
    size_t need = L.scales_off + align_up((size_t)W * M * (K / 32), 1024);
    return need <= L.stage_bytes;
}

// ---------------------------------------------------------------------------------------------
// launches
// ---------------------------------------------------------------------------------------------
int quant_grid(const RankCtx& rc)
{
    int per_sm = 0;
    const void* fn = (const void*)mx_quant_push_kernel<false>;
    // An SM keeps one shared-memory carve-out for all resident CTAs.  The GEMM needs the largest one;
    // asking for the same carve-out here lets quantise CTAs and a GEMM CTA share an SM when the two run
    // as separate kernels.
    static bool carveout_set[kMaxRanks * 2] = {};
    if (rc.device < kMaxRanks * 2 && !carveout_set[rc.device]) {
        cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        cudaGetLastError();
        carveout_set[rc.device] = true;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kQuantThreads, 0) != cudaSuccess || per_sm < 1) {
        per_sm = 1;
    }
    if (per_sm > 6) {
        per_sm = 6;
    }
    return per_sm * rc.num_sms;
}

// The ordered quantise-and-push kernel (several ranks, GEMM beside it): per_sm CTAs per SM.
int launch_quant_push_ordered(RankCtx& rc, cudaStream_t st, QuantPushParams& p, bool prequant, int per_sm);

uint32_t quant_mode(bool prequant)
{
    return prequant ? kQuantPreQuantised : (g.tiny_block_rule != 0 ? kQuantDeviceTiny : kQuantGolden);
}

uint32_t quant_sys_scope(uint32_t world) { return world > 1 ? 1u : 0u; }

constexpr uint32_t kQuantItemsPerSm = 4;  // work items per SM the quantiser's K-segment choice aims for

// max_cols (0 = none): an upper bound on the columns of a K segment.
void choose_segments(uint32_t M, uint32_t K, int num_sms, QuantPushParams& p, uint32_t max_cols = 0)
{
    const uint32_t chunks = (M + kQuantRowsPerItem - 1) / kQuantRowsPerItem;
    const uint32_t max_segs = (K + kQuantColsPerWarpStep - 1) / kQuantColsPerWarpStep;
    uint32_t want = ((uint32_t)num_sms * kQuantItemsPerSm + chunks - 1) / chunks;
    if (want < 1) want = 1;
    if (want > max_segs) want = max_segs;
    uint32_t seg_cols = (uint32_t)align_up((K + want - 1) / want, kQuantColsPerWarpStep);
    if (max_cols != 0 && seg_cols > max_cols) {
        seg_cols = max_cols;
    }
    p.seg_cols = seg_cols;
    p.segs_per_chunk = (K + seg_cols - 1) / seg_cols;
}

// max_grid (0 = no limit): an upper bound on the CTAs, for a push that has to leave in item order.
int launch_quant_push(RankCtx& rc, cudaStream_t st, QuantPushParams& p, bool prequant, bool produce,
                      bool local_only = false, int max_grid = 0)
{
    int grid = quant_grid(rc);
    if (max_grid > 0 && grid > max_grid) grid = max_grid;
    const uint32_t chunks = (p.M + kQuantRowsPerItem - 1) / kQuantRowsPerItem;
    uint32_t items = produce ? chunks * p.segs_per_chunk : 0;
    if (p.consume) {
        uint32_t peer_items = (p.world - 1) * chunks;
        if (peer_items > items) items = peer_items;
    }
    if (items == 0) {
        return 0;
    }
    if ((uint32_t)grid > items) grid = (int)items;
    p.produce = produce ? 1u : 0u;
    p.mode = quant_mode(prequant);
    p.e5m2 = g.a_dtype == 1 ? 1u : 0u;
    p.sys_scope = local_only ? quant_sys_scope(1) : quant_sys_scope(p.world);  // no peer sees these stores directly
    if (grid <= 2 * rc.num_sms && items > (uint32_t)grid) {
        mx_quant_push_kernel<true><<<grid, kQuantThreads, 0, st>>>(p);
    } else {
        mx_quant_push_kernel<false><<<grid, kQuantThreads, 0, st>>>(p);
    }
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int launch_quant_push_ordered(RankCtx& rc, cudaStream_t st, QuantPushParams& p, bool prequant, int per_sm)
{
    const uint32_t chunks = (p.M + kQuantRowsPerItem - 1) / kQuantRowsPerItem;
    const uint32_t items = chunks * p.segs_per_chunk;
    if (items == 0 || p.seg_cols > kOrderedMaxSteps * kQuantColsPerWarpStep) {
        return CATCCOS_B200_EINVAL;
    }
    static bool carveout_set[kMaxRanks * 2] = {};
    if (rc.device < kMaxRanks * 2 && !carveout_set[rc.device]) {
        // the GEMM's CTA, which needs the largest shared-memory carve-out, shares the SM with these CTAs
        cudaFuncSetAttribute((const void*)mx_quant_push_ordered_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        cudaGetLastError();
        carveout_set[rc.device] = true;
    }
    uint32_t grid = (uint32_t)(per_sm * rc.num_sms);
    if (grid > items) grid = items;
    p.produce = 1u;
    p.consume = 0u;
    p.mode = quant_mode(prequant);
    p.e5m2 = g.a_dtype == 1 ? 1u : 0u;
    p.sys_scope = 1u;
    mx_quant_push_ordered_kernel<<<grid, kQuantThreads, 0, st>>>(p);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

// Tensor maps depend on (address, extents, box) only; a decode loop calls with the same few buffers over and
// over, and an encode costs about as much as the launch it precedes.  A small most-recently-used table keeps the
// last maps (calls of one process are serialised by its callers: one host thread per rank).
struct MapKey {
    const void* base;
    uint64_t inner, outer;
    uint32_t box_inner, box_outer;
    bool fp4;
    bool operator==(const MapKey& o) const
    {
        return base == o.base && inner == o.inner && outer == o.outer && box_inner == o.box_inner &&
               box_outer == o.box_outer && fp4 == o.fp4;
    }
};
constexpr int kMapCacheSize = 16;
struct MapCache {
    MapKey key[kMapCacheSize] = {};
    CUtensorMap map[kMapCacheSize];
    uint64_t used[kMapCacheSize] = {};
    uint64_t clock = 0;
} g_maps;

int encode_map_2d_uncached(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                           uint32_t box_outer, bool fp4);

// inner / outer / box in elements; fp4: two E2M1 values per byte in global memory
int encode_map_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                  uint32_t box_outer, bool fp4 = false)
{
    const MapKey k{base, inner, outer, box_inner, box_outer, fp4};
    int victim = 0;
    for (int i = 0; i < kMapCacheSize; ++i) {
        if (g_maps.used[i] != 0 && g_maps.key[i] == k) {
            g_maps.used[i] = ++g_maps.clock;
            *map = g_maps.map[i];
            return 0;
        }
        if (g_maps.used[i] < g_maps.used[victim]) {
            victim = i;
        }
    }
    int rc = encode_map_2d_uncached(map, base, inner, outer, box_inner, box_outer, fp4);
    if (rc == 0) {
        g_maps.key[victim] = k;
        g_maps.map[victim] = *map;
        g_maps.used[victim] = ++g_maps.clock;
    }
    return rc;
}

int encode_map_2d_uncached(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                           uint32_t box_outer, bool fp4)
{
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {fp4 ? inner / 2 : inner};  // bytes: 8-bit elements, or 4-bit ones packed in pairs
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    // packed 4-bit values land in shared memory sixteen to a 16-byte chunk (8 bytes of values, 8 bytes of gap):
    // the same 128 bytes per 128 values as the 8-bit types, so boxes, swizzle and descriptors stay as they are
    const CUtensorMapDataType dt = fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CU_TRY(g.drv.TensorMapEncodeTiled(map, dt, 2, const_cast<void*>(base), dims, strides, box,
                                      estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return 0;
}

template <uint32_t BLOCK_N, typename OutT, bool FUSED>
int launch_gemm_inst(int grid, cudaStream_t st, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                     bool overlap_predecessor)
{
    auto kern = mx_gemm_kernel<BLOCK_N, OutT, FUSED>;
    static bool attr_done[kMaxRanks * 2] = {};
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < kMaxRanks * 2 && !attr_done[dev]) {
        CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)GemmSmem<BLOCK_N>::kDynamicBytes));
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(FUSED ? kGemmFusedThreads : kGemmThreads);
    cfg.dynamicSmemBytes = GemmSmem<BLOCK_N>::kDynamicBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = overlap_predecessor ? 1 : 0;
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

template <typename OutT, bool FUSED>
int launch_gemm_pair_inst(int max_pairs_hint, uint32_t tiles, cudaStream_t st, const CUtensorMap& ta,
                          const CUtensorMap& tb, const GemmParams& p, bool overlap_predecessor)
{
    auto kern = mx_gemm_pair_kernel<OutT, FUSED>;
    const int threads = FUSED ? kGemmFusedThreads : kGemmThreads;
    static bool attr_done[kMaxRanks * 2] = {};
    static int max_clusters[kMaxRanks * 2] = {};
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < kMaxRanks * 2 && !attr_done[dev]) {
        CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairSmem::kDynamicBytes));
        // how many pairs can be resident at once: the grid never exceeds it, because CTAs of one launch wait
        // on flags that the quantise warps of other CTAs of the same launch publish
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * max_pairs_hint);
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = PairSmem::kDynamicBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = max_pairs_hint;
        }
        max_clusters[dev] = n;
        attr_done[dev] = true;
    }
    uint32_t pairs = (uint32_t)(dev < kMaxRanks * 2 ? max_clusters[dev] : max_pairs_hint);
    if (pairs > (uint32_t)max_pairs_hint) pairs = (uint32_t)max_pairs_hint;
    if (pairs > tiles) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = PairSmem::kDynamicBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr;  // the cluster shape is the kernel's own (__cluster_dims__)
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = overlap_predecessor ? 1 : 0;
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

// Rough K-tile periods (microseconds) measured on B200 for the three tilings; used only to pick one.
constexpr double kPeriodPair256 = 0.43, kPeriodSingle256 = 0.47, kPeriodSingle128 = 0.32;

struct GemmPlan {
    bool use_pair;
    uint32_t block_n, ksplit;
};

// Tiling of one GEMM launch: CTA pairs or single CTAs, tile width, and the number of K parts.
GemmPlan plan_gemm(const RankCtx& rc, uint32_t Mg, uint32_t N, uint32_t K, bool no_split = false)
{
    // waves x K-tile period of each candidate (same K for all, so K drops out)
    const uint32_t m128 = (Mg + 127) / 128, m256 = (Mg + 255) / 256;
    const uint32_t n128 = (N + 127) / 128, n256 = (N + 255) / 256;
    const uint32_t sms = (uint32_t)rc.num_sms, max_pairs = sms / 2;
    auto waves = [](uint32_t tiles, uint32_t slots) { return (double)((tiles + slots - 1) / slots); };
    const double t_pair = waves(m256 * n256, max_pairs) * kPeriodPair256;
    const double t_256 = waves(m128 * n256, sms) * kPeriodSingle256;
    const double t_128 = waves(m128 * n128, sms) * kPeriodSingle128;
    GemmPlan plan;
    plan.use_pair = (g.cta_pair == 1 || (g.cta_pair == 0 && g.block_n == 0 && t_pair < t_256 && t_pair < t_128));
    plan.ksplit = 1;
    uint32_t bn = (uint32_t)g.block_n;
    // Split K when the tiles would leave at least half of the SMs idle: every (tile, K part) pair gets its
    // own CTA, the parts' partial tiles meet in this rank's scratch.  Needs the scratch (the allocation-free
    // entry point has none), an even split and at least four K tiles per part.
    if (rc.splitk_ws != nullptr && g.split_k != 1 && g.cta_pair != 1 && !no_split) {
        const uint32_t sbn = (bn == 128 || N <= 128) ? 128u : 256u;
        const uint32_t stiles = m128 * (sbn == 128 ? n128 : n256);
        const uint32_t k_tiles = K / kGemmBlockK;
        // a power of two, at most one part per 32 output columns of the tile
        const uint32_t cap_opt = g.split_k >= 2 ? (uint32_t)g.split_k : 8u;
        const uint32_t cap = std::min(std::min(sms / stiles, sbn / 32u), cap_opt);
        uint32_t s = 1;
        for (uint32_t t = 2; t <= cap; t *= 2) {
            if (k_tiles % t == 0 && k_tiles / t >= 4) {
                s = t;
            }
        }
        if (s >= 2) {
            plan.ksplit = s;
            bn = sbn;
            plan.use_pair = false;
        }
    }
    if (bn != 128 && bn != 256) {
        bn = (N > 128 && t_256 <= t_128) ? 256 : 128;
    }
    plan.block_n = bn;
    return plan;
}

// overlap_predecessor: the kernel launched just before on `st` is this library's quantise kernel, whose output
// the GEMM reads only behind grid_dep_wait(); the GEMM may then be scheduled while that kernel drains.
// epilogue: what the epilogue warps do with a finished tile (never combined with the quantise warps inside)
enum Epilogue { kEpiStore = 0,    // round to bf16 / fp16 and store C
                kEpiMxQuant = 1,  // MX-quantise the output (p.c = codes, p.c_scales)
                kEpiScatter = 2 };  // Matmul + ReduceScatter: fp32 partial rows to the stage of the rank that owns them

int launch_gemm(RankCtx& rc, cudaStream_t st, const void* a, const void* b, GemmParams& p, bool fused_quant = false,
                bool overlap_predecessor = false, Epilogue epilogue = kEpiStore)
{
    const bool mx_out = epilogue == kEpiMxQuant, scatter = epilogue == kEpiScatter;
    if (!g.drv.Load()) {
        return CATCCOS_B200_ECUDA;
    }
    if (p.Mg == 0 || p.N == 0 || p.K == 0 || p.K % kGemmBlockK != 0 || p.N % 16 != 0) {
        ERROR_LOG("mx gemm needs K %% 128 == 0 and N %% 16 == 0 (got M=%u N=%u K=%u)", p.Mg, p.N, p.K);
        return CATCCOS_B200_EINVAL;
    }
    if ((((uintptr_t)a | (uintptr_t)b) & 15u) || (!scatter && ((uintptr_t)p.c & 31u)) || ((uintptr_t)p.a_scales & 3u) ||
        ((uintptr_t)p.b_scales & 1u)) {
        ERROR_LOG("mx gemm operands must be 16-byte aligned (the output 32-byte aligned)");
        return CATCCOS_B200_EINVAL;
    }
    const bool f16 = g.c_dtype == 1;
    p.status = rc.status;
    p.timeout_ns = g.timeout_ns;
    // a barrier inside the kernel may have to wait for as long as the flag wait it depends on
    p.bar_timeout_ns = 2 * g.timeout_ns + 1000000000ull;
#ifdef CATCCOS_TRACE
    if (g.trace_armed && rc.trace != nullptr) {
        g.trace_armed = false;
        p.trace = p.q.trace = p.push.trace = rc.trace;
    }
#endif
    p.a_fmt = g.a_dtype == 2 ? 5u : (g.a_dtype == 1 ? 1u : 0u);
    p.b_fmt = g.b_dtype == 2 ? 5u : (g.b_dtype == 1 ? 1u : 0u);
    const bool a_fp4 = g.a_dtype == 2, b_fp4 = g.b_dtype == 2;
    if ((a_fp4 && (((uintptr_t)a & 31u) || p.K % 128 != 0)) || (b_fp4 && (((uintptr_t)b & 31u) || p.N % 128 != 0))) {
        ERROR_LOG("mx gemm: packed E2M1 operands must be 32-byte aligned, with K a multiple of 128 (and N, for B)");
        return CATCCOS_B200_EINVAL;
    }
    if (b_fp4) {
        // the tensor core takes 4-bit operands K-major only: transpose the weight [K, N/2] -> [N, K/2] into this
        // rank's scratch (grown on first use; a few microseconds for a weight of some megabytes)
        const size_t need = (size_t)p.N * (p.K / 2);
        if (rc.fp4_bt == nullptr) {
            return CATCCOS_B200_ESTATE;  // the allocation-free entry point has no scratch for it
        }
        if (need > rc.fp4_bt_bytes) {
            CUDA_TRY(cudaStreamSynchronize(st));
            CUDA_TRY(cudaFree(rc.fp4_bt));
            CUDA_TRY(cudaMalloc(&rc.fp4_bt, need));
            rc.fp4_bt_bytes = need;
        }
        dim3 tg((p.N + kFp4TransN - 1) / kFp4TransN, (p.K + kFp4TransK - 1) / kFp4TransK);
        fp4_transpose_kernel<<<tg, 256, 0, st>>>(static_cast<const uint8_t*>(b), rc.fp4_bt, p.K, p.N);
        g_launches++;
        CUDA_TRY(cudaGetLastError());
        b = rc.fp4_bt;
        p.b_kmajor = 1;
        overlap_predecessor = false;
    }
    GemmPlan plan = plan_gemm(rc, p.Mg, p.N, p.K);
    if (scatter && plan.ksplit > 1) {
        plan = plan_gemm(rc, p.Mg, p.N, p.K, true);  // the owner adds whole tiles: K stays in one piece
    }
    const bool use_pair = plan.use_pair;
    const uint32_t bn = plan.block_n, ksplit = plan.ksplit;
    const uint32_t m256 = (p.Mg + 255) / 256, n256 = (p.N + 255) / 256;
    const uint32_t max_pairs = (uint32_t)rc.num_sms / 2;
    if (use_pair) {
        CUtensorMap pa, pb;
        int rc2 = encode_map_2d(&pa, a, p.K, p.Mg, kGemmBlockK, 128, a_fp4);
        if (rc2 != 0) return rc2;
        rc2 = b_fp4 ? encode_map_2d(&pb, b, p.K, p.N, kGemmBlockK, 128, true)
                    : encode_map_2d(&pb, b, p.N, p.K, 128, kGemmBlockK, false);
        if (rc2 != 0) return rc2;
        const uint32_t tiles = m256 * n256;
#ifdef CATCCOS_TRACE
        rc.trace_grid = (int)(2 * std::min(tiles, max_pairs));
#endif
        if (mx_out) {
            return launch_gemm_pair_inst<MxOut, false>((int)max_pairs, tiles, st, pa, pb, p, overlap_predecessor);
        }
        if (scatter) {
            return launch_gemm_pair_inst<ScatterOut, false>((int)max_pairs, tiles, st, pa, pb, p, overlap_predecessor);
        }
        if (fused_quant) {
            return f16 ? launch_gemm_pair_inst<__half, true>((int)max_pairs, tiles, st, pa, pb, p, overlap_predecessor)
                       : launch_gemm_pair_inst<__nv_bfloat16, true>((int)max_pairs, tiles, st, pa, pb, p, overlap_predecessor);
        }
        return f16 ? launch_gemm_pair_inst<__half, false>((int)max_pairs, tiles, st, pa, pb, p, overlap_predecessor)
                   : launch_gemm_pair_inst<__nv_bfloat16, false>((int)max_pairs, tiles, st, pa, pb, p, overlap_predecessor);
    }
    CUtensorMap ta, tb;
    int rcode = encode_map_2d(&ta, a, p.K, p.Mg, kGemmBlockK, kGemmBlockM, a_fp4);
    if (rcode != 0) return rcode;
    rcode = b_fp4 ? encode_map_2d(&tb, b, p.K, p.N, kGemmBlockK, bn, true) : encode_map_2d(&tb, b, p.N, p.K, 128, kGemmBlockK, false);
    if (rcode != 0) return rcode;
    const uint32_t tiles = ((p.Mg + kGemmBlockM - 1) / kGemmBlockM) * ((p.N + bn - 1) / bn);
    int grid = (int)(tiles < (uint32_t)rc.num_sms ? tiles : (uint32_t)rc.num_sms);
    p.ksplit = ksplit;
    if (ksplit > 1) {
        grid = (int)(tiles * ksplit);  // <= SMs by construction: all units are resident at once
        p.splitk_ws = rc.splitk_ws;
        p.splitk_flags = rc.splitk_flags;
        p.splitk_epoch = ++rc.splitk_epoch;
    }
#ifdef CATCCOS_TRACE
    rc.trace_grid = grid;
#endif
#define CATCCOS_GEMM_CASE(BN)                                                                         \
    if (bn == BN) {                                                                                   \
        if (mx_out) {                                                                                 \
            return launch_gemm_inst<BN, MxOut, false>(grid, st, ta, tb, p, overlap_predecessor);      \
        }                                                                                             \
        if (scatter) {                                                                                \
            return launch_gemm_inst<BN, ScatterOut, false>(grid, st, ta, tb, p, overlap_predecessor); \
        }                                                                                             \
        if (fused_quant) {                                                                            \
            return f16 ? launch_gemm_inst<BN, __half, true>(grid, st, ta, tb, p, overlap_predecessor)         \
                       : launch_gemm_inst<BN, __nv_bfloat16, true>(grid, st, ta, tb, p, overlap_predecessor); \
        }                                                                                             \
        return f16 ? launch_gemm_inst<BN, __half, false>(grid, st, ta, tb, p, overlap_predecessor)           \
                   : launch_gemm_inst<BN, __nv_bfloat16, false>(grid, st, ta, tb, p, overlap_predecessor);   \
    }
    CATCCOS_GEMM_CASE(256)
    CATCCOS_GEMM_CASE(128)
#undef CATCCOS_GEMM_CASE
    return CATCCOS_B200_EINVAL;
}

// Sets n flag words to the epoch (the rows they stand for were put in place by stream-ordered copies).
__global__ void fill_flags_kernel(uint32_t* flags, uint32_t n, uint32_t epoch)
{
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        flags[i] = epoch;
    }
}

// Ends once every listed flag word carries the epoch (bounded): what follows on the stream may read the rows the
// peers' copy engines wrote.  One thread per word.
__global__ void wait_flags_kernel(const uint32_t* flags, uint32_t flag_stride, uint32_t world, uint32_t rank, uint32_t chunks,
                                  uint32_t segs, uint32_t epoch, uint64_t timeout_ns, StatusBlock* status)
{
    for (uint32_t i = threadIdx.x; i + 1 < world; i += blockDim.x) {
        const uint32_t src = (rank + 1 + i) % world;
        const uint32_t last_chunk = chunks - 1u;
        // the last word a peer's stream writes: everything before it on that stream has landed
        const uint32_t* f = flags + (size_t)src * flag_stride + (size_t)last_chunk * segs + (segs - 1u);
        if (!wait_flag_ge(f, epoch, timeout_ns, status)) {
            report_status(status, kStatusFlagTimeout, src, last_chunk, epoch);
        }
    }
}

constexpr uint32_t kCopySliceRows = 256;  // rows the copy engines move (and flag) at a time: one row of GEMM tiles

// AllGather of this rank's quantised shard by the copy engines.  Behind the quantise kernel on `st` (an event),
// one stream per peer copies the shard into that peer's stage: all scales first (they are small), then slice by
// slice the codes followed by the slice's flag words, which the quantise kernel has set to the epoch in this
// rank's own flag array.  Copies of one stream run in order, so a peer sees a slice's flags only after the
// slice's data; the streams of the peers run side by side and share the NVLink egress, which hides the few
// microseconds every copy costs to start.  No SM takes part: the GEMM that runs meanwhile keeps its load/store
// units to itself, and the slices arrive in the order the GEMM visits them.
int copy_engine_push(RankCtx& rc, cudaStream_t st, uint32_t W, uint32_t rank, uint32_t M, uint32_t K, uint32_t segs,
                     uint32_t slice_rows, const uint8_t* src_codes, const uint8_t* src_scales, const uint32_t* src_flags,
                     uint8_t* const* dst_codes, uint8_t* const* dst_scales, uint32_t* const* dst_flags,
                     size_t code_row_bytes = 0)
{
    const uint32_t sf = K / 32;
    const size_t row_bytes = code_row_bytes != 0 ? code_row_bytes : K;  // a row of codes: K bytes, K / 2 for packed E2M1
    CUDA_TRY(cudaEventRecord(rc.ev_quant, st));
    for (uint32_t t = 0; t + 1 < W; ++t) {
        const uint32_t d = (rank + 1 + t) % W;
        cudaStream_t cs = rc.copy[t];
        CUDA_TRY(cudaStreamWaitEvent(cs, rc.ev_quant, 0));
        CUDA_TRY(cudaMemcpyAsync(dst_scales[d], src_scales, (size_t)M * sf, cudaMemcpyDeviceToDevice, cs));
        for (uint32_t r0 = 0; r0 < M; r0 += slice_rows) {
            const uint32_t rows = std::min(slice_rows, M - r0);
            const uint32_t c0 = r0 / kRowsPerChunk, chunks = (rows + kRowsPerChunk - 1) / kRowsPerChunk;
            CUDA_TRY(cudaMemcpyAsync(dst_codes[d] + (size_t)r0 * row_bytes, src_codes + (size_t)r0 * row_bytes,
                                     (size_t)rows * row_bytes, cudaMemcpyDeviceToDevice, cs));
            CUDA_TRY(cudaMemcpyAsync(dst_flags[d] + (size_t)c0 * segs, src_flags + (size_t)c0 * segs,
                                     (size_t)chunks * segs * sizeof(uint32_t), cudaMemcpyDeviceToDevice, cs));
        }
        CUDA_TRY(cudaEventRecord(rc.ev_copy[t], cs));
    }
    return 0;
}

// The caller's stream does not run past the call before this rank's shard has left: the next call but one
// writes the same stage, and the flag words the copies read are rewritten by the very next call.
int copy_engine_join(RankCtx& rc, cudaStream_t st, uint32_t W)
{
    for (uint32_t t = 0; t + 1 < W; ++t) {
        CUDA_TRY(cudaStreamWaitEvent(st, rc.ev_copy[t], 0));
    }
    return 0;
}

// Common part of the two AllGather-Matmul entry points.
int allgather_matmul(void* stream, const void* a, const void* a_scale, bool prequant, const void* b,
                     const void* b_scale, void* c, void* symm, const catccos_b200_tiling_t* t)
{
    if (!t || !a || !b || !b_scale || !c || (prequant && !a_scale)) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    const uint32_t M = t->m, K = t->k, N = t->n, W = t->rankSize;
    if (W != (uint32_t)g.world || M == 0 || K % kGemmBlockK != 0 || N % 16 != 0) {
        ERROR_LOG("allgather matmul: rankSize %u (world %d), M=%u K=%u N=%u unsupported", W, g.world, M, K, N);
        return CATCCOS_B200_EINVAL;
    }
    SymmAlloc* sa = find_symm(symm);
    if (sa == nullptr) {
        ERROR_LOG("allgather matmul: symm must come from catccos_b200_symm_alloc");
        return CATCCOS_B200_ENOTSYMM;
    }
    RankCtx& rc = cur();
    StageLayout L;
    const uint32_t chunks = (M + kRowsPerChunk - 1) / kRowsPerChunk;
    QuantPushParams seg = {};
    // the same split on every rank and in both kernels; with several ranks a work item is at most 2048 columns wide
    // (what the ordered quantise-and-push kernel keeps in registers)
    choose_segments(M, K, rc.num_sms, seg, W > 1 ? kOrderedMaxSteps * kQuantColsPerWarpStep : 0u);
    if (!stage_layout(sa->size, W, M, K, L) || (size_t)chunks * seg.segs_per_chunk > kMaxFlags) {
        ERROR_LOG("allgather matmul: symmetric buffer of %zu bytes too small", sa->size);
        return CATCCOS_B200_ENOMEM;
    }
    CUDA_TRY(cudaSetDevice(rc.device));
    cudaStream_t st = (cudaStream_t)stream;
    const bool produce = (g.phase_mask & 1) != 0, consume = (g.phase_mask & 2) != 0;
    if (produce) {
        sa->epoch[g.rank] += 1;
    }
    const uint32_t epoch = sa->epoch[g.rank];
    const size_t stage_off = kHeaderBytes + (size_t)(epoch & 1u) * L.stage_bytes;
    const uint32_t rank = (uint32_t)g.rank;

    QuantPushParams q = {};
    q.in = a;
    q.in_scales = (const uint8_t*)a_scale;
    q.M = M;
    q.K = K;
    q.rank = rank;
    q.world = W;
    q.epoch = epoch;
    q.num_dst = W;
    q.publish = 1;
    q.segs_per_chunk = seg.segs_per_chunk;
    q.seg_cols = seg.seg_cols;
    {
        // A GEMM with more tiles than SMs runs in waves: send complete 256-row groups one after another so
        // that the first wave's rows are whole early.  A single-wave GEMM starts every tile at once and is
        // better served by one group (segment-major over all rows).
        const uint32_t tiles = ((W * M + 127) / 128) * ((N + 255) / 256);
        q.group_chunks = tiles > (uint32_t)rc.num_sms ? 256u / kRowsPerChunk : 0u;
    }
    {
        // a split-K GEMM on this rank wants the first K segment of each of its K parts first, then the second
        // of each, ... (every rank takes the same decision)
        const GemmPlan plan = plan_gemm(rc, W * M, N, K);
        const uint32_t segs = seg.segs_per_chunk;
        if (plan.ksplit > 1 && segs <= 32 && segs > 1) {
            const uint32_t kper = K / kGemmBlockK / plan.ksplit, seg_ktiles = seg.seg_cols / kGemmBlockK;
            uint32_t start[9];
            for (uint32_t a = 0; a < plan.ksplit; ++a) {
                start[a] = a * kper / seg_ktiles;
            }
            start[plan.ksplit] = segs;
            uint32_t n = 0;
            for (uint32_t round = 0; n < segs && round < segs; ++round) {
                for (uint32_t a = 0; a < plan.ksplit; ++a) {
                    const uint32_t sg = start[a] + round;
                    if (sg < start[a + 1]) {
                        q.seg_order[n++] = (uint8_t)sg;
                    }
                }
            }
            q.seg_order_n = n == segs ? n : 0u;
        }
    }
    for (uint32_t d = 0; d < W; ++d) {
        uint8_t* base = sa->base[d] + stage_off;
        q.dst_codes[d] = base + L.codes_off + (size_t)rank * M * K;
        q.dst_scales[d] = base + L.scales_off + (size_t)rank * M * (K / 32);
        q.dst_flags[d] = reinterpret_cast<uint32_t*>(sa->base[d] + kFlagsOff) + (size_t)rank * kMaxFlags;
    }
    q.status = rc.status;
    q.timeout_ns = g.timeout_ns;

    GemmParams p = {};
    {
        uint8_t* base = sa->base[rank] + stage_off;
        p.a_scales = base + L.scales_off;
        p.b_scales = (const uint8_t*)b_scale;
        p.c = c;
        p.Mg = W * M;
        p.N = N;
        p.K = K;
        p.flags = reinterpret_cast<const uint32_t*>(sa->base[rank] + kFlagsOff);
        p.flag_stride = kMaxFlags;
        p.segs = seg.segs_per_chunk;
        p.seg_ktiles = seg.seg_cols / kGemmBlockK;
        p.world = W;
        p.rank = rank;
        p.m_local = M;
        p.epoch = epoch;
    }
    const uint8_t* a_stage = sa->base[rank] + stage_off + L.codes_off;

    // With one rank there is no transfer to hide: the quantise kernel uses every SM for a few microseconds and
    // the GEMM follows it on the same stream, which measures faster than sharing the SMs between the two.
    // Several ranks: the quantise kernel stores every item to all ranks and the flag-gated GEMM follows on the
    // same stream (mode 6).  Measured at 2 and 4 ranks it is the fastest arrangement for the prefill shape and,
    // by a third, for the decode shape (one short dependency chain: quantise, store, fence, flag).
    const int auto_mode = 6;
    const int fuse_mode = W == 1 ? ((g.fuse_mode == 5 || g.fuse_mode < 0) ? 3 : g.fuse_mode)
                                 : (g.fuse_mode == 3 ? 0 : (g.fuse_mode >= 0 ? g.fuse_mode : auto_mode));
    // Tile order of the gated GEMM.  Where this rank's shard is in its own stage long before the peers' rows
    // (quantise kernel first, warps or copy engines forward it), the own shard's tiles go first.  Where the
    // quantiser stores an item to every rank before it takes the next, the own rows appear at the pace of the
    // transfer like everybody's: the tiles then follow the send groups, slice by slice over all ranks.
    p.own_first = g.tile_order >= 0 ? (uint32_t)g.tile_order : ((fuse_mode == 6 || fuse_mode == 7) ? 0u : 1u);
    if (produce && consume && fuse_mode == 3) {
        q.publish = 0;
        rcode = launch_quant_push(rc, st, q, prequant, true);
        if (rcode != 0) return rcode;
        p.flags = nullptr;  // stream order is the only dependency
        return launch_gemm(rc, st, a_stage, b, p, false, true);
    }
    if (fuse_mode == 6) {
        // Two kernels on the caller's stream.  The quantise kernel stores every work item to all ranks (one pass:
        // quantise and allgather) and flags it; the flag-gated GEMM kernel follows (with programmatic stream
        // serialisation: it may set itself up while the quantise kernel drains).  The quantise grid shrinks with
        // the number of ranks so that about the same number of bytes is on its way at any time.
        if (produce) {
            const int cap = std::max(rc.num_sms, (4 * rc.num_sms) / (int)std::max(1u, W - 1u) / rc.num_sms * rc.num_sms);
            rcode = launch_quant_push(rc, st, q, prequant, true, false, cap);
            if (rcode != 0) return rcode;
        }
        if (consume) {
            return launch_gemm(rc, st, a_stage, b, p, false, produce);
        }
        return 0;
    }
    if (fuse_mode == 7) {
        // Two kernels side by side.  The ordered quantise-and-push kernel (mx_quant.cuh), on a side stream of high
        // priority, one CTA per SM, never waits for anybody; the GEMM kernel, launched after it on the caller's
        // stream, takes one CTA per SM beside it and follows the flags, its own rows included.
        if (produce && consume) {
            CUDA_TRY(cudaEventRecord(rc.ev_fork, st));
            CUDA_TRY(cudaStreamWaitEvent(rc.side, rc.ev_fork, 0));
        }
        if (produce) {
#ifdef CATCCOS_TRACE
            if (g.trace_armed && rc.trace != nullptr) {
                q.trace = rc.trace;
            }
#endif
            rcode = launch_quant_push_ordered(rc, consume ? rc.side : st, q, prequant, 1);
            if (rcode != 0) return rcode;
            if (consume) {
                CUDA_TRY(cudaEventRecord(rc.ev_join, rc.side));
            }
        }
        if (consume) {
            rcode = launch_gemm(rc, st, a_stage, b, p);
            if (rcode != 0) return rcode;
            if (produce) {
                CUDA_TRY(cudaStreamWaitEvent(st, rc.ev_join, 0));
            }
        }
        return 0;
    }
    if (fuse_mode == 5) {
        if (produce) {
            QuantPushParams ql = q;  // the quantise kernel writes this rank's stage and its own flag words only
            for (uint32_t d = 0; d < W; ++d) {
                if (d != rank) {
                    ql.dst_codes[d] = nullptr;
                    ql.dst_scales[d] = nullptr;
                    ql.dst_flags[d] = nullptr;
                }
            }
            rcode = launch_quant_push(rc, st, ql, prequant, true, true);
            if (rcode != 0) return rcode;
            rcode = copy_engine_push(rc, st, W, rank, M, K, seg.segs_per_chunk, kCopySliceRows, q.dst_codes[rank],
                                     q.dst_scales[rank], q.dst_flags[rank], q.dst_codes, q.dst_scales, q.dst_flags);
            if (rcode != 0) return rcode;
        }
        if (consume) {
            rcode = launch_gemm(rc, st, a_stage, b, p);  // gated on the flags, own rows included
            if (rcode != 0) return rcode;
        }
        return produce ? copy_engine_join(rc, st, W) : 0;
    }
    if (produce) {
        // one GEMM launch: quantise warps fill the local stage, pusher warps forward it to the peers, the GEMM
        // warps of all ranks consume behind them.  The producer half alone (the harness that hosts several ranks
        // on one GPU runs every rank's producer before any consumer) is the same launch with the GEMM warps idle.
        p.gemm_off = consume ? 0u : 1u;
        p.q = q;
        p.q.produce = 1;
        p.q.mode = quant_mode(prequant);
        p.q.e5m2 = g.a_dtype == 1 ? 1u : 0u;
        p.q.sys_scope = 0;
        const bool quant_first = fuse_mode == 4;
        PushParams& ps = p.push;
        ps.src_codes = q.dst_codes[rank];
        ps.src_scales = q.dst_scales[rank];
        ps.src_flags = q.dst_flags[rank];
        for (uint32_t d = 0; d < W; ++d) {
            ps.dst_codes[d] = d == rank ? nullptr : q.dst_codes[d];
            ps.dst_scales[d] = d == rank ? nullptr : q.dst_scales[d];
            ps.dst_flags[d] = d == rank ? nullptr : q.dst_flags[d];
            if (d != rank) {
                p.q.dst_codes[d] = nullptr;  // the quantise warps write the local stage only
                p.q.dst_scales[d] = nullptr;
                p.q.dst_flags[d] = nullptr;
            }
        }
        ps.M = M;
        ps.K = K;
        ps.rank = rank;
        ps.world = W;
        ps.epoch = epoch;
        ps.segs_per_chunk = seg.segs_per_chunk;
        ps.seg_cols = seg.seg_cols;
        ps.group_chunks = q.group_chunks;
        ps.seg_order_n = q.seg_order_n;
        memcpy(ps.seg_order, q.seg_order, sizeof(ps.seg_order));
        ps.timeout_ns = g.timeout_ns;
        ps.status = rc.status;
        if (quant_first) {
            // the quantiser runs first, alone on every SM (48 resident warps per SM instead of the eight inside
            // the GEMM kernel) and fills the local stage (p.q names no peer any more); the GEMM-and-push kernel
            // follows on the same stream and may be scheduled while the quantiser drains
            QuantPushParams ql = p.q;
            rcode = launch_quant_push(rc, st, ql, prequant, true, true);
            if (rcode != 0) return rcode;
            p.q.produce = 0;
        }
        return launch_gemm(rc, st, a_stage, b, p, true, quant_first);
    }
    if (consume) {  // the consumer half alone: the flag-gated GEMM
        return launch_gemm(rc, st, a_stage, b, p);
    }
    return 0;
}

}  // namespace

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

int catccos_b200_init(int rank, int world, int device, const char* ip_port)
{
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.mode != Mode::kNone) {
        ERROR_LOG("catccos_b200_init: already initialised");
        return CATCCOS_B200_ESTATE;
    }
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) {
        ERROR_LOG("catccos_b200_init: rank %d of %d unsupported (at most %d ranks)", rank, world, kMaxRanks);
        return CATCCOS_B200_EINVAL;
    }
    g.world = world;
    g.rank = rank;
    g.ranks.resize(1);
    int rc = setup_rank_ctx(g.ranks[0], device);
    if (rc != 0) return rc;
    if (world > 1) {
        if (!g.drv.Load()) return CATCCOS_B200_ECUDA;
        if (!g.boot.Init(rank, world, ip_port)) {
            ERROR_LOG("catccos_b200_init: rendezvous failed: %s", g.boot.error().c_str());
            return CATCCOS_B200_ENET;
        }
    }
    g.mode = Mode::kProcess;
    return 0;
}

int catccos_b200_init_local(int world, const int* devices)
{
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.mode != Mode::kNone) {
        ERROR_LOG("catccos_b200_init_local: already initialised");
        return CATCCOS_B200_ESTATE;
    }
    if (world < 1 || world > kMaxRanks || devices == nullptr) {
        return CATCCOS_B200_EINVAL;
    }
    g.world = world;
    g.rank = 0;
    g.ranks.resize(world);
    g.local_alloc_cursor.assign(world, 0);
    for (int r = 0; r < world; ++r) {
        int rc = setup_rank_ctx(g.ranks[r], devices[r]);
        if (rc != 0) return rc;
    }
    // ranks on different GPUs reach one another's memory through peer access
    for (int r = 0; r < world; ++r) {
        for (int s = 0; s < world; ++s) {
            if (devices[r] != devices[s]) {
                cudaSetDevice(devices[r]);
                cudaError_t e = cudaDeviceEnablePeerAccess(devices[s], 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                    fprintf(stderr, "%s:%d cudaError:%d (peer access %d->%d)\n", __FILE__, __LINE__, (int)e, devices[r],
                            devices[s]);
                    return CATCCOS_B200_ECUDA;
                }
                cudaGetLastError();
            }
        }
    }
    g.mode = Mode::kLocal;
    return 0;
}

int catccos_b200_set_rank(int rank)
{
    if (g.mode != Mode::kLocal || rank < 0 || rank >= g.world) {
        return CATCCOS_B200_ESTATE;
    }
    g.rank = rank;
    CUDA_TRY(cudaSetDevice(g.ranks[rank].device));
    return 0;
}

int catccos_b200_finalize(void)
{
    std::lock_guard<std::mutex> lock(g.mu);
    if (g.mode == Mode::kNone) {
        return 0;
    }
    for (auto& rc : g.ranks) {
        cudaSetDevice(rc.device);
        cudaDeviceSynchronize();
    }
    for (auto& a : g.allocs) {
        if (!a) continue;
        if (a->vmm) {
            g.drv.MemUnmap(a->va, a->va_size);
            for (auto h : a->handles) g.drv.MemRelease(h);
            g.drv.MemAddressFree(a->va, a->va_size);
        } else if (g.mode == Mode::kLocal) {
            for (int r = 0; r < g.world; ++r) {
                cudaSetDevice(g.ranks[r].device);
                cudaFree(a->base[r]);
            }
        } else {
            cudaFree(a->base[0]);
        }
    }
    g.allocs.clear();
    for (auto& rc : g.ranks) destroy_rank_ctx(rc);
    g.ranks.clear();
    g.boot.Close();
    g.mode = Mode::kNone;
    g.world = 1;
    g.rank = 0;
    return 0;
}

int catccos_b200_symm_alloc(size_t bytes, void** local_ptr)
{
    if (local_ptr == nullptr || bytes == 0) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    std::lock_guard<std::mutex> lock(g.mu);
    const int W = g.world;
    if (g.mode == Mode::kLocal) {
        // the k-th call of every rank names the same allocation
        uint32_t idx = g.local_alloc_cursor[g.rank]++;
        uint32_t seen = 0;
        SymmAlloc* sa = nullptr;
        for (auto& a : g.allocs) {
            if (a && seen++ == idx) {
                sa = a.get();
                break;
            }
        }
        if (sa == nullptr) {
            auto na = std::make_unique<SymmAlloc>();
            na->size = align_up(bytes, 1024);
            na->base.assign(W, nullptr);
            na->epoch.assign(W, 0);
            na->released.assign(W, false);
            for (int r = 0; r < W; ++r) {
                CUDA_TRY(cudaSetDevice(g.ranks[r].device));
                CUDA_TRY(cudaMalloc(&na->base[r], na->size));
                CUDA_TRY(cudaMemset(na->base[r], 0, na->size));
            }
            for (int r = 0; r < W; ++r) {
                CUDA_TRY(cudaSetDevice(g.ranks[r].device));
                CUDA_TRY(cudaDeviceSynchronize());
            }
            CUDA_TRY(cudaSetDevice(g.ranks[g.rank].device));
            sa = na.get();
            g.allocs.push_back(std::move(na));
        } else if (sa->size < bytes) {
            ERROR_LOG("symm_alloc: ranks disagree on the size of allocation %u", idx);
            return CATCCOS_B200_EINVAL;
        }
        *local_ptr = sa->base[g.rank];
        return 0;
    }
    RankCtx& rc = g.ranks[0];
    CUDA_TRY(cudaSetDevice(rc.device));
    auto na = std::make_unique<SymmAlloc>();
    na->base.assign(W, nullptr);
    na->epoch.assign(W, 0);
    if (W == 1) {
        na->size = align_up(bytes, 1024);
        CUDA_TRY(cudaMalloc(&na->base[0], na->size));
        CUDA_TRY(cudaMemset(na->base[0], 0, na->size));
        CUDA_TRY(cudaDeviceSynchronize());
    } else {
        Driver& d = g.drv;
        CUmemAllocationProp prop = {};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = rc.device;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t gran = 0;
        CU_TRY(d.MemGetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
        na->size = align_up(bytes, gran);
        na->vmm = true;
        na->handles.assign(W, 0);
        CU_TRY(d.MemCreate(&na->handles[g.rank], na->size, &prop, 0));
        int my_fd = -1;
        CU_TRY(d.MemExport(&my_fd, na->handles[g.rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        std::vector<int> fds;
        if (!g.boot.ExchangeFds(my_fd, fds)) {
            ERROR_LOG("symm_alloc: handle exchange failed: %s", g.boot.error().c_str());
            return CATCCOS_B200_ENET;
        }
        for (int r = 0; r < W; ++r) {
            if (r != g.rank) {
                CU_TRY(d.MemImport(&na->handles[r], (void*)(uintptr_t)fds[r], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
            }
            close(fds[r]);
        }
        na->va_size = na->size * W;
        CU_TRY(d.MemAddressReserve(&na->va, na->va_size, gran, 0, 0));
        CUmemAccessDesc acc = {};
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = rc.device;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        for (int r = 0; r < W; ++r) {
            CU_TRY(d.MemMap(na->va + (size_t)r * na->size, na->size, 0, na->handles[r], 0));
            na->base[r] = reinterpret_cast<uint8_t*>(na->va + (size_t)r * na->size);
        }
        CU_TRY(d.MemSetAccess(na->va, na->va_size, &acc, 1));
        CUDA_TRY(cudaMemset(na->base[g.rank], 0, na->size));
        CUDA_TRY(cudaDeviceSynchronize());
        if (!g.boot.Barrier()) {  // nobody pushes into a buffer that is still being cleared
            return CATCCOS_B200_ENET;
        }
    }
    *local_ptr = na->base[g.rank];
    g.allocs.push_back(std::move(na));
    return 0;
}

int catccos_b200_symm_free(void* local_ptr)
{
    std::lock_guard<std::mutex> lock(g.mu);
    for (auto& a : g.allocs) {
        if (!a || a->base[g.rank] != local_ptr) {
            continue;
        }
        if (g.mode == Mode::kLocal) {
            a->released[g.rank] = true;  // freed once every rank has let go
            bool all = true;
            for (int r = 0; r < g.world; ++r) all = all && a->released[r];
            if (!all) return 0;
            for (int r = 0; r < g.world; ++r) {
                cudaSetDevice(g.ranks[r].device);
                cudaDeviceSynchronize();
                cudaFree(a->base[r]);
            }
            cudaSetDevice(g.ranks[g.rank].device);
        } else {
            CUDA_TRY(cudaDeviceSynchronize());
            if (a->vmm) {
                g.boot.Barrier();  // peers may still be storing into this rank's copy
                g.drv.MemUnmap(a->va, a->va_size);
                for (auto h : a->handles) g.drv.MemRelease(h);
                g.drv.MemAddressFree(a->va, a->va_size);
            } else {
                cudaFree(a->base[0]);
            }
        }
        a.reset();
        return 0;
    }
    return CATCCOS_B200_ENOTSYMM;
}

size_t catccos_b200_symm_bytes_needed(const catccos_b200_tiling_t* t, int quant_op)
{
    if (t == nullptr) return 0;
    const size_t W = t->rankSize ? t->rankSize : 1;
    const size_t M = t->m;
    if (quant_op == 2) {  // Matmul + ReduceScatter: two stages of the whole fp32 product (m is the whole M there)
        return kHeaderBytes + 2 * align_up(M * (size_t)t->n * sizeof(float), 1024) + 2048;
    }
    const size_t K = quant_op ? t->n : t->k;
    return kHeaderBytes + 2 * (align_up(W * M * K, 1024) + align_up(W * M * (K / 32), 1024)) + 2048;
}

int catccos_b200_mx_quant(void* stream, const void* in_bf16, uint32_t rows, uint32_t k, void* codes, void* scales)
{
    if (!in_bf16 || !codes || !scales || rows == 0 || k == 0 || k % 32 != 0) {
        return CATCCOS_B200_EINVAL;
    }
    if (((uintptr_t)in_bf16 | (uintptr_t)codes) & 15u) {
        return CATCCOS_B200_EINVAL;
    }
    if (k % 128 == 0 && ((uintptr_t)scales & 3u)) {
        return CATCCOS_B200_EINVAL;  // four scale bytes go out as one 32-bit store when a row holds a multiple of four
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    RankCtx& rc = cur();
    QuantPushParams q = {};
    q.in = in_bf16;
    q.M = rows;
    q.K = k;
    q.world = 1;
    q.num_dst = 1;
    q.dst_codes[0] = (uint8_t*)codes;
    q.dst_scales[0] = (uint8_t*)scales;
    choose_segments(rows, k, rc.num_sms, q);
    q.publish = 0;
    q.status = rc.status;
    q.timeout_ns = g.timeout_ns;
    return launch_quant_push(rc, (cudaStream_t)stream, q, false, true);
}

int catccos_b200_mx_quant_fp4(void* stream, const void* in_bf16, uint32_t rows, uint32_t k, void* packed, void* scales)
{
    if (!in_bf16 || !packed || !scales || rows == 0 || k == 0 || k % 32 != 0) {
        return CATCCOS_B200_EINVAL;
    }
    if (((uintptr_t)in_bf16 & 15u) || ((uintptr_t)packed & 7u)) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    RankCtx& rc = cur();
    const uint32_t rows_per_cta = kQuantThreads / 32;
    uint32_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
    const uint32_t cap = (uint32_t)rc.num_sms * 6u;
    if (grid > cap) grid = cap;
    mx_quant_e2m1_kernel<<<grid, kQuantThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const uint16_t*>(in_bf16), rows, k, static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scales),
        g.tiny_block_rule != 0 ? 1u : 0u);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int catccos_b200_mx_quant_allgather(void* stream, const void* in_bf16, void* out_codes, void* out_scales, void* symm,
                                    const catccos_b200_tiling_t* t, uint32_t magic)
{
    (void)magic;
    if (!t || !in_bf16 || !out_codes || !out_scales) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    const uint32_t M = t->m, K = t->n, W = t->rankSize;  // the quantised axis is called n here
    if (W != (uint32_t)g.world || M == 0 || K == 0 || K % 32 != 0) {
        ERROR_LOG("mx quant allgather: rankSize %u (world %d), M=%u N=%u: N must be a positive multiple of 32", W,
                  g.world, M, K);
        return CATCCOS_B200_EINVAL;
    }
    if (((uintptr_t)in_bf16 | (uintptr_t)out_codes) & 15u) {
        return CATCCOS_B200_EINVAL;
    }
    if (K % 128 == 0 && ((uintptr_t)out_scales & 3u)) {
        return CATCCOS_B200_EINVAL;  // scales are stored and copied as 32-bit words when a row holds a multiple of four
    }
    RankCtx& rc = cur();
    CUDA_TRY(cudaSetDevice(rc.device));
    const uint32_t rank = (uint32_t)g.rank;
    QuantPushParams q = {};
    q.in = in_bf16;
    q.M = M;
    q.K = K;
    q.rank = rank;
    q.world = W;
    q.num_dst = W;
    q.status = rc.status;
    q.timeout_ns = g.timeout_ns;
    choose_segments(M, K, rc.num_sms, q);
    uint8_t* oc = (uint8_t*)out_codes;
    uint8_t* os = (uint8_t*)out_scales;
    if (W == 1) {
        q.dst_codes[0] = oc;
        q.dst_scales[0] = os;
        return launch_quant_push(rc, (cudaStream_t)stream, q, false, true);
    }
    SymmAlloc* sa = find_symm(symm);
    if (sa == nullptr) {
        ERROR_LOG("mx quant allgather: symm must come from catccos_b200_symm_alloc");
        return CATCCOS_B200_ENOTSYMM;
    }
    StageLayout L;
    const uint32_t chunks = (M + kRowsPerChunk - 1) / kRowsPerChunk;
    if (!stage_layout(sa->size, W, M, K, L) || (size_t)chunks * q.segs_per_chunk > kMaxFlags) {
        ERROR_LOG("mx quant allgather: symmetric buffer of %zu bytes too small", sa->size);
        return CATCCOS_B200_ENOMEM;
    }
    const bool produce = (g.phase_mask & 1) != 0, consume = (g.phase_mask & 2) != 0;
    if (produce) {
        sa->epoch[g.rank] += 1;
    }
    const uint32_t epoch = sa->epoch[g.rank];
    const size_t stage_off = kHeaderBytes + (size_t)(epoch & 1u) * L.stage_bytes;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* my_flags = reinterpret_cast<uint32_t*>(sa->base[rank] + kFlagsOff);
    // Outputs that live in symmetric memory (the same offset on every rank) receive the peers' shards directly;
    // other outputs receive them through this rank's stage and one more local copy.
    size_t off_c = 0, off_s = 0;
    SymmAlloc* sc = find_symm_containing(oc, (size_t)W * M * K, &off_c);
    SymmAlloc* ss = find_symm_containing(os, (size_t)W * M * (K / 32), &off_s);
    const bool direct = sc != nullptr && ss != nullptr;
    // the quantise kernel writes this rank's shard into the caller's output and sets this rank's own flag words
    q.epoch = epoch;
    q.publish = 1;
    q.dst_codes[rank] = oc + (size_t)rank * M * K;
    q.dst_scales[rank] = os + (size_t)rank * M * (K / 32);
    q.dst_flags[rank] = my_flags + (size_t)rank * kMaxFlags;
    if (produce) {
        rcode = launch_quant_push(rc, st, q, false, true, true);
        if (rcode != 0) return rcode;
        // the copy engines forward it, slice by slice, to every peer: into the peer's output or its stage
        uint8_t* dc[kMaxRanks] = {};
        uint8_t* ds[kMaxRanks] = {};
        uint32_t* df[kMaxRanks] = {};
        for (uint32_t d = 0; d < W; ++d) {
            if (d == rank) continue;
            uint8_t* base = sa->base[d] + stage_off;
            dc[d] = (direct ? sc->base[d] + off_c : base + L.codes_off) + (size_t)rank * M * K;
            ds[d] = (direct ? ss->base[d] + off_s : base + L.scales_off) + (size_t)rank * M * (K / 32);
            df[d] = reinterpret_cast<uint32_t*>(sa->base[d] + kFlagsOff) + (size_t)rank * kMaxFlags;
        }
        // nobody consumes this operator's rows early: one slice per peer (three copies: scales, codes, flags)
        // keeps the copies long and their fixed start-up cost small
        const uint32_t slice_rows = (uint32_t)align_up(M, kRowsPerChunk);
        rcode = copy_engine_push(rc, st, W, rank, M, K, q.segs_per_chunk, slice_rows, q.dst_codes[rank], q.dst_scales[rank],
                                 q.dst_flags[rank], dc, ds, df);
        if (rcode != 0) return rcode;
    }
    if (consume) {
        if (direct) {
            wait_flags_kernel<<<1, 128, 0, st>>>(my_flags, kMaxFlags, W, rank, chunks, q.segs_per_chunk, epoch, g.timeout_ns,
                                                 rc.status);
            g_launches++;
            CUDA_TRY(cudaGetLastError());
        } else {
            QuantPushParams qc = q;
            qc.consume = 1;
            qc.stage_codes = sa->base[rank] + stage_off + L.codes_off;
            qc.stage_scales = sa->base[rank] + stage_off + L.scales_off;
            qc.out_codes = oc;
            qc.out_scales = os;
            qc.flags = my_flags;
            qc.flag_stride = kMaxFlags;
            rcode = launch_quant_push(rc, st, qc, false, false);
            if (rcode != 0) return rcode;
        }
    }
    return produce ? copy_engine_join(rc, st, W) : 0;
}

int catccos_b200_fp8_mx_allgather_matmul(void* stream, const void* a, const void* b, const void* a_scale,
                                         const void* b_scale, void* c, void* symm, const catccos_b200_tiling_t* t,
                                         uint32_t magic)
{
    (void)magic;
    return allgather_matmul(stream, a, a_scale, true, b, b_scale, c, symm, t);
}

int catccos_b200_fp4_mx_allgather_matmul(void* stream, const void* a, const void* b, const void* a_scale,
                                         const void* b_scale, void* c, void* symm, const catccos_b200_tiling_t* t,
                                         uint32_t magic)
{
    (void)magic;
    if (!t || !a || !b || !a_scale || !b_scale || !c) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    const uint32_t M = t->m, K = t->k, N = t->n, W = t->rankSize;
    if (W != (uint32_t)g.world || M == 0 || K % kGemmBlockK != 0 || N % 16 != 0) {
        ERROR_LOG("fp4 allgather matmul: rankSize %u (world %d), M=%u K=%u N=%u unsupported", W, g.world, M, K, N);
        return CATCCOS_B200_EINVAL;
    }
    RankCtx& rc = cur();
    CUDA_TRY(cudaSetDevice(rc.device));
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t rank = (uint32_t)g.rank;
    // both operands are packed E2M1 for the length of this call, whatever the options say
    struct DtypeGuard {
        int a, b;
        DtypeGuard() : a(g.a_dtype), b(g.b_dtype) { g.a_dtype = 2; g.b_dtype = 2; }
        ~DtypeGuard() { g.a_dtype = a; g.b_dtype = b; }
    } guard;
    GemmParams p = {};
    p.a_scales = (const uint8_t*)a_scale;
    p.b_scales = (const uint8_t*)b_scale;
    p.c = c;
    p.Mg = W * M;
    p.N = N;
    p.K = K;
    p.world = W;
    p.rank = rank;
    p.m_local = M;
    if (W == 1) {
        return launch_gemm(rc, st, a, b, p);
    }
    SymmAlloc* sa = find_symm(symm);
    if (sa == nullptr) {
        ERROR_LOG("fp4 allgather matmul: symm must come from catccos_b200_symm_alloc");
        return CATCCOS_B200_ENOTSYMM;
    }
    // a stage: the gathered packed codes [W * M, K / 2], then the gathered scales [W * M, K / 32]
    const size_t row_bytes = K / 2, sf = K / 32;
    const size_t stage_bytes = ((sa->size - kHeaderBytes) / 2) & ~(size_t)1023;
    const size_t scales_off = align_up((size_t)W * M * row_bytes, 1024);
    const uint32_t chunks = (M + kRowsPerChunk - 1) / kRowsPerChunk;
    if (sa->size < kHeaderBytes + 2048 || scales_off + align_up((size_t)W * M * sf, 1024) > stage_bytes || chunks > kMaxFlags) {
        ERROR_LOG("fp4 allgather matmul: symmetric buffer of %zu bytes too small", sa->size);
        return CATCCOS_B200_ENOMEM;
    }
    const bool produce = (g.phase_mask & 1) != 0, consume = (g.phase_mask & 2) != 0;
    if (produce) {
        sa->epoch[g.rank] += 1;
    }
    const uint32_t epoch = sa->epoch[g.rank];
    const size_t stage_off = kHeaderBytes + (size_t)(epoch & 1u) * stage_bytes;
    uint8_t* dc[kMaxRanks] = {};
    uint8_t* ds[kMaxRanks] = {};
    uint32_t* df[kMaxRanks] = {};
    for (uint32_t d = 0; d < W; ++d) {
        uint8_t* base = sa->base[d] + stage_off;
        dc[d] = base + (size_t)rank * M * row_bytes;
        ds[d] = base + scales_off + (size_t)rank * M * sf;
        df[d] = reinterpret_cast<uint32_t*>(sa->base[d] + kFlagsOff) + (size_t)rank * kMaxFlags;
    }
    if (produce) {
        // A arrives quantised: this rank's shard goes into its own stage by two copies, its flag words are set,
        // and the copy engines forward all three to the peers (one flag word per 16-row chunk, one K segment)
        CUDA_TRY(cudaMemcpyAsync(dc[rank], a, (size_t)M * row_bytes, cudaMemcpyDeviceToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(ds[rank], a_scale, (size_t)M * sf, cudaMemcpyDeviceToDevice, st));
        fill_flags_kernel<<<(chunks + 255) / 256, 256, 0, st>>>(df[rank], chunks, epoch);
        g_launches++;
        CUDA_TRY(cudaGetLastError());
        rcode = copy_engine_push(rc, st, W, rank, M, K, 1, kCopySliceRows, dc[rank], ds[rank], df[rank], dc, ds, df, row_bytes);
        if (rcode != 0) return rcode;
    }
    if (consume) {
        p.a_scales = sa->base[rank] + stage_off + scales_off;
        p.flags = reinterpret_cast<const uint32_t*>(sa->base[rank] + kFlagsOff);
        p.flag_stride = kMaxFlags;
        p.segs = 1;
        p.seg_ktiles = K / kGemmBlockK;
        p.epoch = epoch;
        rcode = launch_gemm(rc, st, sa->base[rank] + stage_off, b, p);
        if (rcode != 0) return rcode;
    }
    return produce ? copy_engine_join(rc, st, W) : 0;
}

int catccos_b200_mx_quant_allgather_matmul(void* stream, const void* a_bf16, const void* b, const void* b_scale,
                                           void* c, void* symm, const catccos_b200_tiling_t* t, uint32_t magic)
{
    (void)magic;
    return allgather_matmul(stream, a_bf16, nullptr, false, b, b_scale, c, symm, t);
}

int catccos_b200_mx_gemm(void* stream, const void* a, const void* a_scale, const void* b, const void* b_scale, void* c,
                         uint32_t m, uint32_t n, uint32_t k)
{
    if (!a || !a_scale || !b || !b_scale || !c) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    RankCtx& rc = cur();
    GemmParams p = {};
    p.a_scales = (const uint8_t*)a_scale;
    p.b_scales = (const uint8_t*)b_scale;
    p.c = c;
    p.Mg = m;
    p.N = n;
    p.K = k;
    p.flags = nullptr;
    p.world = 1;
    p.m_local = m;
    return launch_gemm(rc, (cudaStream_t)stream, a, b, p);
}

int catccos_b200_mx_gemm_quant_out(void* stream, const void* a, const void* a_scale, const void* b, const void* b_scale,
                                   void* c_codes, void* c_scales, uint32_t m, uint32_t n, uint32_t k)
{
    if (!a || !a_scale || !b || !b_scale || !c_codes || !c_scales) {
        return CATCCOS_B200_EINVAL;
    }
    if (n % 32 != 0) {
        ERROR_LOG("mx gemm with quantised output: n must be a multiple of 32 (got %u)", n);
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    RankCtx& rc = cur();
    GemmParams p = {};
    p.a_scales = (const uint8_t*)a_scale;
    p.b_scales = (const uint8_t*)b_scale;
    p.c = c_codes;
    p.c_scales = (uint8_t*)c_scales;
    p.c_tiny_rule = g.tiny_block_rule != 0 ? kQuantDeviceTiny : kQuantGolden;
    p.Mg = m;
    p.N = n;
    p.K = k;
    p.flags = nullptr;
    p.world = 1;
    p.m_local = m;
    return launch_gemm(rc, (cudaStream_t)stream, a, b, p, false, false, kEpiMxQuant);
}

// Matmul + ReduceScatter: what plan_gemm will choose for the N tile (the reducer walks the same tiles)
static uint32_t scatter_block_n(const RankCtx& rc, uint32_t M, uint32_t N, uint32_t K)
{
    GemmPlan plan = plan_gemm(rc, M, N, K);
    if (plan.ksplit > 1) {
        plan = plan_gemm(rc, M, N, K, true);
    }
    return plan.use_pair ? kPairBlockN : plan.block_n;
}

int catccos_b200_mxfp8_matmul_reduce_scatter(void* stream, const void* a, const void* b, const void* a_scale,
                                             const void* b_scale, void* d, void* symm, const catccos_b200_tiling_t* t,
                                             uint32_t magic)
{
    (void)magic;
    if (!t || !a || !b || !a_scale || !b_scale || !d) {
        return CATCCOS_B200_EINVAL;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    const uint32_t M = t->m, K = t->k, N = t->n, W = t->rankSize;  // m is the whole M: every rank holds all rows of its K slice
    if (W != (uint32_t)g.world || M == 0 || K % kGemmBlockK != 0 || N % 16 != 0 || M % W != 0 || (M / W) % 32 != 0) {
        ERROR_LOG("matmul reduce scatter: rankSize %u (world %d), M=%u K=%u N=%u unsupported (M / rankSize must be a "
                  "multiple of 32, K of 128, N of 16)", W, g.world, M, K, N);
        return CATCCOS_B200_EINVAL;
    }
    RankCtx& rc = cur();
    CUDA_TRY(cudaSetDevice(rc.device));
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t rank = (uint32_t)g.rank, rows = M / W;
    const bool produce = (g.phase_mask & 1) != 0, consume = (g.phase_mask & 2) != 0;
    if (W == 1) {
        // nothing to reduce: the plain GEMM writes D
        GemmParams p = {};
        p.a_scales = (const uint8_t*)a_scale;
        p.b_scales = (const uint8_t*)b_scale;
        p.c = d;
        p.Mg = M;
        p.N = N;
        p.K = K;
        p.world = 1;
        p.m_local = M;
        return launch_gemm(rc, st, a, b, p);
    }
    SymmAlloc* sa = find_symm(symm);
    if (sa == nullptr) {
        ERROR_LOG("matmul reduce scatter: symm must come from catccos_b200_symm_alloc");
        return CATCCOS_B200_ENOTSYMM;
    }
    const uint32_t bn = scatter_block_n(rc, M, N, K);
    const uint32_t n_tiles = (N + bn - 1) / bn;
    const size_t stage_bytes = ((sa->size - kHeaderBytes) / 2) & ~(size_t)1023;
    const size_t need = (size_t)M * N * sizeof(float);  // world slots of [rows, N] fp32
    if (sa->size < kHeaderBytes + 2048 || need > stage_bytes || (size_t)(rows / 32) * n_tiles > kMaxFlags) {
        ERROR_LOG("matmul reduce scatter: symmetric buffer of %zu bytes too small (needs %zu)", sa->size,
                  kHeaderBytes + 2 * need + 2048);
        return CATCCOS_B200_ENOMEM;
    }
    if (produce) {
        sa->epoch[g.rank] += 1;
    }
    const uint32_t epoch = sa->epoch[g.rank];
    const size_t stage_off = kHeaderBytes + (size_t)(epoch & 1u) * stage_bytes;
    if (produce) {
        GemmParams p = {};
        p.a_scales = (const uint8_t*)a_scale;
        p.b_scales = (const uint8_t*)b_scale;
        p.c = nullptr;
        p.Mg = M;
        p.N = N;
        p.K = K;
        p.world = W;
        p.rank = rank;
        p.m_local = M;
        p.epoch = epoch;
        p.rs_rows = rows;
        for (uint32_t dr = 0; dr < W; ++dr) {
            p.rs_dst[dr] = reinterpret_cast<float*>(sa->base[dr] + stage_off);
            p.rs_flags[dr] = reinterpret_cast<uint32_t*>(sa->base[dr] + kFlagsOff) + (size_t)rank * kMaxFlags;
        }
        rcode = launch_gemm(rc, st, a, b, p, false, false, kEpiScatter);
        if (rcode != 0) return rcode;
    }
    if (consume) {
        const uint32_t units = (rows / 32) * n_tiles;
        const uint32_t grid = std::min(units, (uint32_t)rc.num_sms * 4u);
        const float* parts = reinterpret_cast<const float*>(sa->base[rank] + stage_off);
        const uint32_t* flags = reinterpret_cast<const uint32_t*>(sa->base[rank] + kFlagsOff);
        if (g.c_dtype == 1) {
            mx_reduce_scatter_kernel<__half><<<grid, 256, 0, st>>>(parts, flags, kMaxFlags, W, rows, N, bn, epoch, (__half*)d,
                                                                   g.timeout_ns, rc.status);
        } else {
            mx_reduce_scatter_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(parts, flags, kMaxFlags, W, rows, N, bn, epoch,
                                                                          (__nv_bfloat16*)d, g.timeout_ns, rc.status);
        }
        g_launches++;
        CUDA_TRY(cudaGetLastError());
    }
    return 0;
}

size_t catccos_b200_packed_row_bytes(uint32_t n) { return packed_row_bytes(n); }

int catccos_b200_mx_quant_scatter_packed(void* stream, const void* in_bf16, const int32_t* expanded_row_idx, void* packed_out,
                                         uint32_t tokens, uint32_t n, uint32_t top_k)
{
    if (!in_bf16 || !expanded_row_idx || !packed_out || n == 0 || n % 32 != 0 || top_k == 0) {
        return CATCCOS_B200_EINVAL;
    }
    if ((((uintptr_t)in_bf16 | (uintptr_t)packed_out) & 15u) != 0) {
        return CATCCOS_B200_EINVAL;  // rows are read and written 16 bytes at a time
    }
    if (tokens == 0) {
        return 0;
    }
    int rcode = ensure_init();
    if (rcode != 0) return rcode;
    RankCtx& rc = cur();
    const uint32_t per_cta = kQuantThreads / 32;
    uint32_t grid = (tokens + per_cta - 1) / per_cta;
    grid = std::min(grid, (uint32_t)rc.num_sms * 6u);
    mx_quant_scatter_packed_kernel<<<grid, kQuantThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const uint16_t*>(in_bf16), expanded_row_idx, static_cast<uint8_t*>(packed_out), tokens, n, top_k,
        g.tiny_block_rule != 0 ? 1u : 0u);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int catccos_b200_last_status(uint32_t out[4])
{
    if (out == nullptr || g.mode == Mode::kNone) {
        return CATCCOS_B200_ESTATE;
    }
    RankCtx& rc = cur();
    CUDA_TRY(cudaSetDevice(rc.device));
    CUDA_TRY(cudaDeviceSynchronize());
    StatusBlock sb;
    CUDA_TRY(cudaMemcpy(&sb, rc.status, sizeof(sb), cudaMemcpyDeviceToHost));
    out[0] = sb.code;
    out[1] = sb.rank;
    out[2] = sb.chunk;
    out[3] = sb.epoch;
    if (sb.code != 0) {
        ERROR_LOG("device wait ran out: code %u rank/barrier %u chunk/stage %u epoch %u", sb.code, sb.rank, sb.chunk,
                  sb.epoch);
        CUDA_TRY(cudaMemset(rc.status, 0, sizeof(sb)));
        return CATCCOS_B200_ETIMEOUT;
    }
    return 0;
}

int catccos_b200_set_option(const char* key, int64_t value)
{
    if (key == nullptr) return CATCCOS_B200_EINVAL;
    std::string k = key;
    if (k == "tiny_block_rule" && (value == 0 || value == 1)) {
        g.tiny_block_rule = (int)value;
    } else if (k == "c_dtype" && (value == 0 || value == 1)) {
        g.c_dtype = (int)value;
    } else if (k == "a_dtype" && value >= 0 && value <= 2) {
        g.a_dtype = (int)value;
    } else if (k == "b_dtype" && value >= 0 && value <= 2) {
        g.b_dtype = (int)value;
    } else if (k == "timeout_ms" && value > 0 && value <= 600000) {
        g.timeout_ns = (uint64_t)value * 1000000ull;
    } else if (k == CATCCOS_B200_OPT_BLOCK_N && (value == 0 || value == 128 || value == 256)) {
        g.block_n = (int)value;
    } else if (k == CATCCOS_B200_OPT_PHASE_MASK && value >= 1 && value <= 3) {
        g.phase_mask = (int)value;
    } else if (k == CATCCOS_B200_OPT_CTA_PAIR && value >= 0 && value <= 2) {
        g.cta_pair = (int)value;
    } else if (k == CATCCOS_B200_OPT_FUSE_MODE && (value == -1 || value == 0 || (value >= 3 && value <= 7))) {
        g.fuse_mode = (int)value;
    } else if (k == CATCCOS_B200_OPT_SPLIT_K && value >= 0 && value <= 8) {
        g.split_k = (int)value;
    } else if (k == CATCCOS_B200_OPT_TILE_ORDER && value >= -1 && value <= 1) {
        g.tile_order = (int)value;
    } else {
        ERROR_LOG("set_option: unknown key or bad value: %s = %lld", key, (long long)value);
        return CATCCOS_B200_EINVAL;
    }
    return 0;
}

uint64_t catccos_b200_launch_count(void) { return g_launches.load(); }

}  // extern "C"

// =============================================================================================
// Allocation-free single-GPU entry point
// =============================================================================================
namespace {

// Scratch of catccos_b200_mx_quant_matmul_static: the quantised copy of A and its ready flags live in
// this file-scope device array instead of a buffer from catccos_b200_symm_alloc.  Every GPU that
// loads the library carries it (about 8.3 MiB) until the process exits.
constexpr size_t kStaticMaxElems = size_t(8) << 20;  // m * k may not exceed this
constexpr uint32_t kStaticMaxFlags = 8192;           // (16-row chunks) x (K segments) may not exceed this
constexpr size_t kStaticFlagsOff = 0;
constexpr size_t kStaticStatusOff = kStaticMaxFlags * sizeof(uint32_t);
constexpr size_t kStaticScalesOff = kStaticStatusOff + 1024;
constexpr size_t kStaticCodesOff = kStaticScalesOff + kStaticMaxElems / 32;
constexpr size_t kStaticBytes = kStaticCodesOff + kStaticMaxElems;
static_assert(kStaticScalesOff % 256 == 0 && kStaticCodesOff % 1024 == 0, "TMA and vector stores need these aligned");

static __device__ __align__(256) uint8_t g_static_scratch[kStaticBytes];

struct StaticDeviceState {
    uint8_t* ptr = nullptr;  // device address of g_static_scratch on this device
    int num_sms = 0;
    uint32_t epoch = 0;
};
StaticDeviceState g_static_dev[kMaxRanks * 2];
std::mutex g_static_mu;

}  // namespace

extern "C" int catccos_b200_mx_quant_matmul_static(void* stream, const void* a_bf16, const void* b, const void* b_scale,
                                                   void* c, uint32_t m, uint32_t n, uint32_t k)
{
    if (!a_bf16 || !b || !b_scale || !c || m == 0 || n == 0 || k == 0) {
        return CATCCOS_B200_EINVAL;
    }
    if (k % kGemmBlockK != 0 || n % 16 != 0) {
        ERROR_LOG("mx_quant_matmul_static: k must be a multiple of 128 and n of 16 (got n=%u k=%u)", n, k);
        return CATCCOS_B200_EINVAL;
    }
    if ((((uintptr_t)a_bf16 | (uintptr_t)b) & 15u) || ((uintptr_t)c & 31u) || ((uintptr_t)b_scale & 1u)) {
        ERROR_LOG("mx_quant_matmul_static: a and b must be 16-byte aligned, c 32-byte aligned, b_scale 2-byte aligned");
        return CATCCOS_B200_EINVAL;  // refused before the shared array or the stream is touched
    }
    if ((size_t)m * k > kStaticMaxElems) {
        ERROR_LOG("mx_quant_matmul_static: m * k = %zu exceeds the built-in scratch of %zu elements; "
                  "use catccos_b200_mx_quant_allgather_matmul with a buffer from catccos_b200_symm_alloc",
                  (size_t)m * k, kStaticMaxElems);
        return CATCCOS_B200_ENOMEM;
    }
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxRanks * 2) {
        return CATCCOS_B200_EINVAL;
    }
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDeviceState& sd = g_static_dev[dev];
    if (sd.ptr == nullptr) {
        // One-time set-up for this device (it is current).  In host code the array's name is only a
        // stand-in; the address a kernel may use comes from the runtime.
        void* p = nullptr;
        int sms = 0;
        CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (!g.drv.Load()) {
            return CATCCOS_B200_ECUDA;
        }
        sd.num_sms = sms;  // the state is filled in only once every step of the set-up has succeeded
        sd.ptr = static_cast<uint8_t*>(p);
    }
    RankCtx rc;  // a view for the launcher: nothing is created or owned here
    rc.device = dev;
    rc.num_sms = sd.num_sms;
    rc.status = reinterpret_cast<StatusBlock*>(sd.ptr + kStaticStatusOff);

    QuantPushParams seg = {};
    choose_segments(m, k, rc.num_sms, seg);
    const uint32_t chunks = (m + kRowsPerChunk - 1) / kRowsPerChunk;
    if ((size_t)chunks * seg.segs_per_chunk > kStaticMaxFlags) {
        ERROR_LOG("mx_quant_matmul_static: %u row chunks x %u K segments exceed the built-in %u flag words", chunks,
                  seg.segs_per_chunk, kStaticMaxFlags);
        return CATCCOS_B200_ENOMEM;
    }
    cudaStream_t st = (cudaStream_t)stream;
    // the array keeps what the last call left: the flag words are epochs that only grow, so stale ones
    // never satisfy this call; the status record must start at zero
    CUDA_TRY(cudaMemsetAsync(rc.status, 0, sizeof(StatusBlock), st));
    const uint32_t epoch = ++sd.epoch;

    GemmParams p = {};
    p.a_scales = sd.ptr + kStaticScalesOff;
    p.b_scales = (const uint8_t*)b_scale;
    p.c = c;
    p.Mg = m;
    p.N = n;
    p.K = k;
    p.flags = reinterpret_cast<const uint32_t*>(sd.ptr + kStaticFlagsOff);
    p.flag_stride = kStaticMaxFlags;
    p.segs = seg.segs_per_chunk;
    p.seg_ktiles = seg.seg_cols / kGemmBlockK;
    p.world = 1;
    p.rank = 0;
    p.m_local = m;
    p.epoch = epoch;
    QuantPushParams& q = p.q;
    q.in = a_bf16;
    q.M = m;
    q.K = k;
    q.world = 1;
    q.epoch = epoch;
    q.num_dst = 1;
    q.publish = 1;
    q.produce = 1;
    q.mode = quant_mode(false);
    q.e5m2 = g.a_dtype == 1 ? 1u : 0u;
    q.sys_scope = 0;
    q.segs_per_chunk = seg.segs_per_chunk;
    q.seg_cols = seg.seg_cols;
    q.dst_codes[0] = sd.ptr + kStaticCodesOff;
    q.dst_scales[0] = sd.ptr + kStaticScalesOff;
    q.dst_flags[0] = reinterpret_cast<uint32_t*>(sd.ptr + kStaticFlagsOff);
    q.status = rc.status;
    q.timeout_ns = g.timeout_ns;
    return launch_gemm(rc, st, sd.ptr + kStaticCodesOff, b, p, true);
}

#ifdef CATCCOS_TRACE
// =============================================================================================
// Device-side timeline (trace build only; declarations: include/catccos_b200_trace.h)
// =============================================================================================
extern "C" int catccos_b200_trace_arm(void)
{
    if (g.mode == Mode::kNone) {
        return CATCCOS_B200_ESTATE;
    }
    RankCtx& rc = cur();
    CUDA_TRY(cudaSetDevice(rc.device));
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemset(rc.trace, 0, (size_t)rc.num_sms * kTraceSlots * sizeof(unsigned long long)));
    // the stand-alone quantise kernel keeps the minimum of its CTAs' start times in this word
    const unsigned long long big = ~0ull;
    CUDA_TRY(cudaMemcpy(rc.trace + kTrQuantKernelStart, &big, sizeof(big), cudaMemcpyHostToDevice));
    g.trace_armed = true;
    return 0;
}

extern "C" int catccos_b200_trace_read(unsigned long long* out, uint32_t max_words, uint32_t* grid, uint32_t* slots)
{
    if (out == nullptr || grid == nullptr || slots == nullptr || g.mode == Mode::kNone) {
        return CATCCOS_B200_ESTATE;
    }
    RankCtx& rc = cur();
    const size_t words = (size_t)rc.trace_grid * kTraceSlots;
    if (rc.trace == nullptr || words == 0 || words > max_words) {
        return CATCCOS_B200_EINVAL;
    }
    CUDA_TRY(cudaSetDevice(rc.device));
    CUDA_TRY(cudaDeviceSynchronize());
    CUDA_TRY(cudaMemcpy(out, rc.trace, words * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    *grid = (uint32_t)rc.trace_grid;
    *slots = kTraceSlots;
    return 0;
}
#endif

// The device-side wait record of the allocation-free entry point lives in the built-in array too (the regular
// record belongs to a rank context, which that entry point never creates).  Synchronises the device and copies
// the 16 bytes out; nothing is allocated.
extern "C" int catccos_b200_mx_quant_matmul_static_status(uint32_t out[4])
{
    if (out == nullptr) {
        return CATCCOS_B200_EINVAL;
    }
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxRanks * 2) {
        return CATCCOS_B200_EINVAL;
    }
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticDeviceState& sd = g_static_dev[dev];
    if (sd.ptr == nullptr) {
        return CATCCOS_B200_ESTATE;  // no call has been made on this device yet
    }
    CUDA_TRY(cudaDeviceSynchronize());
    StatusBlock sb;
    CUDA_TRY(cudaMemcpy(&sb, sd.ptr + kStaticStatusOff, sizeof(sb), cudaMemcpyDeviceToHost));
    out[0] = sb.code;
    out[1] = sb.rank;
    out[2] = sb.chunk;
    out[3] = sb.epoch;
    if (sb.code != 0) {
        ERROR_LOG("device wait ran out in mx_quant_matmul_static: code %u rank/barrier %u chunk/stage %u epoch %u", sb.code,
                  sb.rank, sb.chunk, sb.epoch);
        return CATCCOS_B200_ETIMEOUT;
    }
    return 0;
}
