// MXFP8 block-scaled GEMM for sm_100a: C[Mg, N] = dequant(A)[Mg, K] x dequant(B)[K, N].
//
// It replaces the cube-core half of the reference's AllGather-Matmul kernel
// (include/catccos/dgemm/kernel/mx_allgather_matmul.hpp:240-297; its main loop is CATLASS
// BlockMmadTla<MmadMx>, instantiated in
// examples/ascend950_fp8_mx_allgather_matmul/ascend950_fp8_mx_allgather_matmul_device.h:47-57).
//
//   A      E4M3 codes, row-major [Mg, K]   (K-major operand; Mg = world * M_local gathered rows)
//   SFA    E8M0 bytes, row-major [Mg, K/32]
//   B      E4M3 codes, row-major [K, N]    (MN-major operand, read in place)
//   SFB    E8M0 bytes in the reference's file layout [K/64, N, 2]
//   C      bf16 or fp16, row-major [Mg, N]
//
// One CTA per 128 x BLOCK_N output tile, persistent over tiles, 320 threads:
//   warps 0-3 epilogue: tcgen05.ld of the fp32 accumulator, convert, 16-byte global stores
//   warp 4    TMA producer: A and B tiles (128-byte swizzle) into a ring of shared-memory stages
//   warp 5    MMA issuer: four tcgen05.mma.kind::mxf8f6f4.block_scale (K = 32 each) and one
//             tcgen05.commit per stage, nothing else (see the scale loaders)
//   warps 6-9 scale loaders: warp j serves every fourth K tile; plain global loads of the E8M0
//             bytes (the next K tile's loads are in flight while the current one is stored),
//             written to shared memory in the 32x16-byte atom layout tcgen05.cp expects, copied into
//             the stage's scale set in tensor memory by lane 0 (tcgen05.cp), whose tcgen05.commit on the
//             stage's full barrier is the warp's arrival
//
// With FUSED_QUANT the CTA carries fourteen more warps (10-23): eight run the quantise producer (mx_quant.cuh)
// on this rank's bf16 shard into the local stage and publish local flags, six are pushers that copy finished
// work items to the peers' stages over NVLink and set the peers' flags.  The GEMM warps of the same launch
// (and of the peers' launches) consume behind them, so the quantisation, the allgather and the matmul are one
// kernel.
//
// When `flags` is set, a K segment of a tile is not touched before every (source rank, 16-row chunk) under
// the tile's rows has published that segment with the current epoch; tiles are visited in the order the
// chunks arrive (own shard first, then slice by slice over the peers).  Only the TMA producer polls the
// flags as a rule (one lane per chunk, relaxed loads, one acquire at the end) and tells the scale loaders
// through a word in shared memory how far the data is known to be there; a scale loader that is ahead of the
// producer polls for itself.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.cuh"
#include "mx_quant.cuh"

namespace catccos {

constexpr uint32_t kGemmBlockM = 128;
constexpr uint32_t kGemmBlockK = 128;   // bytes == elements (8-bit codes): one 128-byte swizzle row
constexpr uint32_t kGemmThreads = 320;
constexpr uint32_t kPushWarps = 6;
constexpr uint32_t kGemmFusedThreads = kGemmThreads + kQuantThreads + kPushWarps * 32;  // + eight quantise warps + six pushers
constexpr uint32_t kSfWarps = 4;
constexpr uint32_t kRowsPerChunk = 16;  // granularity of the ready flags
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
    const uint8_t* a_scales;  // [Mg, K/32]
    const uint8_t* b_scales;  // [K/64, N, 2]
    void* c;                  // [Mg, N]: bf16 / fp16, or E4M3 codes when the epilogue quantises (MxOut)
    uint8_t* c_scales;        // MxOut only: E8M0 [Mg, N/32], one scale per 32 output columns of a row
    uint32_t c_tiny_rule;     // MxOut only: kQuantGolden / kQuantDeviceTiny
    // ScatterOut only (Matmul + ReduceScatter): rows [d * rs_rows, (d + 1) * rs_rows) of this rank's fp32 partial
    // product go to rank d's stage, slot `rank`; one flag word per (32-row block, N tile) says they have landed
    float* rs_dst[kMaxRanks];       // rank d's partials [world][rs_rows][N] (this rank's own for d == rank)
    uint32_t* rs_flags[kMaxRanks];  // rank d's flag words for this source: [(rs_rows / 32) * n_tiles]
    uint32_t rs_rows;
    uint32_t Mg, N, K;
    uint32_t b_kmajor;        // 1: B is the transposed copy [N, K] (K-major operand); the tensor core takes 4-bit
                              // operands in that form only, so packed E2M1 weights are transposed once per call
    uint32_t a_fmt, b_fmt;    // element type of the A / B codes as tcgen05 names it: 0 = E4M3, 1 = E5M2, 5 = E2M1
                              // (E2M1: packed two per byte in global memory, unpacked by TMA into the
                              // 16-values-per-16-bytes form kind::mxf8f6f4 reads from shared memory)
    // gating on the quantise-and-push kernel (flags == nullptr: all of A is already in place)
    const uint32_t* flags;  // [world][flag_stride] epoch words in this GPU's symmetric header,
                            // word chunk * segs + seg covers 16 rows x (seg_ktiles * 128) columns of K
    uint32_t flag_stride;
    uint32_t segs, seg_ktiles;
    uint32_t world, rank, m_local, epoch;
    uint32_t gemm_off;        // 1: the GEMM warps stay idle (the producer half of a call, run apart)
    uint32_t own_first;       // tile order of a gated launch: 1 = this rank's whole shard first (it is there before any
                              // peer's rows), 0 = slice by slice over ALL ranks, own slice leading (every rank's
                              // rows, this rank's included, are produced at the pace of the transfer)
    uint64_t timeout_ns;      // limit of a wait for ready flags
    uint64_t bar_timeout_ns;  // limit of a wait on an intra-kernel barrier (set above timeout_ns by the host)
    StatusBlock* status;
    unsigned long long* trace;  // timeline side buffer (trace build only), else nullptr
    QuantPushParams q;  // the producer's work when the quantise warps ride in this kernel (local stage only)
    PushParams push;    // the pusher warps' work: local stage -> the peers' stages
    // Split K (ksplit > 1): K is cut in ksplit equal parts and every (tile, part) pair is a work unit of its
    // own CTA (units == grid, so all of them are resident together).  Every part owns an equal share of the
    // tile's columns, writes the rest of its fp32 partial tile to the workspace, and adds the other parts'
    // pieces of its own columns in ascending part order.  ksplit is a power of two <= BLOCK_N / 32.
    uint32_t ksplit;
    float* splitk_ws;        // [tiles][ksplit][BLOCK_N / 32][128][32]
    uint32_t* splitk_flags;  // [tiles][ksplit][4] epoch words, one per epilogue warp
    uint32_t splitk_epoch;
};

template <uint32_t BLOCK_N>
struct GemmSmem {
    static constexpr uint32_t kStages = (BLOCK_N == 256) ? 4 : 6;
    static constexpr uint32_t kABytes = kGemmBlockM * kGemmBlockK;
    static constexpr uint32_t kBBytes = BLOCK_N * kGemmBlockK;
    static constexpr uint32_t kSfaBytes = 512;
    static constexpr uint32_t kSfbAtoms = (BLOCK_N + 127) / 128;
    static constexpr uint32_t kSfbBytes = kSfbAtoms * 512;
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOffA + kStages * kABytes;
    static constexpr uint32_t kOffSfa = kOffB + kStages * kBBytes;
    static constexpr uint32_t kOffSfb = kOffSfa + kStages * kSfaBytes;
    static constexpr uint32_t kOffBar = kOffSfb + kStages * kSfbBytes;
    // barriers: full[S] (TMA bytes + one scale-loader arrival), empty[S], tmem_full[2], tmem_empty[2],
    // overlap_free[2]
    static constexpr uint32_t kNumBars = 2 * kStages + 6 + 4;  // + one per epilogue warp for the split-K reduction
    static constexpr uint32_t kOffTmemPtr = kOffBar + kNumBars * 8;
    static constexpr uint32_t kOffGate = kOffTmemPtr + 8;  // K-tile iterations whose rows the producer has seen ready
    static constexpr uint32_t kBytes = kOffTmemPtr + 16;
    static constexpr uint32_t kDynamicBytes = kBytes + 1024;  // slack to align the base to 1024 bytes
    // Tensor memory: two 128 x BLOCK_N fp32 accumulators and one set of scale factors per stage (12 columns:
    // SFA 4, then SFB 4 per 128 columns of N).  For BLOCK_N = 256 the accumulators overlap by 64 columns
    // (192..255) to leave room for the four sets; the epilogue drains the two shared 32-column chunks first and
    // then lets the next tile start.
    static constexpr bool kOverlap = (BLOCK_N == 256);
    static constexpr uint32_t kOverlapChunks = 2;
    static constexpr uint32_t kAccCol1 = kOverlap ? 192 : 256;
    static constexpr uint32_t kSfCol = kOverlap ? 448 : 384;
    static constexpr uint32_t kSfSetCols = 12;
    static_assert(kSfCol + kStages * kSfSetCols <= 512, "scale-factor sets must fit in tensor memory");
};

struct TileCoord {
    uint32_t m_tile, n_tile;
};

// Tile visiting order.  n runs fastest so that concurrently running CTAs share one A panel in L2.
// With gating, m tiles follow arrival.  own_first: this rank's own shard, then for each 128-row slice of a
// shard, the peers in ring order starting after this rank.  Otherwise slice by slice over all ranks, this
// rank's slice leading and the peers behind it in ring order.
__host__ __device__ __forceinline__ uint32_t arrival_m_tile(uint32_t mo, uint32_t tps, const GemmParams& p)
{
    if (p.own_first == 0u) {
        return ((p.rank + mo % p.world) % p.world) * tps + mo / p.world;
    }
    if (mo < tps) {
        return p.rank * tps + mo;
    }
    const uint32_t j = mo - tps;
    return ((p.rank + 1 + j % (p.world - 1)) % p.world) * tps + j / (p.world - 1);
}

__host__ __device__ __forceinline__ TileCoord tile_coord(uint32_t idx, uint32_t n_tiles, uint32_t m_tiles, const GemmParams& p)
{
    uint32_t mo = idx / n_tiles;
    TileCoord t;
    t.n_tile = idx - mo * n_tiles;
    if (p.flags != nullptr && p.world > 1) {
        if (p.m_local % kGemmBlockM == 0) {
            t.m_tile = arrival_m_tile(mo, p.m_local / kGemmBlockM, p);
        } else {
            uint32_t first = (p.rank * p.m_local) / kGemmBlockM;
            t.m_tile = (mo + first) % m_tiles;
        }
    } else {
        t.m_tile = mo;
    }
    return t;
}

// Waits (whole warp) until K segment `seg0` of every chunk under gathered rows [m0, m0 + 128) carries the epoch,
// and returns how many K segments from seg0 on are there for ALL of those chunks (0 when the wait ran out): a
// tile whose rows arrived long ago is checked once, not once per segment.  A lane looks at four rows and polls
// only for a row that is the first of its (source, chunk) inside the tile, so every chunk is polled by exactly
// one lane.  The polls are relaxed loads, several in flight; the acquire that orders the data behind the flags
// is one load per polling lane, on the last flag it counted.
__device__ __forceinline__ uint32_t wait_rows_ready(const GemmParams& p, uint32_t m0, uint32_t lane, uint32_t seg0)
{
    const uint32_t nseg = p.segs - seg0;
    uint32_t ready = nseg;
    bool ok = true;
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t row = m0 + lane * 4 + i;
        if (row >= p.Mg) {
            break;
        }
        const uint32_t src = row / p.m_local;
        const uint32_t in_src = row - src * p.m_local;
        // first row of the tile, of a source's shard, or of a 16-row chunk
        if (row != m0 && in_src != 0u && (in_src % kRowsPerChunk) != 0u) {
            continue;
        }
        const uint32_t chunk = in_src / kRowsPerChunk;
        const uint32_t* f = p.flags + (size_t)src * p.flag_stride + chunk * p.segs + seg0;
        uint32_t cnt = 0;
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (true) {
            bool stop = false;
            cnt = 0;
            for (uint32_t base = 0; base < nseg && !stop; base += 8) {
                uint32_t v[8];
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    v[j] = base + j < nseg ? ld_relaxed_sys(f + base + j) : p.epoch - 1u;
                }
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    if (!stop && (int32_t)(v[j] - p.epoch) >= 0) {
                        ++cnt;
                    } else {
                        stop = true;
                    }
                }
            }
            if (cnt > 0) {
                break;
            }
            if (spins == 0) {
                t0 = globaltimer_ns();
            }
            if ((++spins & 0x1Fu) == 0u) {
                if (globaltimer_ns() - t0 > p.timeout_ns || status_tripped(p.status)) {
                    report_status(p.status, kStatusFlagTimeout, src, chunk, p.epoch);
                    ok = false;
                    break;
                }
                __nanosleep(64);
            }
        }
        if (cnt > 0) {
            (void)ld_acquire_sys(f + cnt - 1);
        }
        ready = min(ready, cnt);
    }
    ready = __reduce_min_sync(0xFFFFFFFFu, ready);
    return __all_sync(0xFFFFFFFFu, ok) ? ready : 0u;
}

__device__ __forceinline__ void st_release_cta_shared(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_cta_shared(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}

// After an aborted pipeline (a wait ran out) operand loads and MMAs may still be in flight: the warp that
// frees the tensor memory, and with it the last warp of the CTA to leave, gives them time to land.
__device__ __forceinline__ void drain_after_abort(const StatusBlock* st)
{
    if (status_tripped(st)) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 50000ull) {
            __nanosleep(1000);
        }
    }
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack2(float a, float b);

template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b)
{
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Writes 32 consecutive columns of one output row from fp32 accumulator values.
template <typename OutT>
__device__ __forceinline__ void store_c_chunk(OutT* c, const GemmParams& p, uint32_t row, uint32_t col, const uint32_t (&r)[32])
{
    if (row < p.Mg && col < p.N) {
        OutT* dst = c + (size_t)row * p.N + col;
        if (col + 32u <= p.N) {
#pragma unroll
            for (uint32_t v = 0; v < 2; ++v) {
                uint32_t o[8];
#pragma unroll
                for (uint32_t e = 0; e < 8; ++e) {
                    o[e] = pack2<OutT>(__uint_as_float(r[v * 16 + 2 * e]), __uint_as_float(r[v * 16 + 2 * e + 1]));
                }
                st_global_v8(dst + v * 16, o);  // one full 32-byte sector per store
            }
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 32u; ++j) {
                if (col + j < p.N) {
                    dst[j] = static_cast<OutT>(__uint_as_float(r[j]));
                }
            }
        }
    }
}

// Output "type" of the epilogue that MX-quantises what it has just computed: the 32 consecutive columns a lane
// holds of one output row are exactly one MX block, so the lane rounds them to bf16 (the 16-bit tile the
// reference's epilogue quantises from), takes the block's exponent, and writes 32 E4M3 codes and one E8M0 byte.
// It replaces CommBlockMxQuant::QuantFromUb / QuantFromUb2D
// (include/catccos/comm/block/comm_block_mx_quant.hpp:209-310): quantising a GEMM output tile before it leaves
// the core, without materialising the 16-bit tensor.
struct MxOut {};

template <>
__device__ __forceinline__ void store_c_chunk<MxOut>(MxOut*, const GemmParams& p, uint32_t row, uint32_t col,
                                                     const uint32_t (&r)[32])
{
    if (row >= p.Mg || col >= p.N) {
        return;  // N is a multiple of 32 here (checked by the host), so a chunk is inside or outside as a whole
    }
    uint32_t w[16];
    uint32_t amax = 0;
#pragma unroll
    for (uint32_t e = 0; e < 16; ++e) {
        w[e] = pack2<__nv_bfloat16>(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
        const uint32_t a = w[e] & 0x7FFF7FFFu;
        amax = max(amax, max(a & 0xFFFFu, a >> 16));
    }
    uint32_t byte;
    float mul;
    bool nonfinite;
    block_scale(amax, p.c_tiny_rule == kQuantDeviceTiny, 8u, byte, mul, nonfinite);
    uint32_t o[8];
#pragma unroll
    for (uint32_t e = 0; e < 8; ++e) {
        o[e] = nonfinite ? 0x7F7F7F7Fu : encode4(w[2 * e], w[2 * e + 1], mul, false);
    }
    st_global_v8(static_cast<uint8_t*>(p.c) + (size_t)row * p.N + col, o);
    p.c_scales[(size_t)row * (p.N / 32u) + col / 32u] = (uint8_t)byte;
}

// Output "type" of the epilogue of Matmul + ReduceScatter: the fp32 accumulator rows go, unrounded, to the stage
// of the rank that owns them (a peer's over NVLink, or this rank's own), where that rank adds the partial
// products of all ranks in rank order.  It replaces the compute half of MatmulReduceScatterMxTla
// (include/catccos/dgemm/kernel/matmul_reduce_scatter_mx_tla.hpp:36-125), whose partial tiles travel through
// the symmetric workspace as 16-bit values; fp32 partials and a fixed order make the sum independent of timing.
struct ScatterOut {};

template <>
__device__ __forceinline__ void store_c_chunk<ScatterOut>(ScatterOut*, const GemmParams& p, uint32_t row, uint32_t col,
                                                          const uint32_t (&r)[32])
{
    if (row >= p.Mg || col >= p.N) {
        return;
    }
    const uint32_t d = row / p.rs_rows;
    float* dst = p.rs_dst[d] + ((size_t)p.rank * p.rs_rows + (row - d * p.rs_rows)) * p.N + col;
    if (col + 32u <= p.N) {
#pragma unroll
        for (uint32_t v = 0; v < 8; ++v) {
            reinterpret_cast<float4*>(dst)[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                             __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
        }
    } else {
        for (uint32_t j = 0; col + j < p.N; ++j) {
            dst[j] = __uint_as_float(r[j]);
        }
    }
}

// After an epilogue warp has stored its 32 rows of a tile: the rows are fenced and flagged at their owner.
template <typename OutT>
__device__ __forceinline__ void publish_tile_rows(const GemmParams& p, uint32_t row0, uint32_t n_tile, uint32_t n_tiles,
                                                  uint32_t lane)
{
    if constexpr (std::is_same<OutT, ScatterOut>::value) {
        __syncwarp();
        if (lane == 0 && row0 < p.Mg) {
            const uint32_t d = row0 / p.rs_rows;
            const uint32_t block = (row0 - d * p.rs_rows) / 32u;
            __threadfence_system();
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.rs_flags[d] + (size_t)block * n_tiles + n_tile), "r"(p.epoch)
                         : "memory");
        }
    }
}

// The consumer half of Matmul + ReduceScatter: this rank's rows of the product, D [rs_rows, N] = the sum over the
// source ranks, in rank order, of the fp32 partials in this rank's stage.  One CTA per (32-row block, N tile) of
// the producing GEMM, as soon as all ranks have flagged it (bounded wait).
template <typename OutT>
__global__ void __launch_bounds__(256) mx_reduce_scatter_kernel(const float* __restrict__ parts, const uint32_t* flags,
                                                                uint32_t flag_stride, uint32_t world, uint32_t rs_rows, uint32_t N,
                                                                uint32_t bn, uint32_t epoch, OutT* __restrict__ d,
                                                                uint64_t timeout_ns, StatusBlock* status)
{
    const uint32_t n_tiles = (N + bn - 1) / bn;
    const uint32_t units = (rs_rows / 32u) * n_tiles;
    for (uint32_t unit = blockIdx.x; unit < units; unit += gridDim.x) {
        const uint32_t rb = unit / n_tiles, nt = unit - rb * n_tiles;
        if (threadIdx.x < world && !wait_flag_ge(flags + (size_t)threadIdx.x * flag_stride + unit, epoch, timeout_ns, status)) {
            report_status(status, kStatusFlagTimeout, threadIdx.x, unit, epoch);
        }
        __syncthreads();
        if (status_tripped(status)) {
            return;  // nothing is written from partials that never arrived
        }
        const uint32_t c0 = nt * bn;
        const uint32_t cols4 = (min(bn, N - c0)) / 4u;
        for (uint32_t i = threadIdx.x; i < 32u * cols4; i += blockDim.x) {
            const uint32_t r = i / cols4, c = c0 + (i - r * cols4) * 4u;
            const size_t row = (size_t)rb * 32u + r;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t s = 0; s < world; ++s) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(parts + ((size_t)s * rs_rows + row) * N + c));
                acc.x += v.x;
                acc.y += v.y;
                acc.z += v.z;
                acc.w += v.w;
            }
            uint2 o;
            o.x = pack2<OutT>(acc.x, acc.y);
            o.y = pack2<OutT>(acc.z, acc.w);
            *reinterpret_cast<uint2*>(d + row * N + c) = o;
        }
        __syncthreads();
    }
}

template <uint32_t BLOCK_N, typename OutT, bool FUSED_QUANT>
__global__ void __launch_bounds__(FUSED_QUANT ? kGemmFusedThreads : kGemmThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p)
{
    using S = GemmSmem<BLOCK_N>;
    constexpr uint32_t kStages = S::kStages;
    static_assert(BLOCK_N == 128 || BLOCK_N == 256, "tile widths wired up: 128 and 256");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kOffBar);
    uint64_t* full = bars;
    uint64_t* empty = bars + kStages;
    uint64_t* tmem_full = bars + 2 * kStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint64_t* overlap_free = tmem_empty + 2;
    uint64_t* red_bar = overlap_free + 2;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + S::kOffTmemPtr);
    uint32_t* gate = reinterpret_cast<uint32_t*>(smem + S::kOffGate);
    uint32_t* push_turn = gate + 1;  // the pushers of this CTA store one after the other (mx_quant.cuh, push_worker)

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    const uint32_t m_tiles = (p.Mg + kGemmBlockM - 1) / kGemmBlockM;
    const uint32_t n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
    const uint32_t num_tiles = p.gemm_off ? 0u : m_tiles * n_tiles;
    const uint32_t k_tiles = p.K / kGemmBlockK;
    const uint64_t bar_ns = p.bar_timeout_ns;

    if (threadIdx.x == 0) {
        CATCCOS_TR_STAMP(p.trace, kTrCtaStart);
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 2);  // the producer's expect_tx arrival and one scale-loader warp
            mbar_init(&empty[s], 1);
        }
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 4);
            mbar_init(&overlap_free[a], 4);
        }
        for (uint32_t w = 0; w < 4; ++w) {
            mbar_init(&red_bar[w], 1);
        }
        *gate = 0u;
        *push_turn = 0u;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 5) {
        tmem_alloc(tmem_ptr_smem, kTmemCols);
        tmem_relinquish();
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;
    if (threadIdx.x == 0) {
        CATCCOS_TR_STAMP(p.trace, kTrSetupDone);
    }

    if (warp == 4) {
        // ------------------------------- TMA producer -------------------------------------
        if (p.flags == nullptr) {
            grid_dep_wait();  // A is the output of the kernel launched just before (no-op for a plain launch);
        }                     // with flags, the flags say when its rows are there
        const uint32_t ksplit = p.ksplit > 1u ? p.ksplit : 1u;
        const uint32_t kper = k_tiles / ksplit;  // K tiles per work unit (the host only splits evenly)
        const uint32_t num_units = num_tiles * ksplit;
        uint32_t it = 0, ti = 0;
        bool alive = true;
        // packed 4-bit operands arrive as half the bytes they occupy in shared memory (the gaps are not written)
        const uint32_t tx_bytes = (p.a_fmt == 5u ? S::kABytes / 2u : S::kABytes) + (p.b_fmt == 5u ? S::kBBytes / 2u : S::kBBytes);
        for (uint32_t unit = blockIdx.x; alive && unit < num_units; unit += gridDim.x, ++ti) {
            const uint32_t ks = unit / num_tiles;
            TileCoord tc = tile_coord(unit - ks * num_tiles, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kGemmBlockM;
            const uint32_t n0 = tc.n_tile * BLOCK_N;
            const uint32_t kt0 = ks * kper;
            uint32_t ready_end = kt0;  // K tiles below this index are known to be there
            for (uint32_t kt = kt0; alive && kt < kt0 + kper; ++kt, ++it) {
                if (p.flags != nullptr && kt >= ready_end) {
                    const unsigned long long t0 = CATCCOS_TR_NOW();
                    (void)t0;
                    const uint32_t seg0 = kt / p.seg_ktiles;
                    const uint32_t nready = wait_rows_ready(p, m0, lane, seg0);
                    alive = nready != 0u;
                    ready_end = min((seg0 + nready) * p.seg_ktiles, kt0 + kper);
                    fence_proxy_async_all();
                    if (lane == 0) {
                        // the scale loaders may go ahead as far as the rows are known to be there
                        st_release_cta_shared(gate, it + (ready_end - kt));
                        CATCCOS_TR_ADD(p.trace, kTrProdFlagWaitNs, CATCCOS_TR_NOW() - t0);
                    }
                }
                if (lane == 0 && alive) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    const unsigned long long t1 = CATCCOS_TR_NOW();
                    (void)t1;
                    alive = mbar_wait(&empty[s], ph ^ 1u, p.status, 100, s, bar_ns);
                    CATCCOS_TR_ADD(p.trace, kTrProdEmptyWaitNs, CATCCOS_TR_NOW() - t1);
                    if (kt == kt0 && ti < kTraceTiles) {
                        CATCCOS_TR_STAMP(p.trace, kTrTileStart + ti);
                    }
                    CATCCOS_TR_STAMP_FIRST(p.trace, kTrProdFirstTma);
                    mbar_arrive_expect_tx(&full[s], tx_bytes);
                    tma_load_2d(smem + S::kOffA + s * S::kABytes, &tmap_a, &full[s], (int32_t)(kt * kGemmBlockK),
                                (int32_t)m0);
                    if (p.b_kmajor) {
                        // the transposed copy [N, K]: box = 128 (K, contiguous) x BLOCK_N rows
                        tma_load_2d(smem + S::kOffB + s * S::kBBytes, &tmap_b, &full[s], (int32_t)(kt * kGemmBlockK),
                                    (int32_t)n0);
                    } else {
                        // B is [K, N] row-major: box = 128 (N, contiguous) x 128 (K); one box per 128 columns
                        for (uint32_t h = 0; h < BLOCK_N / 128; ++h) {
                            tma_load_2d(smem + S::kOffB + s * S::kBBytes + h * 16384u, &tmap_b, &full[s],
                                        (int32_t)(n0 + h * 128u), (int32_t)(kt * kGemmBlockK));
                        }
                    }
                    CATCCOS_TR_STAMP(p.trace, kTrProdLastTma);
                }
                alive = __all_sync(0xFFFFFFFFu, alive);
            }
        }
    } else if (warp == 5) {
        // ------------------------------- MMA issuer ---------------------------------------
        // One thread gets a tcgen05 instruction out only every ~70 cycles, so this thread issues what nobody
        // else can (the MMAs, and the commit that releases the stage) and nothing more: four MMAs of 128 cycles
        // each leave it enough time for the commit, the wait for the next stage and its address arithmetic.
        if (lane == 0) {
            const bool bk = p.b_kmajor != 0u;
            const uint32_t idesc = make_idesc_mxf8(kGemmBlockM, BLOCK_N, !bk) | ((p.a_fmt & 7u) << 7) |
                                   ((p.b_fmt & 7u) << 10);  // operand formats: E4M3 = 0, E5M2 = 1, E2M1 = 5
            const uint32_t ksplit = p.ksplit > 1u ? p.ksplit : 1u;
            const uint32_t kper = k_tiles / ksplit;  // K tiles per work unit (the host only splits evenly)
            const uint32_t num_units = num_tiles * ksplit;
            const uint32_t my_units = (num_units > blockIdx.x) ? (num_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
            const uint32_t total_it = my_units * kper;

            // descriptor halves: the high words are constants, the low words are start addresses >> 4
            // A: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart; K advances 32 bytes in the row.
            // B: MN-major, 128-byte swizzle: 128 columns contiguous, K rows 128 bytes apart, 8-row K groups
            // 1024 bytes apart (SBO), 128-column groups 16 KiB apart (LBO).
            const uint32_t hi_a = (uint32_t)(make_smem_desc(0, 16, 1024, 2) >> 32);
            const uint32_t hi_b = bk ? hi_a : (uint32_t)(make_smem_desc(0, 16384, 1024, 2) >> 32);
            const uint32_t a_lo0 = (uint32_t)make_smem_desc(0, 16, 1024, 2) | (smem_u32(smem + S::kOffA) >> 4);
            const uint32_t b_lo0 = (uint32_t)make_smem_desc(0, bk ? 16 : 16384, 1024, 2) | (smem_u32(smem + S::kOffB) >> 4);
            constexpr uint32_t kKbStepA = 32u >> 4;                // 32 bytes along K
            const uint32_t kKbStepB = (bk ? 32u : 4096u) >> 4;     // 32 bytes along K, or 32 K rows of 128 bytes
            const uint32_t sf_tmem0 = tmem_base + S::kSfCol;
            bool alive = true;

            auto stage_wait = [&](uint32_t s, uint32_t ph) {
                const unsigned long long t0 = CATCCOS_TR_NOW();
                (void)t0;
                alive = mbar_wait(&full[s], ph, p.status, 103, s, bar_ns);
                tcgen05_fence_after();
                CATCCOS_TR_ADD(p.trace, kTrMmaFullWaitNs, CATCCOS_TR_NOW() - t0);
            };
            auto issue_mma = [&](uint32_t a_lo, uint32_t b_lo, uint32_t sf, uint32_t kb, uint32_t d_col, uint32_t accumulate) {
                umma_mxf8_lohi(d_col, a_lo + kb * kKbStepA, hi_a, b_lo + kb * kKbStepB, hi_b, idesc_with_sf_id(idesc, kb), sf,
                               sf + 4, accumulate);
            };

            if (total_it > 0) {
                stage_wait(0, 0);
            }
            uint32_t it = 0, s = 0, ph = 0;
            for (uint32_t ti = 0; alive && ti < my_units; ++ti) {
                const uint32_t acc = ti & 1u;
                const uint32_t acc_ph = (ti >> 1) & 1u;
                const uint32_t d_col = tmem_base + (acc ? S::kAccCol1 : 0u);
                const unsigned long long t0 = CATCCOS_TR_NOW();
                (void)t0;
                alive = mbar_wait(&tmem_empty[acc], acc_ph ^ 1u, p.status, 101, acc, bar_ns);
                if (S::kOverlap && ti > 0 && alive) {
                    alive = mbar_wait(&overlap_free[acc ^ 1u], ((ti - 1) >> 1) & 1u, p.status, 102, acc, bar_ns);
                }
                CATCCOS_TR_ADD(p.trace, kTrMmaAccWaitNs, CATCCOS_TR_NOW() - t0);
                tcgen05_fence_after();
                CATCCOS_TR_STAMP_FIRST(p.trace, kTrMmaFirst);
                for (uint32_t kt = 0; alive && kt < kper; ++kt, ++it) {
                    const uint32_t a_lo = a_lo0 + s * (S::kABytes >> 4);
                    const uint32_t b_lo = b_lo0 + s * (S::kBBytes >> 4);
                    const uint32_t sf = sf_tmem0 + s * S::kSfSetCols;
                    const uint32_t s_next = (s + 1 == kStages) ? 0u : s + 1;
                    const uint32_t ph_next = ph ^ (s_next == 0u ? 1u : 0u);
                    const bool more = it + 1 < total_it;
                    issue_mma(a_lo, b_lo, sf, 0, d_col, kt != 0 ? 1u : 0u);
                    issue_mma(a_lo, b_lo, sf, 1, d_col, 1u);
                    issue_mma(a_lo, b_lo, sf, 2, d_col, 1u);
                    issue_mma(a_lo, b_lo, sf, 3, d_col, 1u);
                    tcgen05_commit(&empty[s]);
                    if (more) {
                        stage_wait(s_next, ph_next);
                    }
                    s = s_next;
                    ph = ph_next;
                }
                tcgen05_commit(&tmem_full[acc]);
                if (ti < kTraceTiles) {
                    CATCCOS_TR_STAMP(p.trace, kTrTileEnd + ti);
                }
                CATCCOS_TR_STAMP(p.trace, kTrMmaLast);
            }
        }
        __syncwarp();
    } else if (FUSED_QUANT && warp >= 10) {
        // ------------------------------- quantise-and-push producer -----------------------
        // Of the fourteen extra warps, eight quantise this rank's shard into the local stage (warps 10-19
        // except 13 and 17, which share a scheduler with the MMA issuer and must not compete with that
        // single thread for issue slots).  The other six (13, 17, 20-23) run the pusher, a copy loop that
        // issues an instruction only every few hundred cycles, and send finished items on to the peers.
        if (warp < 20u && (warp & 3u) != (5u & 3u)) {
            const uint32_t qw = warp - 10u - (warp > 13u ? 1u : 0u) - (warp > 17u ? 1u : 0u);  // 0..7
            quant_push_producer<true>(p.q, qw * 32u + lane, blockIdx.x, gridDim.x, 1);
        } else {
            const uint32_t pw = warp == 13u ? 0u : (warp == 17u ? 1u : warp - 18u);  // 0..5
            // pusher pw of CTA b is worker pw * grid + b: a short item list spreads over all SMs instead of
            // filling the first CTAs' six pushers
            push_worker(p.push, lane, pw * gridDim.x + blockIdx.x, gridDim.x * kPushWarps, pw, gridDim.x, push_turn);
        }
    } else if (warp >= 6) {
        // ------------------------------- scale loaders ------------------------------------
        // Warp j takes the K tiles whose running index is j modulo 4.  For its K tile it loads, per
        // lane, four A-scale words (rows lane, lane + 32, ...: exactly the 16 bytes of atom row `lane`)
        // and for every 128 columns of B four pairs of 16-bit halves (the file layout keeps the two
        // scales of a 64-deep K group together), and stores them as 16-byte atom rows.
        constexpr uint32_t kNB = BLOCK_N / 32;  // B words per lane
        const uint32_t j = warp - 6;
        if (p.flags == nullptr) {
            grid_dep_wait();  // the A scales are the output of the kernel launched just before (or: see the flags)
        }
        const uint32_t sf_row_bytes = p.K / 32;
        const uint32_t ksplit = p.ksplit > 1u ? p.ksplit : 1u;
        const uint32_t kper = k_tiles / ksplit;  // K tiles per work unit (the host only splits evenly)
        const uint32_t num_units = num_tiles * ksplit;
        const uint32_t my_units = (num_units > blockIdx.x) ? (num_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
        const uint32_t total_it = my_units * kper;
        uint32_t cur_a[4], cur_lo[kNB], cur_hi[kNB];
        uint32_t nxt_a[4], nxt_lo[kNB], nxt_hi[kNB];
        uint32_t known_end = 0;  // K-tile iterations below this index have their rows in place
        bool alive = true;

        auto issue_loads = [&](uint32_t it, uint32_t (&ra)[4], uint32_t (&rlo)[kNB], uint32_t (&rhi)[kNB]) {
            const uint32_t seq = it / kper;
            const uint32_t unit = blockIdx.x + seq * gridDim.x;
            const uint32_t ks = unit / num_tiles;
            const uint32_t kt = ks * kper + (it - seq * kper);
            TileCoord tc = tile_coord(unit - ks * num_tiles, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kGemmBlockM;
            const uint32_t n0 = tc.n_tile * BLOCK_N;
            if (p.flags != nullptr && it >= known_end) {
                // the producer has usually seen these rows' flags already and said so in shared memory
                // one lane reads the word for the warp: the producer may be updating it, and the branch below holds
                // warp-wide operations, so every lane has to take the same side
                const uint32_t g = __shfl_sync(0xFFFFFFFFu, ld_acquire_cta_shared(gate), 0);
                if (g > it) {
                    known_end = g;
                } else {
                    const unsigned long long t0 = CATCCOS_TR_NOW();
                    (void)t0;
                    const uint32_t seg0 = kt / p.seg_ktiles;
                    const uint32_t nready = wait_rows_ready(p, m0, lane, seg0);
                    alive = alive && nready != 0u;
                    known_end = it + (min((seg0 + nready) * p.seg_ktiles, ks * kper + kper) - kt);
                    if (lane == 0) {
                        CATCCOS_TR_ADD(p.trace, kTrSfGateWaitNs + j, CATCCOS_TR_NOW() - t0);
                    }
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                const uint32_t row = m0 + i * 32 + lane;
                ra[i] = 0x7F7F7F7Fu;
                if (row < p.Mg) {
                    ra[i] = __ldcg(reinterpret_cast<const uint32_t*>(p.a_scales + (size_t)row * sf_row_bytes + kt * 4u));
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < kNB; ++i) {
                const uint32_t n = n0 + i * 32 + lane;
                rlo[i] = 0x7F7Fu;
                rhi[i] = 0x7F7Fu;
                if (n < p.N) {
                    rlo[i] = __ldg(reinterpret_cast<const uint16_t*>(p.b_scales + ((size_t)(2 * kt) * p.N + n) * 2));
                    rhi[i] = __ldg(reinterpret_cast<const uint16_t*>(p.b_scales + ((size_t)(2 * kt + 1) * p.N + n) * 2));
                }
            }
        };

        uint32_t it = j;
        if (it < total_it) {
            issue_loads(it, cur_a, cur_lo, cur_hi);
        }
        for (; alive && it < total_it; it += kSfWarps) {
            const bool has_next = it + kSfWarps < total_it;
            if (has_next) {
                issue_loads(it + kSfWarps, nxt_a, nxt_lo, nxt_hi);
            }
            const uint32_t s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            const unsigned long long t1 = CATCCOS_TR_NOW();
            (void)t1;
            alive = mbar_wait_warp(&empty[s], ph ^ 1u, p.status, 105, s, bar_ns) && alive;
            if (lane == 0) {
                CATCCOS_TR_ADD(p.trace, kTrSfEmptyWaitNs + j, CATCCOS_TR_NOW() - t1);
            }
            uint8_t* sfa = smem + S::kOffSfa + s * S::kSfaBytes;
            uint8_t* sfb = smem + S::kOffSfb + s * S::kSfbBytes;
            *reinterpret_cast<uint4*>(sfa + lane * 16u) = make_uint4(cur_a[0], cur_a[1], cur_a[2], cur_a[3]);
#pragma unroll
            for (uint32_t h = 0; h < kNB / 4; ++h) {
                uint4 v;
                v.x = cur_lo[h * 4 + 0] | (cur_hi[h * 4 + 0] << 16);
                v.y = cur_lo[h * 4 + 1] | (cur_hi[h * 4 + 1] << 16);
                v.z = cur_lo[h * 4 + 2] | (cur_hi[h * 4 + 2] << 16);
                v.w = cur_lo[h * 4 + 3] | (cur_hi[h * 4 + 3] << 16);
                *reinterpret_cast<uint4*>(sfb + h * 512u + lane * 16u) = v;
            }
            fence_proxy_async_shared();
            __syncwarp();
            if (lane == 0) {
                // Copy the atoms into tensor memory from here, not from the MMA issuer: one thread gets a tcgen05
                // instruction out only every ~70 cycles, and four MMAs, three copies and a commit per K tile kept
                // the issuer behind the tensor pipe.  Every stage has its own scale set in tensor memory, so the
                // wait for the stage (above) also covers the set; the commit below stands in for this warp's
                // arrival on the full barrier: the issuer sees the stage only when its scales are in place.
                tcgen05_fence_after();
                const uint32_t hi_sf = (uint32_t)(make_smem_desc(0, 0, 128, 0) >> 32);  // 32 rows x 16 bytes, no swizzle
                const uint32_t sf_t = tmem_base + S::kSfCol + s * S::kSfSetCols;
                tcgen05_cp_sf_lohi(sf_t, smem_u32(sfa) >> 4, hi_sf);
#pragma unroll
                for (uint32_t h = 0; h < S::kSfbAtoms; ++h) {
                    tcgen05_cp_sf_lohi(sf_t + 4 + 4 * h, (smem_u32(sfb) >> 4) + h * (512u >> 4), hi_sf);
                }
                tcgen05_commit(&full[s]);
            }
            if (has_next) {
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) cur_a[i] = nxt_a[i];
#pragma unroll
                for (uint32_t i = 0; i < kNB; ++i) {
                    cur_lo[i] = nxt_lo[i];
                    cur_hi[i] = nxt_hi[i];
                }
            }
        }
    } else {
        // ------------------------------- epilogue -----------------------------------------
        const uint32_t q = warp;  // TMEM lane quarter == warp index modulo 4
        OutT* c = reinterpret_cast<OutT*>(p.c);
        constexpr uint32_t kChunks = BLOCK_N / 32;
        const uint32_t ksplit = p.ksplit > 1u ? p.ksplit : 1u;
        const uint32_t num_units = num_tiles * ksplit;
        if (ksplit > 1u && num_tiles > 0u) {
            // Split K: this CTA is work unit blockIdx.x = (tile, part ks) and the only one on its SM.  Each part
            // owns kChunks / ksplit of the tile's 32-column chunks.  A part first writes the chunks it does not
            // own to its partial tile in the workspace ([part][chunk][128 rows x 32 floats], 4 KiB per chunk and
            // warp) and raises a flag per epilogue warp; then lane 0 of every warp pulls the other parts' pieces
            // of the owned chunks into the (now idle) operand stages with bulk copies, all in flight at once,
            // and the warp adds them to its own accumulator in ascending part order and writes C.
            const uint32_t unit = blockIdx.x;
            const uint32_t ks = unit / num_tiles;
            const uint32_t tile = unit - ks * num_tiles;
            TileCoord tc = tile_coord(tile, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kGemmBlockM;
            const uint32_t n0 = tc.n_tile * BLOCK_N;
            const uint32_t row = m0 + q * 32 + lane;
            const uint32_t cps = kChunks / ksplit;
            const uint32_t own0 = ks * cps;
            constexpr size_t kPartFloats = (size_t)kGemmBlockM * BLOCK_N;
            constexpr uint32_t kPieceBytes = 32u * 32u * 4u;  // 32 rows x 32 floats
            float* parts = p.splitk_ws + (size_t)tile * ksplit * kPartFloats;
            uint32_t* flags = p.splitk_flags + (size_t)tile * ksplit * 4u;
            bool alive = mbar_wait_warp(&tmem_full[0], 0, p.status, 106, 0, bar_ns);
            tcgen05_fence_after();
            // a warp whose 32 rows all lie below the matrix has nothing to add up (its peers in the other
            // parts take the same decision, so nobody waits for its flag); lanes below the matrix skip
            // their partial stores
            const bool warp_rows = m0 + q * 32u < p.Mg;
            const bool lane_row = row < p.Mg;
            for (uint32_t chunk = 0; warp_rows && chunk < kChunks; ++chunk) {
                if (chunk - own0 < cps) {
                    continue;
                }
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + chunk * 32u, r);
                tmem_ld_wait();
                // inside a 4 KiB piece (32 rows x 32 floats) the 16-byte vector v of row `lane` sits at slot
                // v * 32 + lane: every store instruction of the warp covers 512 contiguous bytes, and the
                // reader's shared-memory loads are free of bank conflicts
                float4* dst = reinterpret_cast<float4*>(parts + ks * kPartFloats + ((size_t)chunk * kGemmBlockM + q * 32u) * 32u) + lane;
#pragma unroll
                for (uint32_t v = 0; v < 8; ++v) {
                    if (lane_row) {
                        dst[v * 32u] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                   __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    }
                }
            }
            __syncwarp();  // every lane's partial stores are ordered before lane 0's release
            uint8_t* red = smem + S::kOffA + q * ((kChunks - 1u) * kPieceBytes);
            if (warp_rows) {
                if (lane == 0) {
                    st_release_gpu(flags + ks * 4u + q, p.splitk_epoch);
                }
                // lanes 0 .. ksplit-1 each watch one part's flag (the polls overlap instead of queueing up)
                bool ok = true;
                if (lane < ksplit && lane != ks &&
                    !wait_flag_ge_gpu(flags + lane * 4u + q, p.splitk_epoch, p.timeout_ns, p.status)) {
                    report_status(p.status, kStatusFlagTimeout, 0x100u + lane, tile, p.splitk_epoch);
                    ok = false;
                }
                alive = __all_sync(0xFFFFFFFFu, ok) && alive;
                if (lane == 0 && alive) {
                    mbar_arrive_expect_tx(&red_bar[q], (ksplit - 1u) * cps * kPieceBytes);
                    fence_proxy_async_all();  // the other parts' generic-proxy stores before this thread's bulk copies
                    uint32_t slot = 0;
                    for (uint32_t part = 0; part < ksplit; ++part) {
                        if (part == ks) {
                            continue;
                        }
                        for (uint32_t oc = 0; oc < cps; ++oc, ++slot) {
                            bulk_load(red + slot * kPieceBytes,
                                      parts + part * kPartFloats + ((size_t)(own0 + oc) * kGemmBlockM + q * 32u) * 32u,
                                      kPieceBytes, &red_bar[q]);
                        }
                    }
                }
                __syncwarp();
                alive = mbar_wait_warp(&red_bar[q], 0, p.status, 107, q, bar_ns) && alive;
                // a part that gave up writes nothing: C keeps what the caller put there
                for (uint32_t oc = 0; alive && oc < cps; ++oc) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + (own0 + oc) * 32u, r);
                    tmem_ld_wait();
                    for (uint32_t pi = 0; pi + 1u < ksplit; ++pi) {
                        // four 16-byte loads at a time: enough to hide the shared-memory latency without
                        // crowding the 32 accumulator registers
                        const uint32_t src = smem_u32(red + (pi * cps + oc) * kPieceBytes + lane * 16u);
#pragma unroll
                        for (uint32_t h = 0; h < 2; ++h) {
                            float4 f[4];
#pragma unroll
                            for (uint32_t v = 0; v < 4; ++v) {
                                f[v] = ld_shared_v4(src + (h * 4u + v) * 512u);
                            }
#pragma unroll
                            for (uint32_t v = 0; v < 4; ++v) {
                                const uint32_t e = (h * 4u + v) * 4u;
                                r[e] = __float_as_uint(__uint_as_float(r[e]) + f[v].x);
                                r[e + 1] = __float_as_uint(__uint_as_float(r[e + 1]) + f[v].y);
                                r[e + 2] = __float_as_uint(__uint_as_float(r[e + 2]) + f[v].z);
                                r[e + 3] = __float_as_uint(__uint_as_float(r[e + 3]) + f[v].w);
                            }
                        }
                    }
                    store_c_chunk<OutT>(c, p, row, n0 + (own0 + oc) * 32u, r);
                }
            }
            tcgen05_fence_before();
            if (q == 0 && lane == 0) {
                CATCCOS_TR_STAMP(p.trace, kTrEpiLast);
            }
        }
        uint32_t ti = 0;
        bool alive = true;
        for (uint32_t unit = blockIdx.x; alive && ksplit == 1u && unit < num_units; unit += gridDim.x, ++ti) {
            const uint32_t ks = unit / num_tiles;
            const uint32_t tile = unit - ks * num_tiles;
            TileCoord tc = tile_coord(tile, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kGemmBlockM;
            const uint32_t n0 = tc.n_tile * BLOCK_N;
            const uint32_t acc = ti & 1u;
            const uint32_t acc_ph = (ti >> 1) & 1u;
            const uint32_t d_col = acc ? S::kAccCol1 : 0u;
            const unsigned long long t0 = CATCCOS_TR_NOW();
            (void)t0;
            alive = mbar_wait_warp(&tmem_full[acc], acc_ph, p.status, 106, acc, bar_ns);
            if (q == 0 && lane == 0) {
                CATCCOS_TR_ADD(p.trace, kTrEpiWaitNs, CATCCOS_TR_NOW() - t0);
            }
            if (!alive) {
                break;  // an accumulator that never filled is not written out
            }
            tcgen05_fence_after();
            const uint32_t row = m0 + q * 32 + lane;
            // the chunks that hold the columns shared with the other accumulator go first: the last two of
            // accumulator 0, the first two of accumulator 1
            for (uint32_t ci = 0; ci < kChunks; ++ci) {
                uint32_t chunk = ci;
                if (S::kOverlap && acc == 0) {
                    chunk = ci < S::kOverlapChunks ? kChunks - S::kOverlapChunks + ci : ci - S::kOverlapChunks;
                }
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + d_col + chunk * 32u, r);
                tmem_ld_wait();
                if (S::kOverlap && ci == S::kOverlapChunks - 1) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&overlap_free[acc]);
                    }
                }
                store_c_chunk<OutT>(c, p, row, n0 + chunk * 32u, r);
            }
            publish_tile_rows<OutT>(p, m0 + q * 32u, tc.n_tile, n_tiles, lane);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&tmem_empty[acc]);
                if (q == 0) {
                    CATCCOS_TR_STAMP(p.trace, kTrEpiLast);
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        CATCCOS_TR_STAMP(p.trace, kTrCtaEnd);
    }
    drain_after_abort(p.status);
    if (warp == 5) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

}  // namespace catccos
