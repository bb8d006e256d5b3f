// Shared device helpers for the sm_100a kernels: status words, bounded waits, mbarrier / TMA /
// tcgen05 PTX wrappers.  Every spin in this library goes through a bounded wait.  When a limit runs
// out the waiter records what it was waiting for in the status block; from then on the status word
// is non-zero and every other wait of the kernel gives up as soon as it looks (a few hundred polls),
// so that the kernel drains within microseconds instead of one limit per wait, frees its tensor
// memory and returns even when a peer never shows up.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace catccos {

constexpr int kMaxRanks = 8;  // one NVSwitch box; the reference scripts cap ranks per host at 8 too

// Error codes written to StatusBlock::code (0 = ok).  The host reads them after the stream
// has been synchronised; the C ABI returns them from catccos_b200_last_status.
enum StatusCode : uint32_t {
    kStatusOk = 0,
    kStatusFlagTimeout = 1,      // a (source rank, chunk) ready flag did not arrive in time
    kStatusBarrierTimeout = 2,   // an intra-kernel mbarrier wait ran out (a bug, never a peer)
    kStatusHandshakeTimeout = 3, // a peer did not enter the collective in time
};

struct StatusBlock {
    uint32_t code;   // first error wins
    uint32_t rank;   // the rank waited for (or the barrier id)
    uint32_t chunk;  // the chunk waited for (or stage index)
    uint32_t epoch;  // the epoch the waiter expected
};

__device__ __forceinline__ void report_status(StatusBlock* st, uint32_t code, uint32_t rank, uint32_t chunk,
                                              uint32_t epoch)
{
    if (st != nullptr && atomicCAS(&st->code, 0u, code) == 0u) {
        st->rank = rank;
        st->chunk = chunk;
        st->epoch = epoch;
        __threadfence_system();
    }
}

// 32-byte store (one full sector); the address must be 32-byte aligned
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&v)[8])
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]),
                 "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// The same pair at GPU scope, for flags that never leave this GPU.
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// True once some waiter of this kernel (or of an earlier, unread one) has given up.
__device__ __forceinline__ bool status_tripped(const StatusBlock* st)
{
    return st != nullptr && *reinterpret_cast<const volatile uint32_t*>(&st->code) != 0u;
}

__device__ __forceinline__ bool wait_flag_ge_gpu(const uint32_t* flag, uint32_t want, uint64_t timeout_ns,
                                                 const StatusBlock* st = nullptr)
{
    if ((int32_t)(ld_acquire_gpu(flag) - want) >= 0) {
        return true;
    }
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if ((int32_t)(ld_acquire_gpu(flag) - want) >= 0) {
            return true;
        }
        if ((++spins & 0x3Fu) == 0u) {
            if (globaltimer_ns() - t0 > timeout_ns || status_tripped(st)) {
                return false;
            }
            __nanosleep(32);
        }
    }
}

// Waits until *flag >= want (epochs only grow).  Returns false when timeout_ns ran out or another waiter
// has already given up.  The spin reads with relaxed system-scope loads (every poll is one L2 access and
// nothing else); the acquire that orders the data behind the flag is done once, when the value is there.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, uint64_t timeout_ns,
                                             const StatusBlock* st = nullptr)
{
    if ((int32_t)(ld_relaxed_sys(flag) - want) < 0) {
        const uint64_t t0 = globaltimer_ns();
        uint32_t spins = 0;
        while ((int32_t)(ld_relaxed_sys(flag) - want) < 0) {
            if ((++spins & 0x3Fu) == 0u) {
                if (globaltimer_ns() - t0 > timeout_ns || status_tripped(st)) {
                    return false;
                }
                __nanosleep(64);
            }
        }
    }
    return (int32_t)(ld_acquire_sys(flag) - want) >= 0;
}

// ------------------------------------------------------------------------------------------
// shared memory / mbarrier
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded mbarrier wait.  limit_ns is set by the host above the peer-flag limit (a barrier may legitimately
// wait for as long as the flag wait it depends on); if it runs out, or another waiter has already given up,
// the caller gets false and carries on with whatever is in shared memory, which keeps the grid from hanging.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, StatusBlock* st, uint32_t id, uint32_t stage,
                                          uint64_t limit_ns)
{
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xFFu) == 0u) {
            if (status_tripped(st)) {
                return false;
            }
            if (globaltimer_ns() - t0 > limit_ns) {
                report_status(st, kStatusBarrierTimeout, id, stage, parity);
                return false;
            }
        }
    }
    return true;
}

// The same wait made by all 32 lanes of a warp, with one answer for the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, StatusBlock* st, uint32_t id,
                                               uint32_t stage, uint64_t limit_ns)
{
    return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, st, id, stage, limit_ns));
}

__device__ __forceinline__ void fence_proxy_async_shared()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_all()
{
    asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, this GPU's memory only, never cluster multicast)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, uint64_t* bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

// Untiled bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may
// start while its predecessor in the stream still runs; grid_dep_wait() then blocks until the predecessor has
// finished and its writes are visible (and returns at once in a plain launch).  grid_dep_launch() in the
// predecessor lets the successor's CTAs be scheduled as soon as SM resources allow.
__device__ __forceinline__ void grid_dep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_dep_launch()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ------------------------------------------------------------------------------------------
// tcgen05: tensor memory, UMMA descriptors, MMA issue
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Makes the mbarrier track completion of all tcgen05 operations issued so far by this thread.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets
// (each >> 4), descriptor version 1 at bit 46, swizzle mode in bits 61..63
// (0 none, 2 = 128-byte swizzle, 4 = 64-byte, 6 = 32-byte).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(layout_type & 7u) << 61;
    return d;
}

// Instruction descriptor for tcgen05.mma.kind::mxf8f6f4.block_scale with E4M3 x E4M3 operands,
// UE8M0 scale factors and fp32 accumulation.
//   bits  4..5  B scale-factor id (which byte of the 32-bit scale word)
//   bits  7..9  A format (0 = E4M3)      bits 10..12 B format (0 = E4M3)
//   bit  15     A major (0 = K)          bit  16     B major (0 = K, 1 = MN)
//   bits 17..22 N >> 3                   bit  23     scale format (1 = UE8M0)
//   bits 24..28 M >> 4                   bits 29..30 A scale-factor id
__host__ __device__ constexpr uint32_t make_idesc_mxf8(uint32_t M, uint32_t N, bool b_mn_major)
{
    return (0u << 7) | (0u << 10) | (0u << 15) | ((b_mn_major ? 1u : 0u) << 16) | ((N >> 3) << 17) | (1u << 23) |
           ((M >> 4) << 24);
}

__device__ __forceinline__ uint32_t idesc_with_sf_id(uint32_t idesc, uint32_t sf_id)
{
    return idesc | (sf_id << 4) | (sf_id << 29);
}

__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// The same instructions taking the 64-bit descriptors as (low, high) halves: the issuing thread keeps the
// constant high halves in registers and only adds to the low half (the start address), which keeps its
// instruction count per K tile small - the tensor pipe queues only a couple of MMAs ahead, so a slow
// issuing thread starves it.
__device__ __forceinline__ void umma_mxf8_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                               uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%7], [%8], p;\n\t"
        "}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(tmem_sfa),
          "r"(tmem_sfb)
        : "memory");
}

__device__ __forceinline__ void tcgen05_cp_sf_lohi(uint32_t tmem_dst, uint32_t lo, uint32_t hi)
{
    asm volatile(
        "{\n\t"
        ".reg .b64 d;\n\t"
        "mov.b64 d, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t"
        "}"
        ::"r"(tmem_dst), "r"(lo), "r"(hi)
        : "memory");
}

// Copies one 512-byte scale-factor atom (32 rows x 16 bytes) from shared memory into four
// tensor-memory columns, replicated over the four 32-lane groups.
__device__ __forceinline__ void tcgen05_cp_sf(uint32_t tmem_dst, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (lane = TMEM lane).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace catccos

// ------------------------------------------------------------------------------------------
// CTA pairs (clusters of two, tcgen05 cta_group::2)
// ------------------------------------------------------------------------------------------
namespace catccos {

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of the location that `local_smem_addr` names in CTA `cta_rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta_rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
    return r;
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
                 "r"(bytes)
                 : "memory");
}

// Bounded wait on a barrier that the other CTA of the pair arrives on.  What these barriers guard moves
// through the async proxies (TMA, tcgen05), so the default CTA-scope acquire is what is needed; a
// cluster-scope acquire on every poll costs several hundred nanoseconds.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, StatusBlock* st, uint32_t id,
                                                  uint32_t stage, uint64_t limit_ns)
{
    return mbar_wait(bar, parity, st, id, stage, limit_ns);
}

// TMA tile load issued by either CTA of a pair; the completion bytes are credited to the barrier at
// `bar_cluster_addr`, which may live in the other CTA.  No multicast: every CTA loads its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int32_t x,
                                                 int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Arrives on the barrier at the same shared-memory offset in every CTA of cta_mask once all tcgen05
// operations issued so far by this thread have completed.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(cta_mask)
                 : "memory");
}

__device__ __forceinline__ void umma_mxf8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

__device__ __forceinline__ void umma_mxf8_pair_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                    uint32_t b_hi, uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                    uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%7], [%8], p;\n\t"
        "}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(tmem_sfa),
          "r"(tmem_sfb)
        : "memory");
}

__device__ __forceinline__ void tcgen05_cp_sf_pair_lohi(uint32_t tmem_dst, uint32_t lo, uint32_t hi)
{
    asm volatile(
        "{\n\t"
        ".reg .b64 d;\n\t"
        "mov.b64 d, {%1, %2};\n\t"
        "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t"
        "}"
        ::"r"(tmem_dst), "r"(lo), "r"(hi)
        : "memory");
}

__device__ __forceinline__ void tcgen05_cp_sf_pair(uint32_t tmem_dst, uint64_t smem_desc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_desc) : "memory");
}

}  // namespace catccos
