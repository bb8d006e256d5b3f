// Device-side timeline of the fused kernels, compiled in only with -DCATCCOS_TRACE (the second library,
// libcatccos_b200_trace.so; the product build carries none of it).  One thread per role writes
// %globaltimer stamps and accumulated wait times into a side buffer, kTraceSlots 64-bit words per CTA, which
// the host reads back after a chosen launch (catccos_b200_trace_arm / catccos_b200_trace_read).  It is the
// stand-in for the reference's AscendTimer hook points
// (include/catccos/comm/kernel/mx_quant_allgather.hpp:105-119,160-162,284-286).
#pragma once

#include <stdint.h>

namespace catccos {

constexpr uint32_t kTraceSlots = 80;
constexpr uint32_t kTraceTiles = 9;   // per-tile stamps are kept for the first nine tiles of a CTA
constexpr uint32_t kTracePushers = 6;

// Slots holding a time are nanoseconds of this GPU's %globaltimer; slots named *Ns are accumulated waits.
enum TraceSlot : uint32_t {
    kTrCtaStart = 0,
    kTrSetupDone = 1,       // barriers initialised, tensor memory allocated, the roles split up
    kTrProdFirstTma = 2,    // TMA producer: first operand load issued
    kTrProdLastTma = 3,     //               last operand load issued
    kTrProdFlagWaitNs = 4,  //               time spent waiting for ready flags
    kTrProdEmptyWaitNs = 5, //               time spent waiting for a free stage
    kTrMmaFirst = 6,        // MMA issuer: first MMA issued
    kTrMmaLast = 7,         //             last tile committed
    kTrMmaFullWaitNs = 8,   //             time spent waiting for full stages (operands or scales late)
    kTrMmaAccWaitNs = 9,    //             time spent waiting for a free accumulator (epilogue late)
    kTrEpiLast = 10,        // epilogue warp 0: last tile written
    kTrEpiWaitNs = 11,      //                  time spent waiting for accumulators
    kTrQuantFirstDone = 12, // quantise group: first work item published
    kTrQuantDone = 13,      //                 last work item published
    kTrQuantPublishNs = 14, //                 time thread 0 spent in barrier + fence + flag stores
    kTrQuantItems = 15,     //                 work items done by this CTA
    kTrPushFirst = 16,      // + pusher index: first item's local flag seen
    kTrPushLast = 22,       // + pusher index: last item's peer flags stored
    kTrPushFlagWaitNs = 28, // + pusher index: time waiting for the quantise warps' local flags
    kTrPushFenceNs = 34,    // + pusher index: time in the system-scope fence before the peer flags
    kTrPushItems = 40,      // + pusher index: items pushed
    kTrTileStart = 46,      // + tile index: TMA producer starts the tile (its first flag wait is over)
    kTrTileEnd = 55,        // + tile index: MMA issuer commits the tile
    kTrSfGateWaitNs = 64,   // + scale-loader index: time waiting for ready flags
    kTrSfEmptyWaitNs = 68,  // + scale-loader index: time waiting for a free stage
    kTrCtaEnd = 72,
    kTrQuantKernelStart = 73,  // row 0 only: earliest CTA start of the stand-alone quantise kernel (atomic min)
    kTrQuantKernelEnd = 74,    // row 0 only: latest CTA end of the stand-alone quantise kernel (atomic max)
};

#ifdef CATCCOS_TRACE
#define CATCCOS_TR_NOW() ::catccos::globaltimer_ns()
#define CATCCOS_TR_STAMP(tr, slot)                                                       \
    do {                                                                                 \
        if ((tr) != nullptr) (tr)[(size_t)blockIdx.x * ::catccos::kTraceSlots + (slot)] = ::catccos::globaltimer_ns(); \
    } while (0)
#define CATCCOS_TR_STAMP_FIRST(tr, slot)                                                 \
    do {                                                                                 \
        if ((tr) != nullptr && (tr)[(size_t)blockIdx.x * ::catccos::kTraceSlots + (slot)] == 0ull)                     \
            (tr)[(size_t)blockIdx.x * ::catccos::kTraceSlots + (slot)] = ::catccos::globaltimer_ns();                  \
    } while (0)
#define CATCCOS_TR_ADD(tr, slot, v)                                                      \
    do {                                                                                 \
        if ((tr) != nullptr) (tr)[(size_t)blockIdx.x * ::catccos::kTraceSlots + (slot)] += (v);                        \
    } while (0)
#else
#define CATCCOS_TR_NOW() 0ull
#define CATCCOS_TR_STAMP(tr, slot) do { } while (0)
#define CATCCOS_TR_STAMP_FIRST(tr, slot) do { } while (0)
#define CATCCOS_TR_ADD(tr, slot, v) do { } while (0)
#endif

}  // namespace catccos
