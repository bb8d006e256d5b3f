/*
 * Device-side timeline of the fused kernels.  Only libcatccos_b200_trace.so (the library built with
 * -DCATCCOS_TRACE) exports these two entry points; the product library carries no timeline code.
 * They have no counterpart in the reference's operator interface; what they stand in for is its AscendTimer
 * hook points (include/catccos/comm/kernel/mx_quant_allgather.hpp:105-119,160-162,284-286).
 */
#ifndef CATCCOS_B200_TRACE_H
#define CATCCOS_B200_TRACE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The next GEMM launch of the acting rank (stand-alone or fused) writes its timeline: one row of `slots`
 * 64-bit words per CTA, nanoseconds of that GPU's %globaltimer or accumulated waits (slot meanings:
 * catccos_b200/csrc/trace.cuh). */
int catccos_b200_trace_arm(void);

/* Synchronises the device and copies the timeline of the last armed launch: out[cta * slots + slot]. */
int catccos_b200_trace_read(unsigned long long* out, uint32_t max_words, uint32_t* grid, uint32_t* slots);

#ifdef __cplusplus
}
#endif

#endif /* CATCCOS_B200_TRACE_H */
