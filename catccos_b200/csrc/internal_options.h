// Keys of catccos_b200_set_option that are test and tuning hooks, not part of the public boundary
// (include/catccos_b200.h lists the keys a caller may rely on).  The GPU tests use them to force every
// kernel variant through the same C ABI the operators use; a caller never needs them.
#pragma once

// 0 = automatic, 128 or 256: width of the single-CTA GEMM tile
#define CATCCOS_B200_OPT_BLOCK_N "block_n"
// bit 0 = launch the producer half, bit 1 = launch the consumer half (default 3).  The harness that hosts
// several ranks on ONE GPU runs every rank's producer before any consumer, because kernels of different
// ranks must not wait on one another while they share a device.
#define CATCCOS_B200_OPT_PHASE_MASK "phase_mask"
// 0 = automatic, 1 = always run the GEMM on CTA pairs (256 x 256 tiles, cta_group::2), 2 = never
#define CATCCOS_B200_OPT_CTA_PAIR "cta_pair"
// -1 = automatic (3 with one rank, 6 with several);
// 0 = quantise and pusher warps inside the GEMM kernel (one launch); 3 = one rank only: quantise kernel, then GEMM
// kernel on the same stream; 4 = quantise kernel into the local stage, then the GEMM kernel whose pusher warps
// forward the stage to the peers; 5 = quantise kernel, copy engines forward the stage slice by slice, flag-gated
// GEMM kernel; 6 = quantise kernel that stores every item to all ranks, flag-gated GEMM kernel launched behind it
// with programmatic stream serialisation; 7 = the ordered quantise-and-push kernel on a side stream, the flag-gated
// GEMM kernel beside it
#define CATCCOS_B200_OPT_FUSE_MODE "fuse_mode"
// 0 = automatic (K is cut in up to eight parts when the output tiles would leave half of the SMs idle),
// 1 = never, 2..8 = at most that many parts
#define CATCCOS_B200_OPT_SPLIT_K "split_k"
// order in which a flag-gated GEMM visits its row tiles: -1 = automatic (follows fuse_mode), 1 = this rank's own
// shard first, then the peers slice by slice, 0 = slice by slice over all ranks, own slice leading
#define CATCCOS_B200_OPT_TILE_ORDER "tile_order"
