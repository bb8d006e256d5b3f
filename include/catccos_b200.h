/*
 * C ABI of libcatccos_b200.so: the B200 (sm_100a) implementation of CATCCOS's MXFP8
 * quantise + AllGather and AllGather-Matmul operators.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns 0 on success
 * or a negative CATCCOS_B200_E* code.  Device errors that can only be seen after the stream has
 * run (a peer that never published a chunk) are read with catccos_b200_last_status().
 * Each comment names the reference interface the entry point stands in for
 * (paths are relative to the reference repository).
 */
#ifndef CATCCOS_B200_H
#define CATCCOS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Same 17 x uint32 layout as CocTilingParams (utils/info.h:97-115); the operators read
 * m, k, n and rankSize, the remaining fields are accepted for source compatibility. */
typedef struct catccos_b200_tiling {
    uint32_t m, k, n, transA, transB, m0, k0, n0;
    uint32_t commTileM, commInterval, commNpuSplit, commDataSplit, commBlockM;
    uint32_t rankSize, epSize, expertNum, topK;
} catccos_b200_tiling_t;

enum {
    CATCCOS_B200_OK = 0,
    CATCCOS_B200_EINVAL = -1,   /* bad shape / argument (N % 32, K % 128, rank count, null pointer) */
    CATCCOS_B200_ESTATE = -2,   /* not initialised, or initialised differently */
    CATCCOS_B200_ECUDA = -3,    /* a CUDA runtime or driver call failed (printed as "cudaError:<n>") */
    CATCCOS_B200_ENOMEM = -4,   /* symmetric buffer too small for the problem */
    CATCCOS_B200_ENET = -5,     /* rendezvous failed (connect / accept / handle exchange) */
    CATCCOS_B200_ENOTSYMM = -6, /* pointer is not inside a buffer from catccos_b200_symm_alloc */
    CATCCOS_B200_ETIMEOUT = -7  /* a device-side wait ran out (see catccos_b200_last_status) */
};

/* ---- process set-up ------------------------------------------------------------------------
 * One process per rank.  Stands in for aclInit + aclrtSetDevice + set_attr + aclshmemx_init_attr
 * (examples/ascend950_mx_quant_allgather/main.cpp:145-153, utils/shmem_init.h:18-45).
 * ip_port is the reference's rendezvous string, e.g. "tcp://127.0.0.1:8789".  world == 1 needs
 * no rendezvous (ip_port may be NULL). */
int catccos_b200_init(int rank, int world, int device, const char* ip_port);

/* Single-process harness: this process hosts all `world` ranks, rank r on devices[r] (devices may
 * repeat: several ranks on one GPU, used to exercise the multi-rank protocol on one device).
 * catccos_b200_set_rank chooses the rank the next calls act as. */
int catccos_b200_init_local(int world, const int* devices);
int catccos_b200_set_rank(int rank);

/* shmem_finalize + aclrtResetDevice + aclFinalize (main.cpp:221-224). */
int catccos_b200_finalize(void);

/* aclshmem_calloc(1, bytes) (main.cpp:169): collective, zero-filled, mapped into every rank.
 * With one process per rank the memory is a cuMem/VMM allocation exported to the peers. */
int catccos_b200_symm_alloc(size_t bytes, void** local_ptr);
/* shmem_free (main.cpp:219). */
int catccos_b200_symm_free(void* local_ptr);
/* CatccosOperator::GetSymmetricSize (utils/catccos_operator.h:43): bytes an operator needs for a problem.
 * quant_op 0 = AllGather-Matmul, 1 = quantise + AllGather (header + two stages of the gathered codes and scales),
 * 2 = Matmul + ReduceScatter (header + two stages of the fp32 product). */
size_t catccos_b200_symm_bytes_needed(const catccos_b200_tiling_t* tiling, int quant_op);

/* ---- operators -----------------------------------------------------------------------------
 * `stream` is a cudaStream_t.  `magic` is accepted and unused, as in the reference
 * (mx_quant_allgather_device.h:111-112). */

/* MxQuantAllGather<bf16, RowMajor, E4M3, RowMajor><<<rankSize, stream>>>(ffts, in, out, scale,
 * symm, tiling, magic) (examples/ascend950_mx_quant_allgather/mx_quant_allgather_device.h:108-141,
 * main.cpp:186).  The quantised axis is tiling->n (mx_quant_allgather_host.h:30-44):
 * in bf16 [m, n]; out_codes uint8 [rankSize*m, n]; out_scales uint8 [rankSize*m, n/32]. */
int catccos_b200_mx_quant_allgather(void* stream, const void* in_bf16, void* out_codes, void* out_scales, void* symm,
                                    const catccos_b200_tiling_t* tiling, uint32_t magic);

/* DeviceDGemm<MxAllGatherMatmulTla>::Arguments + Initialize + Run
 * (include/catccos/dgemm/kernel/mx_allgather_matmul.hpp:121-135,
 * include/catccos/dgemm/device/device_dgemm.hpp:77,116): A already quantised.
 * a E4M3 [m, k]; a_scale E8M0 [m, k/32]; b E4M3 [k, n]; b_scale E8M0 [k/64, n, 2];
 * c [rankSize*m, n] (bf16 by default, fp16 with option "c_dtype" = 1). */
int catccos_b200_fp8_mx_allgather_matmul(void* stream, const void* a, const void* b, const void* a_scale,
                                         const void* b_scale, void* c, void* symm,
                                         const catccos_b200_tiling_t* tiling, uint32_t magic);

/* The FP4 variant of the operator above: DeviceDGemm<MxAllGatherMatmulTla> composed with float4_e2m1x2_t operands
 * (examples/ascend950_fp4_mx_allgather_matmul/ascend950_fp4_mx_allgather_matmul_device.h:42-104).
 * a packed E2M1 [m, k/2] and b packed E2M1 [k, n/2] (two values per byte, low nibble = even column, the layout
 * examples/utils/gen_data_fp4_mx_allgather_matmul.py:521-544 writes); a_scale E8M0 [m, k/32]; b_scale E8M0
 * [k/64, n, 2]; c [rankSize*m, n].  The shards travel by the copy engines; the GEMM reads the packed codes through
 * TMA (unpacked on the way into shared memory) and runs tcgen05.mma kind::mxf8f6f4 with E2M1 operands.
 * k % 128 == 0, n % 128 == 0; a and b 32-byte aligned. */
int catccos_b200_fp4_mx_allgather_matmul(void* stream, const void* a, const void* b, const void* a_scale,
                                         const void* b_scale, void* c, void* symm,
                                         const catccos_b200_tiling_t* tiling, uint32_t magic);

/* The fused form of the two operators above (quantise kernel pushes, GEMM kernel consumes as
 * chunks land): a bf16 [m, k] quantised on the fly, everything else as above.  The reference has
 * no single entry point for it; it is MxQuantAllGather feeding MxAllGatherMatmulTla. */
int catccos_b200_mx_quant_allgather_matmul(void* stream, const void* a_bf16, const void* b, const void* b_scale,
                                           void* c, void* symm, const catccos_b200_tiling_t* tiling, uint32_t magic);

/* DeviceDGemm<MatmulReduceScatterMxTla>::Arguments + Run, the row-parallel partner of the operator above
 * (include/catccos/dgemm/kernel/matmul_reduce_scatter_mx_tla.hpp:36-135,
 * examples/ascend950_mxfp8_matmul_reduce_scatter/): every rank holds its K slice, a [m, k] and b [k, n] in MXFP8
 * with a_scale [m, k/32] and b_scale [k/64, n, 2]; the products are added over the ranks and rank r receives rows
 * [r * m / rankSize, (r + 1) * m / rankSize) as d [m / rankSize, n] (bf16, or fp16 with "c_dtype" = 1).
 * tiling->m is the WHOLE m, as in the reference's Arguments.  The GEMM's epilogue sends fp32 partial rows straight to
 * the stage of the rank that owns them; that rank adds them in rank order (the result does not depend on timing).
 * symm: catccos_b200_symm_bytes_needed(tiling, 2) bytes.  m / rankSize % 32 == 0, k % 128 == 0, n % 16 == 0. */
int catccos_b200_mxfp8_matmul_reduce_scatter(void* stream, const void* a, const void* b, const void* a_scale,
                                             const void* b_scale, void* d, void* symm,
                                             const catccos_b200_tiling_t* tiling, uint32_t magic);

/* ---- single-GPU building blocks (the compute halves, also the unfused baseline) ------------ */

/* CommBlockMxQuant::operator() (include/catccos/comm/block/comm_block_mx_quant.hpp:155-207):
 * bf16 [rows, k] -> codes [rows, k] + scales [rows, k/32], no communication. */
int catccos_b200_mx_quant(void* stream, const void* in_bf16, uint32_t rows, uint32_t k, void* codes, void* scales);

/* The FP4 branch of the same quantiser (comm_block_mx_quant.hpp:525-568; the reference's float4_e2m1x2_t output
 * type, emax 2, +-6): bf16 [rows, k] -> packed E2M1 codes [rows, k/2] (two per byte, low nibble = even column,
 * as gen_mx_quant_allgather_data.py:400-411 packs them) + scales [rows, k/32].  Round to nearest even, as the
 * reference's device cast; its CPU golden rounds ties toward zero instead, and the two agree on the dequantised
 * tensors the reference feeds its kernel.  No communication, and no GEMM reads these codes yet. */
int catccos_b200_mx_quant_fp4(void* stream, const void* in_bf16, uint32_t rows, uint32_t k, void* packed, void* scales);

/* BlockMmadTla<MmadMx> main loop on data that is already gathered
 * (ascend950_fp8_mx_allgather_matmul_device.h:47-57): c [m, n] = dequant(a)[m, k] x dequant(b)[k, n]. */
int catccos_b200_mx_gemm(void* stream, const void* a, const void* a_scale, const void* b, const void* b_scale, void* c,
                         uint32_t m, uint32_t n, uint32_t k);

/* The same GEMM with the MX quantiser in its epilogue: every 32 consecutive output columns of a row are rounded to
 * bf16, quantised (E4M3 codes + one E8M0 scale) and written as c_codes [m, n] and c_scales [m, n/32]; the 16-bit
 * tensor is never materialised.  CommBlockMxQuant::QuantFromUb / QuantFromUb2D
 * (include/catccos/comm/block/comm_block_mx_quant.hpp:209-310), the reference's quantise-in-epilogue producer.
 * n % 32 == 0.  The result equals catccos_b200_mx_quant applied to the bf16 output of catccos_b200_mx_gemm. */
int catccos_b200_mx_gemm_quant_out(void* stream, const void* a, const void* a_scale, const void* b, const void* b_scale,
                                   void* c_codes, void* c_scales, uint32_t m, uint32_t n, uint32_t k);

/* CommBlockMxQuant::QuantScatterPacked (comm_block_mx_quant.hpp:312-368), the routing-side producer of the packed
 * MoE dispatch: token t (bf16 [n]) is quantised once and its packed row is written to rows
 * expanded_row_idx[t * top_k + r], r < top_k, of packed_out (negative entries drop the route).  A packed row is
 * [n E4M3 codes | n/32 E8M0 scales, padded to an even count | zeros to a multiple of 32 bytes];
 * catccos_b200_packed_row_bytes(n) is its length.  n % 32 == 0; in_bf16 and packed_out 16-byte aligned. */
size_t catccos_b200_packed_row_bytes(uint32_t n);
int catccos_b200_mx_quant_scatter_packed(void* stream, const void* in_bf16, const int32_t* expanded_row_idx, void* packed_out,
                                         uint32_t tokens, uint32_t n, uint32_t top_k);

/* Fused quantise + matmul on one GPU that allocates nothing.  It has no counterpart in the reference.
 * c [m, n] = dequant(quantise(a_bf16 [m, k])) x dequant(b [k, n], b_scale [k/64, n, 2]): the same two
 * fused stages as catccos_b200_mx_quant_allgather_matmul at rankSize 1, but the quantised copy of A and
 * its ready flags live in an array that is part of the library image (a file-scope __device__ array of
 * about 8.3 MiB that every GPU loading the library holds until the process exits) instead of a buffer
 * from catccos_b200_symm_alloc.
 *
 * It is meant for callers that must not allocate device memory where the call is made: code that runs
 * inside a region whose memory was planned ahead of time (an inference server that reserved all of HBM
 * for its own pools at start-up, so a late cudaMalloc fails or fragments them), and latency-critical
 * loops where an allocation would serialise the device.  The call itself makes no cudaMalloc, cudaFree
 * or other allocating call; inputs and the output are the caller's.
 *
 * Limits: m * k <= 8 Mi elements (8 388 608) and at most 8192 (16-row chunk, K segment) pairs, else
 * CATCCOS_B200_ENOMEM with an [ERROR] line; k % 128 == 0, n % 16 == 0.  The first call on each device
 * looks up the array's device address (that device must be current) and should therefore be made
 * before any stream capture begins.  All calls on a device share the one array, which keeps the last
 * call's contents: calls are correct back to back on one stream, but two calls whose kernels overlap
 * on the GPU (different streams, no dependency) race on it.  The kernels that the first call of a new shape
 * class (tile width, output type) launches are configured on that first launch as well, so make one call per
 * shape class before capture.  Device-side wait records of this path are kept in the same array and read with
 * catccos_b200_mx_quant_matmul_static_status, not with catccos_b200_last_status. */
int catccos_b200_mx_quant_matmul_static(void* stream, const void* a_bf16, const void* b, const void* b_scale, void* c,
                                        uint32_t m, uint32_t n, uint32_t k);

/* catccos_b200_last_status for the entry point above: synchronises the current device and copies the 16-byte
 * record of its last call out of the built-in array (out[] as below).  Allocates nothing.  Returns
 * CATCCOS_B200_ESTATE before the first call on the device, CATCCOS_B200_ETIMEOUT when a wait ran out.
 * No counterpart in the reference. */
int catccos_b200_mx_quant_matmul_static_status(uint32_t out[4]);

/* ---- status and options ---------------------------------------------------------------------
 * out[0] code (0 ok, 1 ready-flag timeout, 2 internal barrier timeout, 3 handshake timeout),
 * out[1] rank waited for, out[2] chunk, out[3] epoch.  Synchronises the device, clears the record.
 * The reference has no counterpart: its waits are unbounded (mx_quant_allgather.hpp:179-185). */
int catccos_b200_last_status(uint32_t out[4]);

/* Options (all ranks must set the same values; set them while no call is in flight):
 *   "tiny_block_rule" 0 = CPU golden (amax < 1e-12 -> scale 0x7F), 1 = reference device kernel
 *   "c_dtype"         0 = bf16, 1 = fp16 (the reference's output type, main.cpp:28)
 *   "a_dtype"         element type of the A codes, written by the quantiser and read by the GEMM: 0 = E4M3
 *                     (emax 8, +-448), 1 = E5M2 (emax 15, +-57344; MX_QUANT_DTYPE = 1 in the reference,
 *                     comm_block_mx_quant.hpp:75-76,410), 2 = packed E2M1 (catccos_b200_mx_gemm only: a is
 *                     [m, k/2]; the fused quantisers write 8-bit codes)
 *   "b_dtype"         element type of the B codes the caller passes: 0 = E4M3, 1 = E5M2, 2 = packed E2M1
 *                     [k, n/2] (transposed into a per-rank scratch on every call: the tensor core reads 4-bit
 *                     operands K-major only)
 *   "timeout_ms"      limit of device-side waits on peers (default 2000)
 * Any other key is rejected with CATCCOS_B200_EINVAL, except the test hooks that
 * catccos_b200/csrc/internal_options.h lists (they force kernel variants and are not part of this boundary).
 * The kernels choose their own tiling: CTA pairs (256 x 256 tiles) for more than one wave of work, K cut in
 * up to eight parts when the tiles would leave half of the SMs idle (the partial tiles meet in a per-rank
 * scratch allocated when the rank is set up; because of it, and of the symmetric buffer's epochs, the operator
 * calls of one rank must not overlap on the GPU). */
int catccos_b200_set_option(const char* key, int64_t value);

/* Number of kernels this library has launched since it was loaded. */
uint64_t catccos_b200_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* CATCCOS_B200_H */
