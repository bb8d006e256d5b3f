// Process set-up for one rank: what the reference does with aclInit + aclrtSetDevice + set_attr +
// aclshmemx_init_attr (utils/shmem_init.h:18-45, examples/ascend950_mx_quant_allgather/main.cpp:145-153)
// is one call into the C ABI here.  The symmetric heap is not pre-sized: buffers are created on demand.
#ifndef CATCCOS_B200_HOST_SHMEM_INIT_H
#define CATCCOS_B200_HOST_SHMEM_INIT_H

#include <cstdint>
#include <cstdlib>

#include "../../../include/catccos_b200.h"

constexpr int CATCCOS_SHMEM_SUCCESS = 0;

inline int set_attr(int rankId, int rankSize, uint64_t /*localMemSize*/, const char* ipPort, int deviceId)
{
    return catccos_b200_init(rankId, rankSize, deviceId, ipPort);
}

inline void* shmem_calloc(size_t count, size_t size)
{
    void* p = nullptr;
    return catccos_b200_symm_alloc(count * size, &p) == 0 ? p : nullptr;
}

inline void shmem_free(void* p) { catccos_b200_symm_free(p); }
inline int shmem_finalize() { return catccos_b200_finalize(); }

#endif  // CATCCOS_B200_HOST_SHMEM_INIT_H
