// The host operator interface callers program against, source-compatible with the reference
// (utils/catccos_operator.h:35-54): same virtuals, same non-virtual ValidateCocTilingParams that ANDs
// the common check with the operator's own, same OperatorCreator alias.
#ifndef CATCCOS_B200_HOST_CATCCOS_OPERATOR_H
#define CATCCOS_B200_HOST_CATCCOS_OPERATOR_H

#include <cstring>
#include <functional>
#include <iostream>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "info.h"
#include "shmem_init.h"
#include "utils.h"

class CatccosOperator {
public:
    virtual ~CatccosOperator() = default;

    bool ValidateCocTilingParams(uint32_t rankSize, const CocTilingParams& cocTiling)
    {
        if (!CheckCommonCocTilingParams(rankSize, cocTiling)) {
            return false;
        }
        return CheckCocTilingParams(rankSize, cocTiling);
    }

    // Bytes of symmetric memory a call needs (data stages and flag words, one allocation the caller
    // frees).  The default is the reference's fixed buffer size; both operators here return the true need.
    virtual size_t GetSymmetricSize(const CocTilingParams&) { return SHMEM_BUFF_BYTES; }

    virtual bool CheckCocTilingParams(uint32_t rankSize, const CocTilingParams& cocTiling) = 0;
    virtual void AllocateDeviceSpace(KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                                     std::string dataFile = "") = 0;
    virtual void WriteResultFile(const KernelParams& params, const CocTilingParams& cocTiling, uint32_t rankId,
                                 std::string dataFile = "") = 0;
    virtual size_t GetWorkspaceSize(const CocTilingParams& cocTiling) = 0;
    virtual CocCommType GetActualKernelType(const CocTilingParams& cocTiling) = 0;
};

using OperatorCreator = std::function<std::unique_ptr<CatccosOperator>()>;

#endif  // CATCCOS_B200_HOST_CATCCOS_OPERATOR_H
