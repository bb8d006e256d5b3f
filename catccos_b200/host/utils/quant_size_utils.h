// Overflow-checked size arithmetic for the quantise operators (same contracts as the reference's
// utils/quant_size_utils.h:20-46: std::overflow_error when a product leaves the ptrdiff_t range,
// std::invalid_argument for a zero rank count).
#ifndef CATCCOS_B200_HOST_QUANT_SIZE_UTILS_H
#define CATCCOS_B200_HOST_QUANT_SIZE_UTILS_H

#include <cstddef>
#include <cstdint>
#include <initializer_list>
#include <limits>
#include <stdexcept>

inline size_t CheckedBufferSize(std::initializer_list<size_t> factors)
{
    const size_t limit = static_cast<size_t>(std::numeric_limits<ptrdiff_t>::max());
    size_t product = 1;
    for (size_t f : factors) {
        if (f != 0 && product > limit / f) {
            throw std::overflow_error("Quant buffer size exceeds the addressable range");
        }
        product *= f;
    }
    return product;
}

inline void CheckQuantBlockCount(size_t elementCount, uint32_t rankSize)
{
    if (rankSize == 0) {
        throw std::invalid_argument("Quant rank size must be positive");
    }
    const size_t tileElements = size_t(1) << 20;
    const size_t maxBlocks = (size_t(1) << 20) - 1;
    const size_t perRank = (elementCount + rankSize - 1) / rankSize;
    if (perRank > maxBlocks * tileElements) {
        throw std::overflow_error("Quant block count exceeds the synchronization flag range");
    }
}

#endif  // CATCCOS_B200_HOST_QUANT_SIZE_UTILS_H
