// Counter-based dropout masks: whether element `id` of dropout site `site` is kept is a pure function of
// (key, site, id), so the forward (a product's epilogue) and the backward (a separate pass, possibly much later)
// regenerate the same mask without storing it.  `key` is read from device memory (seed + step counter, advanced
// by the host once per training step with an ordinary kernel), so a step captured in a CUDA graph draws new masks
// at every replay.
#pragma once

#include <stdint.h>

namespace hsa {

__host__ __device__ __forceinline__ uint32_t mix32(uint32_t h) {   // the 32-bit finaliser of MurmurHash3
    h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return h;
}

// true = keep.  threshold = p * 2^32 (p the drop probability).
__host__ __device__ __forceinline__ bool dropout_keep(unsigned long long key, uint32_t site, unsigned long long id, uint32_t threshold) {
    const uint32_t lo = (uint32_t)id, hi = (uint32_t)(id >> 32);
    const uint32_t salt = mix32(hi * 0x9e3779b9u + site * 0x85ebca77u + (uint32_t)key) ^ (uint32_t)(key >> 32);
    return mix32(lo ^ salt) >= threshold;
}

}  // namespace hsa
