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

__host__ __device__ __forceinline__ uint32_t dropout_salt(unsigned long long key, uint32_t site, uint32_t hi) {
    return mix32(hi * 0x9e3779b9u + site * 0x85ebca77u + (uint32_t)key) ^ (uint32_t)(key >> 32);
}

// One hash decides a pair of neighbouring elements (ids 2q and 2q + 1) with 16 bits each: the low half for the even
// element, the high half for the odd one.  true = keep.  threshold = p * 2^32 (p the drop probability), of which the
// upper 16 bits are compared (p is honoured to 2^-16).
__host__ __device__ __forceinline__ bool dropout_keep(unsigned long long key, uint32_t site, unsigned long long id, uint32_t threshold) {
    const unsigned long long q = id >> 1;
    const uint32_t h = mix32((uint32_t)q ^ dropout_salt(key, site, (uint32_t)(q >> 32)));
    const uint32_t t = threshold & 0xffff0000u;
    return (id & 1ull) ? (h >= t) : ((h << 16) >= t);
}

// Largest logical tensor (in elements) the run form below covers: pair indices must fit 32 bits.
constexpr unsigned long long kDropoutRunMaxElems = 1ull << 33;

// The same decisions for NE consecutive elements starting at an EVEN id below 2^33, applied to v in place (kept values
// times `scale`): one hash per pair, the salts (dropout_salt(key, site, 0)) computed once by the caller.  `two`: a
// second, independent mask on top (values dropped twice).
template <int NE>
__device__ __forceinline__ void dropout_run(float (&v)[NE], uint32_t salt0, uint32_t salt1, bool two, unsigned long long id0,
                                            uint32_t threshold, float scale) {
    const uint32_t q0 = (uint32_t)(id0 >> 1), t = threshold & 0xffff0000u;
    if (!two) {
#pragma unroll
        for (int p = 0; p < NE / 2; ++p) {
            const uint32_t h = mix32((q0 + p) ^ salt0);
            v[2 * p] = ((h << 16) >= t) ? v[2 * p] * scale : 0.f;
            v[2 * p + 1] = (h >= t) ? v[2 * p + 1] * scale : 0.f;
        }
    } else {
#pragma unroll
        for (int p = 0; p < NE / 2; ++p) {
            const uint32_t h = mix32((q0 + p) ^ salt0), g = mix32((q0 + p) ^ salt1);
            v[2 * p] = ((h << 16) >= t && (g << 16) >= t) ? v[2 * p] * scale : 0.f;
            v[2 * p + 1] = (h >= t && g >= t) ? v[2 * p + 1] * scale : 0.f;
        }
    }
}

}  // namespace hsa
