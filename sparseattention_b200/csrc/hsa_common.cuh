// Shared device/host helpers for the hsa_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hsa_b200.h"

namespace hsa {

// ---------------------------------------------------------------- errors ----
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define HSA_CHECK_ARG(cond, ...)                                  \
    do {                                                          \
        if (!(cond)) return ::hsa::fail(HSA_ERR_ARG, __VA_ARGS__); \
    } while (0)

inline int launch_status(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
    return 0;
}

inline int dtype_size(int dtype) { return dtype == HSA_F32 ? 4 : 2; }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Can rows of this view be read with 16-byte vector accesses?
inline bool view_vec_ok(const hsa_view &v, int esize) {
    const int64_t vec = 16 / esize;
    return aligned16(v.ptr) && (v.batch_stride % vec == 0) && (v.row_stride % vec == 0);
}

// ------------------------------------------------------------ tree closed forms
// Row of the first node of level l (l >= 1) in the [leaves | parents] ordering; level 0 = leaves.
__host__ __device__ __forceinline__ int level_base(int N, int l) {
    return l == 0 ? 0 : 2 * N - (N >> (l - 1));
}
// Key row leaf n attends to at level l: the sibling of n's ancestor at that level.
__host__ __device__ __forceinline__ int sibling_row(int N, int n, int l) {
    return level_base(N, l) + ((n >> l) ^ 1);
}

// --------------------------------------------------------------- dtype traits
template <typename T> struct Traits;
template <> struct Traits<float> {
    static constexpr int kVec = 4;
    __device__ static __forceinline__ float to_f(float v) { return v; }
    __device__ static __forceinline__ float from_f(float v) { return v; }
};
template <> struct Traits<__nv_bfloat16> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Traits<__half> {
    static constexpr int kVec = 8;
    __device__ static __forceinline__ float to_f(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

// Load / store VEC consecutive elements as floats.  VEC is either the 16-byte width of T or 1.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T *__restrict__ p, float (&out)[VEC]) {
    if constexpr (VEC == 1) {
        out[0] = Traits<T>::to_f(*p);
    } else if constexpr (sizeof(T) == 4) {
        const float4 v = *reinterpret_cast<const float4 *>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) out[i] = Traits<T>::to_f(e[i]);
    }
}

template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T *__restrict__ p, const float (&in)[VEC]) {
    if constexpr (VEC == 1) {
        *p = Traits<T>::from_f(in[0]);
    } else if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4 *>(p) = make_float4(in[0], in[1], in[2], in[3]);
    } else {
        uint4 raw;
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) e[i] = Traits<T>::from_f(in[i]);
        *reinterpret_cast<uint4 *>(p) = raw;
    }
}

// Lane mask of the calling thread's row group (LPR a power of two <= 32, groups aligned in the warp).
// Groups of one warp may sit in loops of different lengths, so shuffles name only their own lanes.
template <int LPR>
__device__ __forceinline__ unsigned group_mask() {
    if constexpr (LPR == 32) return 0xffffffffu;
    else return ((1u << LPR) - 1u) << ((threadIdx.x & 31u) / LPR * LPR);
}

// Sum over the LPR lanes of a row group.
template <int LPR>
__device__ __forceinline__ float group_sum(float v, unsigned mask = group_mask<LPR>()) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
    return v;
}

// A row of D elements spread over LPR lanes, CPL vector chunks of VEC elements per lane:
// lane g owns chunks g, g+LPR, ... (chunk c covers elements [c*VEC, (c+1)*VEC)).
template <typename T, int VEC, int LPR, int CPL>
struct RowFrag {
    float v[CPL][VEC];

    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[c][i] = 0.f;
    }
    __device__ __forceinline__ void load(const T *__restrict__ row, int g, int nchunks) {
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            const int ch = g + c * LPR;
            if (ch < nchunks) {
                load_vec<T, VEC>(row + (int64_t)ch * VEC, v[c]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[c][i] = 0.f;
            }
        }
    }
    __device__ __forceinline__ void store(T *__restrict__ row, int g, int nchunks) const {
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            const int ch = g + c * LPR;
            if (ch < nchunks) store_vec<T, VEC>(row + (int64_t)ch * VEC, v[c]);
        }
    }
    __device__ __forceinline__ float dot_partial(const RowFrag &o) const {
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
            for (int i = 0; i < VEC; ++i) s = fmaf(v[c][i], o.v[c][i], s);
        return s;
    }
    __device__ __forceinline__ void axpy(float a, const RowFrag &o) {
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[c][i] = fmaf(a, o.v[c][i], v[c][i]);
    }
    __device__ __forceinline__ void scale(float a) {
#pragma unroll
        for (int c = 0; c < CPL; ++c)
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[c][i] *= a;
    }
};

// ------------------------------------------------- row-group shape dispatch
// Chooses (VEC, LPR, CPL) for rows of D elements and calls f.template operator()<T,VEC,LPR,CPL>().
// Vector path: D a multiple of the 16-byte width and all views 16-byte addressable.
// Returns false if D is too large for the instantiated shapes.
template <typename T, typename F>
bool dispatch_row_shape(int D, bool vec_ok, F &&f) {
    constexpr int V = Traits<T>::kVec;
    if (vec_ok && D % V == 0) {
        const int chunks = D / V;
        if (chunks <= 4) { f.template operator()<T, V, 4, 1>(); return true; }
        if (chunks <= 8) { f.template operator()<T, V, 8, 1>(); return true; }
        if (chunks <= 16) { f.template operator()<T, V, 16, 1>(); return true; }
        if (chunks <= 32) { f.template operator()<T, V, 32, 1>(); return true; }
        if (chunks <= 64) { f.template operator()<T, V, 32, 2>(); return true; }
        return false;
    }
    if (D <= 32) { f.template operator()<T, 1, 32, 1>(); return true; }
    if (D <= 64) { f.template operator()<T, 1, 32, 2>(); return true; }
    if (D <= 128) { f.template operator()<T, 1, 32, 4>(); return true; }
    if (D <= 256) { f.template operator()<T, 1, 32, 8>(); return true; }
    return false;
}

template <typename F>
int dispatch_dtype(int dtype, F &&f) {
    switch (dtype) {
        case HSA_F32: return f.template operator()<float>();
        case HSA_BF16: return f.template operator()<__nv_bfloat16>();
        case HSA_F16: return f.template operator()<__half>();
        default: return fail(HSA_ERR_DTYPE, "unknown dtype code %d", dtype);
    }
}

// Largest D the row-group kernels accept for a dtype (vector path / scalar path).
inline int max_head_dim(int dtype, bool vec) { return vec ? 64 * (16 / dtype_size(dtype)) : 256; }

__host__ __device__ __forceinline__ int ilog2(unsigned v) {
    int l = 0;
    while (v > 1) { v >>= 1; ++l; }
    return l;
}

}  // namespace hsa
