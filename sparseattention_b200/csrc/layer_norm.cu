// LayerNorm over the last dimension, forward and backward, for the LM that calls the attention layer.
//
// One warp per row; the row lives in registers (NV float4 pieces per lane, d = 128 * NV).  The backward
// walks rows with a grid stride, so every warp also accumulates its share of the weight / bias gradients in
// registers; warps of a CTA are combined in warp order in shared memory, CTAs by a second kernel in CTA order
// (deterministic, no atomics).  HBM traffic: x once forward (+ y); x, dy once backward (+ dx).
#include "hsa_common.cuh"

namespace hsa {

constexpr int kLnWarps = 8;

template <typename T>
__device__ __forceinline__ float4 ln_load4(const T *p) {
    if constexpr (sizeof(T) == 4) {
        return *reinterpret_cast<const float4 *>(p);
    } else {
        const uint2 raw = *reinterpret_cast<const uint2 *>(p);
        const T *e = reinterpret_cast<const T *>(&raw);
        return make_float4(Traits<T>::to_f(e[0]), Traits<T>::to_f(e[1]), Traits<T>::to_f(e[2]), Traits<T>::to_f(e[3]));
    }
}
template <typename T>
__device__ __forceinline__ void ln_store4(T *p, float4 v) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4 *>(p) = v;
    } else {
        uint2 raw;
        T *e = reinterpret_cast<T *>(&raw);
        e[0] = Traits<T>::from_f(v.x); e[1] = Traits<T>::from_f(v.y); e[2] = Traits<T>::from_f(v.z); e[3] = Traits<T>::from_f(v.w);
        *reinterpret_cast<uint2 *>(p) = raw;
    }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// lane l owns columns 4*(l + 32*i) .. +3 for i < NV (consecutive lanes read consecutive 16-byte pieces)
template <typename T, int NV, typename TY = T>
__global__ void __launch_bounds__(kLnWarps * 32)
layer_norm_fwd_kernel(const T *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                      TY *__restrict__ y, float *__restrict__ mean, float *__restrict__ rstd, int64_t rows, float eps,
                      TY *__restrict__ xcopy = nullptr /* optional: the input rows themselves, converted to TY */) {
    constexpr int d = 128 * NV;
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * kLnWarps;
    float4 g[NV], bt[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        g[i] = *reinterpret_cast<const float4 *>(gamma + 4 * (lane + 32 * i));
        bt[i] = *reinterpret_cast<const float4 *>(beta + 4 * (lane + 32 * i));
    }
    for (int64_t r = (int64_t)blockIdx.x * kLnWarps + (threadIdx.x >> 5); r < rows; r += warps) {
        float4 v[NV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            v[i] = ln_load4<T>(x + r * d + 4 * (lane + 32 * i));
            s += v[i].x + v[i].y + v[i].z + v[i].w;
        }
        if (xcopy != nullptr) {
#pragma unroll
            for (int i = 0; i < NV; ++i) ln_store4<TY>(xcopy + r * d + 4 * (lane + 32 * i), v[i]);
        }
        const float mu = warp_sum(s) * (1.f / d);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            v[i].x -= mu; v[i].y -= mu; v[i].z -= mu; v[i].w -= mu;
            q += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        const float rs = rsqrtf(warp_sum(q) * (1.f / d) + eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float4 o;
            o.x = v[i].x * rs * g[i].x + bt[i].x; o.y = v[i].y * rs * g[i].y + bt[i].y;
            o.z = v[i].z * rs * g[i].z + bt[i].z; o.w = v[i].w * rs * g[i].w + bt[i].w;
            ln_store4<TY>(y + r * d + 4 * (lane + 32 * i), o);
        }
        if (lane == 0) { mean[r] = mu; rstd[r] = rs; }
    }
}

template <typename T, int NV, typename TY = T>
__global__ void __launch_bounds__(kLnWarps * 32)
layer_norm_bwd_kernel(const T *__restrict__ x, const TY *__restrict__ dy, const float *__restrict__ gamma,
                      const float *__restrict__ mean, const float *__restrict__ rstd, T *dx,
                      float *__restrict__ partial /* [gridDim.x][2][d] */, int64_t rows, const T *add = nullptr) {
    constexpr int d = 128 * NV;
    __shared__ float4 red[kLnWarps][2][NV][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warps = (int64_t)gridDim.x * kLnWarps;
    float4 g[NV], dg[NV], db[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        g[i] = *reinterpret_cast<const float4 *>(gamma + 4 * (lane + 32 * i));
        dg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        db[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int64_t r = (int64_t)blockIdx.x * kLnWarps + warp; r < rows; r += warps) {
        const float mu = mean[r], rs = rstd[r];
        float4 xh[NV], gy[NV], old[NV];
        float s1 = 0.f, s2 = 0.f;
        // every load of the row is issued before the first reduction waits: the residual's gradient too
#pragma unroll
        for (int i = 0; i < NV; ++i)
            old[i] = add != nullptr ? ln_load4<T>(add + r * d + 4 * (lane + 32 * i)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 xv = ln_load4<T>(x + r * d + 4 * (lane + 32 * i));
            const float4 dv = ln_load4<TY>(dy + r * d + 4 * (lane + 32 * i));
            xh[i] = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
            gy[i] = make_float4(dv.x * g[i].x, dv.y * g[i].y, dv.z * g[i].z, dv.w * g[i].w);
            s1 += gy[i].x + gy[i].y + gy[i].z + gy[i].w;
            s2 += gy[i].x * xh[i].x + gy[i].y * xh[i].y + gy[i].z * xh[i].z + gy[i].w * xh[i].w;
            dg[i].x += dv.x * xh[i].x; dg[i].y += dv.y * xh[i].y; dg[i].z += dv.z * xh[i].z; dg[i].w += dv.w * xh[i].w;
            db[i].x += dv.x; db[i].y += dv.y; db[i].z += dv.z; db[i].w += dv.w;
        }
        const float m1 = warp_sum(s1) * (1.f / d), m2 = warp_sum(s2) * (1.f / d);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            float4 o;
            o.x = rs * (gy[i].x - m1 - xh[i].x * m2); o.y = rs * (gy[i].y - m1 - xh[i].y * m2);
            o.z = rs * (gy[i].z - m1 - xh[i].z * m2); o.w = rs * (gy[i].w - m1 - xh[i].w * m2);
            o.x += old[i].x; o.y += old[i].y; o.z += old[i].z; o.w += old[i].w;   // the gradient arriving through the residual connection
            ln_store4<T>(dx + r * d + 4 * (lane + 32 * i), o);
        }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        red[warp][0][i][lane] = dg[i];
        red[warp][1][i][lane] = db[i];
    }
    __syncthreads();
    // warp w of the CTA adds the kLnWarps partial rows of piece set w, w + kLnWarps, ... in warp order
    for (int item = warp; item < 2 * NV; item += kLnWarps) {
        const int which = item / NV, i = item % NV;
        float4 acc = red[0][which][i][lane];
#pragma unroll
        for (int w = 1; w < kLnWarps; ++w) {
            const float4 t = red[w][which][i][lane];
            acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
        }
        *reinterpret_cast<float4 *>(partial + ((int64_t)blockIdx.x * 2 + which) * d + 4 * (lane + 32 * i)) = acc;
    }
}

// dgamma[c] = sum over CTAs of partial[cta][0][c], dbeta likewise.  A block owns 32 columns; its 32 warps sum
// interleaved slices of the CTA list (CTA w, w+32, ...) and the 32 slice sums are added in slice order: the
// order of additions is fixed, so the result is reproducible.
__global__ void __launch_bounds__(1024)
layer_norm_bwd_reduce_kernel(const float *__restrict__ partial, float *__restrict__ dgamma,
                             float *__restrict__ dbeta, int nctas, int d) {
    __shared__ float slice[32][33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;                      // column in [0, 2d): dgamma then dbeta
    float s0 = 0.f, s1 = 0.f;
    if (c < 2 * d) {
        int k = w;
        for (; k + 32 < nctas; k += 64) {
            s0 += partial[(int64_t)k * 2 * d + c];
            s1 += partial[(int64_t)(k + 32) * 2 * d + c];
        }
        for (; k < nctas; k += 32) s0 += partial[(int64_t)k * 2 * d + c];
    }
    slice[w][lane] = s0 + s1;
    __syncthreads();
    if (w == 0 && c < 2 * d) {
        float t = slice[0][lane];
#pragma unroll
        for (int i = 1; i < 32; ++i) t += slice[i][lane];
        (c < d ? dgamma : dbeta)[c % d] = t;
    }
}

template <typename F>
static bool ln_dispatch_width(int d, F &&f) {
    switch (d) {
        case 128: f.template operator()<1>(); return true;
        case 256: f.template operator()<2>(); return true;
        case 512: f.template operator()<4>(); return true;
        case 384: f.template operator()<3>(); return true;
        case 768: f.template operator()<6>(); return true;
        default: return false;
    }
}

static int ln_grid(int64_t rows) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 148;
    const int64_t want = (rows + kLnWarps - 1) / kLnWarps;
    const int64_t cap = (int64_t)sms * 2;
    return (int)(want < cap ? want : cap);
}

}  // namespace hsa

using namespace hsa;

extern "C" int hsa_layer_norm_supported(int d) { return d == 128 || d == 256 || d == 384 || d == 512 || d == 768; }

extern "C" int hsa_layer_norm_bwd_ctas(int64_t rows) { return rows < 1 ? 0 : ln_grid(rows); }

extern "C" int hsa_layer_norm_fwd(const void *x, const float *gamma, const float *beta, void *y, float *mean,
                                  float *rstd, int64_t rows, int d, float eps, int dtype, void *stream) {
    HSA_CHECK_ARG(x && gamma && beta && y && mean && rstd, "hsa_layer_norm_fwd: null pointer");
    HSA_CHECK_ARG(rows >= 1, "hsa_layer_norm_fwd: rows=%lld", (long long)rows);
    HSA_CHECK_ARG(aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta), "hsa_layer_norm_fwd: pointers must be 16-byte aligned");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        int rc = 0;
        const bool ok = ln_dispatch_width(d, [&]<int NV>() {
            layer_norm_fwd_kernel<T, NV><<<ln_grid(rows), kLnWarps * 32, 0, (cudaStream_t)stream>>>(
                (const T *)x, gamma, beta, (T *)y, mean, rstd, rows, eps);
            rc = launch_status("hsa_layer_norm_fwd");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_layer_norm_fwd: width %d not supported (128, 256, 384, 512, 768)", d);
        return rc;
    });
}

extern "C" int hsa_layer_norm_bwd(const void *x, const void *dy, const float *gamma, const float *mean, const float *rstd,
                                  void *dx, float *dgamma, float *dbeta, float *partial, int64_t rows, int d, int dtype,
                                  void *stream) {
    HSA_CHECK_ARG(x && dy && gamma && mean && rstd && dx && dgamma && dbeta && partial, "hsa_layer_norm_bwd: null pointer");
    HSA_CHECK_ARG(rows >= 1, "hsa_layer_norm_bwd: rows=%lld", (long long)rows);
    HSA_CHECK_ARG(aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(gamma) && aligned16(partial),
                  "hsa_layer_norm_bwd: pointers must be 16-byte aligned");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        int rc = 0;
        const int ctas = ln_grid(rows);
        const bool ok = ln_dispatch_width(d, [&]<int NV>() {
            layer_norm_bwd_kernel<T, NV><<<ctas, kLnWarps * 32, 0, (cudaStream_t)stream>>>(
                (const T *)x, (const T *)dy, gamma, mean, rstd, (T *)dx, partial, rows);
            if ((rc = launch_status("hsa_layer_norm_bwd"))) return;
            layer_norm_bwd_reduce_kernel<<<(2 * d + 31) / 32, 1024, 0, (cudaStream_t)stream>>>(partial, dgamma, dbeta, ctas, d);
            rc = launch_status("hsa_layer_norm_bwd(reduce)");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_layer_norm_bwd: width %d not supported (128, 256, 384, 512, 768)", d);
        return rc;
    });
}

// float32 rows in, bfloat16 rows out (the normalised activations feed bfloat16 products), and the matching backward:
// bfloat16 upstream gradient, float32 gradient of the input, optionally ADDED to what dx already holds (the gradient
// arriving through the residual connection around the normalised branch).
extern "C" int hsa_layer_norm_fwd_mixed(const float *x, const float *gamma, const float *beta, void *y_bf16, void *x_bf16,
                                        float *mean, float *rstd, int64_t rows, int d, float eps, void *stream) {
    HSA_CHECK_ARG(x && gamma && beta && y_bf16 && mean && rstd, "hsa_layer_norm_fwd_mixed: null pointer");
    HSA_CHECK_ARG(rows >= 1, "hsa_layer_norm_fwd_mixed: rows=%lld", (long long)rows);
    HSA_CHECK_ARG(aligned16(x) && aligned16(y_bf16) && aligned16(x_bf16) && aligned16(gamma) && aligned16(beta),
                  "hsa_layer_norm_fwd_mixed: pointers must be 16-byte aligned");
    int rc = 0;
    const bool ok = ln_dispatch_width(d, [&]<int NV>() {
        layer_norm_fwd_kernel<float, NV, __nv_bfloat16><<<ln_grid(rows), kLnWarps * 32, 0, (cudaStream_t)stream>>>(
            x, gamma, beta, (__nv_bfloat16 *)y_bf16, mean, rstd, rows, eps, (__nv_bfloat16 *)x_bf16);
        rc = launch_status("hsa_layer_norm_fwd_mixed");
    });
    if (!ok) return fail(HSA_ERR_ARG, "hsa_layer_norm_fwd_mixed: width %d not supported (128, 256, 384, 512, 768)", d);
    return rc;
}

extern "C" int hsa_layer_norm_bwd_mixed(const float *x, const void *dy_bf16, const float *gamma, const float *mean,
                                        const float *rstd, const float *add, float *dx, float *dgamma, float *dbeta,
                                        float *partial, int64_t rows, int d, void *stream) {
    HSA_CHECK_ARG(x && dy_bf16 && gamma && mean && rstd && dx && dgamma && dbeta && partial, "hsa_layer_norm_bwd_mixed: null pointer");
    HSA_CHECK_ARG(rows >= 1, "hsa_layer_norm_bwd_mixed: rows=%lld", (long long)rows);
    HSA_CHECK_ARG(aligned16(x) && aligned16(dy_bf16) && aligned16(dx) && aligned16(gamma) && aligned16(partial) && aligned16(add),
                  "hsa_layer_norm_bwd_mixed: pointers must be 16-byte aligned");
    int rc = 0;
    const int ctas = ln_grid(rows);
    const bool ok = ln_dispatch_width(d, [&]<int NV>() {
        layer_norm_bwd_kernel<float, NV, __nv_bfloat16><<<ctas, kLnWarps * 32, 0, (cudaStream_t)stream>>>(
            x, (const __nv_bfloat16 *)dy_bf16, gamma, mean, rstd, dx, partial, rows, add);
        if ((rc = launch_status("hsa_layer_norm_bwd_mixed"))) return;
        layer_norm_bwd_reduce_kernel<<<(2 * d + 31) / 32, 1024, 0, (cudaStream_t)stream>>>(partial, dgamma, dbeta, ctas, d);
        rc = launch_status("hsa_layer_norm_bwd_mixed(reduce)");
    });
    if (!ok) return fail(HSA_ERR_ARG, "hsa_layer_norm_bwd_mixed: width %d not supported (128, 256, 384, 512, 768)", d);
    return rc;
}
