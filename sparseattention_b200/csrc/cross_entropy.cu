// Label-smoothed cross entropy over rows of (possibly column-padded) logits, forward and backward.
//
// One CTA per row.  Forward: a single pass keeps a running (max, sum of exponentials, sum of logits)
// per thread over 16-byte pieces of the row and combines them across the block; it emits the row loss
//   (1 - eps) * (lse - x[target]) + eps * (lse - mean_j x[j])
// and the row's log-sum-exp.  Backward: one pass writes
//   dx[j] = g * (exp(x[j] - lse) - (1 - eps) * [j == target] - eps / V)      (0 in the padding columns)
// in the logits' dtype.  Rows whose target equals ignore_index give zero loss and zero gradient.
// HBM traffic: the logits once forward, once backward, plus the gradient once.
#include "hsa_common.cuh"

namespace hsa {

constexpr int kCeThreads = 256;

struct RowStat {
    float m, s, sx;   // running max, sum exp(x - m), sum x
};
__device__ __forceinline__ void stat_add(RowStat &a, float x) {
    const float nm = fmaxf(a.m, x);
    a.s = a.s * expf(a.m - nm) + expf(x - nm);
    a.m = nm;
    a.sx += x;
}
__device__ __forceinline__ RowStat stat_merge(const RowStat &a, const RowStat &b) {
    RowStat r;
    r.m = fmaxf(a.m, b.m);
    const float ea = (a.m == -INFINITY) ? 0.f : expf(a.m - r.m);
    const float eb = (b.m == -INFINITY) ? 0.f : expf(b.m - r.m);
    r.s = a.s * ea + b.s * eb;
    r.sx = a.sx + b.sx;
    return r;
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_fwd_kernel(const T *__restrict__ logits, int64_t row_stride, const int64_t *__restrict__ targets,
                         float *__restrict__ loss_rows, float *__restrict__ lse_out, int V, float eps,
                         int64_t ignore_index, bool vec_ok) {
    constexpr int VEC = Traits<T>::kVec;
    const int64_t row = blockIdx.x;
    const T *x = logits + row * row_stride;
    const int64_t tgt = targets[row];
    RowStat st{-INFINITY, 0.f, 0.f};
    if (vec_ok) {
        const int nfull = V / VEC;
        for (int c = threadIdx.x; c < nfull; c += kCeThreads) {
            float v[VEC];
            load_vec<T, VEC>(x + (int64_t)c * VEC, v);
            // one rescale per 16-byte piece: VEC + 1 exponentials instead of 2 * VEC
            float pm = v[0], px = 0.f;
#pragma unroll
            for (int e = 1; e < VEC; ++e) pm = fmaxf(pm, v[e]);
            const float nm = fmaxf(st.m, pm);
            float ps = 0.f;
#pragma unroll
            for (int e = 0; e < VEC; ++e) { ps += expf(v[e] - nm); px += v[e]; }
            st.s = st.s * expf(st.m - nm) + ps;
            st.m = nm;
            st.sx += px;
        }
        for (int j = nfull * VEC + threadIdx.x; j < V; j += kCeThreads) stat_add(st, Traits<T>::to_f(x[j]));
    } else {
        for (int j = threadIdx.x; j < V; j += kCeThreads) stat_add(st, Traits<T>::to_f(x[j]));
    }
    // block combine: warp shuffles, then one warp over the warp results
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        RowStat other{__shfl_xor_sync(0xffffffffu, st.m, o), __shfl_xor_sync(0xffffffffu, st.s, o),
                      __shfl_xor_sync(0xffffffffu, st.sx, o)};
        st = stat_merge(st, other);
    }
    __shared__ RowStat ws[kCeThreads / 32];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = st;
    __syncthreads();
    if (threadIdx.x < 32) {
        st = threadIdx.x < kCeThreads / 32 ? ws[threadIdx.x] : RowStat{-INFINITY, 0.f, 0.f};
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            RowStat other{__shfl_xor_sync(0xffffffffu, st.m, o), __shfl_xor_sync(0xffffffffu, st.s, o),
                          __shfl_xor_sync(0xffffffffu, st.sx, o)};
            st = stat_merge(st, other);
        }
        if (threadIdx.x == 0) {
            const float lse = st.m + logf(st.s);
            lse_out[row] = lse;
            float loss = 0.f;
            if (tgt != ignore_index) {
                // a target outside [0, V) that is not the ignore index is a corrupt label: the row's loss is NaN,
                // so the mean is NaN and the caller sees it (nn.CrossEntropyLoss raises a device assertion there)
                const float xt = (tgt >= 0 && tgt < V) ? Traits<T>::to_f(x[tgt]) : __int_as_float(0x7fffffff);
                loss = (1.f - eps) * (lse - xt) + eps * (lse - st.sx / (float)V);
            }
            loss_rows[row] = loss;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_bwd_kernel(const T *__restrict__ logits, int64_t row_stride, const int64_t *__restrict__ targets,
                         const float *__restrict__ lse_in, const float *__restrict__ grad_scale, T *__restrict__ dlogits,
                         int64_t drow_stride, int V, int Vp, float eps, int64_t ignore_index, bool vec_ok) {
    constexpr int VEC = Traits<T>::kVec;
    const int64_t row = blockIdx.x;
    const T *x = logits + row * row_stride;
    T *dx = dlogits + row * drow_stride;
    const int64_t tgt = targets[row];
    const float g = (tgt == ignore_index) ? 0.f : grad_scale[0];
    const float lse = lse_in[row];
    const float sm = eps / (float)V;
    auto grad = [&](float xv, int j) -> float {
        if (j >= V) return 0.f;
        float p = expf(xv - lse) - sm;
        if (j == tgt) p -= (1.f - eps);
        return g * p;
    };
    if (vec_ok) {
        const int nchunks = Vp / VEC;
        for (int c = threadIdx.x; c < nchunks; c += kCeThreads) {
            float v[VEC], o[VEC];
            load_vec<T, VEC>(x + (int64_t)c * VEC, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[e] = grad(v[e], c * VEC + e);
            store_vec<T, VEC>(dx + (int64_t)c * VEC, o);
        }
        for (int j = nchunks * VEC + threadIdx.x; j < Vp; j += kCeThreads) dx[j] = Traits<T>::from_f(grad(Traits<T>::to_f(x[j]), j));
    } else {
        for (int j = threadIdx.x; j < Vp; j += kCeThreads) dx[j] = Traits<T>::from_f(grad(Traits<T>::to_f(x[j]), j));
    }
}

}  // namespace hsa

using namespace hsa;

extern "C" int hsa_cross_entropy_fwd(const void *logits, int64_t row_stride, const int64_t *targets, float *loss_rows,
                                     float *lse, int64_t M, int V, float smoothing, int64_t ignore_index, int dtype,
                                     void *stream) {
    HSA_CHECK_ARG(logits && targets && loss_rows && lse, "hsa_cross_entropy_fwd: null pointer");
    HSA_CHECK_ARG(M >= 1 && M <= 0x7fffffffLL && V >= 1 && row_stride >= V, "hsa_cross_entropy_fwd: bad shape M=%lld V=%d stride=%lld",
                  (long long)M, V, (long long)row_stride);
    HSA_CHECK_ARG(smoothing >= 0.f && smoothing < 1.f, "hsa_cross_entropy_fwd: label smoothing %f outside [0, 1)", smoothing);
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const bool vec = aligned16(logits) && row_stride % Traits<T>::kVec == 0;
        cross_entropy_fwd_kernel<T><<<(unsigned)M, kCeThreads, 0, (cudaStream_t)stream>>>(
            (const T *)logits, row_stride, targets, loss_rows, lse, V, smoothing, ignore_index, vec);
        return launch_status("hsa_cross_entropy_fwd");
    });
}

extern "C" int hsa_cross_entropy_bwd(const void *logits, int64_t row_stride, const int64_t *targets, const float *lse,
                                     const float *grad_scale, void *dlogits, int64_t drow_stride, int64_t M, int V, int Vp,
                                     float smoothing, int64_t ignore_index, int dtype, void *stream) {
    HSA_CHECK_ARG(logits && targets && lse && grad_scale && dlogits, "hsa_cross_entropy_bwd: null pointer");
    HSA_CHECK_ARG(M >= 1 && M <= 0x7fffffffLL && V >= 1 && Vp >= V && row_stride >= Vp && drow_stride >= Vp,
                  "hsa_cross_entropy_bwd: bad shape M=%lld V=%d Vp=%d", (long long)M, V, Vp);
    HSA_CHECK_ARG(smoothing >= 0.f && smoothing < 1.f, "hsa_cross_entropy_bwd: label smoothing %f outside [0, 1)", smoothing);
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const int vecw = Traits<T>::kVec;
        const bool vec = aligned16(logits) && aligned16(dlogits) && row_stride % vecw == 0 && drow_stride % vecw == 0;
        cross_entropy_bwd_kernel<T><<<(unsigned)M, kCeThreads, 0, (cudaStream_t)stream>>>(
            (const T *)logits, row_stride, targets, lse, grad_scale, (T *)dlogits, drow_stride, V, Vp, smoothing,
            ignore_index, vec);
        return launch_status("hsa_cross_entropy_bwd");
    });
}
