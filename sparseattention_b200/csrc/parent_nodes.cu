// Parent-node update for one tree level: every parent attends to itself and its two children.
//
// Work decomposition: a group of LPR lanes owns one (batch, parent, head) and spreads the head
// dimension over its lanes in 16-byte chunks, so every global access of a warp is a run of
// consecutive 16-byte pieces (the [H, D] block of a node is contiguous, and the two children of a
// parent are adjacent rows).  Dot products finish with sub-warp shuffles; no shared memory.
// HBM traffic is the algorithmic 8 rows per parent forward and 15 rows backward.
#include "hsa_common.cuh"

namespace hsa {

struct ParentViews {
    const void *qp, *kp, *vp, *kc, *vc;
    void *out;
    int64_t qp_bs, qp_rs, kp_bs, kp_rs, vp_bs, vp_rs, kc_bs, kc_rs, vc_bs, vc_rs, out_bs, out_rs;
};

template <typename T, int VEC, int LPR, int CPL>
__global__ void __launch_bounds__(256)
parent_fwd_kernel(ParentViews a, float *__restrict__ W, int P, int H, int D, float scale) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    const int g = threadIdx.x % LPR;
    const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const int b = blockIdx.y;
    const bool active = group < (int64_t)P * H;
    const int64_t gi = active ? group : 0;          // idle groups shadow group 0 (shuffles stay converged)
    const int p = (int)(gi / H), h = (int)(gi % H);
    const int nchunks = D / VEC;
    const int64_t hoff = (int64_t)h * D;

    Frag q, k0, k1, k2;
    q.load((const T *)a.qp + b * a.qp_bs + p * a.qp_rs + hoff, g, nchunks);
    k0.load((const T *)a.kp + b * a.kp_bs + p * a.kp_rs + hoff, g, nchunks);
    k1.load((const T *)a.kc + b * a.kc_bs + (2 * (int64_t)p) * a.kc_rs + hoff, g, nchunks);
    k2.load((const T *)a.kc + b * a.kc_bs + (2 * (int64_t)p + 1) * a.kc_rs + hoff, g, nchunks);
    float s0 = q.dot_partial(k0), s1 = q.dot_partial(k1), s2 = q.dot_partial(k2);
    Frag v0, v1, v2;
    v0.load((const T *)a.vp + b * a.vp_bs + p * a.vp_rs + hoff, g, nchunks);
    v1.load((const T *)a.vc + b * a.vc_bs + (2 * (int64_t)p) * a.vc_rs + hoff, g, nchunks);
    v2.load((const T *)a.vc + b * a.vc_bs + (2 * (int64_t)p + 1) * a.vc_rs + hoff, g, nchunks);
    s0 = group_sum<LPR>(s0) * scale;
    s1 = group_sum<LPR>(s1) * scale;
    s2 = group_sum<LPR>(s2) * scale;
    const float m = fmaxf(s0, fmaxf(s1, s2));
    const float e0 = __expf(s0 - m), e1 = __expf(s1 - m), e2 = __expf(s2 - m);
    const float inv = 1.f / (e0 + e1 + e2);
    const float w0 = e0 * inv, w1 = e1 * inv, w2 = e2 * inv;
    Frag o;
    o.zero();
    o.axpy(w0, v0);
    o.axpy(w1, v1);
    o.axpy(w2, v2);
    if (active) {
        o.store((T *)a.out + b * a.out_bs + p * a.out_rs + hoff, g, nchunks);
        if (W != nullptr && g == 0) {
            float *w = W + (((int64_t)b * P + p) * H + h) * 3;
            w[0] = w0; w[1] = w1; w[2] = w2;
        }
    }
}

struct ParentGradViews {
    const void *go;
    void *dqp, *dkp, *dvp, *dkc, *dvc;
    int64_t go_bs, go_rs, dqp_bs, dqp_rs, dkp_bs, dkp_rs, dvp_bs, dvp_rs, dkc_bs, dkc_rs, dvc_bs, dvc_rs;
};

// dv_j = w_j g;  dp_j = v_j.g;  ds_j = w_j (dp_j - sum_i w_i dp_i) scale;  dq = sum ds_j k_j;  dk_j = ds_j q.
template <typename T, int VEC, int LPR, int CPL>
__global__ void __launch_bounds__(256)
parent_bwd_kernel(ParentViews a, ParentGradViews d, int P, int H, int D, float scale) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    const int g = threadIdx.x % LPR;
    const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const int b = blockIdx.y;
    const bool active = group < (int64_t)P * H;
    const int64_t gi = active ? group : 0;
    const int p = (int)(gi / H), h = (int)(gi % H);
    const int nchunks = D / VEC;
    const int64_t hoff = (int64_t)h * D;
    const int64_t c0 = 2 * (int64_t)p, c1 = c0 + 1;

    Frag q, k0, k1, k2;
    q.load((const T *)a.qp + b * a.qp_bs + p * a.qp_rs + hoff, g, nchunks);
    k0.load((const T *)a.kp + b * a.kp_bs + p * a.kp_rs + hoff, g, nchunks);
    k1.load((const T *)a.kc + b * a.kc_bs + c0 * a.kc_rs + hoff, g, nchunks);
    k2.load((const T *)a.kc + b * a.kc_bs + c1 * a.kc_rs + hoff, g, nchunks);
    float s0 = q.dot_partial(k0), s1 = q.dot_partial(k1), s2 = q.dot_partial(k2);
    Frag go, v;
    go.load((const T *)d.go + b * d.go_bs + p * d.go_rs + hoff, g, nchunks);
    v.load((const T *)a.vp + b * a.vp_bs + p * a.vp_rs + hoff, g, nchunks);
    float dp0 = go.dot_partial(v);
    v.load((const T *)a.vc + b * a.vc_bs + c0 * a.vc_rs + hoff, g, nchunks);
    float dp1 = go.dot_partial(v);
    v.load((const T *)a.vc + b * a.vc_bs + c1 * a.vc_rs + hoff, g, nchunks);
    float dp2 = go.dot_partial(v);
    s0 = group_sum<LPR>(s0) * scale;
    s1 = group_sum<LPR>(s1) * scale;
    s2 = group_sum<LPR>(s2) * scale;
    dp0 = group_sum<LPR>(dp0);
    dp1 = group_sum<LPR>(dp1);
    dp2 = group_sum<LPR>(dp2);
    const float m = fmaxf(s0, fmaxf(s1, s2));
    const float e0 = __expf(s0 - m), e1 = __expf(s1 - m), e2 = __expf(s2 - m);
    const float inv = 1.f / (e0 + e1 + e2);
    const float w0 = e0 * inv, w1 = e1 * inv, w2 = e2 * inv;
    const float delta = w0 * dp0 + w1 * dp1 + w2 * dp2;
    const float ds0 = w0 * (dp0 - delta) * scale, ds1 = w1 * (dp1 - delta) * scale,
                ds2 = w2 * (dp2 - delta) * scale;
    if (!active) return;
    Frag t;
    // dV
    t = go; t.scale(w0); t.store((T *)d.dvp + b * d.dvp_bs + p * d.dvp_rs + hoff, g, nchunks);
    t = go; t.scale(w1); t.store((T *)d.dvc + b * d.dvc_bs + c0 * d.dvc_rs + hoff, g, nchunks);
    t = go; t.scale(w2); t.store((T *)d.dvc + b * d.dvc_bs + c1 * d.dvc_rs + hoff, g, nchunks);
    // dQ
    t.zero(); t.axpy(ds0, k0); t.axpy(ds1, k1); t.axpy(ds2, k2);
    t.store((T *)d.dqp + b * d.dqp_bs + p * d.dqp_rs + hoff, g, nchunks);
    // dK
    t = q; t.scale(ds0); t.store((T *)d.dkp + b * d.dkp_bs + p * d.dkp_rs + hoff, g, nchunks);
    t = q; t.scale(ds1); t.store((T *)d.dkc + b * d.dkc_bs + c0 * d.dkc_rs + hoff, g, nchunks);
    t = q; t.scale(ds2); t.store((T *)d.dkc + b * d.dkc_bs + c1 * d.dkc_rs + hoff, g, nchunks);
}

// ------------------------------------------------------------------------------------------------
// Streaming variants (16-byte vector path, one chunk per lane).  The kernels above keep one item's rows
// in flight per thread, which leaves HBM half idle: bytes in flight per SM = latency x bandwidth is more
// than the register file can hold as pending loads.  Here every thread owns a private ring of kStages
// shared-memory slots and prefetches the rows of its next kStages-1 items with cp.async, so ~170 KB per
// SM are in flight.  A slot is written and read by the same thread only: cp.async.wait_group is the only
// synchronisation, there is no barrier.  Grid = one CTA of 512 threads per SM, items strided over it.
// ------------------------------------------------------------------------------------------------
constexpr int kPipeThreads = 512;
constexpr int kStages = 3;

__device__ __forceinline__ void pp_cp_async16(void *dst, const void *src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void pp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// The "memory" clobbers keep the compiler from moving the slot reads across the wait.
template <int N> __device__ __forceinline__ void pp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &raw, float (&out)[Traits<T>::kVec]) {
    if constexpr (sizeof(T) == 4) {
        out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
        out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
    } else {
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < Traits<T>::kVec; ++i) out[i] = Traits<T>::to_f(e[i]);
    }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&in)[Traits<T>::kVec]) {
    uint4 raw;
    if constexpr (sizeof(T) == 4) {
        raw = make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]), __float_as_uint(in[3]));
    } else {
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < Traits<T>::kVec; ++i) e[i] = Traits<T>::from_f(in[i]);
    }
    return raw;
}

template <typename T, int LPR, bool BWD>
__global__ void __launch_bounds__(kPipeThreads, 1)
parent_stream_kernel(ParentViews a, ParentGradViews d, float *__restrict__ W, int B, int P, int H, int D, float scale) {
    constexpr int VEC = Traits<T>::kVec;
    constexpr int NV = BWD ? 8 : 7;                    // 16-byte pieces loaded per item and lane
    extern __shared__ uint4 slots[];                   // [kStages][NV][kPipeThreads]
    const int tid = threadIdx.x;
    const int g = tid % LPR;
    const int nchunks = D / VEC;
    const bool lane_on = g < nchunks;
    const int64_t groups_total = (int64_t)gridDim.x * (kPipeThreads / LPR);
    const int64_t group = (int64_t)blockIdx.x * (kPipeThreads / LPR) + tid / LPR;
    const int64_t total = (int64_t)B * P * H;
    const int64_t eoff = (int64_t)g * VEC;

    auto issue = [&](int64_t item, int stage) {
        if (item < total && lane_on) {
            const int h = (int)(item % H);
            const int64_t bp = item / H;
            const int p = (int)(bp % P), b = (int)(bp / P);
            const int64_t ho = (int64_t)h * D + eoff;
            const int64_t c0 = 2 * (int64_t)p;
            uint4 *s = slots + (size_t)stage * NV * kPipeThreads + tid;
            pp_cp_async16(s + 0 * kPipeThreads, (const T *)a.qp + b * a.qp_bs + p * a.qp_rs + ho);
            pp_cp_async16(s + 1 * kPipeThreads, (const T *)a.kp + b * a.kp_bs + p * a.kp_rs + ho);
            pp_cp_async16(s + 2 * kPipeThreads, (const T *)a.kc + b * a.kc_bs + c0 * a.kc_rs + ho);
            pp_cp_async16(s + 3 * kPipeThreads, (const T *)a.kc + b * a.kc_bs + (c0 + 1) * a.kc_rs + ho);
            pp_cp_async16(s + 4 * kPipeThreads, (const T *)a.vp + b * a.vp_bs + p * a.vp_rs + ho);
            pp_cp_async16(s + 5 * kPipeThreads, (const T *)a.vc + b * a.vc_bs + c0 * a.vc_rs + ho);
            pp_cp_async16(s + 6 * kPipeThreads, (const T *)a.vc + b * a.vc_bs + (c0 + 1) * a.vc_rs + ho);
            if constexpr (BWD) pp_cp_async16(s + 7 * kPipeThreads, (const T *)d.go + b * d.go_bs + p * d.go_rs + ho);
        }
        pp_commit();
    };

#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) issue(group + st * groups_total, st);

    int stage = 0;
    for (int64_t item = group; item < total; item += groups_total) {
        issue(item + (kStages - 1) * groups_total, (stage + kStages - 1) % kStages);
        pp_wait<kStages - 1>();
        float v[NV][VEC];
        const uint4 *s = slots + (size_t)stage * NV * kPipeThreads + tid;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (lane_on) {
                unpack8<T>(s[j * kPipeThreads], v[j]);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[j][e] = 0.f;
            }
        }
        stage = (stage + 1) % kStages;
        // rows: 0 q, 1 k_self, 2 k_left, 3 k_right, 4 v_self, 5 v_left, 6 v_right, (7 dOut)
        float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            s0 = fmaf(v[0][e], v[1][e], s0);
            s1 = fmaf(v[0][e], v[2][e], s1);
            s2 = fmaf(v[0][e], v[3][e], s2);
        }
        s0 = group_sum<LPR>(s0) * scale;
        s1 = group_sum<LPR>(s1) * scale;
        s2 = group_sum<LPR>(s2) * scale;
        const float m = fmaxf(s0, fmaxf(s1, s2));
        const float e0 = __expf(s0 - m), e1 = __expf(s1 - m), e2 = __expf(s2 - m);
        const float inv = 1.f / (e0 + e1 + e2);
        const float w0 = e0 * inv, w1 = e1 * inv, w2 = e2 * inv;

        const int h = (int)(item % H);
        const int64_t bp = item / H;
        const int p = (int)(bp % P), b = (int)(bp / P);
        const int64_t ho = (int64_t)h * D + eoff;
        const int64_t c0 = 2 * (int64_t)p;
        if constexpr (!BWD) {
            float o[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[e] = w0 * v[4][e] + w1 * v[5][e] + w2 * v[6][e];
            if (lane_on) *reinterpret_cast<uint4 *>((T *)a.out + b * a.out_bs + p * a.out_rs + ho) = pack8<T>(o);
            if (W != nullptr && g == 0) {
                float *w = W + (((int64_t)b * P + p) * H + h) * 3;
                w[0] = w0; w[1] = w1; w[2] = w2;
            }
        } else {
            float dp0 = 0.f, dp1 = 0.f, dp2 = 0.f;
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                dp0 = fmaf(v[7][e], v[4][e], dp0);
                dp1 = fmaf(v[7][e], v[5][e], dp1);
                dp2 = fmaf(v[7][e], v[6][e], dp2);
            }
            dp0 = group_sum<LPR>(dp0);
            dp1 = group_sum<LPR>(dp1);
            dp2 = group_sum<LPR>(dp2);
            const float delta = w0 * dp0 + w1 * dp1 + w2 * dp2;
            const float ds0 = w0 * (dp0 - delta) * scale, ds1 = w1 * (dp1 - delta) * scale, ds2 = w2 * (dp2 - delta) * scale;
            if (lane_on) {
                float t[VEC];
                auto put = [&](void *base, int64_t bs, int64_t rs, int64_t row) {
                    *reinterpret_cast<uint4 *>((T *)base + b * bs + row * rs + ho) = pack8<T>(t);
                };
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = w0 * v[7][e];
                put(d.dvp, d.dvp_bs, d.dvp_rs, p);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = w1 * v[7][e];
                put(d.dvc, d.dvc_bs, d.dvc_rs, c0);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = w2 * v[7][e];
                put(d.dvc, d.dvc_bs, d.dvc_rs, c0 + 1);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = ds0 * v[1][e] + ds1 * v[2][e] + ds2 * v[3][e];
                put(d.dqp, d.dqp_bs, d.dqp_rs, p);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = ds0 * v[0][e];
                put(d.dkp, d.dkp_bs, d.dkp_rs, p);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = ds1 * v[0][e];
                put(d.dkc, d.dkc_bs, d.dkc_rs, c0);
#pragma unroll
                for (int e = 0; e < VEC; ++e) t[e] = ds2 * v[0][e];
                put(d.dkc, d.dkc_bs, d.dkc_rs, c0 + 1);
            }
        }
    }
    pp_wait<0>();
}

// Launch the streaming kernel when the row shape allows it (vector path, one chunk per lane); returns false otherwise.
template <typename T, bool BWD>
static bool launch_parent_stream(const ParentViews &a, const ParentGradViews &d, float *W, int B, int P, int H, int D,
                                 bool vec, float scale, cudaStream_t st, int &rc) {
    constexpr int VEC = Traits<T>::kVec;
    if (!vec || D % VEC != 0 || D / VEC > 32) return false;
    const int chunks = D / VEC;
    const int lpr = chunks <= 4 ? 4 : chunks <= 8 ? 8 : chunks <= 16 ? 16 : 32;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) return false;
    const int64_t total = (int64_t)B * P * H;
    const int64_t groups_per_cta = kPipeThreads / lpr;
    int64_t ctas = (total + groups_per_cta - 1) / groups_per_cta;
    if (ctas > sms) ctas = sms;
    const size_t smem = (size_t)kStages * (BWD ? 8 : 7) * kPipeThreads * sizeof(uint4);
    auto go = [&](auto kernel) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { rc = fail((int)e, "hsa_parent_nodes: shared memory %zu: %s", smem, cudaGetErrorString(e)); return; }
        kernel<<<(unsigned)ctas, kPipeThreads, smem, st>>>(a, d, W, B, P, H, D, scale);
        rc = launch_status(BWD ? "hsa_parent_nodes_bwd" : "hsa_parent_nodes_fwd");
    };
    switch (lpr) {
        case 4: go(parent_stream_kernel<T, 4, BWD>); break;
        case 8: go(parent_stream_kernel<T, 8, BWD>); break;
        case 16: go(parent_stream_kernel<T, 16, BWD>); break;
        default: go(parent_stream_kernel<T, 32, BWD>); break;
    }
    return true;
}

static int check_parent_shape(const char *fn, int B, int P, int H, int D) {
    HSA_CHECK_ARG(B >= 1 && B <= 65535, "%s: batch %d out of range [1, 65535]", fn, B);
    HSA_CHECK_ARG(P >= 1 && H >= 1 && D >= 1, "%s: bad shape P=%d H=%d D=%d", fn, P, H, D);
    HSA_CHECK_ARG((int64_t)P * H < (1LL << 40), "%s: P*H too large", fn);
    return 0;
}

}  // namespace hsa

using namespace hsa;

extern "C" int hsa_parent_nodes_fwd(hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view Kc, hsa_view Vc,
                                    hsa_view Out, float *W, int B, int P, int H, int D, int dtype,
                                    void *stream) {
    if (int rc = check_parent_shape("hsa_parent_nodes_fwd", B, P, H, D)) return rc;
    HSA_CHECK_ARG(Qp.ptr && Kp.ptr && Vp.ptr && Kc.ptr && Vc.ptr && Out.ptr, "hsa_parent_nodes_fwd: null pointer");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const int es = sizeof(T);
        const bool vec = view_vec_ok(Qp, es) && view_vec_ok(Kp, es) && view_vec_ok(Vp, es) && view_vec_ok(Kc, es) &&
                         view_vec_ok(Vc, es) && view_vec_ok(Out, es);
        ParentViews a{Qp.ptr, Kp.ptr, Vp.ptr, Kc.ptr, Vc.ptr, Out.ptr,
                      Qp.batch_stride, Qp.row_stride, Kp.batch_stride, Kp.row_stride, Vp.batch_stride, Vp.row_stride,
                      Kc.batch_stride, Kc.row_stride, Vc.batch_stride, Vc.row_stride, Out.batch_stride, Out.row_stride};
        const float scale = 1.0f / sqrtf((float)D);
        int rc = 0;
        if (launch_parent_stream<T, false>(a, ParentGradViews{}, W, B, P, H, D, vec, scale, (cudaStream_t)stream, rc)) return rc;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            const int threads = 256;
            const int64_t groups = (int64_t)P * H;
            const int64_t blocks = (groups * LPR + threads - 1) / threads;
            dim3 grid((unsigned)blocks, (unsigned)B);
            parent_fwd_kernel<U, VEC, LPR, CPL><<<grid, threads, 0, (cudaStream_t)stream>>>(a, W, P, H, D, scale);
            rc = launch_status("hsa_parent_nodes_fwd");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_parent_nodes_fwd: head dim %d not supported (max %d)", D,
                             max_head_dim(dtype, vec));
        return rc;
    });
}

extern "C" int hsa_parent_nodes_bwd(hsa_view dOut, hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view Kc,
                                    hsa_view Vc, hsa_view dQp, hsa_view dKp, hsa_view dVp, hsa_view dKc,
                                    hsa_view dVc, int B, int P, int H, int D, int dtype, void *stream) {
    if (int rc = check_parent_shape("hsa_parent_nodes_bwd", B, P, H, D)) return rc;
    HSA_CHECK_ARG(dOut.ptr && Qp.ptr && Kp.ptr && Vp.ptr && Kc.ptr && Vc.ptr && dQp.ptr && dKp.ptr && dVp.ptr &&
                      dKc.ptr && dVc.ptr, "hsa_parent_nodes_bwd: null pointer");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const int es = sizeof(T);
        const hsa_view *all[] = {&dOut, &Qp, &Kp, &Vp, &Kc, &Vc, &dQp, &dKp, &dVp, &dKc, &dVc};
        bool vec = true;
        for (const hsa_view *v : all) vec = vec && view_vec_ok(*v, es);
        ParentViews a{Qp.ptr, Kp.ptr, Vp.ptr, Kc.ptr, Vc.ptr, nullptr,
                      Qp.batch_stride, Qp.row_stride, Kp.batch_stride, Kp.row_stride, Vp.batch_stride, Vp.row_stride,
                      Kc.batch_stride, Kc.row_stride, Vc.batch_stride, Vc.row_stride, 0, 0};
        ParentGradViews d{dOut.ptr, dQp.ptr, dKp.ptr, dVp.ptr, dKc.ptr, dVc.ptr,
                          dOut.batch_stride, dOut.row_stride, dQp.batch_stride, dQp.row_stride,
                          dKp.batch_stride, dKp.row_stride, dVp.batch_stride, dVp.row_stride,
                          dKc.batch_stride, dKc.row_stride, dVc.batch_stride, dVc.row_stride};
        const float scale = 1.0f / sqrtf((float)D);
        int rc = 0;
        if (launch_parent_stream<T, true>(a, d, nullptr, B, P, H, D, vec, scale, (cudaStream_t)stream, rc)) return rc;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            const int threads = 256;
            const int64_t groups = (int64_t)P * H;
            const int64_t blocks = (groups * LPR + threads - 1) / threads;
            dim3 grid((unsigned)blocks, (unsigned)B);
            parent_bwd_kernel<U, VEC, LPR, CPL><<<grid, threads, 0, (cudaStream_t)stream>>>(a, d, P, H, D, scale);
            rc = launch_status("hsa_parent_nodes_bwd");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_parent_nodes_bwd: head dim %d not supported (max %d)", D,
                             max_head_dim(dtype, vec));
        return rc;
    });
}
