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
