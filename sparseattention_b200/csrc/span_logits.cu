// Logits ops and single-query (decode) span attention: small CUDA-core kernels, one row group per
// (batch, leaf or node, head).
//
//   span_logits_kernel     the per-leaf candidate logits (or softmax weights) of span attention,
//                          [B, N, H, 2R+1+L]: window slots first, then one slot per tree level — the layout of the
//                          `Weights` tensor the reference's forward saves.
//   sibling_logits_kernel  the "logits" op of the reference's first Triton prototype: for every node its own
//                          q.k and the q.k with its sibling node.
//   span_decode_kernel     span attention of ONE new leaf per sequence against a key/value cache: what an
//                          incremental decoder needs (a leaf attends only to leaves and completed left
//                          siblings before it).
#include "hsa_common.cuh"

namespace hsa {

constexpr float kLg2e = 1.4426950408889634f;

struct LogitsArgs {
    const void *q, *k;
    float *out;                  // [B, N, H, C] contiguous, C = 2R+1+L
    int64_t q_bs, q_rs, k_bs, k_rs;
    int N, L, H, D, R, C;
    float scale;
    int weights;                 // 0: scaled logits, -inf where masked; 1: softmax weights, 0 where masked
};

template <typename T, int VEC, int LPR, int CPL, bool CAUSAL>
__global__ void __launch_bounds__(256)
span_logits_kernel(LogitsArgs a) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    constexpr int GPB = 256 / LPR;
    const int g = threadIdx.x % LPR;
    const int nq = blockIdx.x * GPB + threadIdx.x / LPR;
    const int h = blockIdx.y, b = blockIdx.z;
    const bool active = nq < a.N;
    const int n = active ? nq : a.N - 1;
    const int nchunks = a.D / VEC;
    const int64_t hoff = (int64_t)h * a.D;
    const T *kb = (const T *)a.k + b * a.k_bs + hoff;
    Frag q;
    q.load((const T *)a.q + b * a.q_bs + n * a.q_rs + hoff, g, nchunks);
    float *dst = a.out + (((int64_t)b * a.N + n) * a.H + h) * a.C;
    float m = -INFINITY, l = 0.f;
    for (int c = 0; c < a.C; ++c) {
        int row = -1;
        if (c <= 2 * a.R) {
            const int r = n - a.R + c;
            if (r >= 0 && r < a.N && (!CAUSAL || r <= n)) row = r;
        } else {
            const int lv = c - 2 * a.R - 1;
            if (!CAUSAL || ((n >> lv) & 1)) row = sibling_row(a.N, n, lv);
        }
        float s = -INFINITY;
        if (row >= 0) {                                   // uniform over the lanes of a group
            Frag kf;
            kf.load(kb + (int64_t)row * a.k_rs, g, nchunks);
            s = group_sum<LPR>(q.dot_partial(kf)) * a.scale;
            const float mn = fmaxf(m, s);
            l = l * exp2f((m - mn) * kLg2e) + exp2f((s - mn) * kLg2e);
            m = mn;
        }
        if (active && g == 0) dst[c] = s;
    }
    if (a.weights && active && g == 0) {
        const float inv = 1.f / l;
        for (int c = 0; c < a.C; ++c) {
            const float s = dst[c];
            dst[c] = (s == -INFINITY) ? 0.f : exp2f((s - m) * kLg2e) * inv;
        }
    }
}

struct SiblingArgs {
    const void *q, *k;
    float *self_out, *cross_out;   // [B, seq, H], [B, M, H]
    int64_t q_bs, q_rs, k_bs, k_rs;
    int M, seq, H, D;
    float scale;
};

template <typename T, int VEC, int LPR, int CPL>
__global__ void __launch_bounds__(256)
sibling_logits_kernel(SiblingArgs a) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    constexpr int GPB = 256 / LPR;
    const int g = threadIdx.x % LPR;
    const int node = blockIdx.x * GPB + threadIdx.x / LPR;
    const int h = blockIdx.y, b = blockIdx.z;
    const int rows = a.M > a.seq ? a.M : a.seq;
    if (node >= rows) return;                             // whole groups leave together
    const int nchunks = a.D / VEC;
    const int64_t hoff = (int64_t)h * a.D;
    const T *qb = (const T *)a.q + b * a.q_bs + hoff;
    const T *kb = (const T *)a.k + b * a.k_bs + hoff;
    Frag q, k;
    q.load(qb + (int64_t)node * a.q_rs, g, nchunks);
    if (node < a.seq && a.self_out != nullptr) {
        k.load(kb + (int64_t)node * a.k_rs, g, nchunks);
        const float s = group_sum<LPR>(q.dot_partial(k)) * a.scale;
        if (g == 0) a.self_out[((int64_t)b * a.seq + node) * a.H + h] = s;
    }
    if (node < a.M && a.cross_out != nullptr) {
        const int sib = node ^ 1;                          // M is even, so the sibling is a row below M as well
        k.load(kb + (int64_t)sib * a.k_rs, g, nchunks);
        const float s = group_sum<LPR>(q.dot_partial(k)) * a.scale;
        if (g == 0) a.cross_out[((int64_t)b * a.M + sib) * a.H + h] = s;
    }
}

struct DecodeArgs {
    const void *q, *k, *v;
    void *out;
    int64_t q_bs, k_bs, k_rs, v_bs, v_rs, o_bs;
    int N, L, H, D, R, n;
    float scale_log2e;
};

// One group per (batch, head): the new leaf a.n attends to leaves max(0, n-R)..n and, for every set bit l of n,
// to the left sibling of its level-l ancestor.
template <typename T, int VEC, int LPR, int CPL>
__global__ void __launch_bounds__(256)
span_decode_kernel(DecodeArgs a) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    constexpr int GPB = 256 / LPR;
    const int g = threadIdx.x % LPR;
    const int hq = blockIdx.x * GPB + threadIdx.x / LPR;
    const int b = blockIdx.y;
    const bool active = hq < a.H;
    const int h = active ? hq : a.H - 1;
    const int nchunks = a.D / VEC;
    const int64_t hoff = (int64_t)h * a.D;
    const T *kb = (const T *)a.k + b * a.k_bs + hoff;
    const T *vb = (const T *)a.v + b * a.v_bs + hoff;
    Frag q, acc;
    q.load((const T *)a.q + b * a.q_bs + hoff, g, nchunks);
    acc.zero();
    const int n = a.n;
    const int lo = max(0, n - a.R);
    const int nwin = n - lo + 1;
    float m = -INFINITY, l = 0.f;
    for (int c = 0; c < nwin + a.L; ++c) {
        int row;
        if (c < nwin) {
            row = lo + c;
        } else {
            const int lv = c - nwin;
            if (((n >> lv) & 1) == 0) continue;
            row = sibling_row(a.N, n, lv);
        }
        Frag kf, vf;
        kf.load(kb + (int64_t)row * a.k_rs, g, nchunks);
        vf.load(vb + (int64_t)row * a.v_rs, g, nchunks);
        const float s = group_sum<LPR>(q.dot_partial(kf)) * a.scale_log2e;
        const float mn = fmaxf(m, s);
        const float corr = exp2f(m - mn), p = exp2f(s - mn);
        acc.scale(corr);
        acc.axpy(p, vf);
        l = l * corr + p;
        m = mn;
    }
    if (!active) return;
    acc.scale(1.f / l);
    acc.store((T *)a.out + b * a.o_bs + hoff, g, nchunks);
}

}  // namespace hsa

using namespace hsa;

extern "C" int hsa_span_attn_logits(hsa_view Q, hsa_view K, float *out, int B, int N, int H, int D, int radius,
                                    int causal, int weights, int dtype, void *stream) {
    HSA_CHECK_ARG(Q.ptr && K.ptr && out, "hsa_span_attn_logits: null pointer");
    HSA_CHECK_ARG(B >= 1 && N >= 1 && (N & (N - 1)) == 0 && H >= 1 && D >= 1 && radius >= 0,
                  "hsa_span_attn_logits: bad shape B=%d N=%d H=%d D=%d radius=%d (N must be a power of two)", B, N, H, D, radius);
    HSA_CHECK_ARG(B <= 65535 && H <= 65535, "hsa_span_attn_logits: B and H are limited to 65535");
    HSA_CHECK_ARG(radius <= (1 << 20), "hsa_span_attn_logits: radius %d is beyond 2^20", radius);
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const bool vec = view_vec_ok(Q, sizeof(T)) && view_vec_ok(K, sizeof(T));
        const int L = ilog2((unsigned)N);
        LogitsArgs a{Q.ptr, K.ptr, out, Q.batch_stride, Q.row_stride, K.batch_stride, K.row_stride,
                     N, L, H, D, radius, 2 * radius + 1 + L, 1.0f / sqrtf((float)D), weights ? 1 : 0};
        int rc = 0;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            constexpr int GPB = 256 / LPR;
            dim3 grid((unsigned)((N + GPB - 1) / GPB), (unsigned)H, (unsigned)B);
            if (causal) span_logits_kernel<U, VEC, LPR, CPL, true><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
            else span_logits_kernel<U, VEC, LPR, CPL, false><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
            rc = launch_status("hsa_span_attn_logits");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_span_attn_logits: head dim %d not supported (max %d)", D, max_head_dim(dtype, vec));
        return rc;
    });
}

extern "C" int hsa_sibling_logits(hsa_view Q, hsa_view K, float *self_out, float *cross_out, int B, int total_nodes,
                                  int seq_len, int H, int D, int dtype, void *stream) {
    HSA_CHECK_ARG(Q.ptr && K.ptr && (self_out || cross_out), "hsa_sibling_logits: null pointer");
    HSA_CHECK_ARG(B >= 1 && total_nodes >= 1 && (total_nodes & 1) == 1 && seq_len >= 0 && seq_len <= total_nodes && H >= 1 && D >= 1,
                  "hsa_sibling_logits: bad shape B=%d nodes=%d seq=%d H=%d D=%d (the node count of a tree is odd)", B, total_nodes,
                  seq_len, H, D);
    HSA_CHECK_ARG(B <= 65535 && H <= 65535, "hsa_sibling_logits: B and H are limited to 65535");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const bool vec = view_vec_ok(Q, sizeof(T)) && view_vec_ok(K, sizeof(T));
        SiblingArgs a{Q.ptr, K.ptr, self_out, cross_out, Q.batch_stride, Q.row_stride, K.batch_stride, K.row_stride,
                      total_nodes - 1, seq_len, H, D, 1.0f / sqrtf((float)D)};
        const int rows = a.M > a.seq ? a.M : a.seq;
        if (rows == 0) return 0;
        int rc = 0;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            constexpr int GPB = 256 / LPR;
            dim3 grid((unsigned)((rows + GPB - 1) / GPB), (unsigned)H, (unsigned)B);
            sibling_logits_kernel<U, VEC, LPR, CPL><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
            rc = launch_status("hsa_sibling_logits");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_sibling_logits: head dim %d not supported (max %d)", D, max_head_dim(dtype, vec));
        return rc;
    });
}

extern "C" int hsa_span_attn_decode(hsa_view q, hsa_view K, hsa_view V, hsa_view out, int B, int N, int H, int D,
                                    int radius, int n, int dtype, void *stream) {
    HSA_CHECK_ARG(q.ptr && K.ptr && V.ptr && out.ptr, "hsa_span_attn_decode: null pointer");
    HSA_CHECK_ARG(B >= 1 && N >= 1 && (N & (N - 1)) == 0 && H >= 1 && D >= 1 && radius >= 0 && n >= 0 && n < N,
                  "hsa_span_attn_decode: bad shape B=%d N=%d H=%d D=%d radius=%d n=%d", B, N, H, D, radius, n);
    HSA_CHECK_ARG(B <= 65535, "hsa_span_attn_decode: B is limited to 65535");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const int es = sizeof(T);
        const bool vec = view_vec_ok(q, es) && view_vec_ok(K, es) && view_vec_ok(V, es) && view_vec_ok(out, es);
        DecodeArgs a{q.ptr, K.ptr, V.ptr, out.ptr, q.batch_stride, K.batch_stride, K.row_stride, V.batch_stride,
                     V.row_stride, out.batch_stride, N, ilog2((unsigned)N), H, D, radius < N ? radius : N, n,
                     kLg2e / sqrtf((float)D)};
        int rc = 0;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            constexpr int GPB = 256 / LPR;
            dim3 grid((unsigned)((H + GPB - 1) / GPB), (unsigned)B);
            span_decode_kernel<U, VEC, LPR, CPL><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
            rc = launch_status("hsa_span_attn_decode");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_span_attn_decode: head dim %d not supported (max %d)", D, max_head_dim(dtype, vec));
        return rc;
    });
}
