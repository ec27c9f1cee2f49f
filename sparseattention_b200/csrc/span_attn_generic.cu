// Span attention, portable CUDA-core kernels (any dtype, any head count, head dims up to the
// row-group limit).  They serve float32 inputs and shapes the tensor-core kernels do not take.
//
// A group of LPR lanes owns one (batch, leaf, head): the query row sits in registers spread over the
// lanes in 16-byte chunks, candidate key/value rows are read straight from global memory (neighbouring
// leaves of a block share almost all of their window, so those reads hit L1), logits are reduced
// with sub-warp shuffles and folded into an online softmax.  Tree rows come from the closed form
// sibling_row(); no tables are read.
#include "hsa_common.cuh"

namespace hsa {

struct SpanArgs {
    const void *q, *k, *v;
    void *out;
    float *lse;
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs;
    int N, L, H, D, R;
    float scale_log2e;   // (1/sqrt(D)) * log2(e)
    float scale;
};

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kBatch = 4;   // candidates handled together, for memory-level parallelism

// Candidate c of leaf n: window slots first (rows lo..hi), then one slot per level.
template <bool CAUSAL>
__device__ __forceinline__ int candidate_row(int c, int n, int lo, int nwin, int N, int L) {
    if (c < nwin) return lo + c;
    const int l = c - nwin;
    if (l >= L) return -1;
    if (CAUSAL && ((n >> l) & 1) == 0) return -1;
    return sibling_row(N, n, l);
}

template <typename T, int VEC, int LPR, int CPL, bool CAUSAL>
__global__ void __launch_bounds__(256)
span_fwd_generic_kernel(SpanArgs a) {
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
    const T *vb = (const T *)a.v + b * a.v_bs + hoff;

    Frag q;
    q.load((const T *)a.q + b * a.q_bs + n * a.q_rs + hoff, g, nchunks);
    const int lo = max(0, n - a.R);
    const int hi = CAUSAL ? n : min(a.N - 1, n + a.R);
    const int nwin = hi - lo + 1;
    const int ncand = nwin + a.L;

    Frag acc;
    acc.zero();
    float m = -INFINITY, l = 0.f;
    for (int c0 = 0; c0 < ncand; c0 += kBatch) {
        int row[kBatch];
        float s[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            row[i] = (c0 + i < ncand) ? candidate_row<CAUSAL>(c0 + i, n, lo, nwin, a.N, a.L) : -1;
            s[i] = 0.f;
            if (row[i] >= 0) {
                Frag kf;
                kf.load(kb + row[i] * a.k_rs, g, nchunks);
                s[i] = q.dot_partial(kf);
            }
        }
        float mb = m;
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            s[i] = group_sum<LPR>(s[i]) * a.scale_log2e;
            if (row[i] < 0) s[i] = -INFINITY;
            mb = fmaxf(mb, s[i]);
        }
        const float corr = exp2f(m - mb);      // first batch holds the leaf itself, so mb is finite
        acc.scale(corr);
        l *= corr;
        m = mb;
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            if (row[i] >= 0) {
                const float p = exp2f(s[i] - m);
                l += p;
                Frag vf;
                vf.load(vb + row[i] * a.v_rs, g, nchunks);
                acc.axpy(p, vf);
            }
        }
    }
    if (!active) return;
    acc.scale(1.f / l);
    acc.store((T *)a.out + b * a.o_bs + n * a.o_rs + hoff, g, nchunks);
    if (a.lse != nullptr && g == 0) a.lse[((int64_t)b * a.N + n) * a.H + h] = (m + log2f(l)) * kLn2;
}

// ------------------------------------------------------------------ backward
struct SpanBwdArgs {
    const void *q, *k, *v, *out, *go;
    const float *lse;
    float *delta;                     // [B, N, H] scratch: rowsum(dOut * Out)
    void *dq, *dk, *dv;
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs, go_bs, go_rs, dq_bs, dq_rs, dk_bs, dk_rs, dv_bs, dv_rs;
    int N, L, H, D, R;
    float scale_log2e, scale;
    int row_begin;                    // first key row of this launch (key-side kernels)
};

// dQ and delta: one group per (batch, leaf, head), same candidate walk as the forward.
template <typename T, int VEC, int LPR, int CPL, bool CAUSAL>
__global__ void __launch_bounds__(256)
span_bwd_dq_generic_kernel(SpanBwdArgs a) {
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
    const T *vb = (const T *)a.v + b * a.v_bs + hoff;

    Frag q, go, t;
    q.load((const T *)a.q + b * a.q_bs + n * a.q_rs + hoff, g, nchunks);
    go.load((const T *)a.go + b * a.go_bs + n * a.go_rs + hoff, g, nchunks);
    t.load((const T *)a.out + b * a.o_bs + n * a.o_rs + hoff, g, nchunks);
    const float delta = group_sum<LPR>(go.dot_partial(t));
    const int64_t stat = ((int64_t)b * a.N + n) * a.H + h;
    const float lse2 = a.lse[stat] * kLog2e;
    if (active && g == 0) a.delta[stat] = delta;

    const int lo = max(0, n - a.R);
    const int hi = CAUSAL ? n : min(a.N - 1, n + a.R);
    const int nwin = hi - lo + 1;
    const int ncand = nwin + a.L;
    Frag dq;
    dq.zero();
    constexpr int NB = 2;
    for (int c0 = 0; c0 < ncand; c0 += NB) {
        int row[NB];
        float s[NB], dp[NB];
        Frag kf[NB];
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            row[i] = (c0 + i < ncand) ? candidate_row<CAUSAL>(c0 + i, n, lo, nwin, a.N, a.L) : -1;
            s[i] = dp[i] = 0.f;
            kf[i].zero();
            if (row[i] >= 0) {
                kf[i].load(kb + row[i] * a.k_rs, g, nchunks);
                s[i] = q.dot_partial(kf[i]);
                Frag vf;
                vf.load(vb + row[i] * a.v_rs, g, nchunks);
                dp[i] = go.dot_partial(vf);
            }
        }
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            s[i] = group_sum<LPR>(s[i]);
            dp[i] = group_sum<LPR>(dp[i]);
            if (row[i] >= 0) {
                const float p = exp2f(s[i] * a.scale_log2e - lse2);
                dq.axpy(p * (dp[i] - delta) * a.scale, kf[i]);
            }
        }
    }
    if (active) dq.store((T *)a.dq + b * a.dq_bs + n * a.dq_rs + hoff, g, nchunks);
}

// Queries that attend to key row r: a window range [w0, w1) (leaf rows only) and a level range
// [t0, t1) (the leaves under r's sibling).  Empty ranges have begin == end.
template <bool CAUSAL>
__device__ __forceinline__ void key_sources(int r, int N, int L, int R, int &w0, int &w1, int &t0, int &t1) {
    w0 = w1 = t0 = t1 = 0;
    if (r < N) {
        w0 = CAUSAL ? r : max(0, r - R);
        w1 = min(N - 1, r + R) + 1;
        if (L > 0 && (!CAUSAL || (r & 1) == 0)) { t0 = r ^ 1; t1 = t0 + 1; }   // level-0 sibling
        return;
    }
    const int rem = 2 * N - r;
    const int l = L - ilog2((unsigned)(rem - 1));
    if (l >= L) return;                                  // root
    const int j = r - level_base(N, l);
    if (CAUSAL && (j & 1)) return;                       // right children are never attended causally
    t0 = (j ^ 1) << l;
    t1 = t0 + (1 << l);
}

// One contribution of query n to key row (kf, vf): accumulates dk += ds * q, dv += p * go.
template <typename Frag, typename T, int LPR>
__device__ __forceinline__ void key_side_step(const SpanBwdArgs &a, int b, int h, int n, int g, int nchunks,
                                              const Frag &kf, const Frag &vf, Frag &dk, Frag &dv) {
    const int64_t hoff = (int64_t)h * a.D;
    Frag q, go;
    q.load((const T *)a.q + b * a.q_bs + n * a.q_rs + hoff, g, nchunks);
    go.load((const T *)a.go + b * a.go_bs + n * a.go_rs + hoff, g, nchunks);
    const float s = group_sum<LPR>(q.dot_partial(kf));
    const float dp = group_sum<LPR>(go.dot_partial(vf));
    const int64_t stat = ((int64_t)b * a.N + n) * a.H + h;
    const float p = exp2f(s * a.scale_log2e - a.lse[stat] * kLog2e);
    const float ds = p * (dp - a.delta[stat]) * a.scale;
    dk.axpy(ds, q);
    dv.axpy(p, go);
}

// dK/dV for key rows with short source lists (leaves and the lowest tree levels): one group per row.
template <typename T, int VEC, int LPR, int CPL, bool CAUSAL>
__global__ void __launch_bounds__(256)
span_bwd_dkdv_rows_kernel(SpanBwdArgs a, int row_end) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    constexpr int GPB = 256 / LPR;
    const int g = threadIdx.x % LPR;
    const int rr = a.row_begin + blockIdx.x * GPB + threadIdx.x / LPR;
    const int h = blockIdx.y, b = blockIdx.z;
    const bool active = rr < row_end;
    const int r = active ? rr : row_end - 1;
    const int nchunks = a.D / VEC;
    const int64_t hoff = (int64_t)h * a.D;
    Frag kf, vf, dk, dv;
    kf.load((const T *)a.k + b * a.k_bs + r * a.k_rs + hoff, g, nchunks);
    vf.load((const T *)a.v + b * a.v_bs + r * a.v_rs + hoff, g, nchunks);
    dk.zero();
    dv.zero();
    int w0, w1, t0, t1;
    key_sources<CAUSAL>(r, a.N, a.L, a.R, w0, w1, t0, t1);
    for (int n = w0; n < w1; ++n) key_side_step<Frag, T, LPR>(a, b, h, n, g, nchunks, kf, vf, dk, dv);
    for (int n = t0; n < t1; ++n) key_side_step<Frag, T, LPR>(a, b, h, n, g, nchunks, kf, vf, dk, dv);
    if (!active) return;
    dk.store((T *)a.dk + b * a.dk_bs + r * a.dk_rs + hoff, g, nchunks);
    dv.store((T *)a.dv + b * a.dv_bs + r * a.dv_rs + hoff, g, nchunks);
}

// dK/dV for tree nodes with long source lists: one block per (row, head, batch); its groups stride
// over the source leaves and the partial sums are combined in a fixed order (deterministic).
template <typename T, int VEC, int LPR, int CPL, bool CAUSAL>
__global__ void __launch_bounds__(256)
span_bwd_dkdv_node_kernel(SpanBwdArgs a) {
    using Frag = RowFrag<T, VEC, LPR, CPL>;
    constexpr int GPB = 256 / LPR;
    extern __shared__ float red[];                 // [2][GPB][D]
    const int g = threadIdx.x % LPR, grp = threadIdx.x / LPR;
    const int r = a.row_begin + blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int nchunks = a.D / VEC;
    const int64_t hoff = (int64_t)h * a.D;
    Frag kf, vf, dk, dv;
    kf.load((const T *)a.k + b * a.k_bs + r * a.k_rs + hoff, g, nchunks);
    vf.load((const T *)a.v + b * a.v_bs + r * a.v_rs + hoff, g, nchunks);
    dk.zero();
    dv.zero();
    int w0, w1, t0, t1;
    key_sources<CAUSAL>(r, a.N, a.L, a.R, w0, w1, t0, t1);
    for (int n = t0 + grp; n < t1; n += GPB) key_side_step<Frag, T, LPR>(a, b, h, n, g, nchunks, kf, vf, dk, dv);
    float *rk = red + (int64_t)grp * a.D, *rv = red + (int64_t)(GPB + grp) * a.D;
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        const int ch = g + c * LPR;
        if (ch < nchunks) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                rk[ch * VEC + i] = dk.v[c][i];
                rv[ch * VEC + i] = dv.v[c][i];
            }
        }
    }
    __syncthreads();
    T *dkp = (T *)a.dk + b * a.dk_bs + r * a.dk_rs + hoff;
    T *dvp = (T *)a.dv + b * a.dv_bs + r * a.dv_rs + hoff;
    for (int e = threadIdx.x; e < 2 * a.D; e += blockDim.x) {
        const int which = e / a.D, col = e % a.D;
        float sum = 0.f;
        for (int i = 0; i < GPB; ++i) sum += red[(int64_t)(which * GPB + i) * a.D + col];
        (which ? dvp : dkp)[col] = Traits<T>::from_f(sum);
    }
}

// Highest level whose nodes are handled one group per row; its source lists hold 2^level leaves.
constexpr int kRowsMaxLevel = 5;

}  // namespace hsa

using namespace hsa;

namespace {
int check_span_shape(const char *fn, int B, int N, int H, int D, int R) {
    HSA_CHECK_ARG(B >= 1 && B <= 65535, "%s: batch %d out of range [1, 65535]", fn, B);
    HSA_CHECK_ARG(H >= 1 && H <= 65535, "%s: heads %d out of range [1, 65535]", fn, H);
    HSA_CHECK_ARG(N >= 1 && (N & (N - 1)) == 0, "%s: N=%d must be a power of two", fn, N);
    HSA_CHECK_ARG(N <= (1 << 28), "%s: N=%d too large", fn, N);
    HSA_CHECK_ARG(D >= 1, "%s: head dim %d", fn, D);
    HSA_CHECK_ARG(R >= 0, "%s: radius %d must be >= 0", fn, R);
    return 0;
}
}  // namespace

int hsa_span_attn_fwd_generic(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H,
                              int D, int radius, int causal, int dtype, cudaStream_t st) {
    if (int rc = check_span_shape("hsa_span_attn_fwd", B, N, H, D, radius)) return rc;
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const int es = sizeof(T);
        const bool vec = view_vec_ok(Q, es) && view_vec_ok(K, es) && view_vec_ok(V, es) && view_vec_ok(Out, es);
        SpanArgs a{Q.ptr, K.ptr, V.ptr, Out.ptr, LSE,
                   Q.batch_stride, Q.row_stride, K.batch_stride, K.row_stride, V.batch_stride, V.row_stride,
                   Out.batch_stride, Out.row_stride, N, ilog2((unsigned)N), H, D, radius < N ? radius : N,
                   kLog2e / sqrtf((float)D), 1.0f / sqrtf((float)D)};
        int rc = 0;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            constexpr int GPB = 256 / LPR;
            dim3 grid((unsigned)((N + GPB - 1) / GPB), (unsigned)H, (unsigned)B);
            if (causal) span_fwd_generic_kernel<U, VEC, LPR, CPL, true><<<grid, 256, 0, st>>>(a);
            else span_fwd_generic_kernel<U, VEC, LPR, CPL, false><<<grid, 256, 0, st>>>(a);
            rc = launch_status("hsa_span_attn_fwd");
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_span_attn_fwd: head dim %d not supported (max %d)", D,
                             max_head_dim(dtype, vec));
        return rc;
    });
}

size_t hsa_span_attn_bwd_generic_workspace(int B, int N, int H) {
    return (size_t)B * N * H * sizeof(float);
}

int hsa_span_attn_bwd_generic(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut,
                              hsa_view dQ, hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D,
                              int radius, int causal, int dtype, cudaStream_t st) {
    if (int rc = check_span_shape("hsa_span_attn_bwd", B, N, H, D, radius)) return rc;
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const int es = sizeof(T);
        const hsa_view *all[] = {&Q, &K, &V, &Out, &dOut, &dQ, &dK, &dV};
        bool vec = true;
        for (const hsa_view *v : all) vec = vec && view_vec_ok(*v, es);
        const int L = ilog2((unsigned)N);
        SpanBwdArgs a{Q.ptr, K.ptr, V.ptr, Out.ptr, dOut.ptr, LSE, (float *)workspace, dQ.ptr, dK.ptr, dV.ptr,
                      Q.batch_stride, Q.row_stride, K.batch_stride, K.row_stride, V.batch_stride, V.row_stride,
                      Out.batch_stride, Out.row_stride, dOut.batch_stride, dOut.row_stride,
                      dQ.batch_stride, dQ.row_stride, dK.batch_stride, dK.row_stride, dV.batch_stride, dV.row_stride,
                      N, L, H, D, radius < N ? radius : N, kLog2e / sqrtf((float)D), 1.0f / sqrtf((float)D), 0};
        int rc = 0;
        const bool ok = dispatch_row_shape<T>(D, vec, [&]<typename U, int VEC, int LPR, int CPL>() {
            constexpr int GPB = 256 / LPR;
            auto launch = [&]<bool CAUSAL>() {
                dim3 gq((unsigned)((N + GPB - 1) / GPB), (unsigned)H, (unsigned)B);
                span_bwd_dq_generic_kernel<U, VEC, LPR, CPL, CAUSAL><<<gq, 256, 0, st>>>(a);
                if ((rc = launch_status("hsa_span_attn_bwd(dq)"))) return;
                // rows [0, split): leaves and levels 1..kRowsMaxLevel; rows [split, 2N-1): higher levels
                const int total = 2 * N - 1;
                const int split = (L > kRowsMaxLevel) ? level_base(N, kRowsMaxLevel + 1) : total;
                SpanBwdArgs lo = a;
                lo.row_begin = 0;
                dim3 gr((unsigned)((split + GPB - 1) / GPB), (unsigned)H, (unsigned)B);
                span_bwd_dkdv_rows_kernel<U, VEC, LPR, CPL, CAUSAL><<<gr, 256, 0, st>>>(lo, split);
                if ((rc = launch_status("hsa_span_attn_bwd(dkdv rows)"))) return;
                if (split < total) {
                    SpanBwdArgs hi = a;
                    hi.row_begin = split;
                    dim3 gn((unsigned)(total - split), (unsigned)H, (unsigned)B);
                    const size_t smem = (size_t)2 * GPB * D * sizeof(float);
                    span_bwd_dkdv_node_kernel<U, VEC, LPR, CPL, CAUSAL><<<gn, 256, smem, st>>>(hi);
                    rc = launch_status("hsa_span_attn_bwd(dkdv nodes)");
                }
            };
            if (causal) launch.template operator()<true>();
            else launch.template operator()<false>();
        });
        if (!ok) return fail(HSA_ERR_ARG, "hsa_span_attn_bwd: head dim %d not supported (max %d)", D,
                             max_head_dim(dtype, vec));
        return rc;
    });
}

// ------------------------------------------------------------------------------------------------
// Allocation-free backward.
//
// Some hosts of this library may not allocate device memory at the point where they call it: an
// inference-engine plugin whose execute hook is handed pre-bound buffers only, or a serving loop
// whose GPU memory was carved up at start-up and where a cudaMalloc would fail or stall every
// stream of the process.  For them the per-(batch, leaf, head) scratch of the backward lives in the
// library image itself, in the fixed array below, instead of a caller-supplied workspace.
//
// The array is a device symbol: in host code its name is only a handle, so the device address is
// looked up once per device with cudaGetSymbolAddress (with that device current) and that address
// is what the kernels receive.
// ------------------------------------------------------------------------------------------------
#include <mutex>

namespace {
static __device__ __align__(256) float g_static_scratch[HSA_STATIC_SCRATCH_MAX_ELEMS];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
float *g_static_addr[kMaxDevices] = {};

// Device address of g_static_scratch on the current device (looked up on first use per device).
int static_scratch_address(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail((int)e, "hsa_span_attn_bwd_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices)
        return fail(HSA_ERR_ARG, "hsa_span_attn_bwd_static: device index %d beyond the %d supported", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_addr[dev] == nullptr) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(e != cudaSuccess ? (int)e : HSA_ERR_WORKSPACE,
                        "hsa_span_attn_bwd_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_addr[dev] = static_cast<float *>(p);
    }
    *out = g_static_addr[dev];
    return 0;
}
}  // namespace

extern "C" int hsa_span_attn_bwd_static(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE,
                                        hsa_view dOut, hsa_view dQ, hsa_view dK, hsa_view dV, int B, int N, int H,
                                        int D, int radius, int causal, int dtype, void *stream) {
    HSA_CHECK_ARG(Q.ptr && K.ptr && V.ptr && Out.ptr && LSE && dOut.ptr && dQ.ptr && dK.ptr && dV.ptr,
                  "hsa_span_attn_bwd_static: null pointer");
    if (int rc = check_span_shape("hsa_span_attn_bwd_static", B, N, H, D, radius)) return rc;
    const long long elems = (long long)B * N * H;
    if (elems > (long long)HSA_STATIC_SCRATCH_MAX_ELEMS)
        return fail(HSA_ERR_WORKSPACE,
                    "hsa_span_attn_bwd_static: B*N*H = %lld exceeds the built-in scratch of %lld entries; "
                    "use hsa_span_attn_bwd with a caller workspace",
                    elems, (long long)HSA_STATIC_SCRATCH_MAX_ELEMS);
    float *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    // Every scratch entry the key-side kernels read is written by the query-side kernel of the same
    // call first, so nothing needs clearing between calls.
    return hsa_span_attn_bwd_generic(Q, K, V, Out, LSE, dOut, dQ, dK, dV, scratch, B, N, H, D, radius, causal, dtype,
                                     (cudaStream_t)stream);
}
