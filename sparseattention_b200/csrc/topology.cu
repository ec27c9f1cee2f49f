// Tree topology tables in closed form, and the pairwise-mean pyramid that seeds the parents.
#include "hsa_common.cuh"

namespace hsa {

// forward_idx / forward_mask: one thread per (leaf, level).  gather: one thread per node.
// The closed forms reproduce hierarchical_attention/ops/topology.py:37-59 and :103-122 exactly:
//   idx[n,l]  = base(l) + ((n >> l) ^ 1)
//   mask[n,l] = causal && bit l of n is clear       (sibling lies to the right = future)
//   gather[r] = ((j^1) << l, ((j^1)+1) << l, l) for node r = (level l, index j) when it has a
//               sibling that may attend to it (causal: j even), else (-1,-1,-1).
__global__ void topology_kernel(int N, int L, int causal, int32_t *__restrict__ idx,
                                uint8_t *__restrict__ mask, int32_t *__restrict__ gather) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n_fwd = (int64_t)N * L;
    if (tid < n_fwd) {
        const int n = (int)(tid / L), l = (int)(tid % L);
        if (idx) idx[tid] = sibling_row(N, n, l);
        if (mask) mask[tid] = (causal && ((n >> l) & 1) == 0) ? 1 : 0;
    }
    const int total = 2 * N - 1;
    if (gather && tid < total) {
        // locate (level, index) of row tid: level l spans [base(l), base(l) + (N >> l))
        int r = (int)tid, l = 0, j = r;
        if (r >= N) {
            const int rem = 2 * N - r;             // in (N >> (l-1)) .. (N >> l) + 1
            l = L - ilog2((unsigned)(rem - 1));    // rem-1 in [N>>l, N>>(l-1))
            j = r - level_base(N, l);
        }
        int s = -1, e = -1, lv = -1;
        const bool is_root = (l == L);
        if (!is_root && (!causal || (j & 1) == 0)) {
            s = (j ^ 1) << l;
            e = ((j ^ 1) + 1) << l;
            lv = l;
        }
        gather[3 * (int64_t)r + 0] = s;
        gather[3 * (int64_t)r + 1] = e;
        gather[3 * (int64_t)r + 2] = lv;
    }
}

// ---- pairwise-mean pyramid ----------------------------------------------------------------
// One thread owns one vector column of one chunk of 2^K consecutive source rows and folds them
// with a binary-counter stack, rounding to T after every level exactly as the reference's
// per-level `0.5*a + 0.5*b` torch ops do (ops/topology.py:153-169).  Nodes of level l (1..K)
// above the source rows land at dst_level[l-1] + chunk * 2^(K-l) + t.  Incomplete pairs (odd
// tails) never merge, which drops them as the reference does.
constexpr int kPyrK = 4;
struct PyramidArgs {
    int64_t dst_level_off[kPyrK];  // element offset (in rows) of each produced level inside y
    int n_src;                     // source rows
    int nlevels;                   // levels produced by this pass (<= kPyrK)
};

template <typename T, int VEC>
__global__ void pyramid_fwd_kernel(const T *__restrict__ src, int64_t src_bs, int64_t src_rs,
                                   T *__restrict__ y, int64_t y_bs, int64_t y_rs, int d,
                                   PyramidArgs a) {
    const int cols = d / VEC;
    const int nchunks = (a.n_src + (1 << kPyrK) - 1) >> kPyrK;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int col = (int)(tid % cols);
    const int chunk = (int)((tid / cols) % nchunks);
    const int b = blockIdx.y;
    if (tid / cols >= nchunks) return;
    const T *s = src + b * src_bs + (int64_t)col * VEC;
    T *out = y + b * y_bs + (int64_t)col * VEC;

    float stack[kPyrK][VEC];
    const int first = chunk << kPyrK;
#pragma unroll
    for (int i = 0; i < (1 << kPyrK); ++i) {
        const int r = first + i;
        if (r >= a.n_src) break;
        float cur[VEC];
        load_vec<T, VEC>(s + (int64_t)r * src_rs, cur);
        // carry: after leaf i, every trailing 1-bit of i merges one level up
#pragma unroll
        for (int l = 0; l < kPyrK; ++l) {
            if (l >= a.nlevels) break;
            if (((i >> l) & 1) == 0) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) stack[l][e] = cur[e];
                break;
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                cur[e] = Traits<T>::to_f(Traits<T>::from_f(0.5f * stack[l][e] + 0.5f * cur[e]));
            const int64_t node = ((int64_t)chunk << (kPyrK - 1 - l)) + (i >> (l + 1));
            store_vec<T, VEC>(out + (a.dst_level_off[l] + node) * y_rs, cur);
        }
    }
}

// gx[n] = 0.5 * G1[n>>1],  G_l[i] = gy_l[i] + 0.5 * G_{l+1}[i>>1]  (terms of missing nodes are 0),
// each G rounded to T as autograd's per-level accumulation does.
template <typename T, int VEC>
__global__ void pyramid_bwd_kernel(const T *__restrict__ gy, int64_t gy_bs, int64_t gy_rs,
                                   T *__restrict__ gx, int64_t gx_bs, int64_t gx_rs, int N, int d,
                                   int nlevels) {
    const int cols = d / VEC;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int col = (int)(tid % cols);
    const int64_t n = tid / cols;
    if (n >= N) return;
    const int b = blockIdx.y;
    const T *g = gy + b * gy_bs + (int64_t)col * VEC;
    // level sizes and offsets: size_l = N >> l (floor), offset_l = sum_{k<l} size_k, l = 1..nlevels
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    // offset of level l = sum of the sizes of the levels below it; walked top-down from the total (no per-thread table)
    int64_t o = 0;
    for (int l = 1; l <= nlevels; ++l) o += (N >> l);
    bool have = false;
    for (int l = nlevels; l >= 1; --l) {
        o -= (N >> l);
        const int64_t i = n >> l;
        if (i < (int64_t)(N >> l)) {
            float v[VEC];
            load_vec<T, VEC>(g + (o + i) * gy_rs, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                acc[e] = have ? Traits<T>::to_f(Traits<T>::from_f(v[e] + Traits<T>::to_f(Traits<T>::from_f(0.5f * acc[e]))))
                              : v[e];
            have = true;
        } else {
            have = false;   // a leaf outside this level's complete pairs has no ancestors above either
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
        }
    }
    float outv[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) outv[e] = have ? 0.5f * acc[e] : 0.f;
    store_vec<T, VEC>(gx + b * gx_bs + n * gx_rs + (int64_t)col * VEC, outv);
}

}  // namespace hsa

using namespace hsa;

extern "C" int hsa_topology_build(int N, int causal, int32_t *fwd_idx, uint8_t *fwd_mask,
                                  int32_t *gather, void *stream) {
    HSA_CHECK_ARG(N >= 1 && (N & (N - 1)) == 0, "hsa_topology_build: N=%d must be a power of two", N);
    HSA_CHECK_ARG(N <= (1 << 29), "hsa_topology_build: N=%d too large for int32 rows", N);
    const int L = ilog2((unsigned)N);
    const int64_t work = ((int64_t)N * L > 2LL * N - 1) ? (int64_t)N * L : 2LL * N - 1;
    const int threads = 256;
    const int64_t blocks = (work + threads - 1) / threads;
    topology_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(N, L, causal ? 1 : 0, fwd_idx,
                                                                            fwd_mask, gather);
    return launch_status("hsa_topology_build");
}

extern "C" int64_t hsa_span_input_y_rows(int64_t N) {
    int64_t m = 0;
    while (N > 1) { N >>= 1; m += N; }
    return m;
}

namespace {
template <typename T, int VEC>
int pyramid_fwd(hsa_view x, hsa_view y, int B, int N, int d, cudaStream_t st) {
    // pass p turns level p*K rows into levels p*K+1 .. p*K+K
    int64_t level_off = 0;     // row offset in y of the next level to be produced
    const T *src = (const T *)x.ptr;
    int64_t src_bs = x.batch_stride, src_rs = x.row_stride;
    int n_src = N;
    while (n_src > 1) {
        PyramidArgs a{};
        a.n_src = n_src;
        int n = n_src, nl = 0;
        int64_t off = level_off;
        int64_t last_off = 0;
        int last_n = 0;
        while (nl < kPyrK && n > 1) {
            n >>= 1;
            a.dst_level_off[nl] = off;
            last_off = off; last_n = n;
            off += n;
            ++nl;
        }
        a.nlevels = nl;
        const int cols = d / VEC;
        const int nchunks = (n_src + (1 << kPyrK) - 1) >> kPyrK;
        const int64_t work = (int64_t)cols * nchunks;
        const int threads = 128;
        dim3 grid((unsigned)((work + threads - 1) / threads), (unsigned)B);
        pyramid_fwd_kernel<T, VEC><<<grid, threads, 0, st>>>(src, src_bs, src_rs, (T *)y.ptr, y.batch_stride,
                                                              y.row_stride, d, a);
        // next pass reads the last level just written
        src = (const T *)y.ptr + last_off * y.row_stride;
        src_bs = y.batch_stride; src_rs = y.row_stride;
        n_src = last_n;
        level_off = off;
    }
    return launch_status("hsa_span_input_y_fwd");
}
}  // namespace

extern "C" int hsa_span_input_y_fwd(hsa_view x, hsa_view y, int B, int N, int d, int dtype, void *stream) {
    HSA_CHECK_ARG(B >= 1 && B <= 65535 && N >= 2 && d >= 1, "hsa_span_input_y_fwd: bad shape B=%d N=%d d=%d", B, N, d);
    HSA_CHECK_ARG(x.ptr && y.ptr, "hsa_span_input_y_fwd: null pointer");
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const bool vec = view_vec_ok(x, sizeof(T)) && view_vec_ok(y, sizeof(T)) && d % Traits<T>::kVec == 0;
        return vec ? pyramid_fwd<T, Traits<T>::kVec>(x, y, B, N, d, (cudaStream_t)stream)
                   : pyramid_fwd<T, 1>(x, y, B, N, d, (cudaStream_t)stream);
    });
}

extern "C" int hsa_span_input_y_bwd(hsa_view gy, hsa_view gx, int B, int N, int d, int dtype, void *stream) {
    HSA_CHECK_ARG(B >= 1 && B <= 65535 && N >= 2 && d >= 1, "hsa_span_input_y_bwd: bad shape B=%d N=%d d=%d", B, N, d);
    HSA_CHECK_ARG(gy.ptr && gx.ptr, "hsa_span_input_y_bwd: null pointer");
    int nlevels = 0;
    for (int n = N; n > 1; n >>= 1) ++nlevels;
    return dispatch_dtype(dtype, [&]<typename T>() -> int {
        const bool vec = view_vec_ok(gy, sizeof(T)) && view_vec_ok(gx, sizeof(T)) && d % Traits<T>::kVec == 0;
        auto go = [&]<int VEC>() -> int {
            const int64_t work = (int64_t)(d / VEC) * N;
            const int threads = 128;
            dim3 grid((unsigned)((work + threads - 1) / threads), (unsigned)B);
            pyramid_bwd_kernel<T, VEC><<<grid, threads, 0, (cudaStream_t)stream>>>(
                (const T *)gy.ptr, gy.batch_stride, gy.row_stride, (T *)gx.ptr, gx.batch_stride, gx.row_stride, N, d,
                nlevels);
            return launch_status("hsa_span_input_y_bwd");
        };
        return vec ? go.template operator()<Traits<T>::kVec>() : go.template operator()<1>();
    });
}
