// Span attention forward for float32 tensors with the working set of a tile staged in shared memory.
//
// The portable kernel (span_attn_generic.cu) lets every (leaf, head) gather its key / value rows straight from global
// memory: correct for every shape, but each row is fetched through L1 once per leaf that attends to it (about 20 times)
// and the kernel sits at an eighth of the HBM roofline.  Here a CTA owns a tile of TL consecutive leaves of one
// (batch, head): the leaf band with its halo, the tree nodes below the tile (only the left children when causal) and
// one sibling node per level above it are copied into shared memory once (cp.async, 16 bytes per thread), then LPR
// lanes per leaf walk the leaf's candidates (window, then one node per level) with an online softmax in float32 FMAs.
// A lane owns every LPR-th 16-byte piece of the head dimension, so the LPR lanes of a leaf read one contiguous run of a
// row; rows are padded by 64 bytes so that two leaves served by the same shared-memory wavefront fall on different banks.
// Results follow the reference's definition exactly (window and level-0 sibling may name the same leaf: it then counts
// twice), in float32 throughout: the parity bound for this dtype is 1e-5.
#include "tc_common.cuh"

namespace hsa {

struct SpanF32Args {
    const float *q, *k, *v;
    float *out, *lse;
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs;
    int N, L, H, R, causal;
    int band_rows;        // TL + R (+ R when not causal)
    int tree_rows;        // nodes of levels 1 .. log2(TL) - 1 under the tile (left children only when causal)
    int rows;             // band + tree + one node per level from log2(TL) up
    float scale_log2e;
};

// TL leaves per CTA, D the head dimension; 256 threads = TL leaves x LPR lanes, 16 floats of the head dim per lane.
template <int TL, int D>
__global__ void __launch_bounds__(256)
span_fwd_f32_kernel(const SpanF32Args a) {
    constexpr int LPR = 256 / TL;
    static_assert(D == 16 * LPR, "a lane owns four 16-byte pieces of a row");
    constexpr int TLOG = TL == 64 ? 6 : 5;
    constexpr int PITCH = D * 4 + 64;                 // bytes; = 64 mod 128
    constexpr int PIECES = D / 4;                     // 16-byte pieces per row
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *Ks = smem;
    unsigned char *Vs = smem + (size_t)a.rows * PITCH;

    const int tid = threadIdx.x;
    const int ntiles = a.N / TL;
    const int h = blockIdx.x % a.H;
    const int tile = (blockIdx.x / a.H) % ntiles;
    const int b = blockIdx.x / (a.H * ntiles);
    const int t0 = tile * TL;
    const int N = a.N, L = a.L, R = a.R;
    const bool causal = a.causal != 0;
    const int64_t hoff = (int64_t)h * D;

    // ---------------------------------------------------------------- stage the tile's rows
    // shared row r -> node row in the [leaves | parents] ordering (or -1: outside the sequence, zero-filled)
    auto node_of = [&](int r) -> int {
        if (r < a.band_rows) {
            const int m = t0 - R + r;
            return (m >= 0 && m < N) ? m : -1;
        }
        r -= a.band_rows;
        if (r < a.tree_rows) {
            // levels 1 .. TLOG-1: level l holds TL >> l nodes under the tile (half of them when causal: the even ones)
            int l = 1, cnt = causal ? (TL >> 2) : (TL >> 1);
            while (r >= cnt) { r -= cnt; ++l; cnt >>= 1; }
            return level_base(N, l) + (t0 >> l) + (causal ? 2 * r : r);
        }
        const int l = TLOG + (r - a.tree_rows);               // the sibling of the tile's ancestor at level l
        return level_base(N, l) + ((t0 >> l) ^ 1);
    };
    {
        const float *kb = a.k + b * a.k_bs + hoff, *vb = a.v + b * a.v_bs + hoff;
        for (int idx = tid; idx < a.rows * PIECES; idx += 256) {
            const int r = idx / PIECES, c = idx % PIECES;
            const int node = node_of(r);
            const bool ok = node >= 0;
            const int64_t nr = ok ? node : 0;
            cp_async16(smem_u32(Ks + (size_t)r * PITCH + c * 16), kb + nr * a.k_rs + c * 4, ok);
            cp_async16(smem_u32(Vs + (size_t)r * PITCH + c * 16), vb + nr * a.v_rs + c * 4, ok);
        }
        cp_async_commit();
    }

    // ---------------------------------------------------------------- this lane's leaf and its slice of q
    const int leaf = tid / LPR, c = tid % LPR;
    const int n = t0 + leaf;
    // the lanes of one leaf always take the same path; leaves of one warp do not (boundaries, causal levels), so the
    // reductions name only the leaf's own lanes
    const unsigned gmask = (LPR == 32 ? 0xffffffffu : ((1u << LPR) - 1u)) << ((tid & 31) / LPR * LPR);
    float4 q[4];
    {
        const float *qp = a.q + b * a.q_bs + (int64_t)n * a.q_rs + hoff;
#pragma unroll
        for (int m = 0; m < 4; ++m) q[m] = __ldg(reinterpret_cast<const float4 *>(qp + 4 * (c + LPR * m)));
    }
    cp_async_wait<0>();
    __syncthreads();

    float mx = -INFINITY, sum = 0.f;
    float4 acc[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) acc[m] = make_float4(0.f, 0.f, 0.f, 0.f);

    // Four candidates at a time (shared rows `row`, weights w: 0 = not attended, 2 = the window and the level-0 sibling
    // name the same leaf): their dot products are independent instruction chains, one softmax update serves all four.
    auto visit4 = [&](const int (&row)[4], const float (&w)[4]) {
        float x[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned char *kr = Ks + (size_t)row[i] * PITCH;
            float d[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const float4 kv = *reinterpret_cast<const float4 *>(kr + (c + LPR * m) * 16);
                d[m] = fmaf(q[m].w, kv.w, fmaf(q[m].z, kv.z, fmaf(q[m].y, kv.y, q[m].x * kv.x)));
            }
            x[i] = (d[0] + d[1]) + (d[2] + d[3]);
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] += __shfl_xor_sync(gmask, x[i], o);
        }
        float mnew = mx;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[i] = w[i] > 0.f ? x[i] * a.scale_log2e : -INFINITY;
            mnew = fmaxf(mnew, x[i]);
        }
        if (mnew > mx) {                                    // rare after the first few candidates
            const float corr = fast_exp2(mx - mnew);        // 0 on the first ones
            sum *= corr;
#pragma unroll
            for (int m = 0; m < 4; ++m) { acc[m].x *= corr; acc[m].y *= corr; acc[m].z *= corr; acc[m].w *= corr; }
            mx = mnew;
        }
        float p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            p[i] = w[i] > 0.f ? w[i] * fast_exp2(x[i] - mx) : 0.f;
            sum += p[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned char *vr = Vs + (size_t)row[i] * PITCH;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const float4 vv = *reinterpret_cast<const float4 *>(vr + (c + LPR * m) * 16);
                acc[m].x = fmaf(p[i], vv.x, acc[m].x); acc[m].y = fmaf(p[i], vv.y, acc[m].y);
                acc[m].z = fmaf(p[i], vv.z, acc[m].z); acc[m].w = fmaf(p[i], vv.w, acc[m].w);
            }
        }
    };

    // the window; the level-0 sibling (leaf n ^ 1) is folded in where it lies inside it
    const int sib = n ^ 1;
    const bool sib_ok = !causal || sib < n;
    const int hi = causal ? 0 : R;
    for (int j0 = -R; j0 <= hi; j0 += 4) {
        int row[4];
        float w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int j = j0 + i, m = n + j;
            const bool ok = j <= hi && m >= 0 && m < N;
            row[i] = ok ? leaf + R + j : leaf + R;              // a row that exists, whatever the weight
            w[i] = ok ? ((sib_ok && m == sib) ? 2.f : 1.f) : 0.f;
        }
        visit4(row, w);
    }
    // one node per level: the sibling of the leaf's ancestor (left siblings only when causal); with radius 0 the level-0
    // sibling, still a leaf of this tile, was not part of the window and joins them
    auto level_row = [&](int l) -> int {
        if (l == 0) return sib - (t0 - R);
        if (l < TLOG) {
            const int idx = ((n >> l) ^ 1) - (t0 >> l);           // node index under the tile; even when causal
            int off = 0;
            for (int ll = 1; ll < l; ++ll) off += causal ? (TL >> (ll + 1)) : (TL >> ll);
            return a.band_rows + off + (causal ? idx >> 1 : idx);
        }
        return a.band_rows + a.tree_rows + (l - TLOG);
    };
    uint32_t levels = causal ? (uint32_t)n : 0xffffffffu;         // bit l: level l is attended
    levels &= L >= 32 ? 0xffffffffu : ((1u << L) - 1u);
    if (R > 0) levels &= ~1u;                                     // level 0 went with the window
    while (levels != 0) {
        int row[4];
        float w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (levels != 0) {
                const int l = __ffs(levels) - 1;
                levels &= levels - 1;
                row[i] = level_row(l);
                w[i] = 1.f;
            } else {
                row[i] = leaf + R;
                w[i] = 0.f;
            }
        }
        visit4(row, w);
    }

    // ---------------------------------------------------------------- normalise and store
    const float inv = 1.f / sum;
    float *op = a.out + b * a.o_bs + (int64_t)n * a.o_rs + hoff;
#pragma unroll
    for (int m = 0; m < 4; ++m)
        *reinterpret_cast<float4 *>(op + 4 * (c + LPR * m)) = make_float4(acc[m].x * inv, acc[m].y * inv, acc[m].z * inv, acc[m].w * inv);
    if (a.lse != nullptr && c == 0) a.lse[((int64_t)b * N + n) * a.H + h] = (mx + log2f(sum)) * 0.6931471805599453f;
}

template <int TL>
static void f32_layout(SpanF32Args &a) {
    constexpr int TLOG = TL == 64 ? 6 : 5;
    a.band_rows = TL + a.R + (a.causal ? 0 : a.R);
    a.tree_rows = a.causal ? (TL / 2 - 1) : (TL - 2);           // sum over levels 1 .. TLOG-1 of (TL >> l) / (causal ? 2 : 1)
    a.rows = a.band_rows + a.tree_rows + (a.L > TLOG ? a.L - TLOG : 0);
}

static size_t f32_smem(int D, int rows) { return (size_t)2 * rows * (D * 4 + 64); }

}  // namespace hsa

using namespace hsa;

// Shapes the staged float32 forward takes: head dim 64 (64-leaf tiles) or 128 (32-leaf tiles), N a power of two of at
// least one tile, 16-byte aligned views, and a window whose rows fit the shared memory of a CTA.
bool hsa_span_attn_fwd_f32_supported(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, int B, int N, int H, int D, int radius,
                                     int causal, int dtype) {
    if (dtype != HSA_F32 || (D != 64 && D != 128)) return false;
    const int TL = D == 64 ? 64 : 32;
    if (B < 1 || H < 1 || N < TL || (N & (N - 1)) != 0 || radius < 0) return false;
    if ((int64_t)(N / TL) * H * B > 0x7fffffffLL) return false;
    if (!view_vec_ok(Q, 4) || !view_vec_ok(K, 4) || !view_vec_ok(V, 4) || !view_vec_ok(Out, 4)) return false;
    SpanF32Args a{};
    a.R = radius; a.causal = causal; a.L = ilog2((unsigned)N);
    if (TL == 64) f32_layout<64>(a); else f32_layout<32>(a);
    return f32_smem(D, a.rows) <= 200 * 1024;
}

int hsa_span_attn_fwd_f32(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H, int D, int radius,
                          int causal, int dtype, cudaStream_t st) {
    if (!hsa_span_attn_fwd_f32_supported(Q, K, V, Out, B, N, H, D, radius, causal, dtype))
        return fail(HSA_ERR_ARG, "hsa_span_attn_fwd: shape not taken by the staged float32 kernel");
    SpanF32Args a{};
    a.q = (const float *)Q.ptr; a.k = (const float *)K.ptr; a.v = (const float *)V.ptr; a.out = (float *)Out.ptr; a.lse = LSE;
    a.q_bs = Q.batch_stride; a.q_rs = Q.row_stride; a.k_bs = K.batch_stride; a.k_rs = K.row_stride;
    a.v_bs = V.batch_stride; a.v_rs = V.row_stride; a.o_bs = Out.batch_stride; a.o_rs = Out.row_stride;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.R = radius; a.causal = causal;
    a.scale_log2e = 1.4426950408889634f / sqrtf((float)D);
    const int TL = D == 64 ? 64 : 32;
    if (TL == 64) f32_layout<64>(a); else f32_layout<32>(a);
    const size_t smem = f32_smem(D, a.rows);
    const unsigned grid = (unsigned)((int64_t)B * (N / TL) * H);
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "hsa_span_attn_fwd(f32): shared memory %zu: %s", smem, cudaGetErrorString(e));
        kernel<<<grid, 256, smem, st>>>(a);
        return launch_status("hsa_span_attn_fwd(f32)");
    };
    return D == 64 ? go(span_fwd_f32_kernel<64, 64>) : go(span_fwd_f32_kernel<32, 128>);
}
