// Element-wise companions of the fused products: regenerating a dropout mask outside a product's epilogue (the
// backward of a dropout whose forward ran inside hsa_gemm_ex), with an optional float32 -> bfloat16 conversion on the way.
#include "hsa_common.cuh"
#include "rng_common.cuh"

namespace hsa {

struct DropArgs {
    const void *in;
    void *out;
    int64_t in_bs, in_rs, out_bs, out_rs;
    int batches, rows, col_begin, ncols;          // the column range [col_begin, col_begin + ncols) of every row is processed
    long long N, rows_total, row_offset, col_shift; // the logical [batches, rows_total, N] tensor element ids refer to;
                                                    // a column c of in/out is column c + col_shift of that tensor
    const unsigned long long *rng_state;
    unsigned int site0, site1, threshold;
    float scale;
};

template <typename TIn>
__global__ void __launch_bounds__(256)
dropout_apply_kernel(DropArgs a) {
    const int vec_per_row = a.ncols / 8;
    const long long total = (long long)a.batches * a.rows * vec_per_row;
    const unsigned long long key = *a.rng_state;
    const uint32_t salt0 = dropout_salt(key, a.site0, 0), salt1 = dropout_salt(key, a.site1, 0);
    for (long long idx = (long long)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
        const int c8 = (int)(idx % vec_per_row);
        const long long br = idx / vec_per_row;
        const int row = (int)(br % a.rows), b = (int)(br / a.rows);
        const int col = a.col_begin + 8 * c8;
        float v[8];
        const TIn *src = (const TIn *)a.in + b * a.in_bs + (int64_t)row * a.in_rs + col;
        if constexpr (sizeof(TIn) == 4) {
            const float4 lo = *reinterpret_cast<const float4 *>(src), hi = *reinterpret_cast<const float4 *>(src + 4);
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        } else {
            const uint4 raw = *reinterpret_cast<const uint4 *>(src);
            const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&raw);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(e[i]);
        }
        const unsigned long long id0 = ((unsigned long long)b * a.rows_total + (unsigned long long)(row + a.row_offset)) *
                                       (unsigned long long)a.N + (unsigned long long)(col + a.col_shift);
        uint4 o;
        __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&o);
        if ((id0 & 1ull) == 0 && id0 + 8 <= kDropoutRunMaxElems) {
            dropout_run(v, salt0, salt1, a.site1 != 0, id0, a.threshold, a.scale);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                bool keep = dropout_keep(key, a.site0, id0 + i, a.threshold);
                if (a.site1 != 0) keep = keep && dropout_keep(key, a.site1, id0 + i, a.threshold);
                v[i] = keep ? v[i] * a.scale : 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>((__nv_bfloat16 *)a.out + b * a.out_bs + (int64_t)row * a.out_rs + col) = o;
    }
}

// ---------------------------------------------------------------------------------------------- column sums
// out[c] = sum over rows of x[r, c] (bias gradients).  A thread owns 8 consecutive columns and every fourth row of a block
// of kCsRows rows; the four row lanes are combined through shared memory, blocks by a second kernel in block order.
constexpr int kCsRows = 256;
// The narrow matrices of the layers (a few hundred columns) take smaller blocks, or too few of them are in flight
constexpr int kCsRowsNarrow = 64;
__host__ __device__ inline int cs_rows_per_block(int cols) { return cols <= 4096 ? kCsRowsNarrow : kCsRows; }

// `rows4(r, n, col, v)` yields the values of rows r, r+4, .. (n <= 4 of them) at columns col..col+7, having issued all
// of their loads before anything depends on one (one load in flight per thread leaves HBM mostly idle).
template <typename F>
__device__ __forceinline__ void colsum_block(int rows_here, int cols, int col0, float *__restrict__ partial_row, F &&rows4) {
    __shared__ float red[4][64][8];
    const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
    const int col = col0 + 8 * cx;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (col < cols) {
        for (int r = ry; r < rows_here; r += 16) {
            float v[4][8];
            const int n = min(4, (rows_here - r + 3) / 4);
            rows4(r, n, col, v);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (u < n) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += v[u][i];
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[ry][cx][i] = acc[i];
    __syncthreads();
    if (ry == 0 && col < cols) {
#pragma unroll
        for (int i = 0; i < 8; ++i) partial_row[col + i] = (red[0][cx][i] + red[1][cx][i]) + (red[2][cx][i] + red[3][cx][i]);
    }
}

__global__ void __launch_bounds__(256)
column_sums_kernel(const __nv_bfloat16 *__restrict__ x, int64_t row_stride, int64_t rows, int cols, float *__restrict__ partial) {
    const int rpb = cs_rows_per_block(cols);
    const int64_t r0 = (int64_t)blockIdx.y * rpb;
    const int rows_here = (int)((rows - r0) < rpb ? (rows - r0) : rpb);
    colsum_block(rows_here, cols, blockIdx.x * 512, partial + (int64_t)blockIdx.y * cols, [&](int r, int n, int col, float (&v)[4][8]) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < n) raw[u] = __ldg(reinterpret_cast<const uint4 *>(x + (r0 + r + 4 * u) * row_stride + col));
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < n) {
                const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&raw[u]);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[u][i] = __bfloat162float(e[i]);
            }
    });
}

// out[c] = sum over blocks of partial[block][c].  A thread block owns 32 columns; its 32 warps sum interleaved slices of
// the block list (block w, w + 32, ..., four loads in flight each) and the 32 slice sums are added in slice order: the
// order of additions is fixed, so the result is reproducible.
__global__ void __launch_bounds__(1024)
column_sums_reduce_kernel(const float *__restrict__ partial, int blocks, int cols, float *__restrict__ out) {
    __shared__ float slice[32][33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (c < cols) {
        int b = w;
        for (; b + 96 < blocks; b += 128) {
            s0 += partial[(int64_t)b * cols + c];
            s1 += partial[(int64_t)(b + 32) * cols + c];
            s2 += partial[(int64_t)(b + 64) * cols + c];
            s3 += partial[(int64_t)(b + 96) * cols + c];
        }
        for (; b < blocks; b += 32) s0 += partial[(int64_t)b * cols + c];
    }
    slice[w][lane] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (w == 0 && c < cols) {
        float t = slice[0][lane];
#pragma unroll
        for (int i = 1; i < 32; ++i) t += slice[i][lane];
        out[c] = t;
    }
}

// out = bfloat16(dropout mask * in) for a float32 matrix [rows, cols] (element id = r * cols + c; no mask when rng_state is
// null) together with the column sums of what was written: the step "gradient through a residual dropout, then the bias
// gradient of the projection under it" in one pass over the gradient instead of three.
__global__ void __launch_bounds__(256)
dropout_cast_colsum_kernel(const float *__restrict__ in, int64_t in_rs, __nv_bfloat16 *__restrict__ out, int64_t out_rs, int64_t rows,
                           int cols, const unsigned long long *__restrict__ rng_state, unsigned int site0, unsigned int site1,
                           unsigned int threshold, float scale, float *__restrict__ partial) {
    const int rpb = cs_rows_per_block(cols);
    const int64_t r0 = (int64_t)blockIdx.y * rpb;
    const int rows_here = (int)((rows - r0) < rpb ? (rows - r0) : rpb);
    const bool drop = rng_state != nullptr;
    const unsigned long long key = drop ? *rng_state : 0ull;
    const uint32_t salt0 = dropout_salt(key, site0, 0), salt1 = dropout_salt(key, site1, 0);
    colsum_block(rows_here, cols, blockIdx.x * 512, partial + (int64_t)blockIdx.y * cols, [&](int r, int n, int col, float (&v)[4][8]) {
        float4 lo[4], hi[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < n) {
                const float *src = in + (r0 + r + 4 * u) * in_rs + col;
                lo[u] = __ldg(reinterpret_cast<const float4 *>(src));
                hi[u] = __ldg(reinterpret_cast<const float4 *>(src + 4));
            }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < n) {
                const int64_t row = r0 + r + 4 * u;
                float w[8] = {lo[u].x, lo[u].y, lo[u].z, lo[u].w, hi[u].x, hi[u].y, hi[u].z, hi[u].w};
                if (drop) dropout_run(w, salt0, salt1, site1 != 0, (unsigned long long)row * (unsigned long long)cols + (unsigned long long)col, threshold, scale);
                uint4 o;
                __nv_bfloat162 *p2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    p2[i] = __floats2bfloat162_rn(w[2 * i], w[2 * i + 1]);
                    v[u][2 * i] = __low2float(p2[i]);              // the sums are those of the stored (rounded) values
                    v[u][2 * i + 1] = __high2float(p2[i]);
                }
                *reinterpret_cast<uint4 *>(out + row * out_rs + col) = o;
            }
    });
}

// Backward of the label-smoothed cross entropy IN PLACE (the logits become their gradient) together with the column
// sums of that gradient (the bias gradient of the layer that produced the logits): a block walks kCsRows rows of a slab
// of 512 columns, so the sums come for free and the separate reduction pass over the [tokens, vocabulary] matrix goes away.
__global__ void __launch_bounds__(256)
ce_bwd_colsum_kernel(__nv_bfloat16 *logits, int64_t row_stride, const long long *__restrict__ targets, const float *__restrict__ lse,
                     const float *__restrict__ grad_scale, int64_t rows, int V, int Vp, float eps, long long ignore_index,
                     float *__restrict__ partial) {
    const int64_t r0 = (int64_t)blockIdx.y * kCsRows;
    const int rows_here = (int)((rows - r0) < kCsRows ? (rows - r0) : kCsRows);
    const float g0 = grad_scale[0], sm = eps / (float)V;
    colsum_block(rows_here, Vp, blockIdx.x * 512, partial + (int64_t)blockIdx.y * Vp, [&](int r, int n, int col, float (&v)[4][8]) {
        uint4 raw[4];
        long long tgt[4];
        float l[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < n) {
                const int64_t row = r0 + r + 4 * u;
                raw[u] = *reinterpret_cast<const uint4 *>(logits + row * row_stride + col);
                tgt[u] = targets[row];
                l[u] = lse[row];
            }
        constexpr float kL2e = 1.4426950408889634f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (u < n) {
                const uint32_t *w = reinterpret_cast<const uint32_t *>(&raw[u]);
                const float g = tgt[u] == ignore_index ? 0.f : g0;
                const float gs = g * sm, gt = g * (1.f - eps), l2 = l[u] * kL2e;
                const long long tdiff = tgt[u] - col;
                const int tcol = (tdiff >= 0 && tdiff < 8) ? (int)tdiff : -1;      // the target's column inside these 8, if any
                const int nv = V - col;                                               // classes among these 8 columns
                uint4 o;
                uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    // two bfloat16 logits per word: the low half is element i, the high half element i+1
                    const float x0 = __uint_as_float(w[i / 2] << 16), x1 = __uint_as_float(w[i / 2] & 0xffff0000u);
                    float d0, d1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(d0) : "f"(fmaf(x0, kL2e, -l2)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(d1) : "f"(fmaf(x1, kL2e, -l2)));
                    d0 = fmaf(d0, g, -gs) - (i == tcol ? gt : 0.f);
                    d1 = fmaf(d1, g, -gs) - (i + 1 == tcol ? gt : 0.f);
                    if (i >= nv) d0 = 0.f;
                    if (i + 1 >= nv) d1 = 0.f;
                    v[u][i] = d0;
                    v[u][i + 1] = d1;
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(d0, d1);
                    ow[i / 2] = *reinterpret_cast<const uint32_t *>(&pk);
                }
                *reinterpret_cast<uint4 *>(logits + (r0 + r + 4 * u) * row_stride + col) = o;
            }
    });
}

}  // namespace hsa

using namespace hsa;

extern "C" size_t hsa_column_sums_partial_bytes(long long rows, int cols) {
    if (rows < 1 || cols < 1) return 0;
    const int rpb = cs_rows_per_block(cols);
    return (size_t)((rows + rpb - 1) / rpb) * cols * sizeof(float);
}

extern "C" int hsa_column_sums(const void *x, long long row_stride, long long rows, int cols, float *out, float *partial, void *stream) {
    HSA_CHECK_ARG(x && out && partial, "hsa_column_sums: null pointer");
    HSA_CHECK_ARG(rows >= 1 && cols >= 8 && cols % 8 == 0 && row_stride % 8 == 0 && aligned16(x), "hsa_column_sums: bad shape or alignment");
    const int rpb = cs_rows_per_block(cols);
    const int blocks = (int)((rows + rpb - 1) / rpb);
    HSA_CHECK_ARG(blocks <= 65535, "hsa_column_sums: too many rows");
    dim3 grid((unsigned)((cols + 511) / 512), (unsigned)blocks);
    column_sums_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, row_stride, rows, cols, partial);
    if (int rc = launch_status("hsa_column_sums")) return rc;
    column_sums_reduce_kernel<<<(unsigned)((cols + 31) / 32), 1024, 0, (cudaStream_t)stream>>>(partial, blocks, cols, out);
    return launch_status("hsa_column_sums(reduce)");
}

extern "C" int hsa_dropout_cast_colsum(const float *in, long long in_row_stride, void *out, long long out_row_stride, long long rows,
                                       int cols, const unsigned long long *rng_state, unsigned int site0, unsigned int site1,
                                       unsigned int threshold, float scale, float *col_sums, float *partial, void *stream) {
    HSA_CHECK_ARG(in && out && col_sums && partial, "hsa_dropout_cast_colsum: null pointer");
    HSA_CHECK_ARG(rows >= 1 && cols >= 8 && cols % 8 == 0 && in_row_stride % 4 == 0 && out_row_stride % 8 == 0 && aligned16(in) && aligned16(out),
                  "hsa_dropout_cast_colsum: bad shape or alignment");
    HSA_CHECK_ARG(rng_state == nullptr || (site0 != 0 && (unsigned long long)rows * (unsigned long long)cols <= kDropoutRunMaxElems),
                  "hsa_dropout_cast_colsum: bad dropout description (site 0, or more than 2^33 elements)");
    const int rpb = cs_rows_per_block(cols);
    const int blocks = (int)((rows + rpb - 1) / rpb);
    HSA_CHECK_ARG(blocks <= 65535, "hsa_dropout_cast_colsum: too many rows");
    dim3 grid((unsigned)((cols + 511) / 512), (unsigned)blocks);
    dropout_cast_colsum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(in, in_row_stride, (__nv_bfloat16 *)out, out_row_stride, rows, cols,
                                                                      rng_state, site0, site1, threshold, scale, partial);
    if (int rc = launch_status("hsa_dropout_cast_colsum")) return rc;
    column_sums_reduce_kernel<<<(unsigned)((cols + 31) / 32), 1024, 0, (cudaStream_t)stream>>>(partial, blocks, cols, col_sums);
    return launch_status("hsa_dropout_cast_colsum(reduce)");
}

extern "C" int hsa_cross_entropy_bwd_inplace(void *logits, long long row_stride, const long long *targets, const float *lse,
                                             const float *grad_scale, long long rows, int V, int Vp, float smoothing,
                                             long long ignore_index, float *col_sums, float *partial, void *stream) {
    HSA_CHECK_ARG(logits && targets && lse && grad_scale && col_sums && partial, "hsa_cross_entropy_bwd_inplace: null pointer");
    HSA_CHECK_ARG(rows >= 1 && V >= 1 && Vp >= V && Vp % 8 == 0 && row_stride >= Vp && row_stride % 8 == 0 && aligned16(logits),
                  "hsa_cross_entropy_bwd_inplace: bad shape or alignment");
    HSA_CHECK_ARG(smoothing >= 0.f && smoothing < 1.f, "hsa_cross_entropy_bwd_inplace: label smoothing %f outside [0, 1)", smoothing);
    const int blocks = (int)((rows + kCsRows - 1) / kCsRows);
    HSA_CHECK_ARG(blocks <= 65535, "hsa_cross_entropy_bwd_inplace: too many rows");
    dim3 grid((unsigned)((Vp + 511) / 512), (unsigned)blocks);
    ce_bwd_colsum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16 *)logits, row_stride, targets, lse, grad_scale, rows, V,
                                                                Vp, smoothing, ignore_index, partial);
    if (int rc = launch_status("hsa_cross_entropy_bwd_inplace")) return rc;
    column_sums_reduce_kernel<<<(unsigned)((Vp + 31) / 32), 1024, 0, (cudaStream_t)stream>>>(partial, blocks, Vp, col_sums);
    return launch_status("hsa_cross_entropy_bwd_inplace(reduce)");
}

extern "C" int hsa_dropout_apply(hsa_view in, int in_dtype, hsa_view out, int batches, int rows, int col_begin, int ncols,
                                 long long N, long long rows_total, long long row_offset, long long col_shift,
                                 const unsigned long long *rng_state, unsigned int site0, unsigned int site1,
                                 unsigned int threshold, float scale, void *stream) {
    HSA_CHECK_ARG(in.ptr && out.ptr && rng_state, "hsa_dropout_apply: null pointer");
    HSA_CHECK_ARG(in_dtype == HSA_F32 || in_dtype == HSA_BF16, "hsa_dropout_apply: the input is float32 or bfloat16");
    HSA_CHECK_ARG(batches >= 1 && rows >= 1 && ncols >= 8 && ncols % 8 == 0 && col_begin >= 0 && col_begin % 8 == 0 && site0 != 0,
                  "hsa_dropout_apply: bad shape (column ranges are multiples of 8)");
    const int ies = in_dtype == HSA_F32 ? 4 : 2;
    if (!aligned16(in.ptr) || !aligned16(out.ptr) || (in.row_stride * ies) % 16 || (in.batch_stride * ies) % 16 ||
        out.row_stride % 8 || out.batch_stride % 8)
        return fail(HSA_ERR_ALIGN, "hsa_dropout_apply: pointers and strides must be 16-byte aligned");
    DropArgs a{in.ptr, out.ptr, in.batch_stride, in.row_stride, out.batch_stride, out.row_stride, batches, rows, col_begin,
               ncols, N, rows_total, row_offset, col_shift, rng_state, site0, site1, threshold, scale};
    const long long total = (long long)batches * rows * (ncols / 8);
    const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (in_dtype == HSA_F32) dropout_apply_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    else dropout_apply_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    return launch_status("hsa_dropout_apply");
}
