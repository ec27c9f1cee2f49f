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
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            bool keep = dropout_keep(key, a.site0, id0 + i, a.threshold);
            if (a.site1 != 0) keep = keep && dropout_keep(key, a.site1, id0 + i, a.threshold);
            v[i] = keep ? v[i] * a.scale : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>((__nv_bfloat16 *)a.out + b * a.out_bs + (int64_t)row * a.out_rs + col) = o;
    }
}

}  // namespace hsa

using namespace hsa;

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
