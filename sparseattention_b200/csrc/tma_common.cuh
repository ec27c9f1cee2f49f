// Tensor maps for the TMA-staged kernels: cuTensorMapEncodeTiled reached through the runtime's driver entry point
// lookup (no link against the driver library), and the one map shape these kernels use.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "hsa_common.cuh"

namespace hsa {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
    // cuTensorMapEncodeTiled is a driver-API call: it needs a context current on the calling thread.  The runtime binds
    // one lazily, so on a thread whose first CUDA call this is (an autograd worker running a backward, for one) it would
    // fail with CUDA_ERROR_INVALID_CONTEXT; cudaFree(0) makes the runtime bind the device's primary context.
    thread_local bool bound = false;
    if (!bound) {
        cudaFree(nullptr);
        bound = true;
    }
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// A view [B, rows, H, D] of 2-byte elements, every `step`-th row; box = 64 elements x 1 head x box_rows rows,
// 128-byte swizzle, rows outside the tensor read as zeros.
inline bool make_map(CUtensorMap *m, const hsa_view &v, int B, int rows, int H, int D, int step, int box_rows) {
    if (encode_tiled() == nullptr) return false;
    const cuuint64_t rows_eff = (cuuint64_t)(rows + step - 1) / step;
    const cuuint64_t row_bytes = (cuuint64_t)v.row_stride * 2 * step;
    cuuint64_t batch_bytes = (cuuint64_t)v.batch_stride * 2;
    if (B == 1) batch_bytes = rows_eff * row_bytes;      // only batch 0 is addressed; any valid stride will do
    const cuuint64_t gdim[4] = {(cuuint64_t)D, (cuuint64_t)H, rows_eff, (cuuint64_t)B};
    const cuuint64_t gstride[3] = {(cuuint64_t)D * 2, row_bytes, batch_bytes};
    const cuuint32_t box[4] = {64u, 1u, (cuuint32_t)box_rows, 1u};
    const cuuint32_t estride[4] = {1u, 1u, 1u, 1u};
    return encode_tiled()(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void *>(v.ptr), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Whether a [B, rows, H, D] view can be described by such a map: heads packed inside a row, batches not overlapping,
// strides inside the descriptor's 40-bit range.
inline bool map_ok(const hsa_view &v, int B, int rows, int H, int D) {
    if (v.row_stride < (int64_t)H * D || v.row_stride * 4 >= (1LL << 40)) return false;
    if (B > 1 && (v.batch_stride * 2 >= (1LL << 40) || v.batch_stride < (int64_t)rows * v.row_stride)) return false;
    return true;
}

// ---------------------------------------------------------------------------------- bounded mbarrier wait
// Every kernel that waits for bulk copies gets two launch arguments from here: how long a CTA waits (clock
// cycles, about a second unless hsa_debug_wait_test changed it) and, for the test of the give-up path only, bytes
// added to what the first barrier of a CTA expects, so that the barrier cannot complete although every copy does.
long long wait_limit_cycles();
unsigned int wait_extra_tx();

#ifdef __CUDACC__
// Wait for phase 0 of an mbarrier.  Returns false when `limit` cycles ran out first.
__device__ __forceinline__ bool mbar_wait_phase0(uint32_t mb, long long limit) {
    uint32_t done = 0;
    const long long start = clock64();
    while (true) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(mb), "r"(0) : "memory");
        if (done) return true;
        if (clock64() - start > limit) return false;
    }
}

// What a CTA that gave up leaves behind instead of results: NaN in every element of `rows` rows of `cols` 2-byte
// elements (bf16 and f16 both read 0x7fff as NaN), so a consumer cannot mistake the tile for data.
__device__ __forceinline__ void fill_rows_nan16(void *base, int64_t row_stride, int rows, int cols, int tid, int nthreads) {
    unsigned short *p = reinterpret_cast<unsigned short *>(base);
    for (int idx = tid; idx < rows * cols; idx += nthreads) p[(int64_t)(idx / cols) * row_stride + idx % cols] = 0x7fffu;
}
#endif

}  // namespace hsa
