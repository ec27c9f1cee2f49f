// C ABI glue: error reporting, version, and the algorithm choice for span attention.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "hsa_common.cuh"
#include "tma_common.cuh"

namespace hsa {
namespace {
thread_local char g_err[512] = "";
}
void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
namespace {
std::atomic<long long> g_wait_limit{2000000000LL};
std::atomic<unsigned int> g_wait_extra{0u};
}
long long wait_limit_cycles() { return g_wait_limit.load(std::memory_order_relaxed); }
unsigned int wait_extra_tx() { return g_wait_extra.load(std::memory_order_relaxed); }
}  // namespace hsa

using namespace hsa;

extern "C" int hsa_debug_wait_test(long long limit_cycles, unsigned int extra_tx_bytes) {
    if (limit_cycles <= 0) return fail(HSA_ERR_ARG, "hsa_debug_wait_test: the limit must be positive");
    g_wait_limit.store(limit_cycles);
    g_wait_extra.store(extra_tx_bytes);
    return 0;
}

int hsa_span_attn_fwd_generic(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H,
                              int D, int radius, int causal, int dtype, cudaStream_t st);
size_t hsa_span_attn_bwd_generic_workspace(int B, int N, int H);
int hsa_span_attn_bwd_generic(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut,
                              hsa_view dQ, hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D,
                              int radius, int causal, int dtype, cudaStream_t st);

bool hsa_span_attn_fwd_tc_supported(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, int B, int N, int H, int D,
                                    int radius, int causal, int dtype);
int hsa_span_attn_fwd_tc(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H, int D,
                         int radius, int causal, int dtype, cudaStream_t st);

bool hsa_span_attn_fwd_tc128_supported(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, int B, int N, int H, int D,
                                       int radius, int causal, int dtype);
int hsa_span_attn_fwd_tc128(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H, int D,
                            int radius, int causal, int dtype, cudaStream_t st);
bool hsa_span_attn_bwd_tc_supported(const hsa_view *views, int nviews, int B, int N, int H, int D, int radius,
                                    int causal, int dtype);
size_t hsa_span_attn_bwd_tc_workspace(int B, int N, int H, int D);
bool hsa_span_attn_bwd_tc8_supported(const hsa_view *views, int nviews, int B, int N, int H, int D, int radius,
                                     int causal, int dtype);
int hsa_span_attn_bwd_tc8(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut, hsa_view dQ,
                          hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D, int radius, int causal,
                          int dtype, cudaStream_t st);
int hsa_span_attn_bwd_tc(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut, hsa_view dQ,
                         hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D, int radius, int causal,
                         int dtype, cudaStream_t st);

bool hsa_span_attn_fwd_f32_supported(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, int B, int N, int H, int D, int radius,
                                     int causal, int dtype);
int hsa_span_attn_fwd_f32(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H, int D, int radius,
                          int causal, int dtype, cudaStream_t st);

extern "C" int hsa_version(void) { return 200; }   // 0.2.0

extern "C" int hsa_copy_rows_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t row_bytes,
                                   size_t rows, int kind, void *stream) {
    HSA_CHECK_ARG(dst && src, "hsa_copy_rows_async: null pointer");
    HSA_CHECK_ARG(kind >= 0 && kind <= 2, "hsa_copy_rows_async: kind must be 0 (host to device), 1 (device to host) or 2");
    HSA_CHECK_ARG(row_bytes <= dst_pitch && row_bytes <= src_pitch, "hsa_copy_rows_async: a row is longer than a pitch");
    if (rows == 0 || row_bytes == 0) return 0;
    const cudaMemcpyKind k = kind == 0 ? cudaMemcpyHostToDevice : kind == 1 ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
    cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, k, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : fail((int)e, "hsa_copy_rows_async: %s", cudaGetErrorString(e));
}

extern "C" const char *hsa_last_error(void) { return g_err; }

extern "C" int hsa_compiled_arch(void) {
#ifdef HSA_TARGET_ARCH
    return HSA_TARGET_ARCH;
#else
    return 0;
#endif
}

extern "C" int hsa_span_attn_fwd(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N,
                                 int H, int D, int radius, int causal, int dtype, int algo, void *stream) {
    HSA_CHECK_ARG(Q.ptr && K.ptr && V.ptr && Out.ptr, "hsa_span_attn_fwd: null pointer");
    HSA_CHECK_ARG(algo >= 0 && algo <= 4, "hsa_span_attn_fwd: unknown algo %d", algo);
    cudaStream_t st = (cudaStream_t)stream;
    if (algo == 4) return hsa_span_attn_fwd_tc128(Q, K, V, Out, LSE, B, N, H, D, radius, causal, dtype, st);
    if (algo == 3) return hsa_span_attn_fwd_tc(Q, K, V, Out, LSE, B, N, H, D, radius, causal, dtype, st);
    if (algo != 1 && hsa_span_attn_fwd_tc128_supported(Q, K, V, Out, B, N, H, D, radius, causal, dtype))
        return hsa_span_attn_fwd_tc128(Q, K, V, Out, LSE, B, N, H, D, radius, causal, dtype, st);
    if (algo == 2 || (algo == 0 && hsa_span_attn_fwd_tc_supported(Q, K, V, Out, B, N, H, D, radius, causal, dtype)))
        return hsa_span_attn_fwd_tc(Q, K, V, Out, LSE, B, N, H, D, radius, causal, dtype, (cudaStream_t)stream);
    // float32: the tile-staged kernel where it applies (head dim 64 / 128), the portable gather otherwise
    if (algo == 0 && hsa_span_attn_fwd_f32_supported(Q, K, V, Out, B, N, H, D, radius, causal, dtype))
        return hsa_span_attn_fwd_f32(Q, K, V, Out, LSE, B, N, H, D, radius, causal, dtype, st);
    return hsa_span_attn_fwd_generic(Q, K, V, Out, LSE, B, N, H, D, radius, causal, dtype, (cudaStream_t)stream);
}

extern "C" size_t hsa_span_attn_bwd_workspace_bytes(int B, int N, int H, int D, int radius, int causal,
                                                    int dtype, int algo) {
    (void)radius; (void)causal;
    if (B < 1 || N < 1 || H < 1 || D < 1) return 0;
    // algo 0 may pick either kernel from the pointers it is given: size for the larger need
    const size_t portable = hsa_span_attn_bwd_generic_workspace(B, N, H);
    const bool tc_dtype = (dtype == HSA_BF16 || dtype == HSA_F16) && (D == 64 || D == 128) && N >= 64;
    const size_t tc = tc_dtype ? hsa_span_attn_bwd_tc_workspace(B, N, H, D) : 0;
    if (algo == 1) return portable;
    if (algo >= 2) return tc;
    return portable > tc ? portable : tc;
}

extern "C" int hsa_span_attn_bwd(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE,
                                 hsa_view dOut, hsa_view dQ, hsa_view dK, hsa_view dV, void *workspace,
                                 size_t workspace_bytes, int B, int N, int H, int D, int radius, int causal,
                                 int dtype, int algo, void *stream) {
    HSA_CHECK_ARG(Q.ptr && K.ptr && V.ptr && Out.ptr && LSE && dOut.ptr && dQ.ptr && dK.ptr && dV.ptr,
                  "hsa_span_attn_bwd: null pointer");
    HSA_CHECK_ARG(algo >= 0 && algo <= 4, "hsa_span_attn_bwd: unknown algo %d", algo);
    const size_t need = hsa_span_attn_bwd_workspace_bytes(B, N, H, D, radius, causal, dtype, algo);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need))
        return fail(HSA_ERR_WORKSPACE, "hsa_span_attn_bwd: workspace of %zu bytes needed, %zu given", need,
                    workspace_bytes);
    if (need > 0 && (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
        return fail(HSA_ERR_ALIGN, "hsa_span_attn_bwd: workspace must be 256-byte aligned");
    const hsa_view views[] = {Q, K, V, Out, dOut, dQ, dK, dV};
    // The 8-warp task-parallel kernel (causal, window radius <= 16) is preferred where it applies; 3 forces the
    // 4-warp kernel, which also takes the non-causal case and wider windows.
    if ((algo == 0 || algo == 4) && hsa_span_attn_bwd_tc8_supported(views, 8, B, N, H, D, radius, causal, dtype))
        return hsa_span_attn_bwd_tc8(Q, K, V, Out, LSE, dOut, dQ, dK, dV, workspace, B, N, H, D, radius, causal, dtype,
                                     (cudaStream_t)stream);
    if (algo >= 2 || (algo == 0 && hsa_span_attn_bwd_tc_supported(views, 8, B, N, H, D, radius, causal, dtype)))
        return hsa_span_attn_bwd_tc(Q, K, V, Out, LSE, dOut, dQ, dK, dV, workspace, B, N, H, D, radius, causal, dtype,
                                    (cudaStream_t)stream);
    return hsa_span_attn_bwd_generic(Q, K, V, Out, LSE, dOut, dQ, dK, dV, workspace, B, N, H, D, radius, causal,
                                     dtype, (cudaStream_t)stream);
}
