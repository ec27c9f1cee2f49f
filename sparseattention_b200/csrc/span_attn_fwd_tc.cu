// Span attention forward on tensor cores (bf16 / f16, head dim 64 or 128, N >= 64).
//
// One CTA = one (batch, head, aligned tile of 64 leaves), 4 warps of 16 leaves each.
// The tile's whole key/value working set is staged in shared memory ONCE with 16-byte cp.async:
//   * the leaf band   [t0 - 16*RB, t0 + 64)            (RB = ceil(R/16); both sides when not causal)
//   * the tree nodes inside the tile's subtree, levels 1..5 (only left children when causal:
//     right children are never attended causally, so they are not even read from HBM)
//   * one node per level >= 6: the sibling of the tile's ancestor (shared by all 64 leaves)
// i.e. about 1.8 rows per leaf instead of the 2R+1+L gathered rows per leaf of a per-query kernel.
// Each warp then scores its 16 leaves against 16-key blocks with mma.sync.m16n8k16 — the band blocks
// it can see plus one or two blocks that pack its tree keys (ldmatrix takes one address per key row,
// so a block may gather arbitrary rows) — masks with the closed-form topology, runs the softmax in
// registers (quad shuffles), and multiplies by V through ldmatrix.trans.  The level-0 sibling n^1 lies
// inside the window; where both slots are valid its probability counts twice (reference semantics),
// done by adding 1 to its base-2 logit.
#include "tc_common.cuh"

namespace hsa {

struct SpanTcArgs {
    const void *q, *k, *v;
    void *out;
    float *lse;
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs;
    int N, L, H, R;
    int RB;          // ceil(R / 16)
    int band_rows;   // leaf rows staged per tile
    int kv_rows;     // all rows staged per tile
    float scale_log2e;
};

template <typename T, int D, bool CAUSAL>
__global__ void __launch_bounds__(128, 3)
span_fwd_tc_kernel(SpanTcArgs a) {
    constexpr int PITCH = D * 2 + 16;          // bytes; the 16-byte skew keeps ldmatrix conflict-free
    constexpr int CPR = D / 8;                 // 16-byte chunks per row
    constexpr int RPI = 128 / CPR;             // rows staged per pass of the CTA
    constexpr int KS = D / 16;                 // k-steps of the QK^T product
    constexpr int TIN = tree_in_rows<CAUSAL>();
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *Ks = smem;
    unsigned char *Vs = Ks + (size_t)a.kv_rows * PITCH;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // work item id -> (batch, tile, head); heads vary fastest so that CTAs running together touch
    // neighbouring 2*D-byte pieces of the same rows
    const int ntiles = a.N / kTile;
    const int h = blockIdx.x % a.H;
    const int tile = (blockIdx.x / a.H) % ntiles;
    const int b = blockIdx.x / (a.H * ntiles);
    const int t0 = tile * kTile;
    const int N = a.N, L = a.L, R = a.R, RB = a.RB;
    const int band_lo = t0 - 16 * RB;
    const int64_t hoff = (int64_t)h * D;
    const T *qg = (const T *)a.q + b * a.q_bs + hoff;
    const T *kg = (const T *)a.k + b * a.k_bs + hoff;
    const T *vg = (const T *)a.v + b * a.v_bs + hoff;

    const int lw = 16 * warp;
    const int quad = lane & 3, qrow = lane >> 2;
    const int n0 = t0 + lw + qrow, n1 = n0 + 8;       // the two leaves this thread holds scores for

    // ---------------------------------------------------------------- Q: global -> A-operand registers
    uint32_t qf[KS][4];
    {
        const T *q0 = qg + (int64_t)n0 * a.q_rs + 2 * quad;
        const T *q1 = qg + (int64_t)n1 * a.q_rs + 2 * quad;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = ldg32(q0 + ks * 16);
            qf[ks][1] = ldg32(q1 + ks * 16);
            qf[ks][2] = ldg32(q0 + ks * 16 + 8);
            qf[ks][3] = ldg32(q1 + ks * 16 + 8);
        }
    }

    // ---------------------------------------------------------------- stage K (group 0) and V (group 1)
    {
        const int c = tid % CPR, rg = tid / CPR;
        const int ntree = TIN + (L - kTileLog);
        auto stage_kv = [&](const T *g, int64_t rs, unsigned char *S) {
            const T *gc = g + c * 8;
            uint32_t dst = smem_u32(S) + rg * PITCH + c * 16;
            int r = band_lo + rg;
            for (int i = rg; i < a.band_rows; i += RPI, r += RPI, dst += RPI * PITCH) {
                const bool ok = (unsigned)r < (unsigned)N;
                cp_async16(dst, gc + (int64_t)(ok ? r : 0) * rs, ok);
            }
            dst = smem_u32(S) + (a.band_rows + rg) * PITCH + c * 16;
            for (int f = rg; f < ntree; f += RPI, dst += RPI * PITCH) {
                int rr;
                bool ok = true;
                if (f < TIN) {
                    const int rem = (CAUSAL ? 32 : 64) - f;
                    const int l = (CAUSAL ? 5 : 6) - (31 - __clz(rem - 1));
                    const int i = f - tree_level_off<CAUSAL>(l);
                    rr = level_base(N, l) + (t0 >> l) + (CAUSAL ? 2 * i : i);
                } else {
                    const int l = kTileLog + (f - TIN);
                    ok = !CAUSAL || ((t0 >> l) & 1);
                    rr = level_base(N, l) + ((t0 >> l) ^ 1);
                }
                cp_async16(dst, gc + (int64_t)rr * rs, ok);
            }
        };
        stage_kv(kg, a.k_rs, Ks);
        cp_async_commit();
        stage_kv(vg, a.v_rs, Vs);
        cp_async_commit();
    }

    const int nbb = CAUSAL ? RB + 1 : 2 * RB + 1;
    const int ntb = (tree_slots<CAUSAL>(L) + 15) >> 4;
    const int nblk = nbb + ntb;

    // ---------------------------------------------------------------- masks (closed-form topology)
    // Tree blocks: one validity bit per score element this thread will hold, bit = tb*8 + nt*4 + e.
    uint32_t tree_bits = 0;
    for (int tb = 0; tb < ntb; ++tb) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int slot = 16 * tb + nt * 8 + 2 * quad + (e & 1);
                const int i = qrow + 8 * (e >> 1);
                int row, jj;
                const int l = tree_slot<CAUSAL>(slot, warp, L, row, jj);
                bool ok = false;
                if (l >= 1 && l <= 3) ok = CAUSAL ? ((i >> l) == jj + 1) : (((i >> l) ^ 1) == jj);
                else if (l >= 4) ok = !CAUSAL || (((t0 + lw) >> l) & 1);
                tree_bits |= (ok ? 1u : 0u) << ((tb & 3) * 8 + nt * 4 + e);
            }
    }
    // Band blocks: key - leaf distance of element (nt, e) in band block bi is dbase + 16*(bi-RB) + nt*8 + (e&1) - 8*(e>>1)
    const int dbase = 2 * quad - qrow;
    const int sib_dlt = (qrow & 1) ? -1 : 1;                     // where the level-0 sibling sits
    const bool sib_ok = !CAUSAL || (qrow & 1);

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    // shared-memory row of key `kk` (0..15) of ordered block o, relative to Ks / Vs
    auto key_row = [&](int o_idx, int kk) -> int {
        const BlockRef br = block_ref<CAUSAL>(o_idx, RB, nbb);
        if (br.band) return lw + 16 * br.idx + kk;
        int row, jj;
        tree_slot<CAUSAL>(16 * br.idx + kk, warp, L, row, jj);
        return a.band_rows + row;
    };

    cp_async_wait<1>();
    __syncthreads();

    const float c2 = a.scale_log2e;
    for (int c0 = 0; c0 < nblk; c0 += kChunk) {
        float s[kChunk][2][4];
        // ---- scores
#pragma unroll
        for (int bi = 0; bi < kChunk; ++bi) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[bi][0][e] = s[bi][1][e] = 0.f;
            if (c0 + bi < nblk) {
                const int krow = key_row(c0 + bi, (lane & 7) + 8 * (lane >> 4));
                const uint32_t kb = smem_u32(Ks + (size_t)krow * PITCH + ((lane >> 3) & 1) * 16);
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, kb + ks * 32);
                    mma16816<T>(s[bi][0], qf[ks], kf[0], kf[1]);
                    mma16816<T>(s[bi][1], qf[ks], kf[2], kf[3]);
                }
                const BlockRef br = block_ref<CAUSAL>(c0 + bi, RB, nbb);
                if (br.band) {
                    const int r0 = t0 + lw + 16 * (br.idx - RB);          // first key row of the block
                    const bool edge = r0 < 0 || r0 + 16 > N;
                    const bool self = br.idx == RB;
                    const int d0 = dbase + 16 * (br.idx - RB);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int dlt = d0 + nt * 8 + (e & 1) - 8 * (e >> 1);
                            bool wv = dlt >= -R && dlt <= (CAUSAL ? 0 : R);
                            if (edge) wv = wv && (unsigned)(r0 + nt * 8 + 2 * quad + (e & 1)) < (unsigned)N;
                            const bool lv = self && sib_ok && dlt == sib_dlt;
                            const float bias = (wv && lv) ? 1.f : ((wv || lv) ? 0.f : -INFINITY);
                            s[bi][nt][e] = fmaf(s[bi][nt][e], c2, bias);
                        }
                } else {
                    const uint32_t bits = tree_bits >> ((br.idx & 3) * 8);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            s[bi][nt][e] = ((bits >> (nt * 4 + e)) & 1u) ? s[bi][nt][e] * c2 : -INFINITY;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[bi][0][e] = s[bi][1][e] = -INFINITY;
            }
        }
        // ---- running max
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int bi = 0; bi < kChunk; ++bi)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                mx0 = fmaxf(mx0, fmaxf(s[bi][nt][0], s[bi][nt][1]));
                mx1 = fmaxf(mx1, fmaxf(s[bi][nt][2], s[bi][nt][3]));
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);   // finite: chunk 0 holds the leaf itself
        if (c0 > 0) {
            const float r0 = fast_exp2(m0 - mn0), r1 = fast_exp2(m1 - mn1);
            l0 *= r0;
            l1 *= r1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1; }
        }
        m0 = mn0;
        m1 = mn1;
        if (c0 == 0) { cp_async_wait<0>(); __syncthreads(); }       // V has landed
        // ---- probabilities and P.V
#pragma unroll
        for (int bi = 0; bi < kChunk; ++bi) {
            if (c0 + bi < nblk) {
                uint32_t pa[4];
                float p[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    p[nt][0] = fast_exp2(s[bi][nt][0] - m0);
                    p[nt][1] = fast_exp2(s[bi][nt][1] - m0);
                    p[nt][2] = fast_exp2(s[bi][nt][2] - m1);
                    p[nt][3] = fast_exp2(s[bi][nt][3] - m1);
                    l0 += p[nt][0] + p[nt][1];
                    l1 += p[nt][2] + p[nt][3];
                }
                pa[0] = pack2<T>(p[0][0], p[0][1]);
                pa[1] = pack2<T>(p[0][2], p[0][3]);
                pa[2] = pack2<T>(p[1][0], p[1][1]);
                pa[3] = pack2<T>(p[1][2], p[1][3]);
                const int vrow = key_row(c0 + bi, (lane & 7) + 8 * ((lane >> 3) & 1));
                const uint32_t vb = smem_u32(Vs + (size_t)vrow * PITCH + (lane >> 4) * 16);
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vb + dp * 32);
                    mma16816<T>(o[2 * dp], pa, vf[0], vf[1]);
                    mma16816<T>(o[2 * dp + 1], pa, vf[2], vf[3]);
                }
            }
        }
    }

    // ---------------------------------------------------------------- epilogue
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.f / l0, i1 = 1.f / l1;
    if (a.lse != nullptr && quad == 0) {
        constexpr float kLn2 = 0.6931471805599453f;
        a.lse[((int64_t)b * N + n0) * a.H + h] = (m0 + log2f(l0)) * kLn2;
        a.lse[((int64_t)b * N + n1) * a.H + h] = (m1 + log2f(l1)) * kLn2;
    }
    // When every warp is done with K, each warp parks its 16 output rows in K's first rows and then
    // stores them 16 bytes per lane (full 32-byte sectors, whole rows per request).
    __syncthreads();
    unsigned char *Os = Ks + lw * PITCH;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int col = nt * 8 + 2 * quad;
        *reinterpret_cast<uint32_t *>(Os + qrow * PITCH + col * 2) = pack2<T>(o[nt][0] * i0, o[nt][1] * i0);
        *reinterpret_cast<uint32_t *>(Os + (qrow + 8) * PITCH + col * 2) = pack2<T>(o[nt][2] * i1, o[nt][3] * i1);
    }
    __syncwarp();
    T *og = (T *)a.out + b * a.o_bs + hoff;
#pragma unroll
    for (int it = 0; it < (16 * CPR) / 32; ++it) {
        const int idx = it * 32 + lane;
        const int r = idx / CPR, c = idx % CPR;
        const uint4 val = *reinterpret_cast<const uint4 *>(Os + r * PITCH + c * 16);
        *reinterpret_cast<uint4 *>(og + (int64_t)(t0 + lw + r) * a.o_rs + c * 8) = val;
    }
}

template <typename T, int D>
static int launch_tc(const SpanTcArgs &a, int B, bool causal, cudaStream_t st) {
    constexpr int PITCH = D * 2 + 16;
    const size_t smem = (size_t)(2 * a.kv_rows) * PITCH;
    const int64_t total = (int64_t)B * (a.N / kTile) * a.H;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "hsa_span_attn_fwd(tc): shared memory %zu: %s", smem, cudaGetErrorString(e));
        kernel<<<(unsigned)total, 128, smem, st>>>(a);
        return launch_status("hsa_span_attn_fwd(tc)");
    };
    return causal ? go(span_fwd_tc_kernel<T, D, true>) : go(span_fwd_tc_kernel<T, D, false>);
}

}  // namespace hsa

using namespace hsa;

// Shapes the tensor-core forward takes.
bool hsa_span_attn_fwd_tc_supported(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, int B, int N, int H, int D,
                                    int radius, int causal, int dtype) {
    if (dtype != HSA_BF16 && dtype != HSA_F16) return false;
    if (D != 64 && D != 128) return false;
    if (N < kTile || (N & (N - 1)) != 0 || N > (1 << 28)) return false;
    if (B < 1 || B > 65535 || H < 1 || radius < 0) return false;
    if ((int64_t)(N / kTile) * H * B > 0x7fffffffLL) return false;      // one CTA per work item, 1-D grid
    if (!view_vec_ok(Q, 2) || !view_vec_ok(K, 2) || !view_vec_ok(V, 2) || !view_vec_ok(Out, 2)) return false;
    const int R = radius < N ? radius : N;
    const int RB = (R + 15) / 16;
    const int L = ilog2((unsigned)N);
    const int band = kTile + 16 * RB * (causal ? 1 : 2);
    const int kv = band + (causal ? 31 : 62) + (L - kTileLog);
    const size_t smem = (size_t)(2 * kv) * (D * 2 + 16);
    return smem <= 200 * 1024;
}

int hsa_span_attn_fwd_tc(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H, int D,
                         int radius, int causal, int dtype, cudaStream_t st) {
    if (!hsa_span_attn_fwd_tc_supported(Q, K, V, Out, B, N, H, D, radius, causal, dtype))
        return fail(HSA_ERR_ARG,
                    "hsa_span_attn_fwd: the tensor-core kernel takes bf16/f16, head dim 64 or 128, N >= 64, "
                    "16-byte aligned views and a window that fits shared memory");
    SpanTcArgs a{};
    a.q = Q.ptr; a.k = K.ptr; a.v = V.ptr; a.out = Out.ptr; a.lse = LSE;
    a.q_bs = Q.batch_stride; a.q_rs = Q.row_stride; a.k_bs = K.batch_stride; a.k_rs = K.row_stride;
    a.v_bs = V.batch_stride; a.v_rs = V.row_stride; a.o_bs = Out.batch_stride; a.o_rs = Out.row_stride;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.R = radius < N ? radius : N;
    a.RB = (a.R + 15) / 16;
    a.band_rows = kTile + 16 * a.RB * (causal ? 1 : 2);
    a.kv_rows = a.band_rows + (causal ? 31 : 62) + (a.L - kTileLog);
    a.scale_log2e = 1.4426950408889634f / sqrtf((float)D);
    if (dtype == HSA_BF16)
        return D == 128 ? launch_tc<__nv_bfloat16, 128>(a, B, causal != 0, st) : launch_tc<__nv_bfloat16, 64>(a, B, causal != 0, st);
    return D == 128 ? launch_tc<__half, 128>(a, B, causal != 0, st) : launch_tc<__half, 64>(a, B, causal != 0, st);
}
