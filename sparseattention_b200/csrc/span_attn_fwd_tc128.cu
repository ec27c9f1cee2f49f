// Span attention forward, tensor cores, 128-leaf tiles: the variant for the common causal case
// (radius <= 16, bf16 / f16, head dim 64 or 128, N >= 128).
//
// Same algorithm as span_attn_fwd_tc.cu, but a CTA covers 128 leaves with 8 warps and keeps its K/V rows
// at an unpadded pitch of 2*D bytes with the 16-byte pieces XOR-swizzled by the row (so ldmatrix stays
// conflict free without the padding).  What that buys: 108.5 KB of staging per CTA, two CTAs = 217 KB of
// the SM's shared memory acting as load buffers (the forward is bound by bytes in flight), 16 warps per SM
// instead of 12, and half the halo rows per leaf.  To stay under 128 registers per thread (two CTAs of 256
// threads) the kernel scores all of a warp's key blocks first (at most two band blocks plus one tree block,
// or two tree blocks once N > 8192), runs one softmax without rescaling, and normalises the probabilities
// before P.V so the accumulators are final: the Q fragments are dead before the output accumulators live.
#include "tc_common.cuh"

namespace hsa {

struct SpanTc128Args {
    const void *q, *k, *v;
    void *out;
    float *lse;
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs;
    int N, L, H, R;
    int RB;          // ceil(R / 16): 0 or 1
    int band_rows;   // 128 + 16 * RB
    int kv_rows;     // band + 63 in-tile tree rows + (L - 7) upper rows
    float scale_log2e;
};

constexpr int kT128 = 128, kT128Log = 7, kT128In = 63;     // causal: even nodes of levels 1..6

// 16-byte piece c of shared-memory row `row` sits at piece swz(row, c)
__device__ __forceinline__ int swz(int row, int c) { return (c & ~7) | ((c ^ row) & 7); }

// Tree key slot s of warp w (causal, 128-leaf tile) -> level and row inside the tile's tree storage.
// Levels 1..3: the even nodes below the warp's 16 leaves (slots 0..6); then one node per level 4.. : the
// sibling of the warp's ancestor (in-tile up to level 6, then the tile's own upper nodes).
__device__ __forceinline__ int tree_slot128(int s, int w, int L, int &row, int &jj) {
    jj = 0;
    if (s < 4) { jj = 2 * s; row = 4 * w + s; return 1; }                       // level 1: offset 0
    if (s < 6) { jj = 2 * (s - 4); row = 32 + 2 * w + (s - 4); return 2; }      // level 2: offset 64 - 32
    if (s == 6) { row = 48 + w; return 3; }                                      // level 3: offset 64 - 16
    const int l = s - 3;
    if (l >= L) { row = 0; return -1; }
    if (l < kT128Log) {                                                          // levels 4, 5, 6
        const int aw = w >> (l - 4);                                             // the warp's ancestor inside the tile
        row = (kT128 / 2 - (kT128 >> l)) + (aw >> 1);                            // its left sibling, stored when aw is odd
        return l;
    }
    row = kT128In + (l - kT128Log);
    return l;
}

template <typename T, int D, int NB>      // NB: key blocks per warp the code is unrolled for (3 or 4)
__global__ void __launch_bounds__(256, 2)
span_fwd_tc128_kernel(SpanTc128Args a) {
    constexpr int PITCH = D * 2;
    constexpr int CPR = D / 8;
    constexpr int RPI = 256 / CPR;
    constexpr int KS = D / 16;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *Ks = smem;
    unsigned char *Vs = Ks + (size_t)a.kv_rows * PITCH;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ntiles = a.N / kT128;
    const int h = blockIdx.x % a.H;
    const int tile = (blockIdx.x / a.H) % ntiles;
    const int b = blockIdx.x / (a.H * ntiles);
    const int t0 = tile * kT128;
    const int N = a.N, L = a.L, R = a.R, RB = a.RB;
    const int64_t hoff = (int64_t)h * D;
    const int lw = 16 * warp;
    const int quad = lane & 3, qrow = lane >> 2;
    const int n0 = t0 + lw + qrow, n1 = n0 + 8;

    // ---------------------------------------------------------------- stage K (group 0) and V (group 1)
    {
        const int c = tid % CPR, rg = tid / CPR;        // RPI is a multiple of 8: (row & 7) == (rg & 7) on every pass
        const int pc = swz(rg, c);
        const int ntree = kT128In + (L - kT128Log);
        auto stage_kv = [&](const void *base, int64_t bs, int64_t rs, unsigned char *S) {
            const T *gc = (const T *)base + b * bs + hoff + c * 8;
            uint32_t dst = smem_u32(S) + rg * PITCH + pc * 16;
            int r = t0 - 16 * RB + rg;
            for (int i = rg; i < a.band_rows; i += RPI, r += RPI, dst += RPI * PITCH) {
                const bool ok = r >= 0;                  // the band never runs past the last leaf
                cp_async16(dst, gc + (int64_t)(ok ? r : 0) * rs, ok);
            }
            dst = smem_u32(S) + (a.band_rows + rg) * PITCH + pc * 16;      // band_rows is a multiple of 16
            for (int f = rg; f < ntree; f += RPI, dst += RPI * PITCH) {
                int rr;
                bool ok = true;
                if (f < kT128In) {
                    const int rem = kT128 / 2 - f;
                    const int l = (kT128Log - 1) - (31 - __clz(rem - 1));
                    const int i = f - (kT128 / 2 - (kT128 >> l));
                    rr = level_base(N, l) + (t0 >> l) + 2 * i;
                } else {
                    const int l = kT128Log + (f - kT128In);
                    ok = (t0 >> l) & 1;
                    rr = level_base(N, l) + ((t0 >> l) ^ 1);
                }
                cp_async16(dst, gc + (int64_t)rr * rs, ok);
            }
        };
        stage_kv(a.k, a.k_bs, a.k_rs, Ks);
        cp_async_commit();
        stage_kv(a.v, a.v_bs, a.v_rs, Vs);
        cp_async_commit();
    }

    // ---------------------------------------------------------------- Q: global -> A-operand registers
    // (after the K/V copies: their latency runs while these 4-byte loads go through the load/store pipe)
    uint32_t qf[KS][4];
    {
        const T *q0 = (const T *)a.q + b * a.q_bs + hoff + (int64_t)n0 * a.q_rs + 2 * quad;
        const T *q1 = q0 + 8 * a.q_rs;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = ldg32(q0 + ks * 16);
            qf[ks][1] = ldg32(q1 + ks * 16);
            qf[ks][2] = ldg32(q0 + ks * 16 + 8);
            qf[ks][3] = ldg32(q1 + ks * 16 + 8);
        }
    }

    const int nbb = RB + 1;                 // band blocks: [the warp's own 16 leaves] (+ the 16 before them)
    const int ntb = (L + 3 + 15) >> 4;      // tree blocks: 7 slots of levels 1..3 + one slot per level 4..L-1
    const int nblk = nbb + ntb;             // <= NB (checked by the launcher)

    // ---------------------------------------------------------------- masks (closed-form topology)
    uint32_t tree_bits = 0;                 // bit tb*8 + nt*4 + e: this thread's score element of tree block tb is attended
    for (int tb = 0; tb < ntb; ++tb) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int slot = 16 * tb + nt * 8 + 2 * quad + (e & 1);
                const int i = qrow + 8 * (e >> 1);
                int row, jj;
                const int l = tree_slot128(slot, warp, L, row, jj);
                bool ok = false;
                if (l >= 1 && l <= 3) ok = (i >> l) == jj + 1;
                else if (l >= 4) ok = ((t0 + lw) >> l) & 1;
                tree_bits |= (ok ? 1u : 0u) << (tb * 8 + nt * 4 + e);
            }
    }
    const int dbase = 2 * quad - qrow;
    const bool odd = qrow & 1;              // odd leaves see their level-0 sibling (the leaf before them)

    // shared-memory row of key kk (0..15) of block o: 0 = own leaves, 1 = the 16 leaves before (when RB = 1), then tree blocks
    auto key_row = [&](int o, int kk) -> int {
        if (o < nbb) return lw + 16 * (o == 0 ? RB : 0) + kk;
        int row, jj;
        tree_slot128(16 * (o - nbb) + kk, warp, L, row, jj);
        return a.band_rows + row;
    };

    cp_async_wait<1>();
    __syncthreads();

    // ---------------------------------------------------------------- scores: NB blocks x 2 n-tiles advance together
    const float c2 = a.scale_log2e;
    float s[NB][2][4];
    {
        uint32_t kb[NB];
        int ksw[NB];
#pragma unroll
        for (int bi = 0; bi < NB; ++bi) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[bi][0][e] = s[bi][1][e] = 0.f;
            const int krow = key_row(min(bi, nblk - 1), (lane & 7) + 8 * (lane >> 4));
            kb[bi] = smem_u32(Ks + (size_t)krow * PITCH);
            ksw[bi] = (((lane >> 3) & 1) ^ krow) & 7;        // piece parity of this lane folded into the row's swizzle
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int bi = 0; bi < NB; ++bi) {
                uint32_t kf[4];
                ldmatrix_x4(kf, kb[bi] + ((((2 * ks) & 7) ^ ksw[bi]) | ((2 * ks) & 8)) * 16);
                mma16816<T>(s[bi][0], qf[ks], kf[0], kf[1]);
                mma16816<T>(s[bi][1], qf[ks], kf[2], kf[3]);
            }
        }
    }
    // ---- masks and base-2 logits
#pragma unroll
    for (int bi = 0; bi < NB; ++bi) {
        if (bi < nbb) {
            const int blk = (bi == 0) ? RB : 0;                   // band block index, 0 = leftmost
            const int r0 = t0 + lw + 16 * (blk - RB);
            const bool self = bi == 0;
            const int d0 = dbase + 16 * (blk - RB);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int dlt = d0 + nt * 8 + (e & 1) - 8 * (e >> 1);           // key - leaf
                    const bool wv = dlt >= -R && dlt <= 0 && (r0 + nt * 8 + 2 * quad + (e & 1)) >= 0;
                    const bool lv = self && odd && dlt == -1;
                    const float bias = (wv && lv) ? 1.f : ((wv || lv) ? 0.f : -INFINITY);
                    s[bi][nt][e] = fmaf(s[bi][nt][e], c2, bias);
                }
        } else if (bi < nblk) {
            const uint32_t bits = tree_bits >> (8 * (bi - nbb));
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    s[bi][nt][e] = ((bits >> (nt * 4 + e)) & 1u) ? s[bi][nt][e] * c2 : -INFINITY;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[bi][0][e] = s[bi][1][e] = -INFINITY;
        }
    }
    // ---- softmax over the whole (single) chunk
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int bi = 0; bi < NB; ++bi)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            m0 = fmaxf(m0, fmaxf(s[bi][nt][0], s[bi][nt][1]));
            m1 = fmaxf(m1, fmaxf(s[bi][nt][2], s[bi][nt][3]));
        }
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int bi = 0; bi < NB; ++bi)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            s[bi][nt][0] = fast_exp2(s[bi][nt][0] - m0);
            s[bi][nt][1] = fast_exp2(s[bi][nt][1] - m0);
            s[bi][nt][2] = fast_exp2(s[bi][nt][2] - m1);
            s[bi][nt][3] = fast_exp2(s[bi][nt][3] - m1);
            l0 += s[bi][nt][0] + s[bi][nt][1];
            l1 += s[bi][nt][2] + s[bi][nt][3];
        }
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
    uint32_t pa[NB][4];                      // normalised probabilities as A operands
#pragma unroll
    for (int bi = 0; bi < NB; ++bi) {
        pa[bi][0] = pack2<T>(s[bi][0][0] * i0, s[bi][0][1] * i0);
        pa[bi][1] = pack2<T>(s[bi][0][2] * i1, s[bi][0][3] * i1);
        pa[bi][2] = pack2<T>(s[bi][1][0] * i0, s[bi][1][1] * i0);
        pa[bi][3] = pack2<T>(s[bi][1][2] * i1, s[bi][1][3] * i1);
    }

    cp_async_wait<0>();
    __syncthreads();                         // V has landed

    // ---------------------------------------------------------------- O = P V
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
    for (int bi = 0; bi < NB; ++bi) {
        if (bi < nblk) {
            const int vrow = key_row(bi, (lane & 7) + 8 * ((lane >> 3) & 1));
            const uint32_t vb = smem_u32(Vs + (size_t)vrow * PITCH);
            const int vsw = ((lane >> 4) ^ vrow) & 7;
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vb + ((((2 * dp) & 7) ^ vsw) | ((2 * dp) & 8)) * 16);
                mma16816<T>(o[2 * dp], pa[bi], vf[0], vf[1]);
                mma16816<T>(o[2 * dp + 1], pa[bi], vf[2], vf[3]);
            }
        }
    }

    // ---------------------------------------------------------------- epilogue: park the rows in K's first rows, store 16 B per lane
    __syncthreads();
    unsigned char *Os = Ks + (size_t)lw * PITCH;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        *reinterpret_cast<uint32_t *>(Os + qrow * PITCH + swz(qrow, nt) * 16 + 4 * quad) = pack2<T>(o[nt][0], o[nt][1]);
        *reinterpret_cast<uint32_t *>(Os + (qrow + 8) * PITCH + swz(qrow, nt) * 16 + 4 * quad) = pack2<T>(o[nt][2], o[nt][3]);
    }
    __syncwarp();
    T *og = (T *)a.out + b * a.o_bs + hoff;
#pragma unroll
    for (int it = 0; it < (16 * CPR) / 32; ++it) {
        const int idx = it * 32 + lane;
        const int r = idx / CPR, c = idx % CPR;
        const uint4 val = *reinterpret_cast<const uint4 *>(Os + r * PITCH + swz(r, c) * 16);
        *reinterpret_cast<uint4 *>(og + (int64_t)(t0 + lw + r) * a.o_rs + c * 8) = val;
    }
}

}  // namespace hsa

using namespace hsa;

// Shapes the 128-leaf-tile forward takes (a subset of what span_attn_fwd_tc.cu takes).
bool hsa_span_attn_fwd_tc128_supported(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, int B, int N, int H, int D,
                                       int radius, int causal, int dtype) {
    if (!causal) return false;
    if (dtype != HSA_BF16 && dtype != HSA_F16) return false;
    if (D != 64 && D != 128) return false;
    if (N < kT128 || (N & (N - 1)) != 0) return false;
    const int L = ilog2((unsigned)N);
    if (L + 3 > 32) return false;                        // the warp's tree keys must fit two 16-key blocks
    if (radius < 0 || radius > 16) return false;
    if (((radius + 15) / 16 + 1) + ((L + 3 + 15) / 16) > 4) return false;
    if (B < 1 || H < 1) return false;
    if ((int64_t)(N / kT128) * H * B > 0x7fffffffLL) return false;
    if (!view_vec_ok(Q, 2) || !view_vec_ok(K, 2) || !view_vec_ok(V, 2) || !view_vec_ok(Out, 2)) return false;
    return true;
}

template <typename T, int D>
static int launch_tc128(const SpanTc128Args &a, int B, cudaStream_t st) {
    const size_t smem = (size_t)2 * a.kv_rows * (D * 2);
    const int64_t total = (int64_t)B * (a.N / kT128) * a.H;
    const int nblk = (a.RB + 1) + ((a.L + 3 + 15) >> 4);
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "hsa_span_attn_fwd(tc128): shared memory %zu: %s", smem, cudaGetErrorString(e));
        kernel<<<(unsigned)total, 256, smem, st>>>(a);
        return launch_status("hsa_span_attn_fwd(tc128)");
    };
    return nblk <= 3 ? go(span_fwd_tc128_kernel<T, D, 3>) : go(span_fwd_tc128_kernel<T, D, 4>);
}

int hsa_span_attn_fwd_tc128(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, float *LSE, int B, int N, int H, int D,
                            int radius, int causal, int dtype, cudaStream_t st) {
    if (!hsa_span_attn_fwd_tc128_supported(Q, K, V, Out, B, N, H, D, radius, causal, dtype))
        return fail(HSA_ERR_ARG, "hsa_span_attn_fwd: shape not taken by the 128-leaf-tile kernel");
    SpanTc128Args a{};
    a.q = Q.ptr; a.k = K.ptr; a.v = V.ptr; a.out = Out.ptr; a.lse = LSE;
    a.q_bs = Q.batch_stride; a.q_rs = Q.row_stride; a.k_bs = K.batch_stride; a.k_rs = K.row_stride;
    a.v_bs = V.batch_stride; a.v_rs = V.row_stride; a.o_bs = Out.batch_stride; a.o_rs = Out.row_stride;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.R = radius;
    a.RB = (radius + 15) / 16;
    a.band_rows = kT128 + 16 * a.RB;
    a.kv_rows = a.band_rows + kT128In + (a.L - kT128Log);
    a.scale_log2e = 1.4426950408889634f / sqrtf((float)D);
    if (dtype == HSA_BF16) return D == 128 ? launch_tc128<__nv_bfloat16, 128>(a, B, st) : launch_tc128<__nv_bfloat16, 64>(a, B, st);
    return D == 128 ? launch_tc128<__half, 128>(a, B, st) : launch_tc128<__half, 64>(a, B, st);
}
