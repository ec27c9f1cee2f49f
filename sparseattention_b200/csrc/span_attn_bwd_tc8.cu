// Span attention backward on tensor cores, 8 warps per 64-leaf tile (bf16 / f16, head dim 64 or 128).
//
// Same decomposition as span_attn_bwd_tc.cu (key-side phase for the tile's leaf keys, query-side phase for
// dQ and the tree slots, deterministic combination of the partial slots), but every 16-row block of the
// tile is worked by a PAIR of warps so that twice as many warps hide each other's latencies at the same
// shared-memory footprint:
//   * the two score-type products of a block are split between the pair — warp "half 0" forms the
//     probabilities (S or S^T, exp with the saved log-sum-exp), warp "half 1" forms dP (or dP^T) — and
//     exchanged through 2 KB of shared memory under a 64-thread named barrier;
//   * both warps then build dS and each accumulates ITS half of the head dimension of dQ / dK / dV and of
//     the tree-slot gradients, so a thread carries 64 accumulators instead of 128 (<= 128 registers:
//     two CTAs of 256 threads per SM).
// Rows sit in shared memory at an unpadded pitch of 2*D bytes with XOR-swizzled 16-byte pieces.
#include "tc_common.cuh"

namespace hsa {

struct SpanBwd8Args {
    const void *q, *k, *v, *out, *go;
    const float *lse;
    void *dq, *dk, *dv;
    float *partial;                 // [B, H, N/64, L-6, 2, D] float32
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs, go_bs, go_rs, dq_bs, dq_rs, dk_bs, dk_rs, dv_bs, dv_rs;
    int N, L, H, R, RB;
    int band_rows, tree_rows, q_rows;
    int kt_off, vt_off, q_off, go_off, stat_off, x_off;      // byte offsets into shared memory (bands start at 0)
    float scale_log2e, scale;
};

__device__ __forceinline__ uint32_t movmatrix_trans8(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}
// 64-thread named barrier of one warp pair (ids 1..4; 0 is __syncthreads).  The id is an immediate so that
// the compiler does not have to reserve all sixteen barriers.
__device__ __forceinline__ void pair_barrier(int id) {
    switch (id) {
        case 1: asm volatile("bar.sync 1, 64;\n" ::: "memory"); break;
        case 2: asm volatile("bar.sync 2, 64;\n" ::: "memory"); break;
        case 3: asm volatile("bar.sync 3, 64;\n" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;\n" ::: "memory"); break;
    }
}

template <typename T>
__device__ __forceinline__ void store_pair8(T *p, float a, float b) {
    *reinterpret_cast<uint32_t *>(p) = pack2<T>(a, b);
}

// byte offset of 16-byte piece `piece` in a row whose (row & 7) ^ lane-piece-parity has been folded into x
__device__ __forceinline__ uint32_t piece_off(int piece_even, int x) {
    return (uint32_t)((((piece_even & 7) ^ x) | (piece_even & 8)) * 16);
}

template <typename T, int D, bool CAUSAL>
__global__ void __launch_bounds__(256, 2)
span_bwd_tc8_kernel(SpanBwd8Args a) {
    constexpr int PITCH = D * 2;
    constexpr int CPR = D / 8;
    constexpr int RPI = 256 / CPR;
    constexpr int KS = D / 16;
    constexpr int DH = D / 2;              // columns of the head dimension this warp accumulates
    constexpr int NTH = DH / 8;            // its 8-column n-tiles
    constexpr int TIN = tree_in_rows<CAUSAL>();
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *Kb = smem;
    unsigned char *Vb = Kb + (size_t)a.band_rows * PITCH;
    float *persist = reinterpret_cast<float *>(smem);          // aliases the bands once they are dead
    unsigned char *Kt = smem + a.kt_off;
    unsigned char *Vt = smem + a.vt_off;
    unsigned char *Qs = smem + a.q_off;
    unsigned char *Gs = smem + a.go_off;
    float *lse_s = reinterpret_cast<float *>(smem + a.stat_off);
    float *dl_s = lse_s + a.q_rows;
    float *xbuf = reinterpret_cast<float *>(smem + a.x_off);   // [4 pairs][2][32 lanes][8]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int blk = warp & 3, half = warp >> 2;                // 16-row block of the tile, and which half of the pair
    const int ntiles = a.N / kTile;
    const int h = blockIdx.x % a.H;
    const int tile = (blockIdx.x / a.H) % ntiles;
    const int b = blockIdx.x / (a.H * ntiles);
    const int t0 = tile * kTile;
    const int N = a.N, L = a.L, R = a.R, RB = a.RB;
    const int band_lo = t0 - 16 * RB;
    const int qoff = CAUSAL ? 0 : 16 * RB;
    const int q_lo = t0 - qoff;
    const int64_t hoff = (int64_t)h * D;
    const T *og = (const T *)a.out + b * a.o_bs + hoff;
    const int lw = 16 * blk;
    const int quad = lane & 3, qrow = lane >> 2;
    const int nup = L - kTileLog;
    const int pbase = half * (DH / 8);                         // first 16-byte piece of this warp's column half
    float *xs = xbuf + ((size_t)(blk * 2 + 0) * 32 + lane) * 8;     // half 0 writes probabilities here
    float *xd = xbuf + ((size_t)(blk * 2 + 1) * 32 + lane) * 8;     // half 1 writes dP here
    const int bar_id = 1 + blk;

    // ---------------------------------------------------------------- staging
    {
        const int c = tid % CPR, rg = tid / CPR;               // RPI is a multiple of 8: (row & 7) == (rg & 7) on every pass
        const int pc = ((c & ~7) | ((c ^ rg) & 7)) * 16;
        auto stage_rows = [&](const void *base, int64_t bs, int64_t rs, unsigned char *S, int first, int rows) {
            const T *gc = (const T *)base + b * bs + hoff + c * 8;
            uint32_t dst = smem_u32(S) + rg * PITCH + pc;
            int r = first + rg;
            for (int i = rg; i < rows; i += RPI, r += RPI, dst += RPI * PITCH) {
                const bool ok = (unsigned)r < (unsigned)N;
                cp_async16(dst, gc + (int64_t)(ok ? r : 0) * rs, ok);
            }
        };
        auto stage_tree = [&](const void *base, int64_t bs, int64_t rs, unsigned char *S) {
            const T *gc = (const T *)base + b * bs + hoff + c * 8;
            uint32_t dst = smem_u32(S) + rg * PITCH + pc;
            for (int f = rg; f < a.tree_rows; f += RPI, dst += RPI * PITCH) {
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
        stage_rows(a.go, a.go_bs, a.go_rs, Gs, q_lo, a.q_rows);
        cp_async_commit();
        stage_rows(a.q, a.q_bs, a.q_rs, Qs, q_lo, a.q_rows);
        stage_rows(a.k, a.k_bs, a.k_rs, Kb, band_lo, a.band_rows);
        stage_rows(a.v, a.v_bs, a.v_rs, Vb, band_lo, a.band_rows);
        stage_tree(a.k, a.k_bs, a.k_rs, Kt);
        stage_tree(a.v, a.v_bs, a.v_rs, Vt);
        cp_async_commit();

        // delta = rowsum(dOut * Out) and base-2 log-sum-exp per staged query row; all global loads of a batch
        // are issued before anything waits
        constexpr int PF = 6;
        for (int i0 = rg; i0 < a.q_rows; i0 += RPI * PF) {
            uint4 ov[PF];
            float lv[PF];
#pragma unroll
            for (int j = 0; j < PF; ++j) {
                const int i = i0 + j * RPI;
                const int n = q_lo + i;
                const bool ok = i < a.q_rows && (unsigned)n < (unsigned)N;
                ov[j] = ok ? __ldg(reinterpret_cast<const uint4 *>(og + (int64_t)n * a.o_rs + c * 8)) : make_uint4(0, 0, 0, 0);
                lv[j] = (ok && c == 0) ? __ldg(a.lse + ((int64_t)b * N + n) * a.H + h) * 1.4426950408889634f : INFINITY;
            }
            if (i0 == rg) { cp_async_wait<1>(); __syncthreads(); }
#pragma unroll
            for (int j = 0; j < PF; ++j) {
                const int i = i0 + j * RPI;
                float part = 0.f;
                if (i < a.q_rows) {
                    const uint4 gv = *reinterpret_cast<const uint4 *>(Gs + i * PITCH + pc);
                    const T *oe = reinterpret_cast<const T *>(&ov[j]);
                    const T *ge = reinterpret_cast<const T *>(&gv);
#pragma unroll
                    for (int e = 0; e < 8; ++e) part = fmaf(Traits<T>::to_f(oe[e]), Traits<T>::to_f(ge[e]), part);
                }
#pragma unroll
                for (int o = CPR / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                if (c == 0 && i < a.q_rows) {
                    dl_s[i] = part;
                    lse_s[i] = lv[j];
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();
    }

    const float c2 = a.scale_log2e, sc = a.scale;

    // A 16x16 product over the whole head dimension: A rows at (Abuf, arow) as m, B rows at (Bbuf, brow) as n.
    // arow / brow are this lane's ldmatrix rows (A: (lane&7)+8*((lane>>3)&1), pieces by lane>>4;
    // B: (lane&7)+8*(lane>>4), pieces by (lane>>3)&1).
    auto product = [&](const unsigned char *Abuf, int arow, const unsigned char *Bbuf, int brow, float (&r)[2][4]) {
#pragma unroll
        for (int e = 0; e < 4; ++e) r[0][e] = r[1][e] = 0.f;
        const uint32_t ab = smem_u32(Abuf + (size_t)arow * PITCH);
        const uint32_t bb = smem_u32(Bbuf + (size_t)brow * PITCH);
        const int ax = ((lane >> 4) ^ arow) & 7, bx = (((lane >> 3) & 1) ^ brow) & 7;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t af[4], bf[4];
            ldmatrix_x4(af, ab + piece_off(2 * ks, ax));
            ldmatrix_x4(bf, bb + piece_off(2 * ks, bx));
            mma16816<T>(r[0], af, bf[0], bf[1]);
            mma16816<T>(r[1], af, bf[2], bf[3]);
        }
    };
    // acc[NTH][4] += A (16x16, register fragments) x rows (Bbuf, trow) restricted to this warp's column half.
    // trow is this lane's transposed-load row: (lane&7)+8*((lane>>3)&1), pieces by lane>>4.
    auto accumulate_half = [&](float (&acc)[NTH][4], const uint32_t (&af)[4], const unsigned char *Bbuf, int trow) {
        const uint32_t tb = smem_u32(Bbuf + (size_t)trow * PITCH);
        const int tx = ((lane >> 4) ^ trow) & 7;
#pragma unroll
        for (int dp = 0; dp < DH / 16; ++dp) {
            uint32_t f[4];
            ldmatrix_x4_trans(f, tb + piece_off(pbase + 2 * dp, tx));
            mma16816<T>(acc[2 * dp], af, f[0], f[1]);
            mma16816<T>(acc[2 * dp + 1], af, f[2], f[3]);
        }
    };
    // Pair exchange: half 0 hands over its 8 probabilities, half 1 its 8 dP values; both end with both.
    auto put8 = [&](float *dst, const float (&v)[2][4]) {
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0][0], v[0][1], v[0][2], v[0][3]);
        *reinterpret_cast<float4 *>(dst + 4) = make_float4(v[1][0], v[1][1], v[1][2], v[1][3]);
    };
    auto get8 = [&](const float *src, float (&v)[2][4]) {
        const float4 u = *reinterpret_cast<const float4 *>(src), w = *reinterpret_cast<const float4 *>(src + 4);
        v[0][0] = u.x; v[0][1] = u.y; v[0][2] = u.z; v[0][3] = u.w;
        v[1][0] = w.x; v[1][1] = w.y; v[1][2] = w.z; v[1][3] = w.w;
    };
    auto exchange = [&](float (&p)[2][4], float (&dp)[2][4]) {
        if (half == 0) {
            put8(xs, p);
            pair_barrier(bar_id);
            get8(xd, dp);
        } else {
            put8(xd, dp);
            pair_barrier(bar_id);
            get8(xs, p);
        }
        pair_barrier(bar_id);                    // the buffers may be rewritten after this
    };

    // ================================================================ phase B: leaf keys of the tile (keys as rows)
    {
        float dk[NTH][4], dv[NTH][4];
#pragma unroll
        for (int i = 0; i < NTH; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) dk[i][e] = dv[i][e] = 0.f;
        const int krow = 16 * RB + lw + (lane & 7) + 8 * ((lane >> 3) & 1);       // own keys as A rows
        const int key0 = t0 + lw;
        for (int qb = (CAUSAL ? 0 : -RB); qb <= RB; ++qb) {
            const int qr0 = qoff + lw + 16 * qb;                                 // local row of the block's first query
            const int nq0 = key0 + 16 * qb;
            if (nq0 >= N || nq0 + 16 <= 0) continue;                            // same decision in both warps of the pair
            float p[2][4], dp[2][4];
            const int brow = qr0 + (lane & 7) + 8 * (lane >> 4);
            if (half == 0) {
                product(Kb, krow, Qs, brow, p);                                  // S^T = K Q^T
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int qc = nt * 8 + 2 * quad + (e & 1);
                        const int kr = qrow + 8 * (e >> 1);
                        const int dlt = kr - qc - 16 * qb;                       // key - query
                        const bool wv = dlt >= -R && dlt <= (CAUSAL ? 0 : R);
                        const bool lv = qb == 0 && ((e & 1) ? (dlt == -1) : (!CAUSAL && dlt == 1));
                        const float bias = (wv && lv) ? 1.f : ((wv || lv) ? 0.f : -INFINITY);
                        p[nt][e] = fast_exp2(fmaf(p[nt][e], c2, bias) - lse_s[qr0 + qc]);     // lse = +inf outside the sequence
                    }
            } else {
                product(Vb, krow, Gs, brow, dp);                                 // dP^T = V dOut^T
            }
            exchange(p, dp);
            float ds[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    ds[nt][e] = p[nt][e] * (dp[nt][e] - dl_s[qr0 + nt * 8 + 2 * quad + (e & 1)]) * sc;
            uint32_t pa[4], da[4];
            pa[0] = pack2<T>(p[0][0], p[0][1]); pa[1] = pack2<T>(p[0][2], p[0][3]);
            pa[2] = pack2<T>(p[1][0], p[1][1]); pa[3] = pack2<T>(p[1][2], p[1][3]);
            da[0] = pack2<T>(ds[0][0], ds[0][1]); da[1] = pack2<T>(ds[0][2], ds[0][3]);
            da[2] = pack2<T>(ds[1][0], ds[1][1]); da[3] = pack2<T>(ds[1][2], ds[1][3]);
            const int trow = qr0 + (lane & 7) + 8 * ((lane >> 3) & 1);
            accumulate_half(dv, pa, Gs, trow);                                   // dV += P^T dOut
            accumulate_half(dk, da, Qs, trow);                                   // dK += dS^T Q
        }
        T *dkg = (T *)a.dk + b * a.dk_bs + hoff + half * DH + 2 * quad;
        T *dvg = (T *)a.dv + b * a.dv_bs + hoff + half * DH + 2 * quad;
        const int64_t r0 = key0 + qrow, r1 = r0 + 8;
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt) {
            store_pair8<T>(dkg + r0 * a.dk_rs + nt * 8, dk[nt][0], dk[nt][1]);
            store_pair8<T>(dkg + r1 * a.dk_rs + nt * 8, dk[nt][2], dk[nt][3]);
            store_pair8<T>(dvg + r0 * a.dv_rs + nt * 8, dv[nt][0], dv[nt][1]);
            store_pair8<T>(dvg + r1 * a.dv_rs + nt * 8, dv[nt][2], dv[nt][3]);
        }
    }

    // ================================================================ phase A: own leaves as queries
    float dq[NTH][4];
#pragma unroll
    for (int i = 0; i < NTH; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
    const int qa0 = qoff + lw;
    const int arow = qa0 + (lane & 7) + 8 * ((lane >> 3) & 1);                   // own leaves as A rows (and as transposed B rows)
    const float lse0 = lse_s[qa0 + qrow], lse1 = lse_s[qa0 + qrow + 8];
    const float dl0 = dl_s[qa0 + qrow], dl1 = dl_s[qa0 + qrow + 8];
    const int dbase = 2 * quad - qrow;
    const int sib_dlt = (qrow & 1) ? -1 : 1;
    const bool sib_ok = !CAUSAL || (qrow & 1);
    const int nbb = CAUSAL ? RB + 1 : 2 * RB + 1;
    const int ntb = (tree_slots<CAUSAL>(L) + 15) >> 4;

    for (int bi = 0; bi < nbb; ++bi) {
        const int r0 = t0 + lw + 16 * (bi - RB);
        if (r0 >= N || r0 + 16 <= 0) continue;
        float p[2][4], dp[2][4];
        const int brow = lw + 16 * bi + (lane & 7) + 8 * (lane >> 4);
        if (half == 0) {
            product(Qs, arow, Kb, brow, p);                                      // S = Q K^T
            const bool edge = r0 < 0 || r0 + 16 > N;
            const bool self = bi == RB;
            const int d0 = dbase + 16 * (bi - RB);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int dlt = d0 + nt * 8 + (e & 1) - 8 * (e >> 1);
                    bool wv = dlt >= -R && dlt <= (CAUSAL ? 0 : R);
                    if (edge) wv = wv && (unsigned)(r0 + nt * 8 + 2 * quad + (e & 1)) < (unsigned)N;
                    const bool lv = self && sib_ok && dlt == sib_dlt;
                    const float bias = (wv && lv) ? 1.f : ((wv || lv) ? 0.f : -INFINITY);
                    p[nt][e] = fast_exp2(fmaf(p[nt][e], c2, bias) - ((e >> 1) ? lse1 : lse0));
                }
        } else {
            product(Gs, arow, Vb, brow, dp);                                     // dP = dOut V^T
        }
        exchange(p, dp);
        uint32_t da[4];
        {
            float ds[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) ds[nt][e] = p[nt][e] * (dp[nt][e] - ((e >> 1) ? dl1 : dl0)) * sc;
            da[0] = pack2<T>(ds[0][0], ds[0][1]); da[1] = pack2<T>(ds[0][2], ds[0][3]);
            da[2] = pack2<T>(ds[1][0], ds[1][1]); da[3] = pack2<T>(ds[1][2], ds[1][3]);
        }
        accumulate_half(dq, da, Kb, lw + 16 * bi + (lane & 7) + 8 * ((lane >> 3) & 1));      // dQ += dS K
    }

    __syncthreads();        // the leaf bands of K and V are dead from here on: `persist` may overwrite them

    const int fps = CAUSAL ? 8 : 15;                                             // first slot that is a partial sum
    const int nps = 1 + nup;
    for (int tb = 0; tb < ntb; ++tb) {
        int rowA, rowB, jj;
        tree_slot<CAUSAL>(16 * tb + (lane & 7) + 8 * (lane >> 4), blk, L, rowA, jj);
        tree_slot<CAUSAL>(16 * tb + (lane & 7) + 8 * ((lane >> 3) & 1), blk, L, rowB, jj);
        float p[2][4], dp[2][4];
        if (half == 0) {
            product(Qs, arow, Kt, rowA, p);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int slot = 16 * tb + nt * 8 + 2 * quad + (e & 1);
                    const int i = qrow + 8 * (e >> 1);
                    int row2, j2;
                    const int l = tree_slot<CAUSAL>(slot, blk, L, row2, j2);
                    bool ok = false;
                    if (l >= 1 && l <= 3) ok = CAUSAL ? ((i >> l) == j2 + 1) : (((i >> l) ^ 1) == j2);
                    else if (l >= 4) ok = !CAUSAL || (((t0 + lw) >> l) & 1);
                    p[nt][e] = ok ? fast_exp2(p[nt][e] * c2 - ((e >> 1) ? lse1 : lse0)) : 0.f;
                }
        } else {
            product(Gs, arow, Vt, rowA, dp);
        }
        exchange(p, dp);
        uint32_t da[4], pt[4], dt[4];
        {
            float ds[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) ds[nt][e] = p[nt][e] * (dp[nt][e] - ((e >> 1) ? dl1 : dl0)) * sc;
            da[0] = pack2<T>(ds[0][0], ds[0][1]); da[1] = pack2<T>(ds[0][2], ds[0][3]);
            da[2] = pack2<T>(ds[1][0], ds[1][1]); da[3] = pack2<T>(ds[1][2], ds[1][3]);
        }
        accumulate_half(dq, da, Kt, rowB);                                       // dQ += dS K_tree
        // slot gradients: transpose the 8x8 fragments so the 16 slots become rows and the warp's 16 leaves the k dimension
        pt[0] = movmatrix_trans8(pack2<T>(p[0][0], p[0][1]));
        pt[1] = movmatrix_trans8(pack2<T>(p[1][0], p[1][1]));
        pt[2] = movmatrix_trans8(pack2<T>(p[0][2], p[0][3]));
        pt[3] = movmatrix_trans8(pack2<T>(p[1][2], p[1][3]));
        dt[0] = movmatrix_trans8(da[0]);
        dt[1] = movmatrix_trans8(da[2]);
        dt[2] = movmatrix_trans8(da[1]);
        dt[3] = movmatrix_trans8(da[3]);
        T *fin_k[2] = {nullptr, nullptr}, *fin_v[2] = {nullptr, nullptr};
        float *par[2] = {nullptr, nullptr};
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int slot = 16 * tb + qrow + 8 * hh;
            int row2, j2;
            const int l = tree_slot<CAUSAL>(slot, blk, L, row2, j2);
            if (l >= 1 && l <= 4) {
                const int node = (l <= 3) ? (((t0 + lw) >> l) + j2) : (((t0 + lw) >> 4) ^ 1);
                const bool ok = l <= 3 || !CAUSAL || (((t0 + lw) >> 4) & 1);
                if (ok) {
                    const int64_t gr = level_base(N, l) + node;
                    fin_k[hh] = (T *)a.dk + b * a.dk_bs + gr * a.dk_rs + hoff + half * DH + 2 * quad;
                    fin_v[hh] = (T *)a.dv + b * a.dv_bs + gr * a.dv_rs + hoff + half * DH + 2 * quad;
                }
            } else if (l >= 5) {
                par[hh] = persist + ((size_t)(blk * nps + (slot - fps)) * 2) * D + half * DH + 2 * quad;
            }
        }
#pragma unroll
        for (int which = 0; which < 2; ++which) {            // 0: dK of the slots (dS^T Q), 1: dV of the slots (P^T dOut)
            float acc[NTH][4];
#pragma unroll
            for (int i = 0; i < NTH; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            if (which) accumulate_half(acc, pt, Gs, arow);
            else accumulate_half(acc, dt, Qs, arow);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                T *fin = which ? fin_v[hh] : fin_k[hh];
                float *pp = par[hh] ? par[hh] + which * D : nullptr;
                if (fin != nullptr) {
#pragma unroll
                    for (int nt = 0; nt < NTH; ++nt) store_pair8<T>(fin + nt * 8, acc[nt][2 * hh], acc[nt][2 * hh + 1]);
                } else if (pp != nullptr) {
#pragma unroll
                    for (int nt = 0; nt < NTH; ++nt)
                        *reinterpret_cast<float2 *>(pp + nt * 8) = make_float2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
                }
            }
        }
    }

    {
        T *dqg = (T *)a.dq + b * a.dq_bs + hoff + half * DH + 2 * quad;
        const int64_t r0 = t0 + lw + qrow, r1 = r0 + 8;
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt) {
            store_pair8<T>(dqg + r0 * a.dq_rs + nt * 8, dq[nt][0], dq[nt][1]);
            store_pair8<T>(dqg + r1 * a.dq_rs + nt * 8, dq[nt][2], dq[nt][3]);
        }
    }
    __syncthreads();

    // ---------------------------------------------------------------- combine the partial slots in block order
    for (int idx = tid; idx < 2 * 2 * D; idx += 256) {
        const int j = idx / (2 * D), rem = idx % (2 * D), which = rem / D, col = rem % D;
        if (CAUSAL && j == 1) continue;
        const int wa = 2 * (j ^ 1);
        const float sum = persist[((size_t)(wa * nps) * 2 + which) * D + col] +
                          persist[((size_t)((wa + 1) * nps) * 2 + which) * D + col];
        const int64_t gr = level_base(N, 5) + (t0 >> 5) + j;
        T *dst = which ? (T *)a.dv + b * a.dv_bs + gr * a.dv_rs + hoff : (T *)a.dk + b * a.dk_bs + gr * a.dk_rs + hoff;
        dst[col] = Traits<T>::from_f(sum);
    }
    for (int idx = tid; idx < nup * 2 * D; idx += 256) {
        const int u = idx / (2 * D), rem = idx % (2 * D);
        const int l = kTileLog + u;
        if (CAUSAL && ((t0 >> l) & 1) == 0) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) sum += persist[((size_t)(w * nps + 1 + u) * 2) * D + rem];
        a.partial[((((size_t)b * a.H + h) * ntiles + tile) * nup + u) * 2 * D + rem] = sum;
    }
    if (CAUSAL) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int idx = tid; idx < 31 * CPR * 2; idx += 256) {
            const int which = idx / (31 * CPR), rem = idx % (31 * CPR);
            const int f = rem / CPR, c = rem % CPR;
            const int remf = 32 - f;
            const int l = 5 - (31 - __clz(remf - 1));
            const int i = f - tree_level_off<true>(l);
            const int64_t gr = level_base(N, l) + (t0 >> l) + 2 * i + 1;
            T *dst = which ? (T *)a.dv + b * a.dv_bs + gr * a.dv_rs + hoff : (T *)a.dk + b * a.dk_bs + gr * a.dk_rs + hoff;
            *reinterpret_cast<uint4 *>(dst + c * 8) = z;
        }
    }
}

struct Bwd8Plan {
    int RB, band_rows, tree_rows, q_rows, nup;
    int kt_off, vt_off, q_off, go_off, stat_off, x_off;
    size_t smem;
};

static Bwd8Plan plan_bwd8(int N, int D, int radius, bool causal) {
    Bwd8Plan p{};
    const int PITCH = D * 2;
    const int R = radius < N ? radius : N;
    const int L = ilog2((unsigned)N);
    p.RB = (R + 15) / 16;
    p.nup = L - kTileLog;
    p.band_rows = kTile + 16 * p.RB * (causal ? 1 : 2);
    p.tree_rows = (causal ? 31 : 62) + p.nup;
    p.q_rows = kTile + 16 * p.RB * (causal ? 1 : 2);
    const size_t bands = (size_t)2 * p.band_rows * PITCH;
    const size_t persist = (size_t)4 * (1 + p.nup) * 2 * D * sizeof(float);
    size_t off = bands > persist ? bands : persist;
    off = (off + 127) / 128 * 128;
    p.kt_off = (int)off; off += (size_t)p.tree_rows * PITCH;
    p.vt_off = (int)off; off += (size_t)p.tree_rows * PITCH;
    off = (off + 127) / 128 * 128;
    p.q_off = (int)off; off += (size_t)p.q_rows * PITCH;
    p.go_off = (int)off; off += (size_t)p.q_rows * PITCH;
    p.stat_off = (int)off; off += (size_t)2 * p.q_rows * sizeof(float);
    off = (off + 15) / 16 * 16;
    p.x_off = (int)off; off += (size_t)4 * 2 * 32 * 8 * sizeof(float);
    p.smem = off;
    return p;
}

}  // namespace hsa

using namespace hsa;

// Defined in span_attn_bwd_tc.cu: sums the tiles' partial rows of the nodes of level >= 6.
int hsa_span_bwd_upper_reduce(float *partial, void *dk, void *dv, int64_t dk_bs, int64_t dk_rs, int64_t dv_bs, int64_t dv_rs,
                              int B, int N, int H, int D, int causal, int dtype, cudaStream_t st);

bool hsa_span_attn_bwd_tc8_supported(const hsa_view *views, int nviews, int B, int N, int H, int D, int radius,
                                     int causal, int dtype) {
    if (dtype != HSA_BF16 && dtype != HSA_F16) return false;
    if (D != 64 && D != 128) return false;
    if (N < kTile || (N & (N - 1)) != 0 || N > (1 << 28)) return false;
    if (B < 1 || B > 65535 || H < 1 || H > 65535 || radius < 0) return false;
    if ((int64_t)(N / kTile) * H * B > 0x7fffffffLL) return false;
    for (int i = 0; i < nviews; ++i)
        if (!view_vec_ok(views[i], 2)) return false;
    // worth it only while two CTAs fit on an SM
    return plan_bwd8(N, D, radius, causal != 0).smem <= 113 * 1024;
}

template <typename T, int D>
static int launch_bwd8(SpanBwd8Args &a, const Bwd8Plan &p, int B, bool causal, cudaStream_t st) {
    const int64_t total = (int64_t)B * (a.N / kTile) * a.H;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess)
            return fail((int)e, "hsa_span_attn_bwd(tc8): shared memory %zu: %s", p.smem, cudaGetErrorString(e));
        kernel<<<(unsigned)total, 256, p.smem, st>>>(a);
        return launch_status("hsa_span_attn_bwd(tc8)");
    };
    return causal ? go(span_bwd_tc8_kernel<T, D, true>) : go(span_bwd_tc8_kernel<T, D, false>);
}

int hsa_span_attn_bwd_tc8(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut, hsa_view dQ,
                          hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D, int radius, int causal,
                          int dtype, cudaStream_t st) {
    const hsa_view views[] = {Q, K, V, Out, dOut, dQ, dK, dV};
    if (!hsa_span_attn_bwd_tc8_supported(views, 8, B, N, H, D, radius, causal, dtype))
        return fail(HSA_ERR_ARG, "hsa_span_attn_bwd: shape not taken by the 8-warp tensor-core kernel");
    const Bwd8Plan p = plan_bwd8(N, D, radius, causal != 0);
    SpanBwd8Args a{};
    a.q = Q.ptr; a.k = K.ptr; a.v = V.ptr; a.out = Out.ptr; a.go = dOut.ptr; a.lse = LSE;
    a.dq = dQ.ptr; a.dk = dK.ptr; a.dv = dV.ptr; a.partial = (float *)workspace;
    a.q_bs = Q.batch_stride; a.q_rs = Q.row_stride; a.k_bs = K.batch_stride; a.k_rs = K.row_stride;
    a.v_bs = V.batch_stride; a.v_rs = V.row_stride; a.o_bs = Out.batch_stride; a.o_rs = Out.row_stride;
    a.go_bs = dOut.batch_stride; a.go_rs = dOut.row_stride; a.dq_bs = dQ.batch_stride; a.dq_rs = dQ.row_stride;
    a.dk_bs = dK.batch_stride; a.dk_rs = dK.row_stride; a.dv_bs = dV.batch_stride; a.dv_rs = dV.row_stride;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.R = radius < N ? radius : N; a.RB = p.RB;
    a.band_rows = p.band_rows; a.tree_rows = p.tree_rows; a.q_rows = p.q_rows;
    a.kt_off = p.kt_off; a.vt_off = p.vt_off; a.q_off = p.q_off; a.go_off = p.go_off; a.stat_off = p.stat_off;
    a.x_off = p.x_off;
    a.scale = 1.0f / sqrtf((float)D);
    a.scale_log2e = 1.4426950408889634f * a.scale;
    int rc;
    if (dtype == HSA_BF16)
        rc = D == 128 ? launch_bwd8<__nv_bfloat16, 128>(a, p, B, causal != 0, st) : launch_bwd8<__nv_bfloat16, 64>(a, p, B, causal != 0, st);
    else
        rc = D == 128 ? launch_bwd8<__half, 128>(a, p, B, causal != 0, st) : launch_bwd8<__half, 64>(a, p, B, causal != 0, st);
    if (rc) return rc;
    return hsa_span_bwd_upper_reduce((float *)workspace, dK.ptr, dV.ptr, dK.batch_stride, dK.row_stride, dV.batch_stride,
                                     dV.row_stride, B, N, H, D, causal, dtype, st);
}
