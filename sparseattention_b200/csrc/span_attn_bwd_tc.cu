// Span attention backward on tensor cores (bf16 / f16, head dim 64 or 128, N >= 64).  Deterministic.
//
// One CTA = one (batch, head, aligned tile of 64 leaves), 4 warps of 16 leaves each.  It stages, once,
// Q and dOut of its leaves plus the halo leaves whose windows reach into the tile, and the same K/V
// working set as the forward (leaf band, in-tile tree nodes, one node per upper level).  Probabilities
// are recomputed from the saved log-sum-exp; delta = rowsum(dOut * Out) is formed while staging.
// Every output row has exactly one writer and every sum a fixed order:
//   phase B (key side)   each warp owns 16 leaf keys of the tile and walks the query blocks that can see
//                        them (its own block and the next RB blocks, halo included; both sides when not
//                        causal): S^T = K Q^T and dP^T = V dOut^T come out with keys as rows, so P^T and
//                        dS^T feed dV += P^T dOut and dK += dS^T Q straight from the accumulators.
//   phase A (query side) each warp owns 16 leaves: dQ += dS K over its band blocks and its tree block(s).
//                        For the tree block the 8x8 fragments of P and dS are transposed in registers
//                        (movmatrix) to get dV/dK of the tree slots: slots of levels 1..4 belong to this
//                        warp alone and are stored; the level-5 slot and the upper-level slots are partial
//                        sums that the CTA combines in warp order.
//   upper levels         a node of level >= 6 collects from 2^(level-6) tiles: each tile writes its partial
//                        row to the workspace and a second kernel adds the tiles of a node in tile order.
// Rows nobody attends to (right children when causal, the root) are written as zeros.
#include "tc_common.cuh"

namespace hsa {

struct SpanBwdTcArgs {
    const void *q, *k, *v, *out, *go;
    const float *lse;
    void *dq, *dk, *dv;
    float *partial;                 // [B, H, N/64, L-6, 2, D] float32
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs, go_bs, go_rs, dq_bs, dq_rs, dk_bs, dk_rs, dv_bs, dv_rs;
    int N, L, H, R, RB;
    int band_rows;      // leaf key rows staged per tile
    int tree_rows;      // tree key rows staged per tile
    int q_rows;         // query rows staged per tile (tile + halo)
    int persist_off;    // byte offsets into shared memory
    int kt_off, vt_off, q_off, go_off, stat_off;
    int ds_off;         // dS^T tiles handed from the key-side phase to the query-side phase
    float scale_log2e, scale;
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(y) : "r"(x));
    return y;
}

template <bool CAUSAL> __device__ __forceinline__ constexpr int first_partial_slot() { return CAUSAL ? 8 : 15; }

template <typename T, int D, bool CAUSAL>
__global__ void __launch_bounds__(128, 2)
span_bwd_tc_kernel(SpanBwdTcArgs a) {
    constexpr int PITCH = D * 2 + 16;
    constexpr int CPR = D / 8;
    constexpr int RPI = 128 / CPR;
    constexpr int KS = D / 16;
    constexpr int TIN = tree_in_rows<CAUSAL>();
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *Kb = smem;                                   // leaf band of K
    unsigned char *Vb = Kb + (size_t)a.band_rows * PITCH;       // leaf band of V
    float *persist = reinterpret_cast<float *>(smem + a.persist_off);   // aliases the bands once they are dead
    unsigned char *Kt = smem + a.kt_off;                        // tree rows of K
    unsigned char *Vt = smem + a.vt_off;
    unsigned char *Qs = smem + a.q_off;
    unsigned char *Gs = smem + a.go_off;                        // dOut rows
    float *lse_s = reinterpret_cast<float *>(smem + a.stat_off);
    float *dl_s = lse_s + a.q_rows;
    // dS^T tiles [query block of the tile][relative key block][16 keys][16 queries] in T, 512 bytes each; the two
    // 16-byte halves of a row are swapped in rows 4..7 and 12..15 so that 8-row matrix loads hit distinct banks
    unsigned char *ds_tiles = smem + a.ds_off;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x % a.H;
    const int tile = blockIdx.x / a.H;
    const int ntiles = a.N / kTile;
    const int b = blockIdx.y;
    const int t0 = tile * kTile;
    const int N = a.N, L = a.L, R = a.R, RB = a.RB;
    const int band_lo = t0 - 16 * RB;
    const int qoff = CAUSAL ? 0 : 16 * RB;          // local row of the tile's first leaf in Qs / Gs
    const int q_lo = t0 - qoff;
    const int64_t hoff = (int64_t)h * D;
    const T *qg = (const T *)a.q + b * a.q_bs + hoff;
    const T *kg = (const T *)a.k + b * a.k_bs + hoff;
    const T *vg = (const T *)a.v + b * a.v_bs + hoff;
    const T *og = (const T *)a.out + b * a.o_bs + hoff;
    const T *gg = (const T *)a.go + b * a.go_bs + hoff;
    const int lw = 16 * warp;
    const int quad = lane & 3, qrow = lane >> 2;
    const int nup = L - kTileLog;

    // ---------------------------------------------------------------- staging
    {
        const int c = tid % CPR, rg = tid / CPR;
        auto stage_rows = [&](const T *g, int64_t rs, unsigned char *S, int first, int rows) {
            const T *gc = g + c * 8;
            uint32_t dst = smem_u32(S) + rg * PITCH + c * 16;
            int r = first + rg;
            for (int i = rg; i < rows; i += RPI, r += RPI, dst += RPI * PITCH) {
                const bool ok = (unsigned)r < (unsigned)N;
                cp_async16(dst, gc + (int64_t)(ok ? r : 0) * rs, ok);
            }
        };
        auto stage_tree = [&](const T *g, int64_t rs, unsigned char *S) {
            const T *gc = g + c * 8;
            uint32_t dst = smem_u32(S) + rg * PITCH + c * 16;
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
        stage_rows(gg, a.go_rs, Gs, q_lo, a.q_rows);
        cp_async_commit();
        stage_rows(qg, a.q_rs, Qs, q_lo, a.q_rows);
        stage_rows(kg, a.k_rs, Kb, band_lo, a.band_rows);
        stage_rows(vg, a.v_rs, Vb, band_lo, a.band_rows);
        stage_tree(kg, a.k_rs, Kt);
        stage_tree(vg, a.v_rs, Vt);
        cp_async_commit();

        // delta = rowsum(dOut * Out) and log-sum-exp (base 2) of every staged query row.  The Out chunks and
        // the statistics come straight from global memory; all loads of a batch are issued before anything
        // waits (the first batch even before dOut has landed), so only one memory latency is exposed.
        constexpr int PF = 10;                       // rows per thread in flight
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
            if (i0 == rg) { cp_async_wait<1>(); __syncthreads(); }      // dOut rows are in shared memory
#pragma unroll
            for (int j = 0; j < PF; ++j) {
                const int i = i0 + j * RPI;
                float part = 0.f;
                if (i < a.q_rows) {
                    const uint4 gv = *reinterpret_cast<const uint4 *>(Gs + i * PITCH + c * 16);
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
    const int nrel = CAUSAL ? RB + 1 : 2 * RB + 1;          // key blocks a query block can see = tiles per query block

    // ================================================================ phase B: leaf keys of the tile
    {
        float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) dk[i][e] = dv[i][e] = 0.f;
        const int krow = 16 * RB + lw + (lane & 7) + 8 * ((lane >> 3) & 1);       // A-operand rows: own keys
        const uint32_t ka = smem_u32(Kb + (size_t)krow * PITCH + (lane >> 4) * 16);
        const uint32_t va = smem_u32(Vb + (size_t)krow * PITCH + (lane >> 4) * 16);
        const int key0 = t0 + lw;                                               // first own key row
        // NQ consecutive query blocks at once: their score-type products advance together through the head
        // dimension (4*NQ independent accumulator chains, the K/V fragments of the own keys loaded once).
        // Query blocks outside the sequence need no special case: their rows are zero-filled and their
        // log-sum-exp is +inf, so every probability comes out as 0.
        auto key_side = [&]<int NQ>(int qb0) {
            float st[NQ][2][4], dpt[NQ][2][4];
            uint32_t qb_addr[NQ], gb_addr[NQ];
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) st[j][0][e] = st[j][1][e] = dpt[j][0][e] = dpt[j][1][e] = 0.f;
                const int brow = qoff + lw + 16 * (qb0 + j) + (lane & 7) + 8 * (lane >> 4);     // B-operand rows: queries
                qb_addr[j] = smem_u32(Qs + (size_t)brow * PITCH + ((lane >> 3) & 1) * 16);
                gb_addr[j] = smem_u32(Gs + (size_t)brow * PITCH + ((lane >> 3) & 1) * 16);
            }
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t af[4], bf[4];
                ldmatrix_x4(af, ka + ks * 32);
#pragma unroll
                for (int j = 0; j < NQ; ++j) {
                    ldmatrix_x4(bf, qb_addr[j] + ks * 32);
                    mma16816<T>(st[j][0], af, bf[0], bf[1]);
                    mma16816<T>(st[j][1], af, bf[2], bf[3]);
                }
                ldmatrix_x4(af, va + ks * 32);
#pragma unroll
                for (int j = 0; j < NQ; ++j) {
                    ldmatrix_x4(bf, gb_addr[j] + ks * 32);
                    mma16816<T>(dpt[j][0], af, bf[0], bf[1]);
                    mma16816<T>(dpt[j][1], af, bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
                const int qb = qb0 + j;
                const int qr0 = qoff + lw + 16 * qb;                             // local row of the block's first query
                // element (nt, e): key row kr = qrow + 8*(e>>1), query column qc = nt*8 + 2*quad + (e&1)
                float p[2][4], ds[2][4];
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
                        const float l2 = lse_s[qr0 + qc];                        // +inf outside the sequence
                        const float pe = fast_exp2(fmaf(st[j][nt][e], c2, bias) - l2);
                        p[nt][e] = pe;
                        ds[nt][e] = pe * (dpt[j][nt][e] - dl_s[qr0 + qc]) * sc;
                    }
                uint32_t pa[4], da[4];
                pa[0] = pack2<T>(p[0][0], p[0][1]); pa[1] = pack2<T>(p[0][2], p[0][3]);
                pa[2] = pack2<T>(p[1][0], p[1][1]); pa[3] = pack2<T>(p[1][2], p[1][3]);
                da[0] = pack2<T>(ds[0][0], ds[0][1]); da[1] = pack2<T>(ds[0][2], ds[0][3]);
                da[2] = pack2<T>(ds[1][0], ds[1][1]); da[3] = pack2<T>(ds[1][2], ds[1][3]);
                // hand dS^T of this (key block, query block) pair to the query-side phase when the queries are the tile's own
                const int qblk = warp + qb;
                if (qblk >= 0 && qblk < 4) {
                    unsigned char *tile_p = ds_tiles + (size_t)(qblk * nrel + (CAUSAL ? qb : qb + RB)) * 512;
                    const int sw = ((qrow >> 2) & 1) * 16;               // same for rows qrow and qrow + 8
                    *reinterpret_cast<uint32_t *>(tile_p + qrow * 32 + (0 ^ sw) + 4 * quad) = da[0];
                    *reinterpret_cast<uint32_t *>(tile_p + (qrow + 8) * 32 + (0 ^ sw) + 4 * quad) = da[1];
                    *reinterpret_cast<uint32_t *>(tile_p + qrow * 32 + (16 ^ sw) + 4 * quad) = da[2];
                    *reinterpret_cast<uint32_t *>(tile_p + (qrow + 8) * 32 + (16 ^ sw) + 4 * quad) = da[3];
                }
                const int trow = qr0 + (lane & 7) + 8 * ((lane >> 3) & 1);       // B rows for [queries x d]
                const uint32_t gt = smem_u32(Gs + (size_t)trow * PITCH + (lane >> 4) * 16);
                const uint32_t qt = smem_u32(Qs + (size_t)trow * PITCH + (lane >> 4) * 16);
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    uint32_t f[4];
                    ldmatrix_x4_trans(f, gt + dp * 32);
                    mma16816<T>(dv[2 * dp], pa, f[0], f[1]);
                    mma16816<T>(dv[2 * dp + 1], pa, f[2], f[3]);
                    ldmatrix_x4_trans(f, qt + dp * 32);
                    mma16816<T>(dk[2 * dp], da, f[0], f[1]);
                    mma16816<T>(dk[2 * dp + 1], da, f[2], f[3]);
                }
            }
        };
        int qb = CAUSAL ? 0 : -RB;
        for (; qb + 1 <= RB; qb += 2) key_side.template operator()<2>(qb);
        if (qb <= RB) key_side.template operator()<1>(qb);
        T *dkg = (T *)a.dk + b * a.dk_bs + hoff;
        T *dvg = (T *)a.dv + b * a.dv_bs + hoff;
        const int64_t r0 = key0 + qrow, r1 = r0 + 8;
        store_acc_rows<T, D / 8>(dkg + r0 * a.dk_rs, dkg + r1 * a.dk_rs, dk, quad);
        store_acc_rows<T, D / 8>(dvg + r0 * a.dv_rs, dvg + r1 * a.dv_rs, dv, quad);
    }

    // ================================================================ phase A: own leaves as queries
    float dq[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
    const int qa0 = qoff + lw;                                                   // local row of the warp's first leaf
    const int arow = qa0 + (lane & 7) + 8 * ((lane >> 3) & 1);
    const uint32_t qa = smem_u32(Qs + (size_t)arow * PITCH + (lane >> 4) * 16);  // A operand: own Q rows
    const uint32_t ga = smem_u32(Gs + (size_t)arow * PITCH + (lane >> 4) * 16);  // A operand: own dOut rows
    const float lse0 = lse_s[qa0 + qrow], lse1 = lse_s[qa0 + qrow + 8];
    const float dl0 = dl_s[qa0 + qrow], dl1 = dl_s[qa0 + qrow + 8];
    const int dbase = 2 * quad - qrow;
    const int sib_dlt = (qrow & 1) ? -1 : 1;
    const bool sib_ok = !CAUSAL || (qrow & 1);
    const int nbb = CAUSAL ? RB + 1 : 2 * RB + 1;
    const int ntb = (tree_slots<CAUSAL>(L) + 15) >> 4;

    // S = Q K^T and dP = dOut V^T of the warp's 16 leaves against 16 keys whose rows are given per lane
    auto score_block = [&](const unsigned char *Kbase, const unsigned char *Vbase, int krow_nt, float (&s)[2][4],
                           float (&dp)[2][4]) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[0][e] = s[1][e] = dp[0][e] = dp[1][e] = 0.f;
        const uint32_t kb = smem_u32(Kbase + (size_t)krow_nt * PITCH + ((lane >> 3) & 1) * 16);
        const uint32_t vb = smem_u32(Vbase + (size_t)krow_nt * PITCH + ((lane >> 3) & 1) * 16);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t af[4], bf[4];
            ldmatrix_x4(af, qa + ks * 32);
            ldmatrix_x4(bf, kb + ks * 32);
            mma16816<T>(s[0], af, bf[0], bf[1]);
            mma16816<T>(s[1], af, bf[2], bf[3]);
            ldmatrix_x4(af, ga + ks * 32);
            ldmatrix_x4(bf, vb + ks * 32);
            mma16816<T>(dp[0], af, bf[0], bf[1]);
            mma16816<T>(dp[1], af, bf[2], bf[3]);
        }
    };
    // dQ += dS K for 16 keys whose rows (k-major operand, transposed load) are given per lane
    auto dq_block = [&](const unsigned char *Kbase, int krow_t, const uint32_t (&da)[4]) {
        const uint32_t kt = smem_u32(Kbase + (size_t)krow_t * PITCH + (lane >> 4) * 16);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t f[4];
            ldmatrix_x4_trans(f, kt + dp * 32);
            mma16816<T>(dq[2 * dp], da, f[0], f[1]);
            mma16816<T>(dq[2 * dp + 1], da, f[2], f[3]);
        }
    };

    __syncthreads();        // every dS^T tile of the key-side phase is in shared memory

    for (int bi = 0; bi < nbb; ++bi) {
        const int r0 = t0 + lw + 16 * (bi - RB);                                 // first key row of the block
        if (r0 >= N || r0 + 16 <= 0) continue;
        const int kblk = warp + bi - RB;                                         // key block relative to the tile
        if (kblk >= 0 && kblk < 4) {
            // the key-side phase already formed dS for this pair: read it back transposed (queries as rows)
            const int rel = RB - bi;                                             // query block = key block + rel
            const unsigned char *tile_p = ds_tiles + (size_t)(warp * nrel + (CAUSAL ? rel : rel + RB)) * 512;
            const int key = (lane & 7) + 8 * (lane >> 4);
            const int hsel = (((lane >> 3) & 1) * 16) ^ (((key >> 2) & 1) * 16);
            uint32_t da[4];
            ldmatrix_x4_trans(da, smem_u32(tile_p + key * 32 + hsel));
            dq_block(Kb, lw + 16 * bi + (lane & 7) + 8 * ((lane >> 3) & 1), da);
            continue;
        }
        float s[2][4], dp[2][4];
        score_block(Kb, Vb, lw + 16 * bi + (lane & 7) + 8 * (lane >> 4), s, dp);
        const bool edge = r0 < 0 || r0 + 16 > N;
        const bool self = bi == RB;
        const int d0 = dbase + 16 * (bi - RB);
        float ds[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int dlt = d0 + nt * 8 + (e & 1) - 8 * (e >> 1);
                bool wv = dlt >= -R && dlt <= (CAUSAL ? 0 : R);
                if (edge) wv = wv && (unsigned)(r0 + nt * 8 + 2 * quad + (e & 1)) < (unsigned)N;
                const bool lv = self && sib_ok && dlt == sib_dlt;
                const float bias = (wv && lv) ? 1.f : ((wv || lv) ? 0.f : -INFINITY);
                const float pe = fast_exp2(fmaf(s[nt][e], c2, bias) - ((e >> 1) ? lse1 : lse0));
                ds[nt][e] = pe * (dp[nt][e] - ((e >> 1) ? dl1 : dl0)) * sc;
            }
        uint32_t da[4];
        da[0] = pack2<T>(ds[0][0], ds[0][1]); da[1] = pack2<T>(ds[0][2], ds[0][3]);
        da[2] = pack2<T>(ds[1][0], ds[1][1]); da[3] = pack2<T>(ds[1][2], ds[1][3]);
        dq_block(Kb, lw + 16 * bi + (lane & 7) + 8 * ((lane >> 3) & 1), da);
    }

    __syncthreads();        // the leaf bands of K and V are dead from here on: `persist` may overwrite them

    const int fps = first_partial_slot<CAUSAL>();
    const int nps = 1 + nup;                                                     // partial slots per warp
    for (int tb = 0; tb < ntb; ++tb) {
        int rowA, rowB, jj;
        tree_slot<CAUSAL>(16 * tb + (lane & 7) + 8 * (lane >> 4), warp, L, rowA, jj);
        tree_slot<CAUSAL>(16 * tb + (lane & 7) + 8 * ((lane >> 3) & 1), warp, L, rowB, jj);
        float s[2][4], dp[2][4];
        score_block(Kt, Vt, rowA, s, dp);
        float p[2][4], ds[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int slot = 16 * tb + nt * 8 + 2 * quad + (e & 1);
                const int i = qrow + 8 * (e >> 1);
                int row2, j2;
                const int l = tree_slot<CAUSAL>(slot, warp, L, row2, j2);
                bool ok = false;
                if (l >= 1 && l <= 3) ok = CAUSAL ? ((i >> l) == j2 + 1) : (((i >> l) ^ 1) == j2);
                else if (l >= 4) ok = !CAUSAL || (((t0 + lw) >> l) & 1);
                const float pe = ok ? fast_exp2(s[nt][e] * c2 - ((e >> 1) ? lse1 : lse0)) : 0.f;
                p[nt][e] = pe;
                ds[nt][e] = pe * (dp[nt][e] - ((e >> 1) ? dl1 : dl0)) * sc;
            }
        uint32_t da[4];
        da[0] = pack2<T>(ds[0][0], ds[0][1]); da[1] = pack2<T>(ds[0][2], ds[0][3]);
        da[2] = pack2<T>(ds[1][0], ds[1][1]); da[3] = pack2<T>(ds[1][2], ds[1][3]);
        dq_block(Kt, rowB, da);

        // gradients of the 16 tree slots: (P^T dOut) and (dS^T Q), slots as rows, the warp's 16 leaves as k
        uint32_t pt[4], dt[4];
        pt[0] = movmatrix_trans(pack2<T>(p[0][0], p[0][1]));      // slots 0-7  x leaves 0-7
        pt[1] = movmatrix_trans(pack2<T>(p[1][0], p[1][1]));      // slots 8-15 x leaves 0-7
        pt[2] = movmatrix_trans(pack2<T>(p[0][2], p[0][3]));      // slots 0-7  x leaves 8-15
        pt[3] = movmatrix_trans(pack2<T>(p[1][2], p[1][3]));      // slots 8-15 x leaves 8-15
        dt[0] = movmatrix_trans(da[0]);
        dt[1] = movmatrix_trans(da[2]);
        dt[2] = movmatrix_trans(da[1]);
        dt[3] = movmatrix_trans(da[3]);
        // destinations of this thread's two slot rows (qrow and qrow + 8)
        T *fin_k[2] = {nullptr, nullptr}, *fin_v[2] = {nullptr, nullptr};
        float *par[2] = {nullptr, nullptr};
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int slot = 16 * tb + qrow + 8 * hh;
            int row2, j2;
            const int l = tree_slot<CAUSAL>(slot, warp, L, row2, j2);
            if (l >= 1 && l <= 4) {
                const int node = (l <= 3) ? (((t0 + lw) >> l) + j2) : ((((t0 + lw) >> 4)) ^ 1);
                const bool ok = l <= 3 || !CAUSAL || (((t0 + lw) >> 4) & 1);
                if (ok) {
                    const int64_t gr = level_base(N, l) + node;
                    fin_k[hh] = (T *)a.dk + b * a.dk_bs + gr * a.dk_rs + hoff;
                    fin_v[hh] = (T *)a.dv + b * a.dv_bs + gr * a.dv_rs + hoff;
                }
            } else if (l >= 5) {
                par[hh] = persist + ((size_t)(warp * nps + (slot - fps)) * 2) * D + 2 * quad;
            }
        }
        const uint32_t gt = smem_u32(Gs + (size_t)arow * PITCH + (lane >> 4) * 16);   // B: own dOut rows, transposed
        const uint32_t qt = smem_u32(Qs + (size_t)arow * PITCH + (lane >> 4) * 16);
#pragma unroll
        for (int which = 0; which < 2; ++which) {            // 0: dK of the slots, 1: dV of the slots
            float acc[D / 8][4];
#pragma unroll
            for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
            for (int dpp = 0; dpp < D / 16; ++dpp) {
                uint32_t f[4];
                ldmatrix_x4_trans(f, (which ? gt : qt) + dpp * 32);
                mma16816<T>(acc[2 * dpp], which ? pt : dt, f[0], f[1]);
                mma16816<T>(acc[2 * dpp + 1], which ? pt : dt, f[2], f[3]);
            }
            // rows owned by this warp alone go out as T (all lanes take part in the transpose; rows that are
            // partial sums or unused pass a null pointer)
            store_acc_rows<T, D / 8>(which ? fin_v[0] : fin_k[0], which ? fin_v[1] : fin_k[1], acc, quad);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float *pp = par[hh] ? par[hh] + which * D : nullptr;
                if (pp != nullptr) {
#pragma unroll
                    for (int nt = 0; nt < D / 8; ++nt)
                        *reinterpret_cast<float2 *>(pp + nt * 8) = make_float2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
                }
            }
        }
    }

    // dQ of the warp's leaves
    {
        T *dqg = (T *)a.dq + b * a.dq_bs + hoff;
        const int64_t r0 = t0 + lw + qrow, r1 = r0 + 8;
        store_acc_rows<T, D / 8>(dqg + r0 * a.dq_rs, dqg + r1 * a.dq_rs, dq, quad);
    }
    __syncthreads();

    // ---------------------------------------------------------------- combine the partial slots, warp order
    // level 5: node j of the tile collects from the two warps under its sibling
    for (int idx = tid; idx < 2 * 2 * D; idx += 128) {
        const int j = idx / (2 * D), rem = idx % (2 * D), which = rem / D, col = rem % D;
        if (CAUSAL && j == 1) continue;
        const int wa = 2 * (j ^ 1);
        const float sum = persist[((size_t)(wa * nps) * 2 + which) * D + col] +
                          persist[((size_t)((wa + 1) * nps) * 2 + which) * D + col];
        const int64_t gr = level_base(N, 5) + (t0 >> 5) + j;
        T *dst = which ? (T *)a.dv + b * a.dv_bs + gr * a.dv_rs + hoff : (T *)a.dk + b * a.dk_bs + gr * a.dk_rs + hoff;
        dst[col] = Traits<T>::from_f(sum);
    }
    // upper levels: the tile's partial rows go to the workspace
    for (int idx = tid; idx < nup * 2 * D; idx += 128) {
        const int u = idx / (2 * D), rem = idx % (2 * D);
        const int l = kTileLog + u;
        if (CAUSAL && ((t0 >> l) & 1) == 0) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) sum += persist[((size_t)(w * nps + 1 + u) * 2) * D + rem];
        a.partial[((((size_t)b * a.H + h) * ntiles + tile) * nup + u) * 2 * D + rem] = sum;
    }
    // rows nobody attends to inside the tile: right children, when causal
    if (CAUSAL) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int idx = tid; idx < 31 * CPR * 2; idx += 128) {
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

// dK/dV rows of the nodes of level >= 6 (root included): sum of the tiles' partial rows, in tile order.
template <typename T, bool CAUSAL>
__global__ void span_bwd_upper_reduce_kernel(SpanBwdTcArgs a, int D) {
    const int N = a.N, L = a.L;
    const int first = level_base(N, kTileLog);
    const int r = first + blockIdx.x;                       // node row
    const int h = blockIdx.y, b = blockIdx.z;
    const int ntiles = N / kTile, nup = L - kTileLog;
    const int rem = 2 * N - r;
    const int l = L - ilog2((unsigned)(rem - 1));
    const int j = r - level_base(N, l);
    const bool attended = l < L && (!CAUSAL || (j & 1) == 0);
    const int span = 1 << (l - kTileLog);                   // tiles under a node of this level
    const int tfirst = (j ^ 1) * span;
    for (int e = threadIdx.x; e < 2 * D; e += blockDim.x) {
        const int which = e / D, col = e % D;
        float sum = 0.f;
        if (attended) {
            const float *src = a.partial + ((((size_t)b * a.H + h) * ntiles + tfirst) * nup + (l - kTileLog)) * 2 * D + e;
            for (int t = 0; t < span; ++t) sum += src[(size_t)t * nup * 2 * D];
        }
        T *dst = which ? (T *)a.dv + b * a.dv_bs + (int64_t)r * a.dv_rs + (int64_t)h * D
                       : (T *)a.dk + b * a.dk_bs + (int64_t)r * a.dk_rs + (int64_t)h * D;
        dst[col] = Traits<T>::from_f(sum);
    }
}

struct BwdTcPlan {
    int RB, band_rows, tree_rows, q_rows, nup;
    int persist_off, kt_off, vt_off, q_off, go_off, stat_off, ds_off;
    size_t smem;
};

static BwdTcPlan plan_bwd_tc(int N, int D, int radius, bool causal) {
    BwdTcPlan p{};
    const int PITCH = D * 2 + 16;
    const int R = radius < N ? radius : N;
    const int L = ilog2((unsigned)N);
    p.RB = (R + 15) / 16;
    p.nup = L - kTileLog;
    p.band_rows = kTile + 16 * p.RB * (causal ? 1 : 2);
    p.tree_rows = (causal ? 31 : 62) + p.nup;
    p.q_rows = kTile + 16 * p.RB * (causal ? 1 : 2);
    const size_t bands = (size_t)2 * p.band_rows * PITCH;
    const size_t persist = (size_t)4 * (1 + p.nup) * 2 * D * sizeof(float);
    p.persist_off = 0;
    size_t off = bands > persist ? bands : persist;
    off = (off + 15) / 16 * 16;
    p.kt_off = (int)off; off += (size_t)p.tree_rows * PITCH;
    p.vt_off = (int)off; off += (size_t)p.tree_rows * PITCH;
    p.q_off = (int)off; off += (size_t)p.q_rows * PITCH;
    p.go_off = (int)off; off += (size_t)p.q_rows * PITCH;
    p.stat_off = (int)off; off += (size_t)2 * p.q_rows * sizeof(float);
    off = (off + 15) / 16 * 16;
    p.ds_off = (int)off; off += (size_t)4 * (causal ? p.RB + 1 : 2 * p.RB + 1) * 512;
    p.smem = off;
    return p;
}

}  // namespace hsa

using namespace hsa;

// Sum of the tiles' partial rows for the nodes of level >= 6 (shared with the 8-warp kernel).
int hsa_span_bwd_upper_reduce(float *partial, void *dk, void *dv, int64_t dk_bs, int64_t dk_rs, int64_t dv_bs, int64_t dv_rs,
                              int B, int N, int H, int D, int causal, int dtype, cudaStream_t st) {
    SpanBwdTcArgs a{};
    a.partial = partial; a.dk = dk; a.dv = dv;
    a.dk_bs = dk_bs; a.dk_rs = dk_rs; a.dv_bs = dv_bs; a.dv_rs = dv_rs;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H;
    const int nodes = 2 * N - 1 - level_base(N, kTileLog);
    dim3 g2((unsigned)nodes, (unsigned)H, (unsigned)B);
    if (dtype == HSA_BF16) {
        if (causal) span_bwd_upper_reduce_kernel<__nv_bfloat16, true><<<g2, 64, 0, st>>>(a, D);
        else span_bwd_upper_reduce_kernel<__nv_bfloat16, false><<<g2, 64, 0, st>>>(a, D);
    } else {
        if (causal) span_bwd_upper_reduce_kernel<__half, true><<<g2, 64, 0, st>>>(a, D);
        else span_bwd_upper_reduce_kernel<__half, false><<<g2, 64, 0, st>>>(a, D);
    }
    return launch_status("hsa_span_attn_bwd(tc, upper levels)");
}

bool hsa_span_attn_bwd_tc_supported(const hsa_view *views, int nviews, int B, int N, int H, int D, int radius,
                                    int causal, int dtype) {
    if (dtype != HSA_BF16 && dtype != HSA_F16) return false;
    if (D != 64 && D != 128) return false;
    if (N < kTile || (N & (N - 1)) != 0 || N > (1 << 28)) return false;
    if (B < 1 || B > 65535 || H < 1 || H > 65535 || radius < 0) return false;
    if ((int64_t)(N / kTile) * H > 0x7fffffffLL) return false;
    for (int i = 0; i < nviews; ++i)
        if (!view_vec_ok(views[i], 2)) return false;
    return plan_bwd_tc(N, D, radius, causal != 0).smem <= 200 * 1024;
}

size_t hsa_span_attn_bwd_tc_workspace(int B, int N, int H, int D) {
    if (N < kTile) return 0;
    const int nup = ilog2((unsigned)N) - kTileLog;
    return (size_t)B * H * (N / kTile) * nup * 2 * D * sizeof(float);
}

template <typename T, int D>
static int launch_bwd_tc(SpanBwdTcArgs &a, const BwdTcPlan &p, int B, bool causal, cudaStream_t st) {
    dim3 grid((unsigned)((a.N / kTile) * a.H), (unsigned)B);
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess)
            return fail((int)e, "hsa_span_attn_bwd(tc): shared memory %zu: %s", p.smem, cudaGetErrorString(e));
        kernel<<<grid, 128, p.smem, st>>>(a);
        return launch_status("hsa_span_attn_bwd(tc)");
    };
    if (int rc = causal ? go(span_bwd_tc_kernel<T, D, true>) : go(span_bwd_tc_kernel<T, D, false>)) return rc;
    const int nodes = 2 * a.N - 1 - level_base(a.N, kTileLog);
    dim3 g2((unsigned)nodes, (unsigned)a.H, (unsigned)B);
    if (causal) span_bwd_upper_reduce_kernel<T, true><<<g2, 64, 0, st>>>(a, D);
    else span_bwd_upper_reduce_kernel<T, false><<<g2, 64, 0, st>>>(a, D);
    return launch_status("hsa_span_attn_bwd(tc, upper levels)");
}

int hsa_span_attn_bwd_tc(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut, hsa_view dQ,
                         hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D, int radius, int causal,
                         int dtype, cudaStream_t st) {
    const hsa_view views[] = {Q, K, V, Out, dOut, dQ, dK, dV};
    if (!hsa_span_attn_bwd_tc_supported(views, 8, B, N, H, D, radius, causal, dtype))
        return fail(HSA_ERR_ARG,
                    "hsa_span_attn_bwd: the tensor-core kernel takes bf16/f16, head dim 64 or 128, N >= 64, "
                    "16-byte aligned views and a window that fits shared memory");
    const BwdTcPlan p = plan_bwd_tc(N, D, radius, causal != 0);
    SpanBwdTcArgs a{};
    a.q = Q.ptr; a.k = K.ptr; a.v = V.ptr; a.out = Out.ptr; a.go = dOut.ptr; a.lse = LSE;
    a.dq = dQ.ptr; a.dk = dK.ptr; a.dv = dV.ptr; a.partial = (float *)workspace;
    a.q_bs = Q.batch_stride; a.q_rs = Q.row_stride; a.k_bs = K.batch_stride; a.k_rs = K.row_stride;
    a.v_bs = V.batch_stride; a.v_rs = V.row_stride; a.o_bs = Out.batch_stride; a.o_rs = Out.row_stride;
    a.go_bs = dOut.batch_stride; a.go_rs = dOut.row_stride; a.dq_bs = dQ.batch_stride; a.dq_rs = dQ.row_stride;
    a.dk_bs = dK.batch_stride; a.dk_rs = dK.row_stride; a.dv_bs = dV.batch_stride; a.dv_rs = dV.row_stride;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.R = radius < N ? radius : N; a.RB = p.RB;
    a.band_rows = p.band_rows; a.tree_rows = p.tree_rows; a.q_rows = p.q_rows;
    a.persist_off = p.persist_off; a.kt_off = p.kt_off; a.vt_off = p.vt_off; a.q_off = p.q_off; a.go_off = p.go_off;
    a.stat_off = p.stat_off; a.ds_off = p.ds_off;
    a.scale = 1.0f / sqrtf((float)D);
    a.scale_log2e = 1.4426950408889634f * a.scale;
    if (dtype == HSA_BF16)
        return D == 128 ? launch_bwd_tc<__nv_bfloat16, 128>(a, p, B, causal != 0, st)
                        : launch_bwd_tc<__nv_bfloat16, 64>(a, p, B, causal != 0, st);
    return D == 128 ? launch_bwd_tc<__half, 128>(a, p, B, causal != 0, st) : launch_bwd_tc<__half, 64>(a, p, B, causal != 0, st);
}
