// Span attention backward on tensor cores, 8 warps per 64-leaf tile, work cut into tasks (bf16 / f16, head
// dim 64 or 128, causal, window radius <= 16).  Deterministic.
//
// Same staging and the same sums as span_attn_bwd_tc.cu, but instead of giving every warp one 16-leaf block
// for the whole kernel (128+ accumulator registers per thread, 8 warps per SM), the tile's work is cut into
// small tasks that exchange 16x16 probability / dS tiles through shared memory, so a thread never holds more
// than 32 accumulators and 16 warps per SM hide each other's latencies:
//   phase 1  8 score tasks, one per warp: (key block kb, query block kb or kb+1) of the leaf band.
//            S^T = K Q^T and dP^T = V dOut^T -> P^T and dS^T (keys as rows) written as bf16/f16 tiles.
//   phase 2  5 score tasks (warps 0-4): the tree block(s) of each of the 4 query blocks (P and dS, queries as
//            rows), and the pair (last key block of the previous tile, first query block);
//            16 output tasks: dV = P^T dOut and dK = dS^T Q of a key block, one half of the head dim each.
//   phase 3  8 output tasks, one per warp: dQ of a query block (two band tiles + its tree tiles), half the
//            head dim each.
//   phase 4  gradients of the tree slots (P^T dOut, dS^T Q with slots as rows): rows owned by one query
//            block are stored, shared nodes go to fp32 partial rows that phase 5 combines in block order.
//   phase 5  level-5 node, per-tile partial rows of the levels >= 6 (summed over tiles by a second kernel in
//            tile order), zero rows for nodes nobody attends to.
// Staged rows sit in [128-byte half][row][128 B] planes with the 128-byte XOR swizzle of the TMA unit: with 256-byte
// rows (D = 128) one cp.async.bulk.tensor box per thread brings them in (bounded mbarrier waits), with 128-byte rows
// per-thread cp.async does (the boxes would be too small to pay off).
#include "tc_common.cuh"
#include "tma_common.cuh"

namespace hsa {

constexpr int kBand8 = kTile + 16;      // staged rows per buffer: the tile and one 16-row block of halo

// Tensor maps of the staged tensors, all over [B, rows, H, D] with a box of 64 elements of one head:
// q, go: box of kBand8 rows; k/v band: every row, box of kBand8 rows; k/v e4, e2: every second row, boxes of 4 and 2
// rows (the left children of levels 1 and 2 below a 16-leaf block); k/v one: every row, box of one row.
struct SpanBwd8Maps {
    CUtensorMap q, go, k_band, k_e4, k_e2, k_one, v_band, v_e4, v_e2, v_one;
};

struct SpanBwd8Args {
    const void *q, *k, *v, *out, *go;
    const float *lse;
    void *dq, *dk, *dv;
    float *partial;                 // [B, H, N/64, L-6, 2, D] float32
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs, o_bs, o_rs, go_bs, go_rs, dq_bs, dq_rs, dk_bs, dk_rs, dv_bs, dv_rs;
    int N, L, H, R;
    int ntb, tree_rows;
    int mbar_off;
    // byte offsets into shared memory (the V band starts at 0)
    int kb_off, vt_off, kt_off, q_off, go_off, stat_off, tiles_off, ttiles_off, persist_off;
    float scale_log2e, scale;
    long long wait_limit;      // cycles a CTA waits for its bulk copies
    unsigned int extra_tx;     // 0 except in the test of the give-up path
};

// CTAs whose wait for their TMA copies ran out (never expected; added to what hsa_span_attn_fwd_wait_expired reports)
__device__ unsigned int g_bwd8_wait_expired = 0;

// Tree rows in shared memory: rows 8*qb .. 8*qb+7 hold what query block qb alone attends to (slots 0..7: four
// even level-1 nodes, two even level-2 nodes, one level-3 node, the level-4 sibling of the block), row 32 the
// tile's left level-5 node, rows 33.. one node per level >= 6.  Any 8 consecutive slots of a block thus sit in 8
// consecutive rows, which the swizzle spreads over all banks.
constexpr int kTreeIn8 = 33;
// Tree key slot s of query block qb -> level (or -1 past the last level) and shared-memory row; jj = node index
// relative to the first node of that level below the block.
__device__ __forceinline__ int tree_slot8(int s, int qb, int L, int &row, int &jj) {
    jj = 0;
    if (s < 8) {
        row = 8 * qb + s;
        if (s < 4) { jj = 2 * s; return 1; }
        if (s < 6) { jj = 2 * (s - 4); return 2; }
        return s == 6 ? 3 : 4;
    }
    const int l = s - 3;
    if (l >= L) { row = 0; return -1; }
    row = 32 + (s - 8);
    return l;
}

template <typename T, int D>
__global__ void __launch_bounds__(256, 2)
span_bwd_tc8_kernel(const SpanBwd8Args a, const __grid_constant__ SpanBwd8Maps maps) {
    constexpr int NH = D / 64;             // 128-byte halves of a row: buffers are [half][row][128 B] planes
    // 256-byte rows come in by TMA; for 128-byte rows the boxes get so small (a 64-leaf tile needs 50 of them for half
    // the bytes) that per-thread 16-byte copies are faster
    constexpr bool TMA = D >= 128;
    constexpr int BP = kBand8 * 128;       // bytes of one plane of a band buffer (Q, dOut, K band, V band)
    constexpr int CPR = D / 8;
    constexpr int RPI = 256 / CPR;
    constexpr int KS = D / 16;
    constexpr int CW = D / 2;              // columns of the head dimension per output task
    constexpr int NTH = CW / 8;            // its 8-column n-tiles
    constexpr int FPS = 8;                 // first tree slot that is a partial sum (level 5)
    constexpr int PR = 2 * D + 8;          // floats per partial row (dK | dV), padded: 8 rows written at once spread over the banks
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the hardware swizzle of the TMA copies XORs address bits 4..6 with bits 7..9: keep the band planes on 1024 bytes
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char *Vb = smem;
    unsigned char *Kb = smem + a.kb_off;
    unsigned char *Vt = smem + a.vt_off;
    unsigned char *Kt = smem + a.kt_off;
    unsigned char *Qs = smem + a.q_off;
    unsigned char *Gs = smem + a.go_off;
    float *lse_s = reinterpret_cast<float *>(smem + a.stat_off);
    float *dl_s = lse_s + kBand8;
    // 512-byte tiles [16 rows][16 columns] of T; the two 16-byte halves of a row are swapped in rows 4..7 and
    // 12..15 so that 8-row matrix loads hit distinct banks
    unsigned char *tiles = smem + a.tiles_off;       // (kb, rel): P^T at ((kb*2+rel)*2), dS^T at +1; halo pair dS^T at 16
    unsigned char *ttiles = smem + a.ttiles_off;     // (qb, tb): P at ((qb*ntb+tb)*2), dS at +1   (inside the dead V band)
    float *persist = reinterpret_cast<float *>(smem + a.persist_off);   // [qb][1+nup] rows of PR floats, inside dead bands
    unsigned long long *mbar = reinterpret_cast<unsigned long long *>(smem + a.mbar_off);
    const int TP = a.tree_rows * 128;      // bytes of one plane of a tree buffer

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ntiles = a.N / kTile;
    const int h = blockIdx.x % a.H;
    const int tile = (blockIdx.x / a.H) % ntiles;
    const int b = blockIdx.x / (a.H * ntiles);
    const int t0 = tile * kTile;
    const int N = a.N, L = a.L, R = a.R, ntb = a.ntb;
    const int64_t hoff = (int64_t)h * D;
    const T *og = (const T *)a.out + b * a.o_bs + hoff;
    const int quad = lane & 3, qrow = lane >> 2;
    const int nup = L - kTileLog;
    const int nps = 1 + nup;

    // What a CTA does when a wait runs out: count itself and leave NaN where its results would go (its dQ rows and its
    // partial rows of the upper levels, which the reduction kernel carries into dK / dV), so nobody mistakes them for data.
    auto give_up = [&]() {
        if (tid == 0) atomicAdd(&g_bwd8_wait_expired, 1u);
        fill_rows_nan16((T *)a.dq + b * a.dq_bs + hoff + (int64_t)t0 * a.dq_rs, a.dq_rs, kTile, D, tid, 256);
        float *mine = a.partial + (((size_t)b * a.H + h) * ntiles + tile) * nup * 2 * D;
        for (int idx = tid; idx < nup * 2 * D; idx += 256) mine[idx] = __int_as_float(0x7fffffff);
    };

    // ---------------------------------------------------------------- staging: one TMA box per thread
    // barrier 0: dOut; barrier 1: Q and the K/V bands; barrier 2: the tree rows.  Rows nobody may attend to are loaded
    // all the same (level-4 siblings of even blocks, upper levels on the causal side) or zero-filled by the copy
    // engine (past the last leaf, before the first), so masked scores and 0 * V products stay finite.
    const uint32_t mbG = smem_u32(&mbar[0]), mbM = smem_u32(&mbar[1]), mbT = smem_u32(&mbar[2]);
    // group 0: dOut, 1: Q and the bands, 2: the tree rows.  TMA: bounded mbarrier wait; per-thread copies: wait_group.
    auto wait_group = [&](int g) -> bool {
        if constexpr (TMA) {
            return mbar_wait_phase0(g == 0 ? mbG : g == 1 ? mbM : mbT, a.wait_limit);
        } else {
            if (g == 0) cp_async_wait<2>(); else if (g == 1) cp_async_wait<1>(); else cp_async_wait<0>();
            return true;
        }
    };
    if (TMA && tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbG), "r"(1) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbM), "r"(1) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbT), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    {
        const int c = tid % CPR, rg = tid / CPR;
        if constexpr (TMA) {
            if (tid == 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbG), "r"((uint32_t)BP * NH + a.extra_tx) : "memory");
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbM), "r"(3u * BP * NH) : "memory");
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbT), "r"(2u * (uint32_t)TP * NH) : "memory");
            }
            // boxes per half: 0 dOut, 1 Q, 2 K band, 3 V band, then per tree tensor (K, V): 16 boxes of the four query
            // blocks (level 1: 4 rows, level 2: 2 rows, level 3, level 4), the level-5 node, one node per upper level
            const int per_tree = 17 + nup;
            const int per_half = 4 + 2 * per_tree;
            if (tid < NH * per_half) {
                const int hf = tid / per_half, j = tid % per_half;
                const CUtensorMap *map;
                unsigned char *S;
                int row, dst_row = 0;
                uint32_t mb;
                if (j < 4) {
                    map = j == 0 ? &maps.go : j == 1 ? &maps.q : j == 2 ? &maps.k_band : &maps.v_band;
                    S = (j == 0 ? Gs : j == 1 ? Qs : j == 2 ? Kb : Vb) + (size_t)hf * BP;
                    row = j < 2 ? t0 : t0 - 16;
                    mb = j == 0 ? mbG : mbM;
                } else {
                    const int isv = (j - 4) / per_tree, f = (j - 4) % per_tree;
                    S = (isv ? Vt : Kt) + (size_t)hf * TP;
                    mb = mbT;
                    if (f < 16) {
                        const int qb = f >> 2, kind = f & 3;
                        if (kind == 0) { map = isv ? &maps.v_e4 : &maps.k_e4; row = (level_base(N, 1) + (t0 >> 1) + 8 * qb) >> 1; dst_row = 8 * qb; }
                        else if (kind == 1) { map = isv ? &maps.v_e2 : &maps.k_e2; row = (level_base(N, 2) + (t0 >> 2) + 4 * qb) >> 1; dst_row = 8 * qb + 4; }
                        else if (kind == 2) { map = isv ? &maps.v_one : &maps.k_one; row = level_base(N, 3) + (t0 >> 3) + 2 * qb; dst_row = 8 * qb + 6; }
                        else { map = isv ? &maps.v_one : &maps.k_one; row = level_base(N, 4) + (t0 >> 4) + (qb ^ 1); dst_row = 8 * qb + 7; }
                    } else if (f == 16) {
                        map = isv ? &maps.v_one : &maps.k_one; row = level_base(N, 5) + (t0 >> 5); dst_row = 32;
                    } else {
                        const int l = kTileLog + (f - 17);
                        map = isv ? &maps.v_one : &maps.k_one; row = level_base(N, l) + ((t0 >> l) ^ 1); dst_row = kTreeIn8 + (f - 17);
                    }
                }
                const uint32_t dst = smem_u32(S + (size_t)dst_row * 128);
                asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
                             ::"r"(dst), "l"(map), "r"(64 * hf), "r"(h), "r"(row), "r"(b), "r"(mb) : "memory");
            }

        } else {
            // one 128-byte plane per buffer: per-thread 16-byte copies, pieces XORed with address bits 7..9 like the
            // copy engine's swizzle.  Groups: dOut | Q and the bands | the tree rows.
            auto put = [&](unsigned char *S, int row, const T *src, bool ok) {
                const uint32_t ra = smem_u32(S + (size_t)row * 128);
                cp_async16(ra + (((c ^ (ra >> 7)) & 7) << 4), src, ok);
            };
            auto stage_rows = [&](const void *base, int64_t bs, int64_t rs, unsigned char *S, int first) {
                const T *gc = (const T *)base + b * bs + hoff + c * 8;
                for (int i = rg; i < kBand8; i += RPI) {
                    const int r = first + i;
                    const bool ok = (unsigned)r < (unsigned)N;
                    put(S, i, gc + (int64_t)(ok ? r : 0) * rs, ok);
                }
            };
            auto stage_tree = [&](const void *base, int64_t bs, int64_t rs, unsigned char *S) {
                const T *gc = (const T *)base + b * bs + hoff + c * 8;
                for (int f = rg; f < a.tree_rows; f += RPI) {
                    int l, node;
                    if (f < 32) {
                        const int qb = f >> 3, sl = f & 7;
                        if (sl < 4) { l = 1; node = 8 * qb + 2 * sl; }
                        else if (sl < 6) { l = 2; node = 4 * qb + 2 * (sl - 4); }
                        else if (sl == 6) { l = 3; node = 2 * qb; }
                        else { l = 4; node = qb ^ 1; }
                        node += t0 >> l;
                    } else if (f == 32) {
                        l = 5; node = t0 >> 5;
                    } else {
                        l = kTileLog + (f - kTreeIn8);
                        node = (t0 >> l) ^ 1;
                    }
                    put(S, f, gc + (int64_t)(level_base(N, l) + node) * rs, true);
                }
            };
            stage_rows(a.go, a.go_bs, a.go_rs, Gs, t0);
            cp_async_commit();
            stage_rows(a.q, a.q_bs, a.q_rs, Qs, t0);
            stage_rows(a.k, a.k_bs, a.k_rs, Kb, t0 - 16);
            stage_rows(a.v, a.v_bs, a.v_rs, Vb, t0 - 16);
            cp_async_commit();
            stage_tree(a.k, a.k_bs, a.k_rs, Kt);
            stage_tree(a.v, a.v_bs, a.v_rs, Vt);
            cp_async_commit();
        }

        // delta = rowsum(dOut * Out) and base-2 log-sum-exp per staged query row; all global loads are issued
        // before anything waits
        constexpr int PF = (kBand8 + RPI - 1) / RPI;
        uint4 ov[PF];
        float lv[PF];
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int i = rg + j * RPI;
            const int n = t0 + i;
            const bool ok = i < kBand8 && n < N;
            ov[j] = ok ? __ldg(reinterpret_cast<const uint4 *>(og + (int64_t)n * a.o_rs + c * 8)) : make_uint4(0, 0, 0, 0);
            lv[j] = (ok && c == 0) ? __ldg(a.lse + ((int64_t)b * N + n) * a.H + h) * 1.4426950408889634f : INFINITY;
        }
        if (!__syncthreads_and(wait_group(0))) {              // dOut rows are in shared memory (the wait is not expected to give up)
            wait_group(1);                                      // a second bounded chance for this CTA's copies to finish
            wait_group(2);
            give_up();
            return;
        }
#pragma unroll
        for (int j = 0; j < PF; ++j) {
            const int i = rg + j * RPI;
            float part = 0.f;
            if (i < kBand8) {
                const uint4 gv = *reinterpret_cast<const uint4 *>(Gs + (c >> 3) * BP + i * 128 + (((c ^ i) & 7) << 4));
                const T *oe = reinterpret_cast<const T *>(&ov[j]);
                const T *ge = reinterpret_cast<const T *>(&gv);
#pragma unroll
                for (int e = 0; e < 8; ++e) part = fmaf(Traits<T>::to_f(oe[e]), Traits<T>::to_f(ge[e]), part);
            }
#pragma unroll
            for (int o = CPR / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (c == 0 && i < kBand8) {
                dl_s[i] = part;
                lse_s[i] = lv[j];
            }
        }
        if (!__syncthreads_and(wait_group(1))) {              // Q and the bands have landed; the statistics are written
            wait_group(2);
            give_up();
            return;
        }
    }

    const float c2 = a.scale_log2e, sc = a.scale;

    // A row of a buffer for ldmatrix: per 128-byte half its shared address and the lane's piece parity folded into the
    // row's swizzle (address bits 7..9).  X = plane 0 of the buffer, ps = bytes per plane.
    struct RowRef { uint32_t addr[NH]; int x[NH]; };
    auto row_ref = [&](const unsigned char *X, int ps, int row, int parity) {
        RowRef r;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
            r.addr[hf] = smem_u32(X + (size_t)hf * ps + (size_t)row * 128);
            r.x[hf] = (parity ^ (r.addr[hf] >> 7)) & 7;
        }
        return r;
    };
    // address of the 16-byte piece pe (even; the lane's parity is already in x) of the head dimension
    auto piece_addr = [&](const RowRef &r, int pe) { return r.addr[pe >> 3] + (uint32_t)((((pe & 7) ^ r.x[pe >> 3])) << 4); };

    // Two 16x16 products over the whole head dimension that share their row patterns:
    //   r1 = A1[arow..] B1[brow..]^T,  r2 = A2[arow..] B2[brow..]^T.
    // arow / brow are this lane's ldmatrix rows (A: (lane&7)+8*((lane>>3)&1), pieces by lane>>4;
    // B: (lane&7)+8*(lane>>4), pieces by (lane>>3)&1).
    auto product2 = [&](const unsigned char *A1, const unsigned char *A2, int arow, const unsigned char *B1,
                        const unsigned char *B2, int bps, int brow, float (&r1)[2][4], float (&r2)[2][4]) {
#pragma unroll
        for (int e = 0; e < 4; ++e) r1[0][e] = r1[1][e] = r2[0][e] = r2[1][e] = 0.f;
        const RowRef a1 = row_ref(A1, BP, arow, lane >> 4), a2 = row_ref(A2, BP, arow, lane >> 4);
        const RowRef b1 = row_ref(B1, bps, brow, (lane >> 3) & 1), b2 = row_ref(B2, bps, brow, (lane >> 3) & 1);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t af[4], bf[4];
            ldmatrix_x4(af, piece_addr(a1, 2 * ks));
            ldmatrix_x4(bf, piece_addr(b1, 2 * ks));
            mma16816<T>(r1[0], af, bf[0], bf[1]);
            mma16816<T>(r1[1], af, bf[2], bf[3]);
            ldmatrix_x4(af, piece_addr(a2, 2 * ks));
            ldmatrix_x4(bf, piece_addr(b2, 2 * ks));
            mma16816<T>(r2[0], af, bf[0], bf[1]);
            mma16816<T>(r2[1], af, bf[2], bf[3]);
        }
    };
    // acc[NTH][4] += A (16x16 register fragments) x rows (Bbuf, trow), columns [8*pb, 8*pb + CW).
    // trow is this lane's transposed-load row: (lane&7)+8*((lane>>3)&1), pieces by lane>>4.
    auto accum_cols = [&](float (&acc)[NTH][4], const uint32_t (&af)[4], const unsigned char *Bbuf, int bps, int trow, int pb) {
        // the CW columns of a task lie inside one 128-byte half
        const uint32_t tb = smem_u32(Bbuf + (size_t)(pb >> 3) * bps + (size_t)trow * 128);
        const int tx = ((lane >> 4) ^ (tb >> 7)) & 7;
#pragma unroll
        for (int dp = 0; dp < CW / 16; ++dp) {
            uint32_t f[4];
            ldmatrix_x4_trans(f, tb + (uint32_t)(((((pb & 7) + 2 * dp)) ^ tx) << 4));
            mma16816<T>(acc[2 * dp], af, f[0], f[1]);
            mma16816<T>(acc[2 * dp + 1], af, f[2], f[3]);
        }
    };
    // a 16x16 tile as written from accumulator-layout words / read back as the A fragment of the tile or of its transpose
    auto tile_store = [&](unsigned char *tp, const uint32_t (&w)[4]) {
        const int sw = ((qrow >> 2) & 1) * 16;               // same for rows qrow and qrow + 8
        *reinterpret_cast<uint32_t *>(tp + qrow * 32 + sw + 4 * quad) = w[0];
        *reinterpret_cast<uint32_t *>(tp + (qrow + 8) * 32 + sw + 4 * quad) = w[1];
        *reinterpret_cast<uint32_t *>(tp + qrow * 32 + (16 ^ sw) + 4 * quad) = w[2];
        *reinterpret_cast<uint32_t *>(tp + (qrow + 8) * 32 + (16 ^ sw) + 4 * quad) = w[3];
    };
    auto tile_load = [&](const unsigned char *tp, uint32_t (&f)[4]) {
        const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
        ldmatrix_x4(f, smem_u32(tp + r * 32 + (((lane >> 4) * 16) ^ (((r >> 2) & 1) * 16))));
    };
    auto tile_load_t = [&](const unsigned char *tp, uint32_t (&f)[4]) {
        const int r = (lane & 7) + 8 * (lane >> 4);
        ldmatrix_x4_trans(f, smem_u32(tp + r * 32 + ((((lane >> 3) & 1) * 16) ^ (((r >> 2) & 1) * 16))));
    };
    auto pack4 = [&](const float (&v)[2][4], uint32_t (&w)[4]) {
        w[0] = pack2<T>(v[0][0], v[0][1]); w[1] = pack2<T>(v[0][2], v[0][3]);
        w[2] = pack2<T>(v[1][0], v[1][1]); w[3] = pack2<T>(v[1][2], v[1][3]);
    };

    // Score task of the leaf band: keys of block kb (band rows 16*(kb+1)..), queries of block qb = kb + rel.
    // Rows outside the sequence are zero-filled and their log-sum-exp is +inf: every probability comes out 0.
    auto band_pair = [&](int kb, int rel, unsigned char *tile_p, unsigned char *tile_ds) {
        const int qr0 = 16 * (kb + rel);
        float st[2][4], dpt[2][4];
        product2(Kb, Vb, 16 * (kb + 1) + (lane & 7) + 8 * ((lane >> 3) & 1), Qs, Gs, BP, qr0 + (lane & 7) + 8 * (lane >> 4), st, dpt);
        // element (nt, e): key row kr = qrow + 8*(e>>1), query column qc = nt*8 + 2*quad + (e&1)
        float p[2][4], ds[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int qc = nt * 8 + 2 * quad + (e & 1);
                const int dlt = qrow + 8 * (e >> 1) - qc - 16 * rel;       // key - query
                const bool wv = dlt >= -R && dlt <= 0;
                const bool lv = rel == 0 && (e & 1) && dlt == -1;           // level-0 sibling of an odd leaf
                const float bias = (wv && lv) ? 1.f : ((wv || lv) ? 0.f : -INFINITY);
                const float pe = fast_exp2(fmaf(st[nt][e], c2, bias) - lse_s[qr0 + qc]);
                p[nt][e] = pe;
                ds[nt][e] = pe * (dpt[nt][e] - dl_s[qr0 + qc]) * sc;
            }
        uint32_t w[4];
        if (tile_p != nullptr) { pack4(p, w); tile_store(tile_p, w); }
        pack4(ds, w);
        tile_store(tile_ds, w);
    };

    // Score task of tree block tb of query block qb: P and dS with the 16 queries as rows, the 16 slots as columns.
    auto tree_pair = [&](int qb, int tb) {
        int rowA, jj;
        tree_slot8(16 * tb + (lane & 7) + 8 * (lane >> 4), qb, L, rowA, jj);
        float s[2][4], dp[2][4];
        product2(Qs, Gs, 16 * qb + (lane & 7) + 8 * ((lane >> 3) & 1), Kt, Vt, TP, rowA, s, dp);
        const float lse0 = lse_s[16 * qb + qrow], lse1 = lse_s[16 * qb + qrow + 8];
        const float dl0 = dl_s[16 * qb + qrow], dl1 = dl_s[16 * qb + qrow + 8];
        float p[2][4], ds[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int slot = 16 * tb + nt * 8 + 2 * quad + (e & 1);
                const int i = qrow + 8 * (e >> 1);
                int row2, j2;
                const int l = tree_slot8(slot, qb, L, row2, j2);
                bool ok = false;
                if (l >= 1 && l <= 3) ok = (i >> l) == j2 + 1;
                else if (l >= 4) ok = ((t0 + 16 * qb) >> l) & 1;
                const float pe = ok ? fast_exp2(s[nt][e] * c2 - ((e >> 1) ? lse1 : lse0)) : 0.f;
                p[nt][e] = pe;
                ds[nt][e] = pe * (dp[nt][e] - ((e >> 1) ? dl1 : dl0)) * sc;
            }
        unsigned char *tp = ttiles + (size_t)((qb * ntb + tb) * 2) * 512;
        uint32_t w[4];
        pack4(p, w);
        tile_store(tp, w);
        pack4(ds, w);
        tile_store(tp + 512, w);
    };

    // Output task: dV (which = 1) or dK (which = 0) of key block kb, columns [ch*CW, (ch+1)*CW).
    auto kv_task = [&](int u) {
        const int kb = u >> 2, which = (u >> 1) & 1, ch = u & 1;
        float acc[NTH][4];
#pragma unroll
        for (int i = 0; i < NTH; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
        for (int rel = 0; rel < 2; ++rel) {
            uint32_t af[4];
            tile_load(tiles + (size_t)((kb * 2 + rel) * 2 + (which ? 0 : 1)) * 512, af);
            accum_cols(acc, af, which ? Gs : Qs, BP, 16 * (kb + rel) + (lane & 7) + 8 * ((lane >> 3) & 1), ch * (CW / 8));
        }
        T *g = which ? (T *)a.dv + b * a.dv_bs : (T *)a.dk + b * a.dk_bs;
        const int64_t rs = which ? a.dv_rs : a.dk_rs;
        g += hoff + ch * CW;
        const int64_t r0 = t0 + 16 * kb + qrow;
        store_acc_rows<T, NTH>(g + r0 * rs, g + (r0 + 8) * rs, acc, quad);
    };

    // Output task: dQ of query block qb, columns [ch*CW, (ch+1)*CW).
    auto dq_task = [&](int u) {
        const int qb = u >> 1, ch = u & 1, pb = ch * (CW / 8);
        float acc[NTH][4];
#pragma unroll
        for (int i = 0; i < NTH; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        uint32_t af[4];
        const int lrow = (lane & 7) + 8 * ((lane >> 3) & 1);
        if (qb > 0 || t0 > 0) {                                // keys of the block before the query block
            tile_load_t(qb == 0 ? tiles + 16 * 512 : tiles + (size_t)(((qb - 1) * 2 + 1) * 2 + 1) * 512, af);
            accum_cols(acc, af, Kb, BP, 16 * qb + lrow, pb);
        }
        tile_load_t(tiles + (size_t)((qb * 2) * 2 + 1) * 512, af);     // keys of the query block itself
        accum_cols(acc, af, Kb, BP, 16 * (qb + 1) + lrow, pb);
        for (int tb = 0; tb < ntb; ++tb) {
            int rowB, jj;
            tree_slot8(16 * tb + lrow, qb, L, rowB, jj);
            tile_load(ttiles + (size_t)((qb * ntb + tb) * 2 + 1) * 512, af);
            accum_cols(acc, af, Kt, TP, rowB, pb);
        }
        T *g = (T *)a.dq + b * a.dq_bs + hoff + ch * CW;
        const int64_t r0 = t0 + 16 * qb + qrow;
        store_acc_rows<T, NTH>(g + r0 * a.dq_rs, g + (r0 + 8) * a.dq_rs, acc, quad);
    };

    // Output task: gradients of the 16 tree slots of block tb seen from query block qb (dV: P^T dOut, dK: dS^T Q).
    auto slot_task = [&](int v) {
        const int ch = v & 1, which = (v >> 1) & 1, qb = (v >> 2) & 3, tb = v >> 4;
        float acc[NTH][4];
#pragma unroll
        for (int i = 0; i < NTH; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
        uint32_t af[4];
        tile_load_t(ttiles + (size_t)((qb * ntb + tb) * 2 + (which ? 0 : 1)) * 512, af);
        accum_cols(acc, af, which ? Gs : Qs, BP, 16 * qb + (lane & 7) + 8 * ((lane >> 3) & 1), ch * (CW / 8));
        // destinations of this thread's two slot rows (qrow and qrow + 8): nodes of levels 1..4 belong to this query
        // block alone; level 5 and above are partial sums
        T *fin[2] = {nullptr, nullptr};
        float *par[2] = {nullptr, nullptr};
        const int q0 = t0 + 16 * qb;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int slot = 16 * tb + qrow + 8 * hh;
            int row2, j2;
            const int l = tree_slot8(slot, qb, L, row2, j2);
            if (l >= 1 && l <= 4) {
                const int node = (l <= 3) ? ((q0 >> l) + j2) : ((q0 >> 4) ^ 1);
                if (l <= 3 || ((q0 >> 4) & 1)) {
                    const int64_t gr = level_base(N, l) + node;
                    fin[hh] = (which ? (T *)a.dv + b * a.dv_bs + gr * a.dv_rs : (T *)a.dk + b * a.dk_bs + gr * a.dk_rs) + hoff + ch * CW;
                }
            } else if (l >= 5) {
                par[hh] = persist + (size_t)(qb * nps + (slot - FPS)) * PR + which * D + ch * CW + 2 * quad;
            }
        }
        store_acc_rows<T, NTH>(fin[0], fin[1], acc, quad);   // all lanes take part in the transpose; null rows are skipped
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
            if (par[hh] != nullptr) {
#pragma unroll
                for (int nt = 0; nt < NTH; ++nt)
                    *reinterpret_cast<float2 *>(par[hh] + nt * 8) = make_float2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
            }
    };

    // ================================================================ phase 1
    {
        const int kb = warp >> 1, rel = warp & 1;
        unsigned char *tp = tiles + (size_t)((kb * 2 + rel) * 2) * 512;
        band_pair(kb, rel, tp, tp + 512);
    }
    if (!__syncthreads_and(wait_group(2))) {         // the tree rows
        give_up();
        return;
    }
    // ================================================================ phase 2
    if (warp < 4) {
        for (int tb = 0; tb < ntb; ++tb) tree_pair(warp, tb);
    } else if (warp == 4 && t0 > 0) {
        band_pair(-1, 1, nullptr, tiles + 16 * 512);
    }
    {
        const int u0 = warp < 5 ? warp : 5 + 4 * (warp - 5);
        const int u1 = warp < 5 ? warp + 1 : (u0 + 4 < 16 ? u0 + 4 : 16);
        for (int u = u0; u < u1; ++u) kv_task(u);
    }
    __syncthreads();
    // ================================================================ phase 3
    dq_task(warp);
    __syncthreads();        // K band, V band and the tree rows are dead: the partial slots may overwrite them
    // ================================================================ phase 4
    for (int v = warp; v < 16 * ntb; v += 8) slot_task(v);
    __syncthreads();

    // ================================================================ phase 5: combine in block order
    // level 5: node 0 of the tile collects from the two query blocks under its sibling (node 1 is never attended)
    for (int idx = tid; idx < 2 * D; idx += 256) {
        const int which = idx / D, col = idx % D;
        const float sum = persist[(size_t)(2 * nps) * PR + idx] + persist[(size_t)(3 * nps) * PR + idx];
        const int64_t gr = level_base(N, 5) + (t0 >> 5);
        T *dst = which ? (T *)a.dv + b * a.dv_bs + gr * a.dv_rs + hoff : (T *)a.dk + b * a.dk_bs + gr * a.dk_rs + hoff;
        dst[col] = Traits<T>::from_f(sum);
    }
    // upper levels: the tile's partial rows go to the workspace
    for (int idx = tid; idx < nup * 2 * D; idx += 256) {
        const int u = idx / (2 * D), rem = idx % (2 * D);
        const int l = kTileLog + u;
        if (((t0 >> l) & 1) == 0) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) sum += persist[(size_t)(w * nps + 1 + u) * PR + rem];
        a.partial[((((size_t)b * a.H + h) * ntiles + tile) * nup + u) * 2 * D + rem] = sum;
    }
    // rows nobody attends to inside the tile: the right children of levels 1..5
    {
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
    int ntb, tree_rows, nup;
    int kb_off, vt_off, kt_off, q_off, go_off, stat_off, tiles_off, ttiles_off, persist_off, mbar_off;
    size_t smem;
    bool fits;
};

// Shared-memory plan.  Every buffer is NH = D/64 planes of [rows][128 B]: V band, K band, V tree, K tree, then Q, dOut.
static Bwd8Plan plan_bwd8(int N, int D) {
    Bwd8Plan p{};
    const int NH = D / 64;
    const size_t BP = (size_t)kBand8 * 128;
    const int L = ilog2((unsigned)N);
    p.nup = L - kTileLog;
    p.ntb = (3 + L + 15) / 16;
    p.tree_rows = kTreeIn8 + p.nup;
    const size_t TP = (size_t)p.tree_rows * 128;
    size_t off = 0;                                            // V band first: most of it is free after the first phase
    off += NH * BP;
    p.kb_off = (int)off; off += NH * BP;
    p.vt_off = (int)off; off += NH * TP;
    p.kt_off = (int)off; off += NH * TP;
    off = (off + 1023) / 1024 * 1024;
    const size_t alias_end = off;
    p.q_off = (int)off; off += NH * BP;
    p.go_off = (int)off; off += NH * BP;
    p.stat_off = (int)off; off += (size_t)2 * kBand8 * sizeof(float);
    off = (off + 15) / 16 * 16;
    p.tiles_off = (int)off; off += (size_t)17 * 512;
    p.mbar_off = (int)off; off += 32;
    p.smem = off + 1024;                                       // slack to put the first plane on a 1024-byte boundary
    // tree tiles reuse rows 16.. of the first V-band plane (its first 16 rows, in every plane, are still read by the
    // pair that reaches into the previous tile); the partial slots reuse what follows that plane
    p.ttiles_off = 16 * 128;
    p.persist_off = (int)BP;
    const size_t persist = (size_t)4 * (1 + p.nup) * (2 * D + 8) * sizeof(float);
    p.fits = p.ntb <= 2 && (size_t)p.ttiles_off + (size_t)p.ntb * 8 * 512 <= BP && (size_t)p.persist_off + persist <= alias_end;
    return p;
}

// The ten tensor maps of a call; the last sixteen results are kept per calling thread (a training loop calls with the
// same buffers again and again).
struct Bwd8MapKey {
    const void *ptr[4];
    int64_t stride[8];
    int B, N, H, D;
    bool operator==(const Bwd8MapKey &o) const {
        for (int i = 0; i < 4; ++i) if (ptr[i] != o.ptr[i]) return false;
        for (int i = 0; i < 8; ++i) if (stride[i] != o.stride[i]) return false;
        return B == o.B && N == o.N && H == o.H && D == o.D;
    }
};
static bool bwd8_maps(const hsa_view &Q, const hsa_view &K, const hsa_view &V, const hsa_view &dOut, int B, int N, int H, int D,
                      SpanBwd8Maps *out) {
    constexpr int kSlots = 16;                                 // a model's layers call with different buffers in turn
    thread_local Bwd8MapKey keys[kSlots] = {};
    thread_local SpanBwd8Maps cached[kSlots];
    thread_local bool valid[kSlots] = {};
    thread_local int next = 0;
    const Bwd8MapKey k{{Q.ptr, K.ptr, V.ptr, dOut.ptr},
                       {Q.batch_stride, Q.row_stride, K.batch_stride, K.row_stride, V.batch_stride, V.row_stride,
                        dOut.batch_stride, dOut.row_stride},
                       B, N, H, D};
    for (int i = 0; i < kSlots; ++i)
        if (valid[i] && keys[i] == k) { *out = cached[i]; return true; }
    SpanBwd8Maps m;
    const int R2 = 2 * N - 1;
    const bool ok = make_map(&m.q, Q, B, N, H, D, 1, kBand8) && make_map(&m.go, dOut, B, N, H, D, 1, kBand8) &&
                    make_map(&m.k_band, K, B, R2, H, D, 1, kBand8) && make_map(&m.v_band, V, B, R2, H, D, 1, kBand8) &&
                    make_map(&m.k_e4, K, B, R2, H, D, 2, 4) && make_map(&m.v_e4, V, B, R2, H, D, 2, 4) &&
                    make_map(&m.k_e2, K, B, R2, H, D, 2, 2) && make_map(&m.v_e2, V, B, R2, H, D, 2, 2) &&
                    make_map(&m.k_one, K, B, R2, H, D, 1, 1) && make_map(&m.v_one, V, B, R2, H, D, 1, 1);
    if (!ok) return false;
    const int slot = next;
    next = (next + 1) % kSlots;
    cached[slot] = m; keys[slot] = k; valid[slot] = true;
    *out = m;
    return true;
}

}  // namespace hsa

using namespace hsa;

// CTAs of the 8-warp backward whose bounded wait for their TMA copies ran out (read by hsa_span_attn_fwd_wait_expired)
int hsa_span_bwd8_wait_expired(unsigned int *count) {
    cudaError_t e = cudaMemcpyFromSymbol(count, g_bwd8_wait_expired, sizeof(unsigned int));
    return e == cudaSuccess ? 0 : fail((int)e, "hsa_span_attn_fwd_wait_expired: %s", cudaGetErrorString(e));
}

// Defined in span_attn_bwd_tc.cu: sums the tiles' partial rows of the nodes of level >= 6.
int hsa_span_bwd_upper_reduce(float *partial, void *dk, void *dv, int64_t dk_bs, int64_t dk_rs, int64_t dv_bs, int64_t dv_rs,
                              int B, int N, int H, int D, int causal, int dtype, cudaStream_t st);

bool hsa_span_attn_bwd_tc8_supported(const hsa_view *views, int nviews, int B, int N, int H, int D, int radius,
                                     int causal, int dtype) {
    if (dtype != HSA_BF16 && dtype != HSA_F16) return false;
    if (D != 64 && D != 128) return false;
    if (!causal || radius < 0 || radius > 16) return false;
    if (N < kTile || (N & (N - 1)) != 0 || N > (1 << 28)) return false;
    if (B < 1 || B > 65535 || H < 1 || H > 65535) return false;
    if ((int64_t)(N / kTile) * H * B > 0x7fffffffLL) return false;
    for (int i = 0; i < nviews; ++i)
        if (!view_vec_ok(views[i], 2)) return false;
    // views[]: Q, K, V, Out, dOut, dQ, dK, dV; the staged ones must be describable by tensor maps
    if (D >= 128 && (nviews < 5 || !map_ok(views[0], B, N, H, D) || !map_ok(views[4], B, N, H, D) ||
                     !map_ok(views[1], B, 2 * N - 1, H, D) || !map_ok(views[2], B, 2 * N - 1, H, D) || encode_tiled() == nullptr))
        return false;
    const Bwd8Plan p = plan_bwd8(N, D);
    // worth it only while two CTAs fit on an SM (227 KB, 1 KB of it reserved per CTA)
    return p.fits && p.smem <= 115200;
}

template <typename T, int D>
static int launch_bwd8(SpanBwd8Args &a, const SpanBwd8Maps &maps, const Bwd8Plan &p, int B, cudaStream_t st) {
    const int64_t total = (int64_t)B * (a.N / kTile) * a.H;
    cudaError_t e = cudaFuncSetAttribute(span_bwd_tc8_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
    if (e != cudaSuccess)
        return fail((int)e, "hsa_span_attn_bwd(tc8): shared memory %zu: %s", p.smem, cudaGetErrorString(e));
    span_bwd_tc8_kernel<T, D><<<(unsigned)total, 256, p.smem, st>>>(a, maps);
    return launch_status("hsa_span_attn_bwd(tc8)");
}

int hsa_span_attn_bwd_tc8(hsa_view Q, hsa_view K, hsa_view V, hsa_view Out, const float *LSE, hsa_view dOut, hsa_view dQ,
                          hsa_view dK, hsa_view dV, void *workspace, int B, int N, int H, int D, int radius, int causal,
                          int dtype, cudaStream_t st) {
    const hsa_view views[] = {Q, K, V, Out, dOut, dQ, dK, dV};
    if (!hsa_span_attn_bwd_tc8_supported(views, 8, B, N, H, D, radius, causal, dtype))
        return fail(HSA_ERR_ARG, "hsa_span_attn_bwd: shape not taken by the 8-warp tensor-core kernel");
    const Bwd8Plan p = plan_bwd8(N, D);
    SpanBwd8Args a{};
    a.q = Q.ptr; a.k = K.ptr; a.v = V.ptr; a.out = Out.ptr; a.go = dOut.ptr; a.lse = LSE;
    a.dq = dQ.ptr; a.dk = dK.ptr; a.dv = dV.ptr; a.partial = (float *)workspace;
    a.q_bs = Q.batch_stride; a.q_rs = Q.row_stride; a.k_bs = K.batch_stride; a.k_rs = K.row_stride;
    a.v_bs = V.batch_stride; a.v_rs = V.row_stride; a.o_bs = Out.batch_stride; a.o_rs = Out.row_stride;
    a.go_bs = dOut.batch_stride; a.go_rs = dOut.row_stride; a.dq_bs = dQ.batch_stride; a.dq_rs = dQ.row_stride;
    a.dk_bs = dK.batch_stride; a.dk_rs = dK.row_stride; a.dv_bs = dV.batch_stride; a.dv_rs = dV.row_stride;
    a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.R = radius < N ? radius : N;
    a.ntb = p.ntb; a.tree_rows = p.tree_rows;
    a.kb_off = p.kb_off; a.vt_off = p.vt_off; a.kt_off = p.kt_off; a.q_off = p.q_off; a.go_off = p.go_off;
    a.stat_off = p.stat_off; a.tiles_off = p.tiles_off; a.ttiles_off = p.ttiles_off; a.persist_off = p.persist_off;
    a.mbar_off = p.mbar_off;
    a.scale = 1.0f / sqrtf((float)D);
    a.scale_log2e = 1.4426950408889634f * a.scale;
    a.wait_limit = wait_limit_cycles();
    a.extra_tx = wait_extra_tx();
    SpanBwd8Maps maps{};                                       // only the 256-byte-row kernel stages by TMA
    if (D >= 128 && !bwd8_maps(Q, K, V, dOut, B, N, H, D, &maps))
        return fail(HSA_ERR_ARG, "hsa_span_attn_bwd(tc8): the driver refused a tensor map for these views");
    int rc;
    if (dtype == HSA_BF16)
        rc = D == 128 ? launch_bwd8<__nv_bfloat16, 128>(a, maps, p, B, st) : launch_bwd8<__nv_bfloat16, 64>(a, maps, p, B, st);
    else
        rc = D == 128 ? launch_bwd8<__half, 128>(a, maps, p, B, st) : launch_bwd8<__half, 64>(a, maps, p, B, st);
    if (rc) return rc;
    return hsa_span_bwd_upper_reduce((float *)workspace, dK.ptr, dV.ptr, dK.batch_stride, dK.row_stride, dV.batch_stride,
                                     dV.row_stride, B, N, H, D, causal, dtype, st);
}
