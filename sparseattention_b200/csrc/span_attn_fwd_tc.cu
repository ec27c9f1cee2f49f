// Span attention forward on tensor cores (bf16 / f16, head dim 64 or 128, N >= 64).
//
// One CTA = one (batch, head, aligned tile of 64 leaves), 4 warps of 16 leaves each.
// The tile's whole key/value working set is staged in shared memory ONCE, into [128-byte half][row][128 B]
// planes with the 128-byte XOR swizzle of the TMA unit — by cp.async.bulk.tensor boxes (one per thread,
// bounded mbarrier waits) when rows are 256 bytes, by per-thread 16-byte cp.async when they are 128 bytes:
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
#include "tma_common.cuh"

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
    int band_box;    // rows per TMA box of the leaf band (the whole band when it fits one box)
    float scale_log2e;
    long long wait_limit;      // cycles a CTA waits for its bulk copies
    unsigned int extra_tx;     // 0 except in the test of the give-up path
};

// Tensor maps of one tensor (K or V), all over [B, rows, H, D] with a box of 64 elements of one head:
// band: every row, box of band_box rows; lv[l-1]: the box of the in-tile nodes of level l = 1..5 (causal: every second
// row, 32 >> l rows; else every row, 64 >> l rows); one: every row, box of one row.
struct SpanTcMaps {
    CUtensorMap band, lv[5], one;
};

// CTAs whose wait for their TMA copies ran out (never expected; added to what hsa_span_attn_fwd_wait_expired reports)
__device__ unsigned int g_fwd64_wait_expired = 0;

template <typename T, int D, bool CAUSAL>
__global__ void __launch_bounds__(128, 3)
span_fwd_tc_kernel(const SpanTcArgs a, const __grid_constant__ SpanTcMaps kmaps, const __grid_constant__ SpanTcMaps vmaps) {
    constexpr int NH = D / 64;                 // 128-byte halves of a row
    constexpr bool TMA = D >= 128;             // 128-byte rows: the boxes get too small to pay off
    constexpr int OPITCH = D * 2 + 16;         // pitch of the output rows parked in shared memory (conflict-free skew)
    constexpr int CPR = D / 8;                 // 16-byte chunks per row
    constexpr int RPI = 128 / CPR;             // rows staged per pass of the CTA
    constexpr int KS = D / 16;                 // k-steps of the QK^T product
    constexpr int TIN = tree_in_rows<CAUSAL>();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
    const int PS = a.kv_rows * 128;            // bytes of one plane
    unsigned char *Ks = smem;                  // [NH][kv_rows][128 B]
    unsigned char *Vs = Ks + (size_t)NH * PS;
    unsigned long long *mbar = reinterpret_cast<unsigned long long *>(Vs + (size_t)NH * PS);

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
    // Rows nobody may attend to are loaded all the same (upper levels on the causal side) or zero-filled (before the
    // first leaf), so masked scores and 0 * V products stay finite.
    const uint32_t mbK = smem_u32(&mbar[0]), mbV = smem_u32(&mbar[1]);
    auto wait_group = [&](int g) -> bool {                       // 0: K, 1: V
        if constexpr (TMA) {
            return mbar_wait_phase0(g == 0 ? mbK : mbV, a.wait_limit);
        } else {
            if (g == 0) cp_async_wait<1>(); else cp_async_wait<0>();
            return true;
        }
    };
    if constexpr (TMA) {
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbK), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbV), "r"(1) : "memory");
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        __syncthreads();
        if (tid == 0) {
            const uint32_t bytes = (uint32_t)PS * NH;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbK), "r"(bytes + a.extra_tx) : "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbV), "r"(bytes) : "memory");
        }
        // boxes of one tensor and half: band_rows / 16 band boxes, one box per level 1..5, one node per upper level
        const int nband = a.band_rows / a.band_box;
        const int per = nband + 5 + (L - kTileLog);
        for (int t = tid; t < 2 * NH * per; t += 128) {
            const int isv = t / (NH * per), rem = t % (NH * per);     // K boxes first
            const int hf = rem / per, j = rem % per;
            const SpanTcMaps &maps = isv ? vmaps : kmaps;
            const CUtensorMap *map;
            int row, dst_row;
            if (j < nband) {
                map = &maps.band; row = band_lo + a.band_box * j; dst_row = a.band_box * j;
            } else if (j < nband + 5) {
                const int l = j - nband + 1;
                map = &maps.lv[l - 1];
                row = level_base(N, l) + (t0 >> l);
                if (CAUSAL) row >>= 1;                                 // index among the even rows
                dst_row = a.band_rows + tree_level_off<CAUSAL>(l);
            } else {
                const int l = kTileLog + (j - nband - 5);
                map = &maps.one; row = level_base(N, l) + ((t0 >> l) ^ 1); dst_row = a.band_rows + TIN + (l - kTileLog);
            }
            const uint32_t dst = smem_u32((isv ? Vs : Ks) + (size_t)hf * PS + (size_t)dst_row * 128);
            asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
                         ::"r"(dst), "l"(map), "r"(64 * hf), "r"(h), "r"(row), "r"(b), "r"(isv ? mbV : mbK) : "memory");
        }
    } else {
        const int c = tid % CPR, rg = tid / CPR;
        const int ntree = TIN + (L - kTileLog);
        auto put = [&](unsigned char *S, int row, const T *src, bool ok) {
            const uint32_t ra = smem_u32(S + (size_t)row * 128);
            cp_async16(ra + (((c ^ (ra >> 7)) & 7) << 4), src, ok);
        };
        auto stage_kv = [&](const T *g, int64_t rs, unsigned char *S) {
            const T *gc = g + c * 8;
            for (int i = rg; i < a.band_rows; i += RPI) {
                const int r = band_lo + i;
                const bool ok = (unsigned)r < (unsigned)N;
                put(S, i, gc + (int64_t)(ok ? r : 0) * rs, ok);
            }
            for (int f = rg; f < ntree; f += RPI) {
                int rr;
                if (f < TIN) {
                    const int rem = (CAUSAL ? 32 : 64) - f;
                    const int l = (CAUSAL ? 5 : 6) - (31 - __clz(rem - 1));
                    const int i = f - tree_level_off<CAUSAL>(l);
                    rr = level_base(N, l) + (t0 >> l) + (CAUSAL ? 2 * i : i);
                } else {
                    const int l = kTileLog + (f - TIN);
                    rr = level_base(N, l) + ((t0 >> l) ^ 1);
                }
                put(S, a.band_rows + f, gc + (int64_t)rr * rs, true);
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

    // What a CTA does when a wait runs out: count itself, leave NaN in its output rows, and go.
    auto give_up = [&]() {
        if (tid == 0) atomicAdd(&g_fwd64_wait_expired, 1u);
        fill_rows_nan16((T *)a.out + b * a.o_bs + hoff + (int64_t)t0 * a.o_rs, a.o_rs, kTile, D, tid, 128);
        if (a.lse != nullptr && tid < kTile) a.lse[((int64_t)b * a.N + t0 + tid) * a.H + h] = __int_as_float(0x7fffffff);
    };
    if (!__syncthreads_and(wait_group(0))) {             // K has landed (the wait is not expected to give up)
        wait_group(1);                                    // a second bounded chance for this CTA's copies to finish
        give_up();
        return;
    }

    // A row of K or V for ldmatrix: per 128-byte half its shared address and the lane's piece parity folded into the
    // row's swizzle (address bits 7..9)
    struct RowRef { uint32_t addr[NH]; int x[NH]; };
    auto row_ref = [&](const unsigned char *X, int row, int parity) {
        RowRef r;
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) {
            r.addr[hf] = smem_u32(X + (size_t)hf * PS + (size_t)row * 128);
            r.x[hf] = (parity ^ (r.addr[hf] >> 7)) & 7;
        }
        return r;
    };
    auto piece_addr = [&](const RowRef &r, int pe) { return r.addr[pe >> 3] + (uint32_t)(((pe & 7) ^ r.x[pe >> 3]) << 4); };

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
                const RowRef kb = row_ref(Ks, krow, (lane >> 3) & 1);
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, piece_addr(kb, 2 * ks));
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
        if (c0 == 0 && !__syncthreads_and(wait_group(1))) {        // V has landed
            give_up();
            return;
        }
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
                const RowRef vb = row_ref(Vs, vrow, lane >> 4);
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, piece_addr(vb, 2 * dp));
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
    unsigned char *Os = Ks + lw * OPITCH;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        const int col = nt * 8 + 2 * quad;
        *reinterpret_cast<uint32_t *>(Os + qrow * OPITCH + col * 2) = pack2<T>(o[nt][0] * i0, o[nt][1] * i0);
        *reinterpret_cast<uint32_t *>(Os + (qrow + 8) * OPITCH + col * 2) = pack2<T>(o[nt][2] * i1, o[nt][3] * i1);
    }
    __syncwarp();
    T *og = (T *)a.out + b * a.o_bs + hoff;
#pragma unroll
    for (int it = 0; it < (16 * CPR) / 32; ++it) {
        const int idx = it * 32 + lane;
        const int r = idx / CPR, c = idx % CPR;
        const uint4 val = *reinterpret_cast<const uint4 *>(Os + r * OPITCH + c * 16);
        *reinterpret_cast<uint4 *>(og + (int64_t)(t0 + lw + r) * a.o_rs + c * 8) = val;
    }
}

static size_t smem_bytes_tc(int D, int kv_rows) {            // planes of K and V, two mbarriers, alignment slack
    return (size_t)2 * (D / 64) * kv_rows * 128 + 16 + 128;
}

// The seven maps of one tensor; the last results are kept per calling thread.
struct TcMapKey {
    const void *ptr;
    int64_t bs, rs;
    int B, rows, H, D, causal, band_box;
    bool operator==(const TcMapKey &o) const {
        return ptr == o.ptr && bs == o.bs && rs == o.rs && B == o.B && rows == o.rows && H == o.H && D == o.D && causal == o.causal &&
               band_box == o.band_box;
    }
};
static bool tc_tensor_maps(const hsa_view &v, int B, int N, int H, int D, bool causal, int band_box, SpanTcMaps *out) {
    constexpr int kSlots = 32;
    thread_local TcMapKey keys[kSlots] = {};
    thread_local SpanTcMaps cached[kSlots];
    thread_local bool valid[kSlots] = {};
    thread_local int next = 0;
    const TcMapKey key{v.ptr, v.batch_stride, v.row_stride, B, 2 * N - 1, H, D, causal ? 1 : 0, band_box};
    for (int i = 0; i < kSlots; ++i)
        if (valid[i] && keys[i] == key) { *out = cached[i]; return true; }
    SpanTcMaps m;
    bool ok = make_map(&m.band, v, B, 2 * N - 1, H, D, 1, band_box) && make_map(&m.one, v, B, 2 * N - 1, H, D, 1, 1);
    for (int l = 1; l <= 5 && ok; ++l)
        ok = causal ? make_map(&m.lv[l - 1], v, B, 2 * N - 1, H, D, 2, 32 >> l) : make_map(&m.lv[l - 1], v, B, 2 * N - 1, H, D, 1, 64 >> l);
    if (!ok) return false;
    const int slot = next;
    next = (next + 1) % kSlots;
    cached[slot] = m; keys[slot] = key; valid[slot] = true;
    *out = m;
    return true;
}

template <typename T, int D>
static int launch_tc(const SpanTcArgs &a, const SpanTcMaps &km, const SpanTcMaps &vm, int B, bool causal, cudaStream_t st) {
    const size_t smem = smem_bytes_tc(D, a.kv_rows);
    const int64_t total = (int64_t)B * (a.N / kTile) * a.H;
    auto go = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "hsa_span_attn_fwd(tc): shared memory %zu: %s", smem, cudaGetErrorString(e));
        kernel<<<(unsigned)total, 128, smem, st>>>(a, km, vm);
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
    if (D >= 128 && (!map_ok(K, B, 2 * N - 1, H, D) || !map_ok(V, B, 2 * N - 1, H, D) || encode_tiled() == nullptr)) return false;
    return smem_bytes_tc(D, kv) <= 200 * 1024;
}

// CTAs of this kernel whose bounded wait for their TMA copies ran out (read by hsa_span_attn_fwd_wait_expired)
int hsa_span_fwd64_wait_expired(unsigned int *count) {
    cudaError_t e = cudaMemcpyFromSymbol(count, g_fwd64_wait_expired, sizeof(unsigned int));
    return e == cudaSuccess ? 0 : fail((int)e, "hsa_span_attn_fwd_wait_expired: %s", cudaGetErrorString(e));
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
    a.band_box = a.band_rows <= 256 ? a.band_rows : 16;
    a.scale_log2e = 1.4426950408889634f / sqrtf((float)D);
    a.wait_limit = wait_limit_cycles();
    a.extra_tx = wait_extra_tx();
    SpanTcMaps km{}, vm{};                                     // only the 256-byte-row kernel stages by TMA
    if (D >= 128 && (!tc_tensor_maps(K, B, N, H, D, causal != 0, a.band_box, &km) || !tc_tensor_maps(V, B, N, H, D, causal != 0, a.band_box, &vm)))
        return fail(HSA_ERR_ARG, "hsa_span_attn_fwd(tc): the driver refused a tensor map for these views");
    if (dtype == HSA_BF16)
        return D == 128 ? launch_tc<__nv_bfloat16, 128>(a, km, vm, B, causal != 0, st) : launch_tc<__nv_bfloat16, 64>(a, km, vm, B, causal != 0, st);
    return D == 128 ? launch_tc<__half, 128>(a, km, vm, B, causal != 0, st) : launch_tc<__half, 64>(a, km, vm, B, causal != 0, st);
}
