// The bottom-up parent refresh above a chosen level as ONE launch per tree (forward) and one for its backward.
//
// Level l of the refresh needs the level below it twice over: the children's keys/values are a projection
// (Wk_y, Wv_y) of the level-(l-1) outputs, and the parents' 3-way attention then reads those.  Run level by level
// this is two dependent launches per level and direction, and above the first few levels the launches are all
// fixed cost: a level has N/2^(l+1) parents per sequence.  Here a persistent grid (one CTA per SM, launched
// cooperatively so that all CTAs are resident) walks the levels itself:
//
//   forward, level l = start .. L-1
//     projection  KVc[rows of level l-1] = R[rows of level l-1] . [Wk_y; Wv_y]^T  (+ dropout of the value half)
//                 128 x 256 tiles on tcgen05 (accumulator in tensor memory, operands by TMA), tiles dealt round-robin
//     grid barrier
//     attention   R[parent] = softmax3(q.k_self, q.k_left, q.k_right) . (v_self, v_left, v_right), one lane group
//                 per (sequence, parent, head)
//     grid barrier
//   backward, level l = L-1 .. start
//     attention backward: dQ/dK/dV of the parents, dK/dV of the children (value half masked like the forward)
//     grid barrier
//     dR[rows of level l-1] += dKVc[rows of level l-1] . [Wk_y; Wv_y]     (float32 running sum + bfloat16 copy)
//     grid barrier
//
// (The weight gradient of the projection is not formed here: over all levels it is one product,
// dKVc^T . R, which the caller runs once.)  The grid barrier is an atomic counter in caller memory with a bounded
// wait: a CTA that waits longer than the limit writes a status word, and every CTA that sees a non-zero status
// leaves; the host reads the word with hsa_parent_tree_status.
#include <type_traits>

#include "hsa_common.cuh"
#include "rng_common.cuh"
#include "tc5_common.cuh"
#include "tma_common.cuh"

namespace hsa {

constexpr int kTreeThreads = 320;          // warp 0: TMA producer, warp 1: MMA issue, warps 2..9: epilogue; all: attention phases
constexpr int kTBN = 256, kTStages = 4;
constexpr int kTStage = 128 * 128 + kTBN * 128;      // A tile + B tile of one 64-wide K step

struct TreeArgs {
    // parents' projections (level slices are rows off(l) .. of [B, M, d] views)
    const __nv_bfloat16 *q, *k, *v;
    int64_t q_bs, q_rs, k_bs, k_rs, v_bs, v_rs;
    __nv_bfloat16 *R;  int64_t r_bs, r_rs;            // forward: refreshed parents [B, M, d];  backward: dR (bfloat16 copy)
    __nv_bfloat16 *C;  int64_t c_bs, c_rs;            // forward: child projections [B, M, 2d]; backward: the same, read only
    // backward only
    float *dRf;        int64_t f_bs, f_rs;            // float32 running gradient of R [B, M, d]
    __nv_bfloat16 *dq, *dk, *dv; int64_t dq_bs, dq_rs, dk_bs, dk_rs, dv_bs, dv_rs;
    __nv_bfloat16 *dC; int64_t dc_bs, dc_rs;          // gradient of the child projections [B, M, 2d]
    int B, N, L, H, D, d, start;
    const unsigned long long *rng;  unsigned int site, threshold;  float drop_scale;
    unsigned int *state;                               // [0] barrier counter (zero at launch), [1] status
    unsigned int extra_arrivals;                       // test hook: arrivals the barrier waits for but nobody makes
    long long wait_limit;
    float scale;                                       // 1 / sqrt(D)
};

__device__ __forceinline__ int tree_off(int N, int l) { return N - (N >> l); }     // first row of level l among the parents

// ---- grid barrier with a bounded wait.  Every thread of every CTA calls it; false = give up (status is set).
__device__ __forceinline__ bool tree_grid_sync(const TreeArgs &a, unsigned int &epoch, volatile int *abort_flag) {
    asm volatile("fence.proxy.async.global;\n" ::: "memory");       // rows written with plain stores are read by TMA next
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        epoch += 1;
        if (*abort_flag) {
            atomicMax(&a.state[1], 2u);
        } else {
            const unsigned int target = epoch * (gridDim.x + a.extra_arrivals);
            atomicAdd(&a.state[0], 1u);
            const long long t0 = clock64();
            while (true) {
                unsigned int seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(a.state) : "memory");
                if (seen >= target) break;
                unsigned int st;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(st) : "l"(a.state + 1) : "memory");
                if (st != 0) { *abort_flag = 1; break; }
                if (clock64() - t0 > a.wait_limit) { atomicMax(&a.state[1], 1u); *abort_flag = 1; break; }
            }
        }
        __threadfence();
    }
    __syncthreads();
    return *abort_flag == 0;
}

template <bool BWD>
__global__ void __launch_bounds__(kTreeThreads, 1)
parent_tree_kernel(const TreeArgs a, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b) {
    using namespace tc5;
    constexpr uint32_t IDESC = instr_desc(128, kTBN, true, false, BWD);      // backward reads the weights as [K, N]
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(smem + (size_t)kTStages * kTStage);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kTStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_addr(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (kTStages + s); };
    auto acc_full = [&](int i) { return bar0 + 8u * (2 * kTStages + i); };
    auto acc_empty = [&](int i) { return bar0 + 8u * (2 * kTStages + 2 + i); };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full(i), 1); mbar_init(acc_empty(i), 8); }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
    }
    if (warp == 1) tmem_alloc(smem_addr(tmem_slot), 2 * kTBN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int N = a.N, M = N - 1, d = a.d, H = a.H, D = a.D;
    // pipeline state of the three roles, carried from level to level
    int st_s = 0; uint32_t st_ph = 0;          // shared-memory stage ring (producer / MMA each keep their own copy)
    int st_acc = 0; uint32_t st_accph = 0;     // accumulator ring (MMA / epilogue)
    unsigned int epoch = 0;
    bool alive = true;

    // ---------------------------------------------------------------- the projection of one level's children rows
    // forward:  C[b, po + r, 0:2d] = R[b, po + r, :] . W^T          K = d,  N = 2d   (W stored [2d, d]: K-major)
    // backward: dRf[b, po + r, 0:d] += dC[b, po + r, :] . W          K = 2d, N = d    (W stored [2d, d] = [K, N])
    auto gemm_phase = [&](int po, int pp) {
        const int KD = BWD ? 2 * d : d, ND = BWD ? d : 2 * d;
        const int k_blocks = KD / 64, n_tiles = ND / kTBN, m_tiles = (pp + 127) / 128;
        const int total = a.B * m_tiles * n_tiles;
        if (warp == 0) {
            if (lane == 0) {
                for (int t = blockIdx.x; t < total && alive; t += gridDim.x) {
                    const int nt = t % n_tiles, mt = (t / n_tiles) % m_tiles, b = t / (n_tiles * m_tiles);
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!(alive = mbar_wait(empty(st_s), st_ph ^ 1, a.wait_limit, abort_flag))) break;
                        mbar_expect_tx(full(st_s), kTStage);
                        const uint32_t sa = smem_addr(smem + (size_t)st_s * kTStage), sb = sa + 128 * 128;
                        tma_load_3d(sa, &map_a, kb * 64, po + mt * 128, b, full(st_s));
                        if constexpr (!BWD) {
                            tma_load_3d(sb, &map_b, kb * 64, nt * kTBN, 0, full(st_s));
                        } else {
#pragma unroll
                            for (int p = 0; p < kTBN / 64; ++p) tma_load_3d(sb + p * 8192, &map_b, nt * kTBN + p * 64, kb * 64, 0, full(st_s));
                        }
                        if (++st_s == kTStages) { st_s = 0; st_ph ^= 1; }
                    }
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                for (int t = blockIdx.x; t < total && alive; t += gridDim.x) {
                    if (!(alive = mbar_wait(acc_empty(st_acc), st_accph ^ 1, a.wait_limit, abort_flag))) break;
                    fence_after_sync();
                    const uint32_t dt = tmem_base + st_acc * kTBN;
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!(alive = mbar_wait(full(st_s), st_ph, a.wait_limit, abort_flag))) break;
                        fence_after_sync();
                        const uint32_t sa = smem_addr(smem + (size_t)st_s * kTStage), sb = sa + 128 * 128;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t da = smem_desc(sa + k * 32, 16, 1024);
                            const uint64_t db = BWD ? smem_desc(sb + k * 2048, 8192, 1024) : smem_desc(sb + k * 32, 16, 1024);
                            mma_f16(dt, da, db, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                        mma_commit(empty(st_s));
                        if (++st_s == kTStages) { st_s = 0; st_ph ^= 1; }
                    }
                    if (!alive) break;
                    mma_commit(acc_full(st_acc));
                    if (++st_acc == 2) { st_acc = 0; st_accph ^= 1; }
                }
            }
        } else {
            const int q4 = warp & 3, col_lo = ((warp - 2) >> 2) * (kTBN / 2);
            for (int t = blockIdx.x; t < total && alive; t += gridDim.x) {
                const int nt = t % n_tiles, mt = (t / n_tiles) % m_tiles, b = t / (n_tiles * m_tiles);
                alive = mbar_wait(acc_full(st_acc), st_accph, a.wait_limit, abort_flag);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                fence_after_sync();
                const int r = mt * 128 + q4 * 32 + lane;                    // row inside the level's children
                const bool row_ok = r < pp;
                const uint32_t tbase = tmem_base + st_acc * kTBN + ((uint32_t)(q4 * 32) << 16);
#pragma unroll 1
                for (int c0 = col_lo; c0 < col_lo + kTBN / 2; c0 += 32) {
                    uint32_t rr[32];
                    tmem_ld32(tbase + c0, rr);
                    tmem_ld_wait();
                    if (!row_ok) continue;
                    const int col = nt * kTBN + c0;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(rr[i]);
                    if constexpr (!BWD) {
                        if (a.rng != nullptr && col >= d) {                 // the value half: dropout, ids of the [B, M, 2d] tensor
                            const unsigned long long key = *a.rng;
                            const unsigned long long id0 = ((unsigned long long)b * M + (unsigned long long)(po + r)) * (2ull * d) + col;
                            dropout_run(v, dropout_salt(key, a.site, 0), 0u, false, id0, a.threshold, a.drop_scale);
                        }
                        __nv_bfloat16 *dst = a.C + b * a.c_bs + (int64_t)(po + r) * a.c_rs + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 o;
                            __nv_bfloat162 *p2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                            for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                            *reinterpret_cast<uint4 *>(dst + i) = o;
                        }
                    } else {
                        float *fd = a.dRf + b * a.f_bs + (int64_t)(po + r) * a.f_rs + col;
                        __nv_bfloat16 *bd = a.R + b * a.r_bs + (int64_t)(po + r) * a.r_rs + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const float4 old = *reinterpret_cast<const float4 *>(fd + i);
                            v[i] += old.x; v[i + 1] += old.y; v[i + 2] += old.z; v[i + 3] += old.w;
                            *reinterpret_cast<float4 *>(fd + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        }
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 o;
                            __nv_bfloat162 *p2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                            for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                            *reinterpret_cast<uint4 *>(bd + i) = o;
                        }
                    }
                }
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(st_acc));
                if (++st_acc == 2) { st_acc = 0; st_accph ^= 1; }
            }
        }
    };

    // ---------------------------------------------------------------- the 3-way attention of one level (all threads)
    // LPR lanes per (sequence, parent, head), 16 bytes of the head dimension per lane.
    auto attention_phase = [&](auto lpr_tag, int lvl) {
        constexpr int LPR = decltype(lpr_tag)::value;
        using Frag = RowFrag<__nv_bfloat16, 8, LPR, 1>;
        const int P = N >> (lvl + 1), off = tree_off(N, lvl), po = tree_off(N, lvl - 1);
        const int g = threadIdx.x % LPR;
        const int groups = kTreeThreads / LPR;
        const long long items = (long long)a.B * P * H;
        const unsigned mask = group_mask<LPR>();
        for (long long base = (long long)blockIdx.x * groups; base < items; base += (long long)gridDim.x * groups) {
            const long long it = base + threadIdx.x / LPR;
            const bool active = it < items;
            const long long gi = active ? it : items - 1;
            const int h = (int)(gi % H), p = (int)((gi / H) % P), b = (int)(gi / ((long long)H * P));
            const int64_t hoff = (int64_t)h * D;
            const int64_t prow = off + p, c0 = po + 2 * (int64_t)p, c1 = c0 + 1;
            const __nv_bfloat16 *kc = a.C + b * a.c_bs + hoff, *vc = kc + d;
            Frag q, k0, k1, k2;
            q.load(a.q + b * a.q_bs + prow * a.q_rs + hoff, g, D / 8);
            k0.load(a.k + b * a.k_bs + prow * a.k_rs + hoff, g, D / 8);
            k1.load(kc + c0 * a.c_rs, g, D / 8);
            k2.load(kc + c1 * a.c_rs, g, D / 8);
            float s0 = q.dot_partial(k0), s1 = q.dot_partial(k1), s2 = q.dot_partial(k2);
            if constexpr (!BWD) {
                Frag v0, v1, v2;
                v0.load(a.v + b * a.v_bs + prow * a.v_rs + hoff, g, D / 8);
                v1.load(vc + c0 * a.c_rs, g, D / 8);
                v2.load(vc + c1 * a.c_rs, g, D / 8);
                s0 = group_sum<LPR>(s0, mask) * a.scale;
                s1 = group_sum<LPR>(s1, mask) * a.scale;
                s2 = group_sum<LPR>(s2, mask) * a.scale;
                const float m = fmaxf(s0, fmaxf(s1, s2));
                const float e0 = __expf(s0 - m), e1 = __expf(s1 - m), e2 = __expf(s2 - m);
                const float inv = 1.f / (e0 + e1 + e2);
                Frag o;
                o.zero();
                o.axpy(e0 * inv, v0);
                o.axpy(e1 * inv, v1);
                o.axpy(e2 * inv, v2);
                if (active) o.store(a.R + b * a.r_bs + prow * a.r_rs + hoff, g, D / 8);
            } else {
                Frag go, v;
                go.load(a.R + b * a.r_bs + prow * a.r_rs + hoff, g, D / 8);            // backward: R holds the bfloat16 dR
                v.load(a.v + b * a.v_bs + prow * a.v_rs + hoff, g, D / 8);
                float dp0 = go.dot_partial(v);
                v.load(vc + c0 * a.c_rs, g, D / 8);
                float dp1 = go.dot_partial(v);
                v.load(vc + c1 * a.c_rs, g, D / 8);
                float dp2 = go.dot_partial(v);
                s0 = group_sum<LPR>(s0, mask) * a.scale;
                s1 = group_sum<LPR>(s1, mask) * a.scale;
                s2 = group_sum<LPR>(s2, mask) * a.scale;
                dp0 = group_sum<LPR>(dp0, mask);
                dp1 = group_sum<LPR>(dp1, mask);
                dp2 = group_sum<LPR>(dp2, mask);
                const float m = fmaxf(s0, fmaxf(s1, s2));
                const float e0 = __expf(s0 - m), e1 = __expf(s1 - m), e2 = __expf(s2 - m);
                const float inv = 1.f / (e0 + e1 + e2);
                const float w0 = e0 * inv, w1 = e1 * inv, w2 = e2 * inv;
                const float delta = w0 * dp0 + w1 * dp1 + w2 * dp2;
                const float ds0 = w0 * (dp0 - delta) * a.scale, ds1 = w1 * (dp1 - delta) * a.scale, ds2 = w2 * (dp2 - delta) * a.scale;
                if (active) {
                    Frag t;
                    t = go; t.scale(w0); t.store(a.dv + b * a.dv_bs + prow * a.dv_rs + hoff, g, D / 8);
                    // the children's values went through dropout in the forward: the same mask on their gradient
                    __nv_bfloat16 *dkc = a.dC + b * a.dc_bs + hoff, *dvc = dkc + d;
                    auto masked_store = [&](float w, int64_t crow) {
                        t = go; t.scale(w);
                        if (a.rng != nullptr) {
                            const unsigned long long key = *a.rng;
                            const unsigned long long id0 = ((unsigned long long)b * M + (unsigned long long)crow) * (2ull * d) + d + hoff + 8 * g;
                            dropout_run(t.v[0], dropout_salt(key, a.site, 0), 0u, false, id0, a.threshold, a.drop_scale);
                        }
                        t.store(dvc + crow * a.dc_rs, g, D / 8);
                    };
                    masked_store(w1, c0);
                    masked_store(w2, c1);
                    t.zero(); t.axpy(ds0, k0); t.axpy(ds1, k1); t.axpy(ds2, k2);
                    t.store(a.dq + b * a.dq_bs + prow * a.dq_rs + hoff, g, D / 8);
                    t = q; t.scale(ds0); t.store(a.dk + b * a.dk_bs + prow * a.dk_rs + hoff, g, D / 8);
                    t = q; t.scale(ds1); t.store(dkc + c0 * a.dc_rs, g, D / 8);
                    t = q; t.scale(ds2); t.store(dkc + c1 * a.dc_rs, g, D / 8);
                }
            }
        }
    };
    auto attention = [&](int lvl) {
        if (D == 64) attention_phase(std::integral_constant<int, 8>{}, lvl);
        else attention_phase(std::integral_constant<int, 16>{}, lvl);
    };

    if constexpr (!BWD) {
        for (int lvl = a.start; lvl < a.L && alive; ++lvl) {
            gemm_phase(tree_off(N, lvl - 1), N >> lvl);
            if (!(alive = tree_grid_sync(a, epoch, abort_flag))) break;
            attention(lvl);
            alive = tree_grid_sync(a, epoch, abort_flag);
        }
    } else {
        for (int lvl = a.L - 1; lvl >= a.start && alive; --lvl) {
            attention(lvl);
            if (!(alive = tree_grid_sync(a, epoch, abort_flag))) break;
            gemm_phase(tree_off(N, lvl - 1), N >> lvl);
            alive = tree_grid_sync(a, epoch, abort_flag);
        }
    }

    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc(tmem_base, 2 * kTBN);
    }
}

static bool tree_map(CUtensorMap *m, const void *ptr, int64_t inner, int64_t rows, int64_t batches, int64_t row_stride,
                     int64_t batch_stride, int box_rows) {
    if (encode_tiled() == nullptr) return false;
    if (batches == 1) batch_stride = rows * row_stride;
    const cuuint64_t gdim[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t gstride[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)batch_stride * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    const cuuint32_t estride[3] = {1u, 1u, 1u};
    return encode_tiled()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool BWD>
static int launch_tree(TreeArgs &a, const CUtensorMap &ma, const CUtensorMap &mb, cudaStream_t st) {
    const size_t smem = (size_t)kTStages * kTStage + (2 * kTStages + 4) * 8 + 16 + 1024;
    auto kernel = parent_tree_kernel<BWD>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail((int)e, "hsa_parent_tree: shared memory %zu: %s", smem, cudaGetErrorString(e));
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kTreeThreads, smem);
    if (e != cudaSuccess || per_sm < 1 || sms < 1)
        return fail(e != cudaSuccess ? (int)e : HSA_ERR_ARG, "hsa_parent_tree: the kernel does not fit an SM");
    // all CTAs have to be resident for the grid barrier: a cooperative launch guarantees it or fails
    e = cudaMemsetAsync(a.state, 0, 2 * sizeof(unsigned int), st);
    if (e != cudaSuccess) return fail((int)e, "hsa_parent_tree: clearing the barrier state: %s", cudaGetErrorString(e));
    void *params[] = {(void *)&a, (void *)&ma, (void *)&mb};
    e = cudaLaunchCooperativeKernel((const void *)kernel, dim3((unsigned)sms), dim3(kTreeThreads), params, smem, st);
    if (e != cudaSuccess) return fail((int)e, "hsa_parent_tree: cooperative launch: %s", cudaGetErrorString(e));
    return launch_status("hsa_parent_tree");
}

static int tree_check(const char *what, int B, int N, int H, int D, int start) {
    HSA_CHECK_ARG(B >= 1 && N >= 4 && (N & (N - 1)) == 0 && H >= 1 && (D == 64 || D == 128), "%s: bad shape B=%d N=%d H=%d D=%d (head dim 64 or 128)",
                  what, B, N, H, D);
    HSA_CHECK_ARG((H * D) % 256 == 0, "%s: the model width H*D = %d must be a multiple of 256", what, H * D);
    HSA_CHECK_ARG(start >= 1 && start < ilog2((unsigned)N), "%s: start_level %d outside [1, log2 N)", what, start);
    HSA_CHECK_ARG((unsigned long long)B * (unsigned long long)(N - 1) * 2ull * (unsigned long long)(H * D) <= kDropoutRunMaxElems,
                  "%s: more than 2^33 child K/V elements", what);
    return 0;
}

}  // namespace hsa

using namespace hsa;

extern "C" size_t hsa_parent_tree_state_bytes(void) { return 256; }

extern "C" int hsa_parent_tree_status(const void *state, unsigned int *status) {
    if (state == nullptr || status == nullptr) return fail(HSA_ERR_ARG, "hsa_parent_tree_status: null pointer");
    cudaError_t e = cudaMemcpy(status, (const unsigned int *)state + 1, sizeof(unsigned int), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? 0 : fail((int)e, "hsa_parent_tree_status: %s", cudaGetErrorString(e));
}

extern "C" int hsa_parent_tree_fwd(hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view R, hsa_view KVc, const void *Wkv, int B, int N,
                                   int H, int D, int start_level, const unsigned long long *rng_state, unsigned int site,
                                   unsigned int threshold, float drop_scale, void *state, void *stream) {
    HSA_CHECK_ARG(Qp.ptr && Kp.ptr && Vp.ptr && R.ptr && KVc.ptr && Wkv && state, "hsa_parent_tree_fwd: null pointer");
    if (int rc = tree_check("hsa_parent_tree_fwd", B, N, H, D, start_level)) return rc;
    const int d = H * D, M = N - 1;
    const hsa_view *vs[] = {&Qp, &Kp, &Vp, &R, &KVc};
    for (const hsa_view *v : vs)
        if (!view_vec_ok(*v, 2)) return fail(HSA_ERR_ALIGN, "hsa_parent_tree_fwd: views must be 16-byte aligned");
    TreeArgs a{};
    a.q = (const __nv_bfloat16 *)Qp.ptr; a.k = (const __nv_bfloat16 *)Kp.ptr; a.v = (const __nv_bfloat16 *)Vp.ptr;
    a.q_bs = Qp.batch_stride; a.q_rs = Qp.row_stride; a.k_bs = Kp.batch_stride; a.k_rs = Kp.row_stride;
    a.v_bs = Vp.batch_stride; a.v_rs = Vp.row_stride;
    a.R = (__nv_bfloat16 *)R.ptr; a.r_bs = R.batch_stride; a.r_rs = R.row_stride;
    a.C = (__nv_bfloat16 *)KVc.ptr; a.c_bs = KVc.batch_stride; a.c_rs = KVc.row_stride;
    a.B = B; a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.D = D; a.d = d; a.start = start_level;
    a.rng = rng_state; a.site = site; a.threshold = threshold; a.drop_scale = drop_scale;
    a.state = (unsigned int *)state; a.extra_arrivals = wait_extra_tx() ? 1u : 0u; a.wait_limit = wait_limit_cycles();
    a.scale = 1.0f / sqrtf((float)D);
    CUtensorMap ma, mb;
    if (!tree_map(&ma, R.ptr, d, M, B, R.row_stride, R.batch_stride, 128) || !tree_map(&mb, Wkv, d, 2 * d, 1, d, 0, kTBN))
        return fail(HSA_ERR_ARG, "hsa_parent_tree_fwd: the driver refused a tensor map for these views");
    return launch_tree<false>(a, ma, mb, (cudaStream_t)stream);
}

extern "C" int hsa_parent_tree_bwd(hsa_view Qp, hsa_view Kp, hsa_view Vp, hsa_view KVc, hsa_view dRf, hsa_view dRb, hsa_view dQp,
                                   hsa_view dKp, hsa_view dVp, hsa_view dKVc, const void *Wkv, int B, int N, int H, int D,
                                   int start_level, const unsigned long long *rng_state, unsigned int site,
                                   unsigned int threshold, float drop_scale, void *state, void *stream) {
    HSA_CHECK_ARG(Qp.ptr && Kp.ptr && Vp.ptr && KVc.ptr && dRf.ptr && dRb.ptr && dQp.ptr && dKp.ptr && dVp.ptr && dKVc.ptr && Wkv && state,
                  "hsa_parent_tree_bwd: null pointer");
    if (int rc = tree_check("hsa_parent_tree_bwd", B, N, H, D, start_level)) return rc;
    const int d = H * D, M = N - 1;
    const hsa_view *vs[] = {&Qp, &Kp, &Vp, &KVc, &dRb, &dQp, &dKp, &dVp, &dKVc};
    for (const hsa_view *v : vs)
        if (!view_vec_ok(*v, 2)) return fail(HSA_ERR_ALIGN, "hsa_parent_tree_bwd: views must be 16-byte aligned");
    if (!view_vec_ok(dRf, 4)) return fail(HSA_ERR_ALIGN, "hsa_parent_tree_bwd: dRf must be 16-byte aligned");
    TreeArgs a{};
    a.q = (const __nv_bfloat16 *)Qp.ptr; a.k = (const __nv_bfloat16 *)Kp.ptr; a.v = (const __nv_bfloat16 *)Vp.ptr;
    a.q_bs = Qp.batch_stride; a.q_rs = Qp.row_stride; a.k_bs = Kp.batch_stride; a.k_rs = Kp.row_stride;
    a.v_bs = Vp.batch_stride; a.v_rs = Vp.row_stride;
    a.R = (__nv_bfloat16 *)dRb.ptr; a.r_bs = dRb.batch_stride; a.r_rs = dRb.row_stride;
    a.C = (__nv_bfloat16 *)KVc.ptr; a.c_bs = KVc.batch_stride; a.c_rs = KVc.row_stride;
    a.dRf = (float *)dRf.ptr; a.f_bs = dRf.batch_stride; a.f_rs = dRf.row_stride;
    a.dq = (__nv_bfloat16 *)dQp.ptr; a.dq_bs = dQp.batch_stride; a.dq_rs = dQp.row_stride;
    a.dk = (__nv_bfloat16 *)dKp.ptr; a.dk_bs = dKp.batch_stride; a.dk_rs = dKp.row_stride;
    a.dv = (__nv_bfloat16 *)dVp.ptr; a.dv_bs = dVp.batch_stride; a.dv_rs = dVp.row_stride;
    a.dC = (__nv_bfloat16 *)dKVc.ptr; a.dc_bs = dKVc.batch_stride; a.dc_rs = dKVc.row_stride;
    a.B = B; a.N = N; a.L = ilog2((unsigned)N); a.H = H; a.D = D; a.d = d; a.start = start_level;
    a.rng = rng_state; a.site = site; a.threshold = threshold; a.drop_scale = drop_scale;
    a.state = (unsigned int *)state; a.extra_arrivals = wait_extra_tx() ? 1u : 0u; a.wait_limit = wait_limit_cycles();
    a.scale = 1.0f / sqrtf((float)D);
    CUtensorMap ma, mb;
    // A = dKVc rows (K = 2d); B = the weights read as [K = 2d, N = d]: boxes of 64 columns x 64 rows
    if (!tree_map(&ma, dKVc.ptr, 2 * d, M, B, dKVc.row_stride, dKVc.batch_stride, 128) || !tree_map(&mb, Wkv, d, 2 * d, 1, d, 0, 64))
        return fail(HSA_ERR_ARG, "hsa_parent_tree_bwd: the driver refused a tensor map for these views");
    return launch_tree<true>(a, ma, mb, (cudaStream_t)stream);
}
