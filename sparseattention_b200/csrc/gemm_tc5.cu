// Dense bf16 / f16 matrix products on the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor
// memory), for the contractions of the attention layer and of the language model around it that share one dense
// operand: the Q/K/V and output projections, the feed-forward pair and the LM head, forward and backward.
//
//   C[b, m, n] (+)= sum_k A[b, m, k] * B[n, k]  (+ bias[n])
//
// Persistent kernel, one CTA per SM, 10 warps with fixed roles:
//   warp 0   producer: one thread issues the TMA tile loads of a stage (A box(es), B box(es)) onto its "full" mbarrier
//   warp 1   one thread issues tcgen05.mma for the stage (four K=16 steps per 64-wide stage), commits the stage's
//            "empty" mbarrier, and after the last stage of a tile commits the accumulator's "full" mbarrier;
//            the warp also owns the tensor-memory allocation
//   warps 2-9 epilogue: tcgen05.ld of the 128 x BN float32 accumulator (a thread owns one row and half of its
//            columns), bias and the fused tail, conversion, 16-byte global stores; two accumulators (2 x BN columns of
//            tensor memory) alternate, so the epilogue of tile i overlaps the main loop of tile i+1.  With the short
//            reductions of this model (K = 512: 2.9 us of MMA per tile) four epilogue warps could not keep up.
//            Measured on this kernel with K = 512: the main loop alone sustains 1.3-1.6 PFLOP/s; reading the accumulators
//            costs 6-8 % of that; conversion, staging and barriers next to nothing; what remains (to 0.9-1.0 PFLOP/s) is
//            the output's way to L2 (2 TB/s of writes), whichever instruction carries it (bulk copies from shared memory
//            are the fastest of three forms tried).  So the epilogue is kept lean: a second instantiation without the
//            optional tail, dropout decisions two per hash, and two staging blocks per column half so that a bulk store
//            drains while the next group is converted
// Operands sit in shared memory as 128-byte rows with the TMA unit's 128-byte swizzle, which is one of the
// canonical tcgen05 operand layouts both for K-major tiles ([row][64 k]) and for MN-major tiles ([k][64 rows]);
// so A and B may each be given as [rows, K] or transposed as [K, rows] without a transposing copy: the three
// products of a linear layer (Y = X W^T, dX = dY W, dW = dY^T X) are the same kernel.
// Long-K products with few output tiles (the weight gradients) are cut along K into `splits` pieces whose
// float32 partial tiles are summed in a fixed order by a second kernel.
// Every mbarrier wait is bounded; a CTA whose wait runs out raises a flag the other roles see, counts itself in
// g_gemm_aborts (hsa_gemm_aborts reads it), frees its tensor memory and returns.
#include <cstdlib>
#include <mutex>

#include "hsa_common.cuh"
#include "tc5_common.cuh"
#include "rng_common.cuh"
#include "tma_common.cuh"

namespace hsa {

constexpr int kBM = 128, kBK = 64;
constexpr int kEpiWarps = 8;                      // two warps per tensor-memory lane quarter, half the columns each
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;

// Stage geometry shared by the kernel and its launcher.
__host__ __device__ constexpr int gemm_bk(bool a_mn, bool b_mn) { return (a_mn && b_mn) ? 128 : kBK; }
__host__ __device__ constexpr int gemm_staging_bytes(bool a_mn, bool b_mn) { return (a_mn && b_mn) ? 0 : 65536; }
__host__ __device__ constexpr int gemm_stages(int stage_bytes, int staging_bytes) {
    int n = (227 * 1024 - 2304 - staging_bytes) / stage_bytes;      // 2304: bias values, barriers, alignment slack
    return n > 6 ? 6 : n;
}

struct GemmArgs {
    void *c;                      // [batches, rows, N] (OutT), element strides below
    int64_t c_bs, c_rs;
    const float *bias;            // [N] or null
    float *partial;               // split-K: [splits, batches * m_tiles * 128, n_tiles * BN] float32, else null
    int rows, batches, N;         // rows per batch of A and C
    int k_blocks;                 // 64-wide K steps of the whole product
    int kb_per_batch;             // A_MN / B_MN with batch-strided K: K steps per batch entry (k_blocks = batches * this)
    int m_tiles, n_tiles, splits; // m tiles of 128 rows (one CTA per tile) or 256 rows (a CTA pair per tile)
    int accumulate;               // C += (float32 outputs only)
    int tma_store;                // output rows leave through the copy engine (needs map_c; not with accumulate / split-K)
    long long wait_limit;
    hsa_gemm_epilogue epi;        // optional fused element-wise tail (all fields zero: none)
};

__device__ unsigned int g_gemm_aborts = 0;


__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// TWO: the tile is 256 x BN and belongs to a pair of CTAs (cluster of two, tcgen05 cta_group::2): each CTA stages its
// own 128 rows of A and half of the B tile, so a stage is 32 KB instead of 48 KB per 128 output rows and every byte
// fetched from L2 feeds twice the arithmetic.  With this model's short reductions (K = 512) the single-CTA form is
// bound by L2 bandwidth (85 flop per byte staged), not by the tensor pipe.
// FULL: the epilogue carries the optional element-wise tail (dropout, gate, residual, second copy, cross-entropy
// statistics).  Products without one run the instantiation that has none of that code: the epilogue loop is the
// kernel's critical path with short reductions, and its instruction footprint matters.
template <int BN, bool A_MN, bool B_MN, typename OutT, bool TWO, bool FULL>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc5_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c) {
    using namespace tc5;
    constexpr int B_ROWS = TWO ? BN / 2 : BN;          // rows of the B tile this CTA stages
    constexpr int MT = TWO ? 2 * kBM : kBM;            // rows of a tile
    // K extent of a stage.  With both operands stored transposed a stage is four boxes of [BK rows][64 elements]; the copy
    // engine takes about as long for an 8 KB box as for a 16 KB one (measured: ~230 cycles either way), so those products
    // use 128-row boxes: the same four boxes then carry twice the K.  They write their (float32) results with plain stores
    // and have no output staging blocks; their room goes to the stages.
    constexpr int BK = gemm_bk(A_MN, B_MN);
    constexpr int A_BYTES = kBM * 2 * BK, B_BYTES = B_ROWS * 2 * BK;
    constexpr int STAGE = A_BYTES + B_BYTES;
    constexpr int STG_BYTES = gemm_staging_bytes(A_MN, B_MN);
    constexpr int STAGES = gemm_stages(STAGE, STG_BYTES);
    constexpr uint32_t IDESC = instr_desc(MT, BN, true, A_MN, B_MN);
    const uint32_t rank = TWO ? cluster_ctarank() : 0;  // 0 = the CTA that issues the MMAs
    const int unit = TWO ? blockIdx.x / 2 : blockIdx.x, nunits = TWO ? gridDim.x / 2 : gridDim.x;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    unsigned char *staging = smem + (size_t)STAGES * STAGE;           // 2 x 2 x 16 KB: two blocks of output rows per column half
    float *bias_s = reinterpret_cast<float *>(staging + STG_BYTES);    // the tile's bias values, 128 per column half
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(staging + STG_BYTES + 1024);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_addr(bars);
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto acc_full = [&](int i) { return bar0 + 8u * (2 * STAGES + i); };
    auto acc_empty = [&](int i) { return bar0 + 8u * (2 * STAGES + 2 + i); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full(i), 1); mbar_init(acc_empty(i), (TWO ? 2 : 1) * kEpiWarps); }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_map(&map_a);
        prefetch_map(&map_b);
        if (a.tma_store) prefetch_map(&map_c);
    }
    if (warp == 1) {
        if constexpr (TWO) tmem_alloc_pair(smem_addr(tmem_slot), 2 * BN);
        else tmem_alloc(smem_addr(tmem_slot), 2 * BN);
    }
    fence_before_sync();
    __syncthreads();
    if constexpr (TWO) cluster_sync();                 // the partner's barriers exist before anything signals them
    fence_after_sync();
    // Programmatic dependent launch: everything above (barriers, tensor memory, descriptor prefetch) may overlap the tail
    // of the previous kernel in the stream; nothing below runs before that kernel has completed and its writes are visible.
    // The next kernel launched this way may in turn begin its own set-up while this one is still working.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_mn = a.m_tiles * a.n_tiles * a.batches;
    const int total = tiles_mn * a.splits;
    const int kb_split = (a.k_blocks + a.splits - 1) / a.splits;

    // tile -> (split, batch, m tile, n tile); n fastest, so CTAs running together share A rows
    auto decode = [&](int t, int &sp, int &b, int &mt, int &nt) {
        nt = t % a.n_tiles; t /= a.n_tiles;
        mt = t % a.m_tiles; t /= a.m_tiles;
        b = t % a.batches;  sp = t / a.batches;
    };

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            bool ok = true;
            // in a pair both CTAs' copies are counted on the even CTA's "full" barrier, which expects both stages
            auto load = [&](uint32_t dst, const CUtensorMap *map, int x0, int y0, int z0, uint32_t mb) {
                if constexpr (TWO) tma_load_3d_pair(dst, map, x0, y0, z0, mb);
                else tma_load_3d(dst, map, x0, y0, z0, mb);
            };
            for (int t = unit; t < total && ok; t += nunits) {
                int sp, b, mt, nt;
                decode(t, sp, b, mt, nt);
                const int kb0 = sp * kb_split, kb1 = min(a.k_blocks, kb0 + kb_split);
                const int m0 = mt * MT + (int)rank * kBM, n0 = nt * BN + (int)rank * B_ROWS;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!(ok = mbar_wait(empty(s), ph ^ 1, a.wait_limit, abort_flag))) break;
                    if (rank == 0) mbar_expect_tx(full(s), (TWO ? 2 : 1) * STAGE);
                    const uint32_t fb = TWO ? map_to_cta(full(s), 0) : full(s);
                    const uint32_t sa = smem_addr(smem + (size_t)s * STAGE), sb = sa + A_BYTES;
                    // K position of this step: a plain K offset, or (batch entry, row offset) when K runs over rows of a
                    // batch-strided tensor
                    const int kbatch = kb / a.kb_per_batch, krow = (kb % a.kb_per_batch) * BK;
                    if constexpr (!A_MN) {
                        load(sa, &map_a, kb * BK, m0, b, fb);
                    } else {
#pragma unroll
                        for (int p = 0; p < kBM / 64; ++p) load(sa + p * (BK * 128), &map_a, m0 + p * 64, krow, kbatch, fb);
                    }
                    if constexpr (!B_MN) {
                        load(sb, &map_b, kb * BK, n0, 0, fb);
                    } else {
#pragma unroll
                        for (int p = 0; p < B_ROWS / 64; ++p) load(sb + p * (BK * 128), &map_b, n0 + p * 64, krow, kbatch, fb);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
            if (!ok) {                                   // let copies already issued land before the CTA goes
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0 && rank == 0) {
            int s = 0; uint32_t ph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool ok = true;
            for (int t = unit; t < total && ok; t += nunits) {
                int sp, b, mt, nt;
                decode(t, sp, b, mt, nt);
                const int kb0 = sp * kb_split, kb1 = min(a.k_blocks, kb0 + kb_split);
                if (!(ok = mbar_wait(acc_empty(acc), acc_ph ^ 1, a.wait_limit, abort_flag))) break;
                fence_after_sync();
                const uint32_t d = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!(ok = mbar_wait(full(s), ph, a.wait_limit, abort_flag))) break;
                    fence_after_sync();
                    const uint32_t sa = smem_addr(smem + (size_t)s * STAGE), sb = sa + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t da = A_MN ? smem_desc(sa + k * 2048, BK * 128, 1024) : smem_desc(sa + k * 32, 16, 1024);
                        const uint64_t db = B_MN ? smem_desc(sb + k * 2048, BK * 128, 1024) : smem_desc(sb + k * 32, 16, 1024);
                        if constexpr (TWO) mma_f16_pair(d, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
                        else mma_f16(d, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    // the stage is free (in both CTAs of a pair) once these MMAs have read it
                    if constexpr (TWO) mma_commit_pair(empty(s)); else mma_commit(empty(s));
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                // the accumulator is complete once all MMAs of the tile are
                if constexpr (TWO) mma_commit_pair(acc_full(acc)); else mma_commit(acc_full(acc));
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;                            // the tensor-memory lane quarter this warp may read
        const int col_lo = ((warp - 2) >> 2) * (BN / 2);   // ... and the half of the tile's columns it owns
        int acc = 0; uint32_t acc_ph = 0;
        bool ok = true;
        uint32_t group = 0;                                // staged groups handed to the copy engine so far (this half)
        const unsigned long long drop_key = (FULL && a.epi.rng_state != nullptr) ? *a.epi.rng_state : 0ull;
        const uint32_t drop_salt0 = dropout_salt(drop_key, a.epi.drop_site0, 0), drop_salt1 = dropout_salt(drop_key, a.epi.drop_site1, 0);
        // Gate / residual blocks ([128 rows][128 bytes] of a tensor shaped like the output) are fetched one block AHEAD into
        // registers, 8 threads per row (whole lines), so their latency hides behind the previous block's work; the first
        // block of a tile is requested before the accumulator is even waited for.
        const bool in_gate = FULL && a.tma_store && a.epi.gate != nullptr && sizeof(OutT) == 2;
        const bool in_res = FULL && a.tma_store && a.epi.residual != nullptr && sizeof(OutT) == 4;
        const int t128 = ((warp & 3) << 5) | lane;                           // thread index inside the column half
        uint4 pre[8];
        auto fetch_block = [&](int bb, int row0, int first_col) {
            const unsigned char *base = in_gate ? (const unsigned char *)a.epi.gate : (const unsigned char *)a.epi.residual;
            const long long bs = in_gate ? a.epi.gate_bs * 2 : a.epi.res_bs * 4, rs = in_gate ? a.epi.gate_rs * 2 : a.epi.res_rs * 4;
            const int esz = in_gate ? 2 : 4, per_piece = 16 / esz;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int idx = it * 128 + t128, rr = idx >> 3, pc = idx & 7;
                pre[it] = make_uint4(0, 0, 0, 0);
                if (row0 + rr < a.rows && first_col + pc * per_piece < a.N)
                    pre[it] = __ldg(reinterpret_cast<const uint4 *>(base + bb * bs + (long long)(row0 + rr) * rs +
                                                                    (long long)first_col * esz + pc * 16));
            }
        };
        for (int t = unit; t < total && ok; t += nunits) {
            int sp, b, mt, nt;
            decode(t, sp, b, mt, nt);
            if (in_gate || in_res) fetch_block(b, mt * MT + (int)rank * kBM, nt * BN + ((warp - 2) >> 2) * (BN / 2));
            if (a.bias != nullptr && a.partial == nullptr) {
                // this half's 128 bias values, fetched before the accumulator is waited for (a global load inside the
                // column loop would sit on the critical path of every chunk)
                const int hb = (warp - 2) >> 2, j = ((warp & 3) << 5) | lane;
                const int cidx = nt * BN + hb * (BN / 2) + j;
                if (j < BN / 2) bias_s[hb * 128 + j] = cidx < a.N ? __ldg(a.bias + cidx) : 0.f;
            }
            ok = mbar_wait(acc_full(acc), acc_ph, a.wait_limit, abort_flag);
            {   // the four warps that share a staging block go on (or give up) together
                uint32_t all_ok;
                asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, %2, 128, q;\nselp.u32 %0, 1, 0, p;\n}\n"
                             : "=r"(all_ok) : "r"((uint32_t)ok), "r"(1 + ((warp - 2) >> 2)) : "memory");
                ok = all_ok != 0;
            }
            if (!ok) break;
            fence_after_sync();
            const int row = mt * MT + (int)rank * kBM + q * 32 + lane;
            const bool row_ok = row < a.rows;
            const uint32_t tbase = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
            // cross-entropy statistics of this thread's row over its half of the tile's columns (when asked for)
            float ce_m = -INFINITY, ce_s = 0.f, ce_sx = 0.f, ce_xt = 0.f;
            long long ce_target = -1;
            if (FULL && a.epi.ce_partial != nullptr && row_ok) ce_target = a.epi.ce_targets[(long long)b * a.rows + row];
            const int half = (warp - 2) >> 2;                 // which half of the tile's columns
            const int row_local = q * 32 + lane;              // row inside this CTA's 128 rows
            // [128 rows][128 B] blocks, 128-byte swizzle, for the TMA stores: two per half, used in turn, so that the copy
            // engine reads one while the next group is converted into the other
            unsigned char *stg = staging + half * 32768 + (group & 1) * 16384;
#pragma unroll 1
            for (int c0 = col_lo; c0 < col_lo + BN / 2; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tbase + c0, r);
                tmem_ld_wait();
                const int col = nt * BN + c0;
                if (a.tma_store && (c0 - col_lo) % (sizeof(OutT) == 2 ? 64 : 32) == 0) {
                    // a new staged group: its block is free once the store issued from it two groups ago has read it, which
                    // the issuing thread waited for right after handing over the group in between
                    asm volatile("bar.sync %0, 128;\n" ::"r"(1 + half) : "memory");
                }
                if (a.partial != nullptr) {
                    // split-K: the raw float32 tile goes to this split's slab (padded to whole tiles: no masks)
                    float *dst = a.partial + ((size_t)sp * a.batches * a.m_tiles * MT + ((size_t)b * a.m_tiles * MT + row)) *
                                                 ((size_t)a.n_tiles * BN) + col;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4 *>(dst + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                          __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    continue;
                }
                const bool live = row_ok && col < a.N;        // dead rows / columns still take part in the staged store
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                const hsa_gemm_epilogue &e = a.epi;
                if (live) {
                    if (a.bias != nullptr) {                 // visible since the barrier that follows the accumulator wait
                        const float *bs = bias_s + half * 128 + (c0 - col_lo);
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            const float4 bv = *reinterpret_cast<const float4 *>(bs + i);
                            v[i] += bv.x; v[i + 1] += bv.y; v[i + 2] += bv.z; v[i + 3] += bv.w;
                        }
                    }
                    if (e.relu) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
                    }
                    if (FULL && e.rng_state != nullptr && col >= e.drop_col_begin && col < e.drop_col_end) {   // ranges are whole chunks
                        // dropout on columns [drop_col_begin, drop_col_end): element id = (batch, row, column) of the logical
                        // [batches, drop_rows_total, N] tensor this product writes a row range of
                        const unsigned long long id0 = ((unsigned long long)b * e.drop_rows_total + (unsigned long long)(row + e.drop_row_offset)) *
                                                       (unsigned long long)a.N + (unsigned long long)col;
                        dropout_run(v, drop_salt0, drop_salt1, e.drop_site1 != 0, id0, e.drop_threshold, e.drop_scale);
                    }
                }
                // Gate and residual blocks are fetched by the four warps of this half together, 8 threads per 128-byte row
                // (whole lines, like the output block leaves), through the staging block; a thread then picks up its own row.
                constexpr int CPG_IN = sizeof(OutT) == 2 ? 64 : 32;          // columns of a staged group (one 128-byte output row)
                const int cg_in = (c0 - col_lo) % CPG_IN;
                auto commit_block = [&]() {                                  // the prefetched block into the staging block
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int idx = it * 128 + t128, rr = idx >> 3, pc = idx & 7;
                        *reinterpret_cast<uint4 *>(stg + rr * 128 + ((pc ^ (rr & 7)) << 4)) = pre[it];
                    }
                    asm volatile("bar.sync %0, 128;\n" ::"r"(1 + half) : "memory");
                };
                auto fetch_next = [&]() {                                    // the block after this group, if the half has one
                    if (c0 + 32 < col_lo + BN / 2) fetch_block(b, mt * MT + (int)rank * kBM, col + 32);
                };
                auto staged_done = [&]() { asm volatile("bar.sync %0, 128;\n" ::"r"(1 + half) : "memory"); };
                if (in_gate) {
                    // one staged group of the gate (64 bfloat16 per row) serves two 32-column chunks
                    if (cg_in == 0) commit_block();
                    const unsigned char *srow = stg + row_local * 128;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 raw = *reinterpret_cast<const uint4 *>(srow + (((cg_in / 8 + i) ^ (row_local & 7)) << 4));
                        const __nv_bfloat16 *ge = reinterpret_cast<const __nv_bfloat16 *>(&raw);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[8 * i + j] = (__bfloat162float(ge[j]) > 0.f) ? v[8 * i + j] * e.gate_scale : 0.f;
                    }
                    if (cg_in + 32 == CPG_IN) { staged_done(); fetch_next(); }
                } else if (FULL && live && e.gate != nullptr) {
                    // pass the value where the gate tensor (same shape as the output) is positive: the backward of
                    // relu followed by dropout, whose forward output is the gate
                    const __nv_bfloat16 *gp = (const __nv_bfloat16 *)e.gate + b * e.gate_bs + (int64_t)row * e.gate_rs + col;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (col + i < a.N) {
                            const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(gp + i));
                            const __nv_bfloat16 *ge = reinterpret_cast<const __nv_bfloat16 *>(&raw);
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[i + j] = (__bfloat162float(ge[j]) > 0.f) ? v[i + j] * e.gate_scale : 0.f;
                        }
                    }
                }
                if (in_res) {
                    commit_block();
                    const unsigned char *srow = stg + row_local * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 rv = *reinterpret_cast<const float4 *>(srow + ((i ^ (row_local & 7)) << 4));
                        v[4 * i] += rv.x; v[4 * i + 1] += rv.y; v[4 * i + 2] += rv.z; v[4 * i + 3] += rv.w;
                    }
                    staged_done();
                    fetch_next();
                } else if (FULL && live && e.residual != nullptr) {
                    const float *rp = e.residual + b * e.res_bs + (int64_t)row * e.res_rs + col;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        if (col + i < a.N) {
                            const float4 rv = __ldg(reinterpret_cast<const float4 *>(rp + i));
                            v[i] += rv.x; v[i + 1] += rv.y; v[i + 2] += rv.z; v[i + 3] += rv.w;
                        }
                    }
                }
                if (FULL && e.ce_partial != nullptr && live) {
                    // classes [0, ce_classes): running max and sum of exponentials (base 2, on log2(e)-scaled logits), the
                    // plain sum (label smoothing) and the target's logit.  Five instructions per element on the common path.
                    constexpr float kL2e = 1.4426950408889634f;
                    const int nvalid = min(32, e.ce_classes - col);             // classes in this chunk (may be <= 0 in padding)
                    if (nvalid > 0) {
                        float cm = ce_m;
                        if (nvalid == 32) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) cm = fmaxf(cm, v[i]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) if (i < nvalid) cm = fmaxf(cm, v[i]);
                        }
                        const float cm2 = cm * kL2e;
                        float add = 0.f, sx = 0.f;
                        if (nvalid == 32) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) { add += fast_ex2(fmaf(v[i], kL2e, -cm2)); sx += v[i]; }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) if (i < nvalid) { add += fast_ex2(fmaf(v[i], kL2e, -cm2)); sx += v[i]; }
                        }
                        ce_s = ce_s * fast_ex2((ce_m - cm) * kL2e) + add;
                        ce_sx += sx;
                        ce_m = cm;
                        const long long tc = ce_target - col;
                        const uint32_t tmask = (tc >= 0 && tc < nvalid) ? (1u << (uint32_t)tc) : 0u;
                        if (tmask != 0) {                                   // bit tests, not an indexed read: v stays in registers
#pragma unroll
                            for (int i = 0; i < 32; ++i) ce_xt = (tmask & (1u << i)) ? v[i] : ce_xt;
                        }
                    }
                }
                OutT *dst = (OutT *)a.c + b * a.c_bs + (int64_t)row * a.c_rs + col;
                auto store_bf16 = [&](__nv_bfloat16 *d16) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (col + i < a.N) {
                            uint4 o;
                            __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                            for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                            *reinterpret_cast<uint4 *>(d16 + i) = o;
                        }
                    }
                };
                if (FULL && e.ce_partial != nullptr && e.ce_skip_store) {
                    // loss only: the logits are never written
                } else if (a.tma_store) {
                    // Rows leave through the copy engine: the 4 warps of this half park a [128 rows][128 B] block in shared
                    // memory (swizzled like the tensor map expects) and one thread stores it with a single bulk copy, which
                    // writes whole lines and clips what lies outside the tensor.  Per-thread 16-byte stores would touch half
                    // a sector each.
                    constexpr int CPG = sizeof(OutT) == 2 ? 64 : 32;          // columns per 128-byte staged row
                    const int cg = (c0 - col_lo) % CPG;                       // first column of this chunk inside the group
                    unsigned char *srow = stg + row_local * 128;
                    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 o;
                            __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                            for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
                            *reinterpret_cast<uint4 *>(srow + (((cg / 8 + i) ^ (row_local & 7)) << 4)) = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<float4 *>(srow + ((i ^ (row_local & 7)) << 4)) =
                                make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                    if (cg + 32 == CPG) {                                     // the group is complete: hand it to the copy engine
                        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                        asm volatile("bar.sync %0, 128;\n" ::"r"(1 + half) : "memory");
                        if (q == 0 && lane == 0) {
                            const int gcol = nt * BN + c0 + 32 - CPG;
                            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];\n"
                                         ::"l"(&map_c), "r"(gcol), "r"(mt * MT + (int)rank * kBM), "r"(b), "r"(smem_addr(stg)) : "memory");
                            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                            asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");   // the previous group's block is free
                        }
                        ++group;
                        stg = staging + half * 32768 + (group & 1) * 16384;
                    }
                    if constexpr (sizeof(OutT) == 4) {
                        if (FULL && live && e.copy_bf16 != nullptr)
                            store_bf16((__nv_bfloat16 *)e.copy_bf16 + b * e.copy_bs + (int64_t)row * e.copy_rs + col);
                    }
                } else if (live) {
                    if constexpr (sizeof(OutT) == 2) {
                        store_bf16(reinterpret_cast<__nv_bfloat16 *>(dst));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            if (col + i < a.N) {
                                if (a.accumulate) {
                                    const float4 old = *reinterpret_cast<const float4 *>(dst + i);
                                    v[i] += old.x; v[i + 1] += old.y; v[i + 2] += old.z; v[i + 3] += old.w;
                                }
                                *reinterpret_cast<float4 *>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                            }
                        }
                        if (FULL && e.copy_bf16 != nullptr)
                            store_bf16((__nv_bfloat16 *)e.copy_bf16 + b * e.copy_bs + (int64_t)row * e.copy_rs + col);
                    }
                }
            }
            if (a.bias != nullptr && a.partial == nullptr && !a.tma_store)      // bias_s is rewritten at the top of the next tile
                asm volatile("bar.sync %0, 128;\n" ::"r"(1 + half) : "memory");
            if (FULL && a.epi.ce_partial != nullptr && row_ok)
                *reinterpret_cast<float4 *>(a.epi.ce_partial + (((long long)b * a.rows + row) * (2 * a.n_tiles) + 2 * nt + half) * 4) =
                    make_float4(ce_m, ce_s, ce_sx, ce_xt);
            fence_before_sync();
            __syncwarp();
            if (lane == 0) {                                  // the MMA thread (even CTA of a pair) may reuse the accumulator
                if constexpr (TWO) mbar_arrive_cluster(map_to_cta(acc_empty(acc), 0));
                else mbar_arrive(acc_empty(acc));
            }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (a.tma_store && q == 0 && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
    }

    // ---------------------------------------------------------------------- teardown
    fence_before_sync();
    __syncthreads();
    if constexpr (TWO) cluster_sync();                 // nobody leaves while the partner may still touch its memory
    if (*abort_flag && threadIdx.x == 0) atomicAdd(&g_gemm_aborts, 1u);
    if (warp == 1) {
        fence_after_sync();
        if constexpr (TWO) tmem_dealloc_pair(tmem_base, 2 * BN);
        else tmem_dealloc(tmem_base, 2 * BN);
    }
}

// Sum the split-K slabs in split order, add the bias, convert, store (one thread per four columns).
template <typename OutT>
__global__ void __launch_bounds__(256)
gemm_splitk_reduce_kernel(const float *__restrict__ partial, int splits, size_t slab, int rows, int batches, int N,
                          int padded_rows, int padded_cols, OutT *c, int64_t c_bs, int64_t c_rs,
                          const float *__restrict__ bias, int accumulate) {
    const int cols4 = N / 4;
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (size_t)batches * rows * cols4) return;
    const int c4 = (int)(idx % cols4);
    const size_t br = idx / cols4;
    const int row = (int)(br % rows), b = (int)(br / rows);
    const float *src = partial + ((size_t)b * padded_rows + row) * padded_cols + 4 * c4;
    float4 s = *reinterpret_cast<const float4 *>(src);
    for (int sp = 1; sp < splits; ++sp) {
        const float4 v = *reinterpret_cast<const float4 *>(src + sp * slab);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    if (bias != nullptr) {
        const float4 bv = *reinterpret_cast<const float4 *>(bias + 4 * c4);
        s.x += bv.x; s.y += bv.y; s.z += bv.z; s.w += bv.w;
    }
    OutT *dst = c + b * c_bs + (int64_t)row * c_rs + 4 * c4;
    if constexpr (sizeof(OutT) == 4) {
        if (accumulate) {
            const float4 old = *reinterpret_cast<const float4 *>(dst);
            s.x += old.x; s.y += old.y; s.z += old.z; s.w += old.w;
        }
        *reinterpret_cast<float4 *>(dst) = s;
    } else {
        uint2 o;
        __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&o);
        p[0] = __floats2bfloat162_rn(s.x, s.y);
        p[1] = __floats2bfloat162_rn(s.z, s.w);
        *reinterpret_cast<uint2 *>(dst) = o;
    }
}

static thread_local int g_last_map_result = 0;      // CUresult of the last cuTensorMapEncodeTiled, for error messages

// A 3-D tensor map over 2-byte elements: dims {inner, rows, batches}, box {64, box_rows, 1}, 128-byte swizzle,
// zero fill outside.
static bool make_map3(CUtensorMap *m, const void *ptr, int64_t inner, int64_t rows, int64_t batches, int64_t row_stride,
                      int64_t batch_stride, int box_rows) {
    if (encode_tiled() == nullptr) return false;
    if (batches == 1) batch_stride = rows * row_stride;
    const cuuint64_t gdim[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t gstride[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)batch_stride * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    const cuuint32_t estride[3] = {1u, 1u, 1u};
    const CUresult r = encode_tiled()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(ptr), gdim, gstride, box, estride,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    g_last_map_result = (int)r;
    return r == CUDA_SUCCESS;
}

// The output tensor [batches, rows, N] for bulk stores of [128 rows][128 bytes] blocks.
static bool make_map_out(CUtensorMap *m, const void *ptr, int64_t N, int64_t rows, int64_t batches, int64_t row_stride,
                         int64_t batch_stride, int esize) {
    if (encode_tiled() == nullptr) return false;
    if (batches == 1) batch_stride = rows * row_stride;
    const cuuint64_t gdim[3] = {(cuuint64_t)N, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t gstride[2] = {(cuuint64_t)row_stride * esize, (cuuint64_t)batch_stride * esize};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / esize), 128u, 1u};
    const cuuint32_t estride[3] = {1u, 1u, 1u};
    return encode_tiled()(m, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                          const_cast<void *>(ptr), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Programmatic dependent launch of the products: off unless HSA_B200_PDL=1 (measured: no gain inside a captured
// training step, where back-to-back products already start within a microsecond of each other).
static bool pdl_enabled() {
    static const bool on = [] {
        const char *v = getenv("HSA_B200_PDL");
        return v != nullptr && v[0] == '1';
    }();
    return on;
}

static int sm_count() {
    static int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
        return v;
    }();
    return n;
}

}  // namespace hsa

using namespace hsa;

namespace hsa {
// Merge the per-tile-half statistics of a row into its loss and log-sum-exp (one thread per row).
__global__ void __launch_bounds__(256)
ce_combine_kernel(const float *__restrict__ partial, int slots, const long long *__restrict__ targets, float *__restrict__ loss_rows,
                  float *__restrict__ lse_out, long long rows, int V, float eps, long long ignore_index) {
    const long long r = (long long)blockIdx.x * 256 + threadIdx.x;
    if (r >= rows) return;
    const float4 *p = reinterpret_cast<const float4 *>(partial) + r * slots;
    float m = -INFINITY;
    for (int i = 0; i < slots; ++i) m = fmaxf(m, p[i].x);
    float s = 0.f, sx = 0.f, xt = 0.f;
    for (int i = 0; i < slots; ++i) {
        const float4 t = p[i];
        if (t.x > -INFINITY) s += t.y * __expf(t.x - m);
        sx += t.z;
        xt += t.w;
    }
    const float lse = m + logf(s);
    lse_out[r] = lse;
    const long long tgt = targets[r];
    float loss = 0.f;
    if (tgt != ignore_index) {
        if (tgt < 0 || tgt >= V) xt = __int_as_float(0x7fffffff);     // a corrupt label shows as NaN
        loss = (1.f - eps) * (lse - xt) + eps * (lse - sx / (float)V);
    }
    loss_rows[r] = loss;
}
}  // namespace hsa

extern "C" size_t hsa_linear_ce_partial_bytes(long long rows, int N) {
    if (rows < 1 || N < 1) return 0;
    const int BN = N > 128 ? 256 : 128;
    return (size_t)rows * 2 * ((N + BN - 1) / BN) * 4 * sizeof(float);
}

extern "C" int hsa_linear_ce_combine(const float *partial, long long rows, int N, const long long *targets, float *loss_rows,
                                     float *lse, int classes, float smoothing, long long ignore_index, void *stream) {
    HSA_CHECK_ARG(partial && targets && loss_rows && lse, "hsa_linear_ce_combine: null pointer");
    HSA_CHECK_ARG(rows >= 1 && N >= 1 && classes >= 1 && classes <= N, "hsa_linear_ce_combine: bad shape");
    HSA_CHECK_ARG(smoothing >= 0.f && smoothing < 1.f, "hsa_linear_ce_combine: label smoothing %f outside [0, 1)", smoothing);
    const int BN = N > 128 ? 256 : 128;
    const int slots = 2 * ((N + BN - 1) / BN);
    ce_combine_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, (cudaStream_t)stream>>>(partial, slots, targets, loss_rows, lse, rows,
                                                                                      classes, smoothing, ignore_index);
    return launch_status("hsa_linear_ce_combine");
}

extern "C" int hsa_gemm_aborts(unsigned int *count) {
    if (count == nullptr) return fail(HSA_ERR_ARG, "hsa_gemm_aborts: null pointer");
    cudaError_t e = cudaMemcpyFromSymbol(count, g_gemm_aborts, sizeof(unsigned int));
    return e == cudaSuccess ? 0 : fail((int)e, "hsa_gemm_aborts: %s", cudaGetErrorString(e));
}

// Tile shape of a product: BN = 256 columns (128 for narrow outputs); 256-row tiles on CTA pairs when a batch entry
// has at least 256 rows, else 128-row tiles on single CTAs.
struct GemmShape { int BN, MT; bool two; };
static GemmShape gemm_shape(int rows, int N) {
    GemmShape s;
    s.BN = N > 128 ? 256 : 128;
    s.two = rows >= 256;
    s.MT = s.two ? 2 * kBM : kBM;
    return s;
}

extern "C" size_t hsa_gemm_workspace_bytes(int batches, int rows, int N, int K, int a_layout, int b_layout, int splits) {
    (void)a_layout; (void)b_layout; (void)K;
    if (splits <= 1 || batches < 1 || rows < 1 || N < 1) return 0;
    const GemmShape sh = gemm_shape(rows, N);
    const size_t m_tiles = (rows + sh.MT - 1) / sh.MT, n_tiles = (N + sh.BN - 1) / sh.BN;
    return (size_t)splits * batches * m_tiles * sh.MT * n_tiles * sh.BN * sizeof(float);
}

extern "C" int hsa_gemm_choose_splits(int batches, int rows, int N, int K) {
    if (batches < 1 || rows < 1 || N < 1 || K < 1) return 1;
    const GemmShape sh = gemm_shape(rows, N);
    const long long m_tiles = (rows + sh.MT - 1) / sh.MT, n_tiles = (N + sh.BN - 1) / sh.BN;
    const long long tiles = (long long)batches * m_tiles * n_tiles;
    const int k_blocks = (K + kBK - 1) / kBK;
    const int units = sh.two ? sm_count() / 2 : sm_count();        // tiles that run at once
    // Estimated time of s splits: waves of tiles, each (k_blocks / s) steps of ~0.38 us, plus writing and reading the
    // float32 partial slabs.  Splitting pays when there are too few tiles to fill the GPU, or when the last wave of
    // tiles would leave most of it idle and K is long enough to absorb the extra pass.
    const double step_us = 0.38, bytes_per_us = 5.0e6;
    double best = 1e30;
    int best_s = 1;
    for (int s = 1; s <= 32 && k_blocks / s >= 4; ++s) {
        const long long waves = (tiles * s + units - 1) / units;
        double t = (double)waves * ((k_blocks + s - 1) / s) * step_us;
        if (s > 1) t += 2.0 * s * batches * m_tiles * sh.MT * n_tiles * sh.BN * 4.0 / bytes_per_us + 3.0;
        if (t < best * 0.97) { best = t; best_s = s; }             // a later s must win by 3 %
    }
    return best_s;
}

// Layout codes: 0 = the operand is stored [rows, K] (K contiguous); 1 = stored transposed, [K, rows].
extern "C" int hsa_gemm(hsa_view A, hsa_view Bm, hsa_view C, const float *bias, int batches, int rows, int N, int K,
                        int a_layout, int b_layout, int out_dtype, int accumulate, int splits, void *workspace,
                        size_t workspace_bytes, void *stream) {
    return hsa_gemm_ex(A, Bm, C, bias, batches, rows, N, K, a_layout, b_layout, out_dtype, accumulate, splits, workspace,
                       workspace_bytes, nullptr, stream);
}

extern "C" int hsa_gemm_ex(hsa_view A, hsa_view Bm, hsa_view C, const float *bias, int batches, int rows, int N, int K,
                           int a_layout, int b_layout, int out_dtype, int accumulate, int splits, void *workspace,
                           size_t workspace_bytes, const hsa_gemm_epilogue *epilogue, void *stream) {
    HSA_CHECK_ARG(A.ptr && Bm.ptr && C.ptr, "hsa_gemm: null pointer");
    HSA_CHECK_ARG(batches >= 1 && rows >= 1 && N >= 8 && K >= 1 && N % 8 == 0,
                  "hsa_gemm: bad shape batches=%d rows=%d N=%d K=%d (N must be a multiple of 8)", batches, rows, N, K);
    HSA_CHECK_ARG((a_layout | 1) == 1 && (b_layout | 1) == 1, "hsa_gemm: layout codes are 0 or 1");
    HSA_CHECK_ARG(out_dtype == HSA_BF16 || out_dtype == HSA_F32, "hsa_gemm: the output is bfloat16 or float32");
    HSA_CHECK_ARG(!accumulate || out_dtype == HSA_F32, "hsa_gemm: accumulation needs a float32 output");
    HSA_CHECK_ARG(a_layout == 0 || rows % 8 == 0, "hsa_gemm: a transposed A needs rows %% 8 == 0");
    HSA_CHECK_ARG(splits >= 1 && splits <= 1024, "hsa_gemm: splits out of range");
    const int esz = out_dtype == HSA_F32 ? 4 : 2;
    if (!aligned16(A.ptr) || !aligned16(Bm.ptr) || !aligned16(C.ptr) || (A.row_stride % 8) || (Bm.row_stride % 8) ||
        (A.batch_stride % 8) || (C.row_stride * esz) % 16 || (C.batch_stride * esz) % 16 || (bias && !aligned16(bias)))
        return fail(HSA_ERR_ALIGN, "hsa_gemm: pointers and strides must be 16-byte aligned");
    const GemmShape sh = gemm_shape(rows, N);
    const int BN = sh.BN;
    GemmArgs g{};
    g.c = C.ptr; g.c_bs = C.batch_stride; g.c_rs = C.row_stride; g.bias = bias;
    g.rows = rows; g.batches = batches; g.N = N;
    g.m_tiles = (rows + sh.MT - 1) / sh.MT;
    g.n_tiles = (N + BN - 1) / BN;
    g.accumulate = accumulate;
    g.wait_limit = wait_limit_cycles();
    if (epilogue != nullptr) {
        g.epi = *epilogue;
        const hsa_gemm_epilogue &e = g.epi;
        HSA_CHECK_ARG(splits == 1, "hsa_gemm_ex: a fused epilogue needs splits == 1");
        HSA_CHECK_ARG(a_layout == 0, "hsa_gemm_ex: a fused epilogue needs a_layout == 0");
        HSA_CHECK_ARG(e.residual == nullptr || (aligned16(e.residual) && e.res_rs % 4 == 0 && e.res_bs % 4 == 0),
                      "hsa_gemm_ex: residual must be 16-byte aligned");
        HSA_CHECK_ARG(e.gate == nullptr || (aligned16(e.gate) && e.gate_rs % 8 == 0 && e.gate_bs % 8 == 0),
                      "hsa_gemm_ex: gate must be 16-byte aligned");
        HSA_CHECK_ARG(e.copy_bf16 == nullptr || (out_dtype == HSA_F32 && aligned16(e.copy_bf16) && e.copy_rs % 8 == 0 && e.copy_bs % 8 == 0),
                      "hsa_gemm_ex: the bfloat16 copy needs a float32 main output and 16-byte alignment");
        HSA_CHECK_ARG(e.ce_partial == nullptr || (e.ce_targets != nullptr && e.ce_classes >= 1 && e.ce_classes <= N && aligned16(e.ce_partial) &&
                                                   out_dtype == HSA_BF16),
                      "hsa_gemm_ex: bad cross-entropy description (bfloat16 logits, targets, 1 <= classes <= N)");
        HSA_CHECK_ARG(e.rng_state == nullptr || (e.drop_col_begin >= 0 && e.drop_col_end <= N && e.drop_site0 != 0 && e.drop_rows_total >= rows),
                      "hsa_gemm_ex: bad dropout description");
        HSA_CHECK_ARG(e.rng_state == nullptr || (e.drop_col_begin % 32 == 0 && (e.drop_col_end % 32 == 0 || e.drop_col_end == N)),
                      "hsa_gemm_ex: the dropout column range starts and ends on multiples of 32 (or ends with the last column)");
        HSA_CHECK_ARG(e.rng_state == nullptr || (unsigned long long)batches * (unsigned long long)e.drop_rows_total * (unsigned long long)N <= kDropoutRunMaxElems,
                      "hsa_gemm_ex: the tensor the dropout ids refer to has more than 2^33 elements");
    }
    // K runs over rows of the stored tensors when an operand is transposed; a transposed A carries the batch dimension
    // in K (the weight gradient sums over every row of every batch entry)
    int out_batches = batches;
    CUtensorMap ma, mb;
    bool ok;
    if (a_layout == 0) {
        g.k_blocks = (K + kBK - 1) / kBK;
        g.kb_per_batch = g.k_blocks;
        ok = make_map3(&ma, A.ptr, K, rows, batches, A.row_stride, A.batch_stride, kBM);
        // B: [N, K] or [K, N], shared by all batch entries
        ok = ok && (b_layout == 0 ? make_map3(&mb, Bm.ptr, K, N, 1, Bm.row_stride, 0, sh.two ? BN / 2 : BN)
                                  : make_map3(&mb, Bm.ptr, N, K, 1, Bm.row_stride, 0, kBK));
    } else {
        // A stored [batches, K, rows]: C[rows, N] = sum over batch entries and k; B must be transposed as well,
        // stored [batches, K, N], so both are cut along the same (batch entry, row) steps
        HSA_CHECK_ARG(b_layout == 1, "hsa_gemm: a transposed A needs a transposed B ([K, N])");
        constexpr int bk = gemm_bk(true, true);
        g.kb_per_batch = (K + bk - 1) / bk;
        g.k_blocks = g.kb_per_batch * batches;
        out_batches = 1;
        g.batches = 1;
        ok = make_map3(&ma, A.ptr, rows, K, batches, A.row_stride, A.batch_stride, bk) &&
             make_map3(&mb, Bm.ptr, N, K, batches, Bm.row_stride, Bm.batch_stride, bk);
    }
    if (!ok)
        return fail(HSA_ERR_ARG,
                    "hsa_gemm: the driver refused a tensor map, CUresult %d (batches=%d rows=%d N=%d K=%d layouts %d/%d; A %p strides %lld/%lld; "
                    "B %p strides %lld/%lld)", g_last_map_result, batches, rows, N, K, a_layout, b_layout, A.ptr, (long long)A.batch_stride,
                    (long long)A.row_stride, Bm.ptr, (long long)Bm.batch_stride, (long long)Bm.row_stride);
    if (splits > g.k_blocks) splits = g.k_blocks;
    {   // every split must own at least one K step (an accumulator nobody wrote holds stale numbers)
        const int per = (g.k_blocks + splits - 1) / splits;
        splits = (g.k_blocks + per - 1) / per;
    }
    g.splits = splits;
    if (splits > 1) {
        const size_t need = hsa_gemm_workspace_bytes(out_batches, rows, N, K, a_layout, b_layout, splits);
        if (workspace == nullptr || workspace_bytes < need)
            return fail(HSA_ERR_WORKSPACE, "hsa_gemm: split-K workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(HSA_ERR_ALIGN, "hsa_gemm: workspace must be 256-byte aligned");
        g.partial = (float *)workspace;
    }
    // the output's tensor map (rows leave by bulk copies), unless the epilogue has to read C back or writes partial slabs
    CUtensorMap mc = ma;
    g.tma_store = 0;
    if (a_layout == 0 && g.partial == nullptr && !accumulate && !(epilogue && epilogue->ce_partial && epilogue->ce_skip_store) && make_map_out(&mc, C.ptr, N, rows, out_batches, C.row_stride, C.batch_stride, esz))
        g.tma_store = 1;
    const long long total = (long long)g.m_tiles * g.n_tiles * g.batches * g.splits;
    if (total > 0x7fffffffLL) return fail(HSA_ERR_ARG, "hsa_gemm: too many tiles");
    const int units = sh.two ? sm_count() / 2 : sm_count();
    const int grid = (int)(total < units ? total : units) * (sh.two ? 2 : 1);
    cudaStream_t st = (cudaStream_t)stream;

    auto launch = [&](auto kernel, int bn) -> int {
        const bool amn = a_layout != 0, bmn = b_layout != 0;
        const int stage = (kBM + (sh.two ? bn / 2 : bn)) * 2 * gemm_bk(amn, bmn);
        const int stg = gemm_staging_bytes(amn, bmn);
        const int stages = gemm_stages(stage, stg);
        const size_t smem = (size_t)stages * stage + stg + 1024 + (2 * stages + 4) * 8 + 16 + 1024;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "hsa_gemm: shared memory %zu: %s", smem, cudaGetErrorString(e));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = sh.two ? 2 : 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, kernel, g, ma, mb, mc);
        if (e != cudaSuccess) return fail((int)e, "hsa_gemm: launch: %s", cudaGetErrorString(e));
        return launch_status("hsa_gemm");
    };
    const bool f32 = out_dtype == HSA_F32 || g.partial != nullptr;
    int rc;
    const bool full = epilogue != nullptr && (epilogue->rng_state != nullptr || epilogue->gate != nullptr || epilogue->residual != nullptr ||
                                              epilogue->copy_bf16 != nullptr || epilogue->ce_partial != nullptr);
#define HSA_GEMM_CASE2(BNV, AMN, BMN, FULLV)                                                                           \
    (sh.two ? (f32 ? launch(gemm_tc5_kernel<BNV, AMN, BMN, float, true, FULLV>, BNV)                                   \
                   : launch(gemm_tc5_kernel<BNV, AMN, BMN, __nv_bfloat16, true, FULLV>, BNV))                          \
            : (f32 ? launch(gemm_tc5_kernel<BNV, AMN, BMN, float, false, FULLV>, BNV)                                  \
                   : launch(gemm_tc5_kernel<BNV, AMN, BMN, __nv_bfloat16, false, FULLV>, BNV)))
#define HSA_GEMM_CASE(BNV, AMN, BMN) (full ? HSA_GEMM_CASE2(BNV, AMN, BMN, true) : HSA_GEMM_CASE2(BNV, AMN, BMN, false))
    if (BN == 256) {
        rc = a_layout ? HSA_GEMM_CASE(256, true, true) : (b_layout ? HSA_GEMM_CASE(256, false, true) : HSA_GEMM_CASE(256, false, false));
    } else {
        rc = a_layout ? HSA_GEMM_CASE(128, true, true) : (b_layout ? HSA_GEMM_CASE(128, false, true) : HSA_GEMM_CASE(128, false, false));
    }
#undef HSA_GEMM_CASE
#undef HSA_GEMM_CASE2
    if (rc != 0 || splits == 1) return rc;
    const size_t slab = (size_t)out_batches * g.m_tiles * sh.MT * g.n_tiles * BN;
    const size_t work = (size_t)out_batches * rows * (N / 4);
    const unsigned blocks = (unsigned)((work + 255) / 256);
    if (out_dtype == HSA_F32)
        gemm_splitk_reduce_kernel<float><<<blocks, 256, 0, st>>>(g.partial, splits, slab, rows, out_batches, N, g.m_tiles * sh.MT,
                                                                 g.n_tiles * BN, (float *)C.ptr, C.batch_stride, C.row_stride, bias, accumulate);
    else
        gemm_splitk_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(g.partial, splits, slab, rows, out_batches, N, g.m_tiles * sh.MT,
                                                                         g.n_tiles * BN, (__nv_bfloat16 *)C.ptr, C.batch_stride,
                                                                         C.row_stride, bias, 0);
    return launch_status("hsa_gemm(split-K reduce)");
}
