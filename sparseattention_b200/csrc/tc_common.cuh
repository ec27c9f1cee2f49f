// Building blocks shared by the tensor-core span attention kernels (forward and backward):
// cp.async / ldmatrix / mma.sync wrappers and the tile-local view of the tree.
//
// A CTA works on an aligned tile of 64 leaves with 4 warps of 16 leaves each.  Its key/value rows in
// shared memory are: the leaf band, then the tree nodes inside the tile's subtree (levels 1..5; only
// left children when causal, since right children are never attended causally), then one node per
// level >= 6 (the sibling of the tile's ancestor, shared by all 64 leaves).
#pragma once

#include <type_traits>

#include "hsa_common.cuh"

namespace hsa {

constexpr int kTile = 64;       // leaves per CTA
constexpr int kTileLog = 6;
constexpr int kChunk = 3;       // 16-key blocks scored together before one softmax update

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
    const int sz = valid ? 16 : 0;   // src-size 0 zero-fills the 16 bytes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    } else {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
}

// ---- tile-local tree storage ------------------------------------------------------------------
// In-tile nodes of levels 1..5 are stored level after level; causal tiles keep only even nodes.
template <bool CAUSAL> __device__ __forceinline__ constexpr int tree_in_rows() { return CAUSAL ? 31 : 62; }
template <bool CAUSAL> __device__ __forceinline__ int tree_level_off(int l) {   // l in 1..5
    return CAUSAL ? 32 - (64 >> l) : 64 - (128 >> l);
}

// Tree key slot s of warp w -> (level, row inside the tile's tree storage).  Slots enumerate the nodes of
// levels 1..3 below the warp's 16 leaves, then one node per level 4, 5, ... (the sibling of the warp's
// ancestor).  Returns the level, or -1 past the last level.  `row` always names a staged, finite row.
template <bool CAUSAL>
__device__ __forceinline__ int tree_slot(int s, int w, int L, int &row, int &jj) {
    if (CAUSAL) {
        if (s < 4) { jj = 2 * s; row = 4 * w + s; return 1; }
        if (s < 6) { jj = 2 * (s - 4); row = 16 + 2 * w + (s - 4); return 2; }
        if (s == 6) { jj = 0; row = 24 + w; return 3; }
        if (s == 7) { jj = 0; row = 28 + (w >> 1); return 4; }          // node w^1, stored when even
        if (s == 8) { jj = 0; row = 30; return 5; }                      // node (w>>1)^1 = 0 when needed
        const int l = s - 3;
        jj = 0;
        if (l >= L) { row = 0; return -1; }
        row = 31 + (l - kTileLog);
        return l;
    } else {
        if (s < 8) { jj = s; row = 8 * w + s; return 1; }
        if (s < 12) { jj = s - 8; row = 32 + 4 * w + (s - 8); return 2; }
        if (s < 14) { jj = s - 12; row = 48 + 2 * w + (s - 12); return 3; }
        if (s == 14) { jj = 0; row = 56 + (w ^ 1); return 4; }
        if (s == 15) { jj = 0; row = 60 + ((w >> 1) ^ 1); return 5; }
        const int l = s - 10;
        jj = 0;
        if (l >= L) { row = 0; return -1; }
        row = 62 + (l - kTileLog);
        return l;
    }
}

template <bool CAUSAL> __device__ __forceinline__ int tree_slots(int L) { return (CAUSAL ? 3 : 10) + L; }

// Ordered block index o of a warp -> what it holds.  Order: the band block with the leaves themselves
// first (so the running maximum is finite from the start), then the other band blocks, then tree blocks.
struct BlockRef {
    bool band;
    int idx;    // band block index (0 = leftmost) or tree block index
};
template <bool CAUSAL>
__device__ __forceinline__ BlockRef block_ref(int o, int RB, int nbb) {
    if (o >= nbb) return {false, o - nbb};
    if (o == 0) return {true, RB};
    if (o <= RB) return {true, o - 1};
    return {true, o};
}

// 4x4 transpose inside every quad of lanes.  In: w[t] = this lane's 32-bit word (two columns) of n-tile t of a
// group of four n-tiles.  Out: lane q holds, in order, the words the four lanes had for n-tile q, i.e. eight
// consecutive columns (16 bytes) of one n-tile.  Two butterfly rounds (lane ^ 1, lane ^ 2).
__device__ __forceinline__ void quad_transpose4(uint32_t (&w)[4], int quad) {
    const bool b0 = quad & 1, b1 = quad & 2;
    uint32_t x0 = b0 ? w[0] : w[1], x1 = b0 ? w[2] : w[3];
    x0 = __shfl_xor_sync(0xffffffffu, x0, 1);
    x1 = __shfl_xor_sync(0xffffffffu, x1, 1);
    if (b0) { w[0] = x0; w[2] = x1; } else { w[1] = x0; w[3] = x1; }
    x0 = b1 ? w[0] : w[2];
    x1 = b1 ? w[1] : w[3];
    x0 = __shfl_xor_sync(0xffffffffu, x0, 2);
    x1 = __shfl_xor_sync(0xffffffffu, x1, 2);
    if (b1) { w[0] = x0; w[1] = x1; } else { w[2] = x0; w[3] = x1; }
}

// Store an accumulator block (NT n-tiles of 8 columns, rows qrow and qrow + 8 of a 16-row block) as T to two
// global rows.  After the quad transpose every lane writes 16 contiguous bytes, so one store instruction
// covers 64 contiguous bytes of each of 8 rows instead of 16.  row0 / row1 point at column 0 of the block.
template <typename T, int NT>
__device__ __forceinline__ void store_acc_rows(T *row0, T *row1, const float (&acc)[NT][4], int quad) {
    static_assert(NT % 4 == 0, "n-tiles come in groups of four");
#pragma unroll
    for (int j = 0; j < NT / 4; ++j) {
        uint32_t w0[4], w1[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            w0[t] = pack2<T>(acc[4 * j + t][0], acc[4 * j + t][1]);
            w1[t] = pack2<T>(acc[4 * j + t][2], acc[4 * j + t][3]);
        }
        quad_transpose4(w0, quad);
        quad_transpose4(w1, quad);
        if (row0 != nullptr) *reinterpret_cast<uint4 *>(row0 + (4 * j + quad) * 8) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
        if (row1 != nullptr) *reinterpret_cast<uint4 *>(row1 + (4 * j + quad) * 8) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
    }
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t ldg32(const void *p) { return __ldg(reinterpret_cast<const unsigned int *>(p)); }

}  // namespace hsa
