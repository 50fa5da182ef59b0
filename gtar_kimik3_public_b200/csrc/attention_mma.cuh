// Building blocks of the bfloat16 tensor-core attention kernels: asynchronous copies of a
// page of keys or values into swizzled shared memory, matrix fragments, and the running
// softmax of a 16-row tile.  Scores, maxima, sums and the output accumulator are 32-bit.
#pragma once

#include "common.cuh"

namespace attn {

constexpr int PAGE = 64;  // keys per page (the cache's page size)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16-byte asynchronous copy; `valid` = false writes zeros instead (nothing is read).
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// A tile of rows x D bfloat16 in shared memory, rows of D*2 bytes, 16-byte chunks XOR-swizzled
// with the row so that the eight rows of an ldmatrix fall into different banks.
template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
    return row * (D / 8) + (chunk ^ (row & 7));
}

// Copies `rows` rows (each D bfloat16, contiguous, `src_row_stride` elements apart) into a swizzled
// tile; rows at or beyond `valid_rows` are zero-filled.  All `n_threads` threads of the group take part.
template <int D>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* tile, const __nv_bfloat16* src, size_t src_row_stride,
                                                int rows, int valid_rows, int tid, int n_threads) {
    constexpr int CHUNKS = D / 8;
    for (int c = tid; c < rows * CHUNKS; c += n_threads) {
        const int row = c / CHUNKS, chunk = c % CHUNKS;
        const bool valid = row < valid_rows;
        const __nv_bfloat16* g = src + (valid ? (size_t)row * src_row_stride + chunk * 8 : 0);
        cp_async_16(reinterpret_cast<uint4*>(tile) + swz<D>(row, chunk), g, valid);
    }
}

// A whole page (PAGE rows of D contiguous bfloat16) into a swizzled tile by N_THREADS threads: what the loop over
// a sequence's pages does for every page, so it is written for that case.  A thread copies the same chunk of every
// (N_THREADS / chunks a row)-th row; that distance is a multiple of eight rows, so the swizzle of its chunk is the
// same for all of them and every copy is one instruction at a constant distance from the thread's first, in shared
// and in global memory alike (the general loop above spends some fifteen instructions of index arithmetic a copy,
// half of what a step of sixteen keys executed).  Rows at or beyond `valid_rows` are zero-filled.
template <int D, int N_THREADS>
__device__ __forceinline__ void load_page_async(__nv_bfloat16* tile, const __nv_bfloat16* src, int valid_rows, int tid) {
    constexpr int CHUNKS = D / 8, ROWS_A_PASS = N_THREADS / CHUNKS, PASSES = PAGE / ROWS_A_PASS;
    static_assert(N_THREADS % CHUNKS == 0 && ROWS_A_PASS % 8 == 0 && PAGE % ROWS_A_PASS == 0, "a pass must be whole groups of eight rows");
    const int row0 = tid / CHUNKS, chunk = tid % CHUNKS;
    const uint32_t dst = smem_u32(tile) + (uint32_t)swz<D>(row0, chunk) * 16;
    const __nv_bfloat16* g = src + row0 * D + chunk * 8;
    if (valid_rows >= PAGE) {
#pragma unroll
        for (int i = 0; i < PASSES; ++i)  // the distances become immediates of the instruction
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + i * ROWS_A_PASS * CHUNKS * 16),
                         "l"(g + i * ROWS_A_PASS * D));
    } else {
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const bool valid = row0 + i * ROWS_A_PASS < valid_rows;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst + i * ROWS_A_PASS * CHUNKS * 16),
                         "l"(valid ? g + i * ROWS_A_PASS * D : src), "r"(valid ? 16 : 0));
        }
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// S(16 x 16 keys) = Q(16 x D) K^T for the 16 keys starting at row `key0` of a swizzled K tile.
// q[ks] are the A fragments of Q for the k-step ks.  s[0] holds keys key0..key0+7, s[1] the next 8.
template <int D>
__device__ __forceinline__ void qk_16keys(float (&s)[2][4], const uint32_t (&q)[D / 16][4], const __nv_bfloat16* k_tile,
                                          int key0, int lane) {
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
    // ldmatrix.x4: lanes 0-7 give the rows of matrix 0 (keys 0-7, dims 0-7), 8-15 matrix 1 (keys 0-7, dims 8-15),
    // 16-23 matrix 2 (keys 8-15, dims 0-7), 24-31 matrix 3 (keys 8-15, dims 8-15).
    const int row = key0 + (lane & 7) + ((lane >> 4) << 3);
    const int chunk_in_step = (lane >> 3) & 1;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(b, reinterpret_cast<const uint4*>(k_tile) + swz<D>(row, ks * 2 + chunk_in_step));
        mma_16816(s[0], q[ks], b[0], b[1]);
        mma_16816(s[1], q[ks], b[2], b[3]);
    }
}

// O(16 x D) += P(16 x 16 keys) V(16 keys x D) for the 16 keys starting at row `key0` of a swizzled V tile.
template <int D>
__device__ __forceinline__ void pv_16keys(float (&o)[D / 8][4], const uint32_t (&p)[4], const __nv_bfloat16* v_tile,
                                          int key0, int lane) {
    // ldmatrix.x4.trans: matrix 0 = keys 0-7 x dims 0-7, 1 = keys 8-15 x dims 0-7, 2 = keys 0-7 x dims 8-15,
    // 3 = keys 8-15 x dims 8-15  ->  (b0, b1) of the dim tile 2j and (b0, b1) of the dim tile 2j+1.
    const int row = key0 + (lane & 7) + (((lane >> 3) & 1) << 3);
    const int chunk_in_pair = lane >> 4;
#pragma unroll
    for (int j = 0; j < D / 16; ++j) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, reinterpret_cast<const uint4*>(v_tile) + swz<D>(row, j * 2 + chunk_in_pair));
        mma_16816(o[2 * j], p, b[0], b[1]);
        mma_16816(o[2 * j + 1], p, b[2], b[3]);
    }
}

// The same two products for a loop over pages: the tile is given by its 32-bit shared-memory address and the lane's
// place in it by a byte offset that the caller forms once (`k_lane_offset`, `v_lane_offset`).  The chunk of a later
// k-step (or pair of dim tiles) differs from the first one's by an XOR inside the offset, (2 ks) ^ c ^ (row & 7) =
// (2 ks) ^ (c ^ (row & 7)), so nothing of the index arithmetic is left in the loop but one addition an ldmatrix.
template <int D>
__device__ __forceinline__ uint32_t k_lane_offset(int key0, int lane) {
    return (uint32_t)swz<D>(key0 + (lane & 7) + ((lane >> 4) << 3), (lane >> 3) & 1) * 16;
}
template <int D>
__device__ __forceinline__ uint32_t v_lane_offset(int key0, int lane) {
    return (uint32_t)swz<D>(key0 + (lane & 7) + (((lane >> 3) & 1) << 3), lane >> 4) * 16;
}
__device__ __forceinline__ void ldmatrix_x4_at(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_at(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
template <int D>
__device__ __forceinline__ void qk_16keys_at(float (&s)[2][4], const uint32_t (&q)[D / 16][4], uint32_t k_tile, uint32_t offset) {
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t b[4];
        ldmatrix_x4_at(b, k_tile + (offset ^ (uint32_t)(ks * 32)));
        mma_16816(s[0], q[ks], b[0], b[1]);
        mma_16816(s[1], q[ks], b[2], b[3]);
    }
}
template <int D>
__device__ __forceinline__ void pv_16keys_at(float (&o)[D / 8][4], const uint32_t (&p)[4], uint32_t v_tile, uint32_t offset) {
#pragma unroll
    for (int j = 0; j < D / 16; ++j) {
        uint32_t b[4];
        ldmatrix_x4_trans_at(b, v_tile + (offset ^ (uint32_t)(j * 32)));
        mma_16816(o[2 * j], p, b[0], b[1]);
        mma_16816(o[2 * j + 1], p, b[2], b[3]);
    }
}

// 2^x by the hardware's approximation alone (relative error 2^-22; results below the normal range become zero, which
// is what a probability that small is to a sum of 32-bit numbers): exp2f() wraps the same instruction in a range
// check and two scalings, three more instructions for each of a step's exponentials.
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Running softmax over a 16-row tile.  A thread owns rows r0 = lane/4 and r0 + 8; index h = 0, 1.
// Scores arrive raw; `sl2` = scale * log2(e).  Entries already set to -inf are masked.
template <int D>
__device__ __forceinline__ void softmax_update(float (&s)[2][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                               uint32_t (&p)[4], float sl2) {
    float corrs[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[h], mx * sl2);
        // a row that has seen no visible key yet keeps m = -inf; use 0 as the reference so exp2 gives 0, not NaN
        const float ref = m_new == -INFINITY ? 0.f : m_new;
        const float corr = m[h] == ref ? 1.f : exp2_fast(m[h] - ref);  // exactly one where the maximum stays
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float e = exp2_fast(fmaf(s[n][2 * h + c], sl2, -ref));
                s[n][2 * h + c] = e;
                sum += e;
            }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[h] = l[h] * corr + sum;
        m[h] = m_new;
        corrs[h] = corr;
    }
    // The accumulator is rescaled only where some row of the warp has a new maximum: a factor of exactly one changes
    // nothing, and after a sequence's first keys that is the usual case (64 multiplications of every 16 keys' 250
    // instructions).
    if (__any_sync(0xffffffffu, corrs[0] != 1.f || corrs[1] != 1.f)) {
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            o[j][0] *= corrs[0];
            o[j][1] *= corrs[0];
            o[j][2] *= corrs[1];
            o[j][3] *= corrs[1];
        }
    }
    p[0] = pack_bf16(s[0][0], s[0][1]);
    p[1] = pack_bf16(s[0][2], s[0][3]);
    p[2] = pack_bf16(s[1][0], s[1][1]);
    p[3] = pack_bf16(s[1][2], s[1][3]);
}

// ---- a whole page (64 keys) at a time: one maximum, one rescale of the accumulator per page ----

// S(16 x 64) = Q K^T for the first `n16` groups of 16 keys of a swizzled K page; s[2g], s[2g+1] hold group g.
template <int D, bool FULL>
__device__ __forceinline__ void qk_page(float (&s)[8][4], const uint32_t (&q)[D / 16][4], const __nv_bfloat16* k_tile,
                                        int n16, int lane) {
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.f;
    const int row = (lane & 7) + ((lane >> 4) << 3);
    const int chunk_in_step = (lane >> 3) & 1;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            if (FULL || g < n16) {
                uint32_t b[4];
                ldmatrix_x4(b, reinterpret_cast<const uint4*>(k_tile) + swz<D>(g * 16 + row, ks * 2 + chunk_in_step));
                mma_16816(s[2 * g], q[ks], b[0], b[1]);
                mma_16816(s[2 * g + 1], q[ks], b[2], b[3]);
            }
        }
    }
}

// Running softmax over a 16 x 64 score tile (entries set to -inf are masked); p[g] = the A fragment of group g.
template <int D>
__device__ __forceinline__ void softmax_page(float (&s)[8][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                             uint32_t (&p)[4][4], float sl2) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n) mx = fmaxf(mx, fmaxf(s[n][2 * h], s[n][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[h], mx * sl2);
        const float ref = m_new == -INFINITY ? 0.f : m_new;
        const float corr = m[h] == ref ? 1.f : exp2_fast(m[h] - ref);
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float e = exp2_fast(fmaf(s[n][2 * h + c], sl2, -ref));
                s[n][2 * h + c] = e;
                sum += e;
            }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[h] = l[h] * corr + sum;
        m[h] = m_new;
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            o[j][2 * h] *= corr;
            o[j][2 * h + 1] *= corr;
        }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        p[g][0] = pack_bf16(s[2 * g][0], s[2 * g][1]);
        p[g][1] = pack_bf16(s[2 * g][2], s[2 * g][3]);
        p[g][2] = pack_bf16(s[2 * g + 1][0], s[2 * g + 1][1]);
        p[g][3] = pack_bf16(s[2 * g + 1][2], s[2 * g + 1][3]);
    }
}

// O(16 x D) += P(16 x 64) V for the first `n16` groups of 16 keys of a swizzled V page.
template <int D, bool FULL>
__device__ __forceinline__ void pv_page(float (&o)[D / 8][4], const uint32_t (&p)[4][4], const __nv_bfloat16* v_tile,
                                        int n16, int lane) {
    const int row = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int chunk_in_pair = lane >> 4;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (FULL || g < n16) {
#pragma unroll
            for (int j = 0; j < D / 16; ++j) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, reinterpret_cast<const uint4*>(v_tile) + swz<D>(g * 16 + row, j * 2 + chunk_in_pair));
                mma_16816(o[2 * j], p[g], b[0], b[1]);
                mma_16816(o[2 * j + 1], p[g], b[2], b[3]);
            }
        }
    }
}

}  // namespace attn
