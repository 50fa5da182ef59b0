// bfloat16 matrix product on the 5th-generation tensor cores:  OUT[a, b] = sum_k A[a, k] * B[b, k]
// for two K-major operands (every projection of the model is  y = x W^T  with x [M, K] and W [N, K],
// src/layers/attention.py:62-65, src/layers/swiglu.py:9-11, so either may be "A").
//
//   prefill  (many tokens):  A = activations, B = weights   -> OUT row-major [M, N]
//   decode   (M <= 64):      A = weights,     B = activations (swap-AB: the 128 rows of the MMA are
//                            filled by weight rows, the few tokens sit on the MMA's N)  -> OUT^T
//
// One block computes a 128 x BN tile.  Operands come in through TMA (cp.async.bulk.tensor, 128-byte
// swizzle, no multicast) into a ring of shared-memory stages guarded by mbarriers; one elected thread
// issues tcgen05.mma with the accumulator in tensor memory; four warps read the accumulator back
// with tcgen05.ld and write the result.  Warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2-5 = epilogue.  Accumulation is 32-bit.
//
// Epilogues: plain store (bfloat16 or float32) and SwiGLU over row pairs (gate and up rows
// interleaved: even index = gate, odd = up, src/layers/swiglu.py:14).  With split-K (2, 4 or 8
// ways) the blocks of one tile form a thread-block cluster: each leaves its float32 partial tile in
// its own shared memory, and after a cluster barrier every block sums one slice of the tile over all
// blocks through distributed shared memory, in the order of the splits, and writes that slice.
//
// Every wait on an mbarrier is bounded: after GK_SPIN_LIMIT polls the thread records a code in
// *error_flag and leaves its loop; the block still drains its own copies, frees its tensor memory
// and returns.

#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;     // rows of A per tile = MMA M
constexpr int BK = 64;      // k elements per stage = one 128-byte swizzle row
constexpr int UMMA_K = 16;  // k per tcgen05.mma for 16-bit inputs
constexpr int THREADS = 192;
constexpr uint32_t GK_SPIN_LIMIT = 1u << 24;

enum Epilogue : int { EPI_STORE = 0, EPI_SWIGLU_A = 1, EPI_SWIGLU_B = 2, EPI_QKV = 3 };

// The attention input stage done where the packed q|k|v projection leaves the tensor cores (many-token
// orientation only: a thread owns one token's row of the tile, hence whole heads): per-head RMSNorm of
// q and k, rotation by the token's position, queries to `q_out`, keys and values into the token's
// place in the pages (src/layers/attention.py:82-89; src/layers/rmsnorm.py:11-16; src/layers/rope.py:17-33).
struct QkvEpilogue {
    int n_q, n_kv, head_dim;
    const void* wq;
    const void* wk;
    int weights_bf16, use_norm;
    float eps;
    const float* cos_table;   // [positions][head_dim / 2]; null = no rotation
    const float* sin_table;
    const int* tok_pos;
    const int* tok_seq;
    const int* slots;
    const int* block_table;
    int max_pages, page_size;
    __nv_bfloat16* q_out;     // [tokens][n_q][head_dim]
    __nv_bfloat16* k_pages;   // null = this layer writes no keys and values
    __nv_bfloat16* v_pages;
};

// The B operand of a skinny product made inside the kernel from the residual stream: x = RMSNorm(h + delta)
// (src/layers/rmsnorm.py:11-16, src/models/transformer.py:47-48), for up to 16 tokens.  Every block reads
// the tokens' whole rows (a few tens of kilobytes from L2) to get the row's mean square, normalises the
// K range it works on straight into shared memory in the MMA's layout, and the blocks of the first tile
// write h + delta back (to `h_out`, another buffer than `h`: other blocks still read `h`).
struct NormInput {
    const float* h;                 // [rows_b][k]; null = B comes through TMA as usual
    const __nv_bfloat16* delta;     // [rows_b][k] or null
    const void* weight;             // norm weight [k]
    int weight_bf16;
    float eps;
    float* h_out;                   // [rows_b][k]
};

// The residual add and the first half of the next RMSNorm done where a skinny product (A = weights) is
// written (src/models/transformer.py:47-48, src/layers/rmsnorm.py:11-16):  h += OUT (32-bit, in place),
// xw = bfloat16(h * weight) and, per token, this block's share of sum(h^2) in `ss[token][partial]`.  The next
// product reads xw and multiplies its own output rows by rsqrt(sum(ss) / size + eps) (RowScale).
struct ResidualOutput {
    float* h;                       // [rows_b][rows_a]
    const void* weight;             // the next norm's weight [rows_a]
    int weight_bf16;
    __nv_bfloat16* xw;              // [rows_b][rows_a]
    float* ss;                      // [rows_b][n_partials], n_partials = tiles along A * splits
    int n_partials;
};

struct RowScale {
    const float* ss;                // [rows_b][n_partials]
    int n_partials;
    float eps, inv_size;            // 1 / (width of the normalised rows)
};

enum Mode : int { MODE_PLAIN = 0, MODE_NORMED = 1, MODE_RESIDUAL = 2, MODE_SCALED = 3 };

struct GemmParams {
    int rows_a, rows_b, k_blocks;      // k_blocks = ceil(K / BK)
    int k_blocks_per_split;
    void* out;
    long long stride_a, stride_b;      // element strides of OUT for the A index and the B index
    int out_dtype;                     // GK_F32 or GK_BF16
    int epilogue;
    int vector_ok;                     // rows of OUT start on 16-byte boundaries (stride_b == 1 case)
    int swiglu_vector_ok;              // rows of the SwiGLU output start on 16-byte boundaries
    int a_static, b_static;            // the operand is not written by the kernel before (weights): it may
                                       // be fetched before that kernel has finished
    int* error_flag;
    QkvEpilogue qkv;                   // read when epilogue == EPI_QKV
    NormInput norm;                    // MODE_NORMED (BN = 16 only)
    ResidualOutput residual;           // MODE_RESIDUAL
    RowScale scale;                    // MODE_SCALED
    int k_total;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < GK_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the 128-byte
// swizzle: start address / 16, leading byte offset 1 (unused for swizzled K-major), stride byte
// offset 1024 / 16 between groups of eight rows, descriptor version 1, layout type SWIZZLE_128B = 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: float32 accumulator, bfloat16 A and B, both K-major, M x N.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float weight_at(const void* w, int is_bf16, int i) {
    return is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]) : reinterpret_cast<const float*>(w)[i];
}

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }

template <typename T>
__device__ __forceinline__ void store_out(void* out, long long index, float v) {
    reinterpret_cast<T*>(out)[index] = from_float<T>(v);
}

// The output stage for sixteen consecutive B indices (col0 .. col0 + 15) of the A index `row_a`.
__device__ __forceinline__ void write_chunk(const GemmParams& p, float (&v)[16], int row_a, bool a_ok, int col0, int lane) {
    char* out = reinterpret_cast<char*>(p.out);
    if (p.epilogue == EPI_STORE && p.stride_b == 1 && a_ok && col0 + 16 <= p.rows_b && p.vector_ok) {
        // sixteen consecutive outputs of one row: 32 bytes (bfloat16) or 64 bytes (float32) in 16-byte stores
        const long long at = (long long)row_a * p.stride_a + col0;
        if (p.out_dtype == GK_F32) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + at);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint4 w;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]);
                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]);
                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
                w.x = *reinterpret_cast<uint32_t*>(&h0);
                w.y = *reinterpret_cast<uint32_t*>(&h1);
                w.z = *reinterpret_cast<uint32_t*>(&h2);
                w.w = *reinterpret_cast<uint32_t*>(&h3);
                dst[i] = w;
            }
        }
    } else if (p.epilogue == EPI_STORE) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int rb = col0 + i;
            if (a_ok && rb < p.rows_b) {
                const long long at = (long long)row_a * p.stride_a + (long long)rb * p.stride_b;
                if (p.out_dtype == GK_F32) store_out<float>(out, at, v[i]);
                else store_out<__nv_bfloat16>(out, at, v[i]);
            }
        }
    } else if (p.epilogue == EPI_SWIGLU_A) {
        // gate and up alternate along A (TMEM lanes): even lane = gate, odd lane = up of channel row_a / 2
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 1);
            const int rb = col0 + i;
            if ((lane & 1) == 0 && a_ok && rb < p.rows_b) {
                const long long at = (long long)(row_a >> 1) * p.stride_a + (long long)rb * p.stride_b;
                store_out<__nv_bfloat16>(out, at, silu(v[i]) * other);
            }
        }
    } else if (a_ok && col0 + 16 <= p.rows_b && p.stride_b == 1 && p.swiglu_vector_ok) {
        // gate and up alternate along B (TMEM columns): eight outputs, one 16-byte store
        const long long at = (long long)row_a * p.stride_a + (col0 >> 1);
        uint4 w;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(silu(v[0]) * v[1], silu(v[2]) * v[3]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(silu(v[4]) * v[5], silu(v[6]) * v[7]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(silu(v[8]) * v[9], silu(v[10]) * v[11]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(silu(v[12]) * v[13], silu(v[14]) * v[15]);
        w.x = *reinterpret_cast<uint32_t*>(&h0);
        w.y = *reinterpret_cast<uint32_t*>(&h1);
        w.z = *reinterpret_cast<uint32_t*>(&h2);
        w.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + at) = w;
    } else {
        // gate and up alternate along B (TMEM columns)
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            const int rb = col0 + i;
            if (a_ok && rb + 1 < p.rows_b) {
                const long long at = (long long)row_a * p.stride_a + (long long)(rb >> 1) * p.stride_b;
                store_out<__nv_bfloat16>(out, at, silu(v[i]) * v[i + 1]);
            }
        }
    }
}

template <int BN, int STAGES>
struct alignas(1024) GemmSmem {
    __nv_bfloat16 a[STAGES][BM * BK];
    __nv_bfloat16 b[STAGES][BN * BK];
    uint64_t full[STAGES], empty[STAGES], acc_ready, b_ready;
    uint32_t tmem_base;
};

template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                             const __grid_constant__ CUtensorMap map_b,
                                                             const GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles must start on a 1024-byte boundary
    GemmSmem<BN, STAGES>& sm =
        *reinterpret_cast<GemmSmem<BN, STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;  // a power of two >= 32 (BN is 16, 32, 64, 128 or 256)
    constexpr bool NORMED = MODE == MODE_NORMED;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_a = blockIdx.x, tile_b = blockIdx.y, split = blockIdx.z;
    const int kb_begin = split * p.k_blocks_per_split;
    const int kb_end = min(kb_begin + p.k_blocks_per_split, p.k_blocks);
    const int n_kb = max(kb_end - kb_begin, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.acc_ready, 1);
        if (NORMED) mbar_init(&sm.b_ready, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = sm.tmem_base;
    constexpr bool b_normed = NORMED;  // B is made here from the residual stream; TMA brings A only
    // the normalised B tiles of this block's K range, one [BN rows][128 bytes] tile per k-block, after the stages
    __nv_bfloat16* b_tiles = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(&sm) + sizeof(GemmSmem<BN, STAGES>));
    // the same place in the other modes: per-token scales (MODE_SCALED), shares of the sums of squares (MODE_RESIDUAL)
    float* extra = reinterpret_cast<float*>(b_tiles);
    const uint32_t STAGE_BYTES = (b_normed ? BM : BM + BN) * BK * sizeof(__nv_bfloat16);

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: stream A and B tiles of each k-block into the ring
            int issued = 0;
            bool ok = true;
            // the first ring of stages: what does not depend on the kernel before is fetched at once,
            // the rest after that kernel has finished
            const int pre = min(STAGES, n_kb);
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(&sm.full[i], STAGE_BYTES);
                const int k = (kb_begin + i) * BK;
                if (p.a_static) tma_load_2d(sm.a[i], &map_a, k, tile_a * BM, &sm.full[i]);
                if (p.b_static && !b_normed) tma_load_2d(sm.b[i], &map_b, k, tile_b * BN, &sm.full[i]);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                const int k = (kb_begin + i) * BK;
                if (!p.a_static) tma_load_2d(sm.a[i], &map_a, k, tile_a * BM, &sm.full[i]);
                if (!p.b_static && !b_normed) tma_load_2d(sm.b[i], &map_b, k, tile_b * BN, &sm.full[i]);
            }
            issued = pre;
            for (int i = pre; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&sm.empty[s], ((i / STAGES) - 1) & 1);
                if (!ok) break;
                mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(sm.a[s], &map_a, k, tile_a * BM, &sm.full[s]);
                if (!b_normed) tma_load_2d(sm.b[s], &map_b, k, tile_b * BN, &sm.full[s]);
                issued = i + 1;
            }
            if (!ok) {
                atomicExch(p.error_flag, 1);
                // drain: copies already issued must land before this block's shared memory is given up
                for (int i = max(issued - STAGES, 0); i < issued; ++i) mbar_wait(&sm.full[i % STAGES], (i / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            const uint32_t idesc = umma_idesc(BM, BN);
            bool ok = true;
            if (b_normed && n_kb > 0) ok = mbar_wait(&sm.b_ready, 0);  // the epilogue warps have made the B tiles
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&sm.full[s], (i / STAGES) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(sm.a[s]);
                const uint32_t b_addr = b_normed ? smem_u32(b_tiles + (size_t)i * BN * BK) : smem_u32(sm.b[s]);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t da = umma_desc(a_addr + k * UMMA_K * 2), db = umma_desc(b_addr + k * UMMA_K * 2);
                    umma(tmem_acc, da, db, idesc, i > 0 || k > 0);
                }
                umma_commit(&sm.empty[s]);  // the stage is free once these MMAs have read it
            }
            if (!ok) atomicExch(p.error_flag, 2);
            umma_commit(&sm.acc_ready);  // arrives when every MMA issued above has finished
        }
    } else {
        // ---- epilogue warps 2..5: TMEM lane quarter = warp % 4
        const int quarter = warp & 3;
        const int row_a = tile_a * BM + quarter * 32 + lane;
        bool ok = true;
        if constexpr (NORMED) {
            // x = RMSNorm(h + delta) for this block's K range, straight into the MMA's shared-memory layout.
            // Eight threads a token: first the whole row's sum of squares, then the range.
            pdl_wait();
            // `tpr` threads a token (a power of two, at most a warp), so that all 128 threads are busy for
            // 4 to 16 tokens; a thread's loads are issued eight chunks of four at a time
            const int e = (warp - 2) * 32 + lane;
            const int rows_pad = p.rows_b <= 4 ? 4 : p.rows_b <= 8 ? 8 : 16;
            const int tpr = 128 / rows_pad;           // 32, 16 or 8
            const int m = e / tpr, part = e % tpr;
            const int K = p.k_total;
            const bool row_ok = m < p.rows_b;
            const float* hrow = p.norm.h + (size_t)m * K;
            const __nv_bfloat16* drow = p.norm.delta ? p.norm.delta + (size_t)m * K : nullptr;
            auto load_sum = [&](int c, float (&v)[4]) {  // h + delta at columns c .. c+3
                const float4 hv = *reinterpret_cast<const float4*>(hrow + c);
                v[0] = hv.x; v[1] = hv.y; v[2] = hv.z; v[3] = hv.w;
                if (drow) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(drow + c);
                    const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v[0] += d0.x; v[1] += d0.y; v[2] += d1.x; v[3] += d1.y;
                }
            };
            float ss = 0.f;
            if (row_ok) {
                const int step = tpr * 4;
                for (int c0 = part * 4; c0 < K; c0 += 8 * step) {
                    float v[8][4];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int c = c0 + u * step;
                        if (c < K) load_sum(c, v[u]);
                        else v[u][0] = v[u][1] = v[u][2] = v[u][3] = 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) ss += v[u][0] * v[u][0] + v[u][1] * v[u][1] + v[u][2] * v[u][2] + v[u][3] * v[u][3];
                }
            }
            for (int o = 1; o < tpr; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = 1.0f / sqrtf(ss / (float)K + p.norm.eps);
            const int k_lo = kb_begin * BK, k_hi = min(kb_end * BK, K);
            const bool write_h = tile_a == 0 && tile_b == 0 && p.norm.h_out != nullptr;
            if (m < BN) {
                // the block's own K range, again eight chunks at a time (the values are in L1 from the pass
                // above): all loads of a batch are issued before the first is used
                const int step = tpr * 4;
                for (int c0 = k_lo + part * 4; c0 < kb_end * BK; c0 += 8 * step) {
                    float v[8][4], wv[8][4];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int c = c0 + u * step;
                        if (row_ok && c < k_hi) {
                            load_sum(c, v[u]);
                            if (p.norm.weight_bf16) {
                                const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.norm.weight) + c);
                                const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                                const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                                wv[u][0] = w0.x; wv[u][1] = w0.y; wv[u][2] = w1.x; wv[u][3] = w1.y;
                            } else {
                                const float4 w4 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm.weight) + c);
                                wv[u][0] = w4.x; wv[u][1] = w4.y; wv[u][2] = w4.z; wv[u][3] = w4.w;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 4; ++j) v[u][j] = wv[u][j] = 0.f;
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int c = c0 + u * step;
                        if (c >= kb_end * BK) continue;
                        if (write_h && row_ok && c < k_hi)
                            *reinterpret_cast<float4*>(p.norm.h_out + (size_t)m * K + c) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
                        float x[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) x[j] = (v[u][j] * inv) * wv[u][j];
                        // element (row m, column col) of k-block kb: 128-byte rows, 16-byte chunks XOR-swizzled with the row
                        const int kb = (c - k_lo) / BK, col = (c - k_lo) % BK;
                        __nv_bfloat16* tile = b_tiles + (size_t)kb * BN * BK;
                        __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
                        uint2 packed;
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(tile + m * BK + (((col >> 3) ^ (m & 7)) << 3) + (col & 7)) = packed;
                    }
                }
            }
            // rows of the tile beyond the padded token count (tokens <= 8 leave rows 8..15, <= 4 rows 4..15)
            for (int idx = e; idx < (BN - rows_pad) * (kb_end - kb_begin) * (BK / 8); idx += 128) {
                const int chunks_per_kb = (BN - rows_pad) * (BK / 8);
                const int kb = idx / chunks_per_kb, rest = idx % chunks_per_kb;
                const int r = rows_pad + rest / (BK / 8), ch = rest % (BK / 8);
                *reinterpret_cast<uint4*>(b_tiles + (size_t)kb * BN * BK + r * BK + (ch << 3)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.b_ready)) : "memory");
        }
        if constexpr (MODE == MODE_SCALED) {
            // 1 / rms of each token of this tile from the shares the product before left, while the MMAs run:
            // 128 / BN threads a token, each adding every (128 / BN)-th share, then a tree over those threads
            pdl_wait();
            constexpr int TPT = BN >= 128 ? 1 : 128 / BN;
            const int e = (warp - 2) * 32 + lane;
            for (int t0 = 0; t0 < BN; t0 += 128 / TPT) {
                const int local = t0 + e / TPT, part = e % TPT, token = tile_b * BN + local;
                float sum = 0.f;
                if (local < BN && token < p.rows_b) {
                    const float* shares = p.scale.ss + (size_t)token * p.scale.n_partials;
#pragma unroll 4
                    for (int j = part; j < p.scale.n_partials; j += TPT) sum += shares[j];
                }
#pragma unroll
                for (int o = 1; o < TPT; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (part == 0 && local < BN) extra[local] = 1.0f / sqrtf(sum * p.scale.inv_size + p.scale.eps);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (n_kb > 0) {
            ok = mbar_wait(&sm.acc_ready, 0);
            if (!ok && lane == 0) atomicExch(p.error_flag, 3);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_wait();  // the kernel before may still read what is overwritten here
        const bool a_ok = row_a < p.rows_a;
        const bool have_acc = n_kb > 0 && ok;
        const uint32_t t_row = tmem_acc + ((uint32_t)(quarter * 32) << 16);
        if (gridDim.z == 1) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                if (have_acc) {
                    tmem_ld16(t_row + c0, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
                if constexpr (MODE == MODE_SCALED) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] *= extra[c0 + i];
                }
                if constexpr (MODE == MODE_RESIDUAL) {
                    // h += v; xw = h * weight; the warp's 32 rows of every token's square go to extra[col][quarter]
                    const float w = a_ok ? weight_at(p.residual.weight, p.residual.weight_bf16, row_a) : 0.f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int rb = tile_b * BN + c0 + i;
                        float sq = 0.f;
                        if (a_ok && rb < p.rows_b) {
                            const size_t at = (size_t)rb * p.rows_a + row_a;
                            const float hn = p.residual.h[at] + v[i];
                            p.residual.h[at] = hn;
                            p.residual.xw[at] = __float2bfloat16(hn * w);
                            sq = hn * hn;
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        if (lane == 0) extra[(c0 + i) * 4 + quarter] = sq;
                    }
                } else {
                    write_chunk(p, v, row_a, a_ok, tile_b * BN + c0, lane);
                }
            }
            if constexpr (MODE == MODE_RESIDUAL) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int e = (warp - 2) * 32 + lane, token = tile_b * BN + e;
                if (e < BN && token < p.rows_b)
                    p.residual.ss[(size_t)token * p.residual.n_partials + tile_a] =
                        ((extra[e * 4] + extra[e * 4 + 1]) + extra[e * 4 + 2]) + extra[e * 4 + 3];
            }
        } else {
            // split-K: this block's partial tile goes to its own shared memory, [column][row] float32,
            // over the pipeline stages (every copy has landed and every MMA has read them by now)
            float* stage = reinterpret_cast<float*>(sm.a[0]);
            const int row_in_tile = quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                if (have_acc) {
                    tmem_ld16(t_row + c0, v);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) stage[(c0 + i) * BM + row_in_tile] = v[i];
            }
        }
    }
    // MODE_RESIDUAL: the stream and norm weights of the first two groups this thread will finish, fetched while
    // the cluster gathers (they do not depend on the partial tiles)
    float4 pre_h[2], pre_w[2];
    if constexpr (MODE == MODE_RESIDUAL) {
        if (gridDim.z > 1 && warp >= 2 && (p.rows_a & 3) == 0) {
            const int rows_per = BM / (int)gridDim.z, quads = rows_per / 4, count = quads * BN;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int idx = (warp - 2) * 32 + lane + u * 128;
                const int row_a = tile_a * BM + (int)blockIdx.z * rows_per + 4 * (idx % quads), rb = tile_b * BN + idx / quads;
                pre_h[u] = pre_w[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (idx < count && row_a + 3 < p.rows_a && rb < p.rows_b) {
                    pre_h[u] = *reinterpret_cast<const float4*>(p.residual.h + (size_t)rb * p.rows_a + row_a);
                    if (p.residual.weight_bf16) {
                        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.residual.weight) + row_a);
                        const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                        const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                        pre_w[u] = make_float4(w0.x, w0.y, w1.x, w1.y);
                    } else {
                        pre_w[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.residual.weight) + row_a);
                    }
                }
            }
        }
    }
    if (gridDim.z > 1) {
        // every thread of every block of the cluster: the partial tiles are complete and visible
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2) {
            // this block sums rows [rank * rows_per, (rank + 1) * rows_per) of the tile over all blocks
            const int n_ranks = gridDim.z, rank = blockIdx.z;
            const int rows_per = BM / n_ranks;
            const uint32_t stage_addr = smem_u32(sm.a[0]);
            const int e = (warp - 2) * 32 + lane;
            // A thread takes four consecutive rows of one column at a time: one 16-byte load from every
            // block's partial tile (all issued before the first is used), added in the order of the
            // splits; two such groups are in flight per thread.
            auto load_parts = [&](int row, int col, float4 (&part)[8]) {
                const uint32_t local = stage_addr + (uint32_t)(col * BM + row) * 4u;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    part[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (r < n_ranks) {
                        uint32_t remote;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(r));
                        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(part[r].x), "=f"(part[r].y), "=f"(part[r].z), "=f"(part[r].w)
                                     : "r"(remote)
                                     : "memory");
                    }
                }
            };
            auto add_up = [&](const float4 (&part)[8]) {
                float4 acc = part[0];
#pragma unroll
                for (int r = 1; r < 8; ++r)
                    if (r < n_ranks) {
                        acc.x += part[r].x;
                        acc.y += part[r].y;
                        acc.z += part[r].z;
                        acc.w += part[r].w;
                    }
                return acc;
            };
            char* out = reinterpret_cast<char*>(p.out);
            const int quads = rows_per / 4, count = quads * BN;
            const bool swiglu = p.epilogue == EPI_SWIGLU_A;
            // 8-byte (plain, bfloat16) / 16-byte (plain, float32) / 4-byte (SwiGLU) stores need aligned rows
            const bool vec = p.stride_a == 1 && !swiglu && ((uintptr_t)out & 15) == 0 &&
                             (p.stride_b * (p.out_dtype == GK_F32 ? 4 : 2)) % 16 == 0;
            constexpr int U = 2;
            for (int base = e; base < count; base += 128 * U) {
                float4 part[U][8];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + u * 128;
                    if (idx < count) load_parts(rank * rows_per + 4 * (idx % quads), idx / quads, part[u]);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int idx = base + u * 128;
                    if (idx >= count) continue;
                    const int row_a = tile_a * BM + rank * rows_per + 4 * (idx % quads), rb = tile_b * BN + idx / quads;
                    if (row_a >= p.rows_a || rb >= p.rows_b) {
                        if constexpr (MODE == MODE_RESIDUAL) extra[(idx / quads) * 16 + idx % quads] = 0.f;
                        continue;
                    }
                    float4 v = add_up(part[u]);
                    if constexpr (MODE == MODE_SCALED) {
                        const float inv = extra[idx / quads];
                        v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
                    }
                    const float vs[4] = {v.x, v.y, v.z, v.w};
                    if constexpr (MODE == MODE_RESIDUAL) {
                        // h += v over four consecutive features of one token; the quad's squares go to extra[col][quad]
                        const size_t at = (size_t)rb * p.rows_a + row_a;
                        float hn[4], sq = 0.f;
                        if (row_a + 3 < p.rows_a && (p.rows_a & 3) == 0) {
                            float4 h4, w4;
                            if (base == e) {
                                h4 = pre_h[u];
                                w4 = pre_w[u];
                            } else {
                                h4 = *reinterpret_cast<const float4*>(p.residual.h + at);
                                w4 = make_float4(weight_at(p.residual.weight, p.residual.weight_bf16, row_a),
                                                 weight_at(p.residual.weight, p.residual.weight_bf16, row_a + 1),
                                                 weight_at(p.residual.weight, p.residual.weight_bf16, row_a + 2),
                                                 weight_at(p.residual.weight, p.residual.weight_bf16, row_a + 3));
                            }
                            hn[0] = h4.x + vs[0]; hn[1] = h4.y + vs[1]; hn[2] = h4.z + vs[2]; hn[3] = h4.w + vs[3];
                            *reinterpret_cast<float4*>(p.residual.h + at) = make_float4(hn[0], hn[1], hn[2], hn[3]);
                            const float w[4] = {w4.x, w4.y, w4.z, w4.w};
                            __nv_bfloat162 lo = __floats2bfloat162_rn(hn[0] * w[0], hn[1] * w[1]);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(hn[2] * w[2], hn[3] * w[3]);
                            uint2 packed;
                            packed.x = *reinterpret_cast<uint32_t*>(&lo);
                            packed.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(p.residual.xw + at) = packed;
#pragma unroll
                            for (int i = 0; i < 4; ++i) sq += hn[i] * hn[i];
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                if (row_a + i < p.rows_a) {
                                    hn[i] = p.residual.h[at + i] + vs[i];
                                    p.residual.h[at + i] = hn[i];
                                    p.residual.xw[at + i] =
                                        __float2bfloat16(hn[i] * weight_at(p.residual.weight, p.residual.weight_bf16, row_a + i));
                                    sq += hn[i] * hn[i];
                                }
                            }
                        }
                        extra[(idx / quads) * 16 + idx % quads] = sq;
                    } else if (swiglu) {
#pragma unroll
                        for (int i = 0; i < 4; i += 2) {
                            if (row_a + i + 1 < p.rows_a) {
                                const long long at = (long long)((row_a + i) >> 1) * p.stride_a + (long long)rb * p.stride_b;
                                store_out<__nv_bfloat16>(out, at, silu(vs[i]) * vs[i + 1]);
                            }
                        }
                    } else if (vec && row_a + 3 < p.rows_a) {
                        const long long at = (long long)row_a + (long long)rb * p.stride_b;
                        if (p.out_dtype == GK_F32) {
                            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at) = v;
                        } else {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                            uint2 w;
                            w.x = *reinterpret_cast<uint32_t*>(&lo);
                            w.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + at) = w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (row_a + i < p.rows_a) {
                                const long long at = (long long)(row_a + i) * p.stride_a + (long long)rb * p.stride_b;
                                if (p.out_dtype == GK_F32) store_out<float>(out, at, vs[i]);
                                else store_out<__nv_bfloat16>(out, at, vs[i]);
                            }
                        }
                    }
                }
            }
        }
        if constexpr (MODE == MODE_RESIDUAL) {
            if (warp >= 2) {
                // this block's share of each token's sum of squares: its quads in order
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int e = (warp - 2) * 32 + lane, token = tile_b * BN + e;
                const int quads = BM / (int)gridDim.z / 4;
                if (e < BN && token < p.rows_b) {
                    float sum = 0.f;
                    for (int q = 0; q < quads; ++q) sum += extra[e * 16 + q];
                    p.residual.ss[(size_t)token * p.residual.n_partials + tile_a * gridDim.z + blockIdx.z] = sum;
                }
            }
        }
        // nobody leaves while its shared memory may still be read
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS));
    }
}

// One token's share of one head: `v` holds the head's HD projection outputs in 32-bit.
template <int HD>
__device__ __forceinline__ void qkv_head(const QkvEpilogue& e, float (&v)[HD], int token, int head) {
    const bool is_q = head < e.n_q, is_k = !is_q && head < e.n_q + e.n_kv;
    const int pos = e.tok_pos[token];
    __nv_bfloat16* dst;
    if (is_q) {
        dst = e.q_out + ((size_t)token * e.n_q + head) * HD;
    } else {
        if (e.k_pages == nullptr) return;
        const int hk = is_k ? head - e.n_q : head - e.n_q - e.n_kv;
        const int page = e.block_table[(size_t)e.slots[e.tok_seq[token]] * e.max_pages + pos / e.page_size];
        const size_t at = (((size_t)page * e.n_kv + hk) * e.page_size + (pos % e.page_size)) * HD;
        dst = (is_k ? e.k_pages : e.v_pages) + at;
    }
    if (is_q || is_k) {
        if (e.use_norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < HD; ++i) ss += v[i] * v[i];
            const float inv = 1.0f / sqrtf(ss / (float)HD + e.eps);
            const void* w = is_q ? e.wq : e.wk;
#pragma unroll
            for (int i = 0; i < HD; ++i) {
                const float wi = e.weights_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i])
                                                : reinterpret_cast<const float*>(w)[i];
                v[i] = (v[i] * inv) * wi;
            }
        }
        if (e.cos_table) {
            const float4* c4 = reinterpret_cast<const float4*>(e.cos_table + (size_t)pos * (HD / 2));
            const float4* s4 = reinterpret_cast<const float4*>(e.sin_table + (size_t)pos * (HD / 2));
#pragma unroll
            for (int i = 0; i < HD / 2; i += 4) {
                const float4 c = c4[i >> 2], sn = s4[i >> 2];
                const float cs[4] = {c.x, c.y, c.z, c.w}, ss4[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float a = v[i + j], b = v[i + j + HD / 2];
                    v[i + j] = a * cs[j] - b * ss4[j];
                    v[i + j + HD / 2] = b * cs[j] + a * ss4[j];
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < HD; i += 8) {
        uint4 w;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[i], v[i + 1]), h1 = __floats2bfloat162_rn(v[i + 2], v[i + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[i + 4], v[i + 5]), h3 = __floats2bfloat162_rn(v[i + 6], v[i + 7]);
        w.x = *reinterpret_cast<uint32_t*>(&h0);
        w.y = *reinterpret_cast<uint32_t*>(&h1);
        w.z = *reinterpret_cast<uint32_t*>(&h2);
        w.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(dst + i) = w;
    }
}

// The heads of one half (`half` = 0, 1) of a 256-wide tile for the token of this thread's row; `t_row`
// addresses the row's accumulator.  Every lane takes part in the tensor-memory loads; rows beyond the tokens do no more.
template <int HD, int BN>
__device__ __forceinline__ void qkv_tile(const GemmParams& p, uint32_t t_row, int row_a, bool a_ok, int tile_b, int half) {
    const int n_heads = p.qkv.n_q + 2 * p.qkv.n_kv;
    constexpr int PER_HALF = BN / HD / 2;  // heads of the tile this warp takes
#pragma unroll 1
    for (int hh = half * PER_HALF; hh < (half + 1) * PER_HALF; ++hh) {
        const int head = tile_b * (BN / HD) + hh;
        if (head >= n_heads) break;  // uniform over the warp
        float v[HD];
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 16) {
            float part[16];
            tmem_ld16(t_row + hh * HD + c0, part);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[c0 + i] = part[i];
        }
        if (a_ok) qkv_head<HD>(p.qkv, v, row_a, head);
    }
}

// ---------------------------------------------------------------- persistent variant for many tokens
// One block per SM walks over 128 x 256 tiles (A index fastest, so the blocks working at the same time
// share their B tiles in L2).  Two accumulators of 256 columns fill the tensor memory: while the
// epilogue warps drain one, the MMA thread already fills the other with the next tile.  No split-K.
template <int BN, int STAGES>
struct alignas(1024) PersistentSmem {
    __nv_bfloat16 a[STAGES][BM * BK];
    __nv_bfloat16 b[STAGES][BN * BK];
    uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
};

constexpr int PERSISTENT_THREADS = 320;  // TMA warp, MMA warp, eight epilogue warps (two per lane quarter)

template <int BN, int STAGES>
__global__ void __launch_bounds__(PERSISTENT_THREADS, 1) gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                        const __grid_constant__ CUtensorMap map_b,
                                                                        const GemmParams p) {
    static_assert(2 * BN <= 512, "two accumulators must fit the tensor memory");
    extern __shared__ unsigned char smem_raw[];
    PersistentSmem<BN, STAGES>& sm =
        *reinterpret_cast<PersistentSmem<BN, STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t TMEM_COLS = 512;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_a = (p.rows_a + BM - 1) / BM, tiles_b = (p.rows_b + BN - 1) / BN;
    const int n_tiles = tiles_a * tiles_b;
    const int n_kb = p.k_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.acc_full[b], 1);
            mbar_init(&sm.acc_empty[b], PERSISTENT_THREADS - 64);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    constexpr uint32_t STAGE_BYTES = (BM + BN) * BK * sizeof(__nv_bfloat16);

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: one stream of k-blocks over all the block's tiles
            pdl_wait();
            bool ok = true;
            long long it = 0, issued = 0;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int tile_a = t % tiles_a, tile_b = t / tiles_a;
                for (int kb = 0; kb < n_kb && ok; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    if (it >= STAGES) ok = mbar_wait(&sm.empty[s], (uint32_t)((it / STAGES) - 1) & 1);
                    if (!ok) break;
                    mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                    tma_load_2d(sm.a[s], &map_a, kb * BK, tile_a * BM, &sm.full[s]);
                    tma_load_2d(sm.b[s], &map_b, kb * BK, tile_b * BN, &sm.full[s]);
                    issued = it + 1;
                }
            }
            if (!ok) {
                atomicExch(p.error_flag, 21);
                for (long long i = issued > STAGES ? issued - STAGES : 0; i < issued; ++i)
                    mbar_wait(&sm.full[i % STAGES], (uint32_t)(i / STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            const uint32_t idesc = umma_idesc(BM, BN);
            bool ok = true;
            long long it = 0;
            int j = 0;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++j) {
                const int buf = j & 1;
                if (j >= 2) ok = mbar_wait(&sm.acc_empty[buf], (uint32_t)((j >> 1) - 1) & 1);  // the epilogue has drained it
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + buf * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    ok = mbar_wait(&sm.full[s], (uint32_t)(it / STAGES) & 1);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma(acc, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, kb > 0 || k > 0);
                    umma_commit(&sm.empty[s]);
                }
                umma_commit(&sm.acc_full[buf]);
            }
            if (!ok) atomicExch(p.error_flag, 22);
        }
    } else {
        // ---- epilogue warps: warp w reads the lanes of quarter w % 4; the two warps of a quarter take
        // one half of the tile's columns each
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        pdl_wait();
        bool ok = true;
        int j = 0;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++j) {
            const int tile_a = t % tiles_a, tile_b = t / tiles_a, buf = j & 1;
            const int row_a = tile_a * BM + quarter * 32 + lane;
            ok = mbar_wait(&sm.acc_full[buf], (uint32_t)(j >> 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t_row = tmem + buf * BN + ((uint32_t)(quarter * 32) << 16);
            const bool a_ok = row_a < p.rows_a;
            if (p.epilogue == EPI_QKV) {
                if (p.qkv.head_dim == 128) qkv_tile<128, BN>(p, t_row, row_a, a_ok, tile_b, half);
                else qkv_tile<64, BN>(p, t_row, row_a, a_ok, tile_b, half);
            } else {
#pragma unroll 1
                for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 16) {
                    float v[16];
                    tmem_ld16(t_row + c0, v);
                    write_chunk(p, v, row_a, a_ok, tile_b * BN + c0, lane);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.acc_empty[buf])) : "memory");
        }
        if (!ok && lane == 0) atomicExch(p.error_flag, 23);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// A K-major matrix [rows, k] of bfloat16 with `ld` elements between rows; boxes of box_rows x 64.
int make_map(CUtensorMap* map, const void* base, int rows, int k, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return gk_fail(GK_CUDA_ERROR, "gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__nv_bfloat16)};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gk_fail(GK_CUDA_ERROR, "gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return GK_OK;
}

constexpr int NORMED_MAX_K_BLOCKS = 16;  // k-blocks of normalised B a block keeps in shared memory

template <int BN, int STAGES, int MODE = MODE_PLAIN>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    static_assert(STAGES * (BM + BN) * BK * 2 >= BM * BN * 4, "the partial tile must fit in the pipeline stages");
    const size_t base = sizeof(GemmSmem<BN, STAGES>) + 1024;
    constexpr size_t EXTRA = MODE == MODE_RESIDUAL ? (size_t)BN * 16 * 4 : MODE == MODE_SCALED ? (size_t)BN * 4 : 0;
    const size_t smem_max = base + (MODE == MODE_NORMED ? (size_t)NORMED_MAX_K_BLOCKS * BN * BK * 2 : EXTRA);
    const size_t smem = base + (MODE == MODE_NORMED ? (size_t)p.k_blocks_per_split * BN * BK * 2 : EXTRA);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(err));
        configured = true;
    }
    gk_launch_cluster(gemm_tc_kernel<BN, STAGES, MODE>, grid, dim3(THREADS), smem, stream, dim3(1, 1, grid.z), ma, mb, p);
    GK_CHECK_LAUNCH("gemm_tc");
    return GK_OK;
}

template <int BN, int STAGES>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
    const size_t smem = sizeof(PersistentSmem<BN, STAGES>) + 1024;
    static bool configured = false;
    static int n_sms = 0;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int device = 0;
        if (err == cudaSuccess) err = cudaGetDevice(&device);
        if (err == cudaSuccess) err = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int n_tiles = ((p.rows_a + BM - 1) / BM) * ((p.rows_b + BN - 1) / BN);
    dim3 grid(n_tiles < n_sms ? n_tiles : n_sms);
    gk_launch(gemm_tc_persistent_kernel<BN, STAGES>, grid, dim3(PERSISTENT_THREADS), smem, stream, ma, mb, p);
    GK_CHECK_LAUNCH("gemm_tc_persistent");
    return GK_OK;
}

}  // namespace

// OUT[a, b] = sum_k A[a, k] B[b, k].  `bn` (16, 32, 64, 128 or 256) is the tile width along B.
// With `splits` = 2, 4 or 8 the K range of a tile is shared by that many blocks (one cluster).  `a_static` / `b_static` mark an operand that no
// kernel earlier in the stream writes (weights): under programmatic dependent launch its first tiles
// are fetched while the kernel before still runs.  `error_flag` is a device int that stays 0 unless a
// wait inside the kernel gave up.
GK_EXPORT int gk_gemm_bf16_tc(const void* a, int rows_a, long long lda, const void* b, int rows_b, long long ldb, int k,
                              void* out, int out_dtype, long long stride_a, long long stride_b, int epilogue, int bn,
                              int splits, int a_static, int b_static, int* error_flag, void* stream) {
    GK_REQUIRE(rows_a > 0 && rows_b > 0 && k > 0, "gemm_tc: bad sizes %d x %d x %d", rows_a, rows_b, k);
    GK_REQUIRE(k % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0,
               "gemm_tc: k and the row strides must be multiples of 8 elements (16 bytes for TMA); got k=%d lda=%lld ldb=%lld",
               k, lda, ldb);
    GK_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)b & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    GK_REQUIRE(GK_VALID_DTYPE(out_dtype), "gemm_tc: bad output dtype");
    GK_REQUIRE(epilogue >= EPI_STORE && epilogue <= EPI_SWIGLU_B, "gemm_tc: bad epilogue %d", epilogue);
    GK_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_tc: splits must be 1, 2, 4 or 8, got %d", splits);
    GK_REQUIRE(splits == 1 || epilogue != EPI_SWIGLU_B, "gemm_tc: split-K does not go with the SwiGLU-over-B epilogue");
    GK_REQUIRE(epilogue == EPI_STORE || out_dtype == GK_BF16, "gemm_tc: the SwiGLU epilogue writes bfloat16");
    GK_REQUIRE(error_flag != nullptr, "gemm_tc: error_flag is required");
    CUtensorMap ma, mb;
    int status = make_map(&ma, a, rows_a, k, lda, BM);
    if (status) return status;
    status = make_map(&mb, b, rows_b, k, ldb, bn);
    if (status) return status;
    GemmParams p = {};
    p.k_total = k;
    p.rows_a = rows_a;
    p.rows_b = rows_b;
    p.k_blocks = (k + BK - 1) / BK;
    p.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    p.out = out;
    p.stride_a = stride_a;
    p.stride_b = stride_b;
    p.out_dtype = out_dtype;
    p.epilogue = epilogue;
    p.vector_ok = stride_b == 1 && ((uintptr_t)out & 15) == 0 && (stride_a * (out_dtype == GK_F32 ? 4 : 2)) % 16 == 0;
    p.swiglu_vector_ok = ((uintptr_t)out & 15) == 0 && (stride_a * 2) % 16 == 0;
    p.a_static = a_static;
    p.b_static = b_static;
    p.error_flag = error_flag;
    if (bn == 256 && splits == 1) return launch_persistent<256, 4>(ma, mb, p, (cudaStream_t)stream);
    dim3 grid((rows_a + BM - 1) / BM, (rows_b + bn - 1) / bn, splits);
    GK_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm_tc: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    switch (bn) {
        // skinny products are bound by memory latency: as many bytes in flight per block as fit
        case 16: return launch<16, 5>(ma, mb, p, grid, s);
        case 32: return launch<32, 9>(ma, mb, p, grid, s);
        case 64: return launch<64, 8>(ma, mb, p, grid, s);
        case 128: return launch<128, 3>(ma, mb, p, grid, s);
        case 256: return launch<256, 4>(ma, mb, p, grid, s);
        default: return gk_fail(GK_BAD_ARGUMENT, "gemm_tc: bn must be 16, 32, 64, 128 or 256, got %d", bn);
    }
}

// The packed q|k|v projection of many tokens with the attention input stage in its epilogue:
// x [n_tokens, k] times w_qkv [(n_q + 2 n_kv) * head_dim, k]^T, then per-head RMSNorm of q and k, rotation,
// queries to q_out [n_tokens, n_q, head_dim], keys and values into the pages (null pages: not written).
// head_dim 64 or 128; runs on the persistent 128 x 256 kernel.
GK_EXPORT int gk_gemm_bf16_tc_qkv(const void* x, int n_tokens, const void* w_qkv, int k, int n_q, int n_kv, int head_dim,
                                  const void* wq, const void* wk, int weight_dtype, int use_norm, float eps,
                                  const float* cos_table, const float* sin_table, int table_positions, int max_position,
                                  const int* tok_pos, const int* tok_seq, const int* slots, const int* block_table,
                                  int max_pages, int page_size, void* q_out, void* k_pages, void* v_pages,
                                  int* error_flag, void* stream) {
    GK_REQUIRE(n_tokens > 0 && k > 0 && k % 8 == 0, "gemm_tc_qkv: bad sizes tokens=%d k=%d", n_tokens, k);
    GK_REQUIRE(head_dim == 64 || head_dim == 128, "gemm_tc_qkv: head_dim %d is not 64 or 128", head_dim);
    GK_REQUIRE(n_q > 0 && n_kv > 0 && page_size > 0 && max_pages > 0, "gemm_tc_qkv: bad head counts or page geometry");
    GK_REQUIRE(GK_VALID_DTYPE(weight_dtype) && (!use_norm || (wq && wk)), "gemm_tc_qkv: bad norm weights");
    GK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "gemm_tc_qkv: cos and sin tables go together");
    GK_REQUIRE(cos_table == nullptr || max_position < table_positions,
               "gemm_tc_qkv: position %d is beyond the rotary table (%d positions)", max_position, table_positions);
    GK_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w_qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 &&
                   ((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0 && ((uintptr_t)cos_table & 15) == 0 &&
                   ((uintptr_t)sin_table & 15) == 0, "gemm_tc_qkv: pointers must be 16-byte aligned");
    GK_REQUIRE(error_flag != nullptr, "gemm_tc_qkv: error_flag is required");
    const int n = (n_q + 2 * n_kv) * head_dim;
    CUtensorMap ma, mb;
    int status = make_map(&ma, x, n_tokens, k, k, BM);
    if (status) return status;
    status = make_map(&mb, w_qkv, n, k, k, 256);
    if (status) return status;
    GemmParams p = {};
    p.rows_a = n_tokens;
    p.rows_b = n;
    p.k_blocks = (k + BK - 1) / BK;
    p.k_blocks_per_split = p.k_blocks;
    p.epilogue = EPI_QKV;
    p.out_dtype = GK_BF16;
    p.b_static = 1;
    p.error_flag = error_flag;
    p.qkv.n_q = n_q;
    p.qkv.n_kv = n_kv;
    p.qkv.head_dim = head_dim;
    p.qkv.wq = wq;
    p.qkv.wk = wk;
    p.qkv.weights_bf16 = weight_dtype == GK_BF16;
    p.qkv.use_norm = use_norm;
    p.qkv.eps = eps;
    p.qkv.cos_table = cos_table;
    p.qkv.sin_table = sin_table;
    p.qkv.tok_pos = tok_pos;
    p.qkv.tok_seq = tok_seq;
    p.qkv.slots = slots;
    p.qkv.block_table = block_table;
    p.qkv.max_pages = max_pages;
    p.qkv.page_size = page_size;
    p.qkv.q_out = (__nv_bfloat16*)q_out;
    p.qkv.k_pages = (__nv_bfloat16*)k_pages;
    p.qkv.v_pages = (__nv_bfloat16*)v_pages;
    return launch_persistent<256, 4>(ma, mb, p, (cudaStream_t)stream);
}

// A skinny product whose activations come straight from the residual stream:
//   OUT[m, :] = RMSNorm(h[m] + delta[m]; norm_weight, eps) @ w^T     for m < n_tokens <= 16,
// and h_out = h + delta.  `w` is [n, k] bfloat16 (rows alternate gate, up with the SwiGLU epilogue);
// `delta` may be null; `h_out` must not alias `h`.  The K range of a tile may be shared by 1, 2, 4 or 8
// blocks (one cluster), each keeping at most 16 k-blocks of 64 of the normalised activations.
GK_EXPORT int gk_gemm_bf16_tc_normed(const void* w, int n, int k, const float* h, const void* delta, int n_tokens,
                                     const void* norm_weight, int norm_weight_dtype, float eps, float* h_out, void* out,
                                     int swiglu, int splits, int* error_flag, void* stream) {
    GK_REQUIRE(n > 0 && k > 0 && k % 8 == 0, "gemm_tc_normed: bad sizes n=%d k=%d", n, k);
    GK_REQUIRE(n_tokens > 0 && n_tokens <= 16, "gemm_tc_normed: takes 1 to 16 tokens, got %d", n_tokens);
    GK_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "gemm_tc_normed: splits must be 1, 2, 4 or 8");
    GK_REQUIRE(GK_VALID_DTYPE(norm_weight_dtype) && norm_weight && h && h_out && h != h_out, "gemm_tc_normed: bad norm inputs");
    GK_REQUIRE(eps > 0.f, "gemm_tc_normed: eps must be positive");
    GK_REQUIRE(((uintptr_t)w & 15) == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)delta & 15) == 0 &&
                   ((uintptr_t)h_out & 15) == 0 && ((uintptr_t)out & 15) == 0, "gemm_tc_normed: pointers must be 16-byte aligned");
    GK_REQUIRE(!swiglu || n % 2 == 0, "gemm_tc_normed: the SwiGLU epilogue needs an even number of weight rows");
    GK_REQUIRE(error_flag != nullptr, "gemm_tc_normed: error_flag is required");
    CUtensorMap ma;
    int status = make_map(&ma, w, n, k, k, BM);
    if (status) return status;
    GemmParams p = {};
    p.k_total = k;
    p.rows_a = n;
    p.rows_b = n_tokens;
    p.k_blocks = (k + BK - 1) / BK;
    p.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    GK_REQUIRE(p.k_blocks_per_split <= NORMED_MAX_K_BLOCKS,
               "gemm_tc_normed: %d k-blocks a block exceed the %d it can keep; use more splits", p.k_blocks_per_split,
               NORMED_MAX_K_BLOCKS);
    p.out = out;
    p.stride_a = 1;
    p.stride_b = swiglu ? n / 2 : n;
    p.out_dtype = GK_BF16;
    p.epilogue = swiglu ? EPI_SWIGLU_A : EPI_STORE;
    p.a_static = 1;
    p.b_static = 0;
    p.error_flag = error_flag;
    p.norm.h = h;
    p.norm.delta = (const __nv_bfloat16*)delta;
    p.norm.weight = norm_weight;
    p.norm.weight_bf16 = norm_weight_dtype == GK_BF16;
    p.norm.eps = eps;
    p.norm.h_out = h_out;
    dim3 grid((n + BM - 1) / BM, 1, splits);
    return launch<16, 5, MODE_NORMED>(ma, ma, p, grid, (cudaStream_t)stream);
}

namespace {

template <int MODE>
int launch_skinny(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t s) {
    switch (bn) {
        case 16: return launch<16, 5, MODE>(ma, mb, p, grid, s);
        case 32: return launch<32, 9, MODE>(ma, mb, p, grid, s);
        case 64: return launch<64, 8, MODE>(ma, mb, p, grid, s);
        default: return gk_fail(GK_BAD_ARGUMENT, "gemm_tc: the token tile of a skinny product is 16, 32 or 64, got %d", bn);
    }
}

int skinny_params(GemmParams& p, CUtensorMap& ma, CUtensorMap& mb, const void* w, int n, int k, const void* x, int n_tokens,
                  long long ldx, int bn, int splits, int* error_flag, const char* who) {
    GK_REQUIRE(n > 0 && k > 0 && k % 8 == 0 && ldx % 8 == 0, "%s: bad sizes n=%d k=%d ldx=%lld (k and ldx in steps of 8)", who, n, k, ldx);
    GK_REQUIRE(n_tokens > 0 && n_tokens <= 64, "%s: takes 1 to 64 tokens, got %d", who, n_tokens);
    GK_REQUIRE((bn == 16 || bn == 32 || bn == 64) && n_tokens <= bn, "%s: token tile %d does not hold %d tokens", who, bn, n_tokens);
    GK_REQUIRE(splits == 1 || splits == 2 || splits == 4 || splits == 8, "%s: splits must be 1, 2, 4 or 8, got %d", who, splits);
    GK_REQUIRE(((uintptr_t)w & 15) == 0 && ((uintptr_t)x & 15) == 0, "%s: operands must be 16-byte aligned", who);
    GK_REQUIRE(error_flag != nullptr, "%s: error_flag is required", who);
    int status = make_map(&ma, w, n, k, k, BM);
    if (status) return status;
    status = make_map(&mb, x, n_tokens, k, ldx, bn);
    if (status) return status;
    p.k_total = k;
    p.rows_a = n;
    p.rows_b = n_tokens;
    p.k_blocks = (k + BK - 1) / BK;
    p.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    p.stride_a = 1;
    p.a_static = 1;
    p.b_static = 0;
    p.error_flag = error_flag;
    return GK_OK;
}

}  // namespace

// A skinny product that ends a branch of a pre-norm block and starts the next norm
// (src/models/transformer.py:47-48, src/layers/rmsnorm.py:11-16), for up to 64 tokens:
//   h[m, :] += x[m, :] @ w^T            (float32, in place)
//   xw[m, :] = bfloat16(h[m, :] * next_weight)
//   ss[m, j] = block j's share of sum(h[m, :]^2),   j < n_partials = ceil(n / 128) * splits.
// The product that follows takes xw and `ss` (gk_gemm_bf16_tc_scaled).
GK_EXPORT int gk_gemm_bf16_tc_residual(const void* w, int n, int k, const void* x, int n_tokens, long long ldx, float* h,
                                       const void* next_weight, int next_weight_dtype, void* xw, float* ss, int n_partials,
                                       int bn, int splits, int* error_flag, void* stream) {
    GemmParams p = {};
    CUtensorMap ma, mb;
    int status = skinny_params(p, ma, mb, w, n, k, x, n_tokens, ldx, bn, splits, error_flag, "gemm_tc_residual");
    if (status) return status;
    GK_REQUIRE(h && next_weight && xw && ss && GK_VALID_DTYPE(next_weight_dtype), "gemm_tc_residual: bad outputs or norm weight");
    GK_REQUIRE(((uintptr_t)h & 15) == 0 && ((uintptr_t)xw & 15) == 0, "gemm_tc_residual: h and xw must be 16-byte aligned");
    dim3 grid((n + BM - 1) / BM, 1, splits);
    GK_REQUIRE(n_partials == (int)grid.x * splits, "gemm_tc_residual: %d shares expected, got room for %d", (int)grid.x * splits,
               n_partials);
    p.stride_b = n;
    p.out_dtype = GK_BF16;
    p.epilogue = EPI_STORE;
    p.residual.h = h;
    p.residual.weight = next_weight;
    p.residual.weight_bf16 = next_weight_dtype == GK_BF16;
    p.residual.xw = (__nv_bfloat16*)xw;
    p.residual.ss = ss;
    p.residual.n_partials = n_partials;
    return launch_skinny<MODE_RESIDUAL>(bn, ma, mb, p, grid, (cudaStream_t)stream);
}

// The product after gk_gemm_bf16_tc_residual:  OUT[m, :] = (xw[m, :] @ w^T) * rsqrt(sum_j ss[m, j] / k + eps),
// which is RMSNorm(h) @ w^T up to the rounding of xw.  `w` is [n, k] bfloat16 (rows alternate gate, up with
// the SwiGLU epilogue, and OUT is [n_tokens, n / 2]); OUT is bfloat16.
GK_EXPORT int gk_gemm_bf16_tc_scaled(const void* w, int n, int k, const void* xw, int n_tokens, long long ldx, const float* ss,
                                     int n_partials, float eps, void* out, int swiglu, int bn, int splits, int* error_flag,
                                     void* stream) {
    GemmParams p = {};
    CUtensorMap ma, mb;
    int status = skinny_params(p, ma, mb, w, n, k, xw, n_tokens, ldx, bn, splits, error_flag, "gemm_tc_scaled");
    if (status) return status;
    GK_REQUIRE(ss && n_partials > 0 && eps > 0.f && out, "gemm_tc_scaled: bad scale inputs");
    GK_REQUIRE(!swiglu || n % 2 == 0, "gemm_tc_scaled: the SwiGLU epilogue needs an even number of weight rows");
    p.out = out;
    p.stride_b = swiglu ? n / 2 : n;
    p.out_dtype = GK_BF16;
    p.epilogue = swiglu ? EPI_SWIGLU_A : EPI_STORE;
    p.scale.ss = ss;
    p.scale.n_partials = n_partials;
    p.scale.eps = eps;
    p.scale.inv_size = 1.0f / (float)k;
    dim3 grid((n + BM - 1) / BM, 1, splits);
    return launch_skinny<MODE_SCALED>(bn, ma, mb, p, grid, (cudaStream_t)stream);
}
