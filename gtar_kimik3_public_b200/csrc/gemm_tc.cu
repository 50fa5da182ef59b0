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

struct GemmParams {
    int rows_a, rows_b, k_blocks;      // k_blocks = ceil(K / BK)
    int k_blocks_per_split;
    void* out;
    long long stride_a, stride_b;      // element strides of OUT for the A index and the B index
    int out_dtype;                     // GK_F32 or GK_BF16
    int epilogue;
    int vector_ok;                     // rows of OUT start on 16-byte boundaries (stride_b == 1 case)
    int swiglu_vector_ok;              // rows of the SwiGLU output start on 16-byte boundaries
    int rows32_ok;                     // rows of a row-major bfloat16 output (plain or SwiGLU) start on 32-byte boundaries
    int a_static, b_static;            // the operand is not written by the kernel before (weights): it may
                                       // be fetched before that kernel has finished
    int* error_flag;
    QkvEpilogue qkv;                   // read when epilogue == EPI_QKV
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

// x * sigmoid(x) with the fast division (two units in the last place of the 32-bit quotient, which is then rounded
// to bfloat16): the exact one is a subroutine of a dozen instructions, and a 2,048-token gate|up product calls
// it 6 million times in its output stage
__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

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

// The output stage for the accumulator columns c_begin .. c_end - 1 of this thread's row (`tile_col0` = B index of
// the tile's first column): whole lines as above where the output is row-major bfloat16 (plain, or SwiGLU over
// neighbouring columns) with aligned rows and the columns are whole, else sixteen at a time, each lane its row.
__device__ __forceinline__ void write_columns(const GemmParams& p, uint32_t t_row, bool have_acc, int row_a, bool a_ok,
                                              int tile_col0, int c_begin, int c_end, int lane) {
    const bool plain = p.epilogue == EPI_STORE && p.stride_b == 1 && p.out_dtype == GK_BF16 && p.rows32_ok;
    const bool swiglu = p.epilogue == EPI_SWIGLU_B && p.stride_b == 1 && p.rows32_ok;
    const int span = plain ? 64 : 128;  // accumulator columns that make 128 bytes of output
    auto load16 = [&](int c, float (&v)[16]) {
        if (have_acc) {
            tmem_ld16(t_row + c, v);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
        }
    };
#pragma unroll 1
    for (int c0 = c_begin; c0 < c_end;) {
        if ((plain || swiglu) && c0 + span <= c_end && tile_col0 + c0 + span <= p.rows_b) {
            uint32_t r[32];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                float v[16];
                if (plain) {
                    load16(c0 + 16 * m, v);
                    pack8(v, r + 8 * m);
                    pack8(v + 8, r + 8 * m + 4);
                } else {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        load16(c0 + 32 * m + 16 * half, v);
                        float o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = silu(v[2 * i]) * v[2 * i + 1];
                        pack8(o, r + 8 * m + 4 * half);
                    }
                }
            }
            swap_pieces<uint32_t, 8>(r, lane);
            const int first_row = row_a - (lane & 3);
            __nv_bfloat16* at = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)first_row * p.stride_a +
                                (plain ? tile_col0 + c0 : (tile_col0 + c0) >> 1) + (lane & 3) * 16;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (first_row + i < p.rows_a) store32(at + (long long)i * p.stride_a, r + 8 * i);
            c0 += span;
        } else {
            float v[16];
            load16(c0, v);
            write_chunk(p, v, row_a, a_ok, tile_col0 + c0, lane);
            c0 += 16;
        }
    }
}

__host__ __device__ constexpr bool split_pushes(int bn) { return bn <= 64; }

template <int BN, int STAGES>
struct alignas(1024) GemmSmem {
    __nv_bfloat16 a[STAGES][BM * BK];
    __nv_bfloat16 b[STAGES][BN * BK];
    uint64_t full[STAGES], empty[STAGES], acc_ready;
    uint32_t tmem_base;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                             const __grid_constant__ CUtensorMap map_b,
                                                             const GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles must start on a 1024-byte boundary
    GemmSmem<BN, STAGES>& sm =
        *reinterpret_cast<GemmSmem<BN, STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;  // a power of two >= 32 (BN is 16, 32, 64, 128 or 256)
    // with K split over a cluster, narrow tiles are summed from a region of their own behind the stages (present
    // only in launches that split K), which the other blocks write into; wide tiles are fetched from the others' stages
    constexpr bool PUSH = split_pushes(BN);
    float* split_sums = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(&sm) + sizeof(GemmSmem<BN, STAGES>));
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
    constexpr uint32_t STAGE_BYTES = (BM + BN) * BK * sizeof(__nv_bfloat16);

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
                if (p.b_static) tma_load_2d(sm.b[i], &map_b, k, tile_b * BN, &sm.full[i]);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                const int k = (kb_begin + i) * BK;
                if (!p.a_static) tma_load_2d(sm.a[i], &map_a, k, tile_a * BM, &sm.full[i]);
                if (!p.b_static) tma_load_2d(sm.b[i], &map_b, k, tile_b * BN, &sm.full[i]);
            }
            issued = pre;
            for (int i = pre; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&sm.empty[s], ((i / STAGES) - 1) & 1);
                if (!ok) break;
                mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(sm.a[s], &map_a, k, tile_a * BM, &sm.full[s]);
                tma_load_2d(sm.b[s], &map_b, k, tile_b * BN, &sm.full[s]);
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
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                ok = mbar_wait(&sm.full[s], (i / STAGES) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(sm.a[s]), b_addr = smem_u32(sm.b[s]);
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
            write_columns(p, t_row, have_acc, row_a, a_ok, tile_b * BN, 0, BN, lane);
        } else {
            const int row_in_tile = quarter * 32 + lane;
            if (PUSH) {
                // split-K, narrow tiles: a row of this block's partial tile goes straight into the shared memory
                // of the block that will sum that row (a region beside its pipeline stages, which its own MMAs may
                // still be reading), as [source block][column][row of the owner's share] float32.  The stores are
                // posted: nobody waits for a trip between SMs, as a block that fetched the others' tiles would.
                const int n_ranks = gridDim.z, rows_per = BM >> (__ffs(n_ranks) - 1);  // the splits are a power of two: no division in the output stage
                const int owner = row_in_tile >> (__ffs(rows_per) - 1), row_local = row_in_tile & (rows_per - 1);  // a power of two
                const uint32_t mine = smem_u32(split_sums) + (uint32_t)((int)blockIdx.z * rows_per * BN + row_local) * 4u;
                uint32_t dst;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(mine), "r"(owner));
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
                    for (int i = 0; i < 16; ++i)
                        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst + (uint32_t)((c0 + i) * rows_per) * 4u), "f"(v[i]) : "memory");
                }
            } else {
                // split-K: this block's partial tile goes to its own shared memory, [column][row] float32,
                // over the pipeline stages (every copy has landed and every MMA has read them by now)
                float* stage = reinterpret_cast<float*>(sm.a[0]);
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
    }
    if (gridDim.z > 1) {
        // every thread of every block of the cluster: the partial tiles are complete and visible
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (warp >= 2) {
            // this block sums rows [rank * rows_per, (rank + 1) * rows_per) of the tile over all blocks
            const int n_ranks = gridDim.z, rank = blockIdx.z;
            const int rows_per = BM >> (__ffs(n_ranks) - 1);
            const uint32_t stage_addr = smem_u32(sm.a[0]);
            const int e = (warp - 2) * 32 + lane;
            // A thread takes four consecutive rows of one column at a time: one 16-byte load from every
            // block's partial tile (all issued before the first is used), added in the order of the
            // splits; two such groups are in flight per thread.
            auto load_parts = [&](int row, int col, float4 (&part)[8]) {
                if (PUSH) {
                    // the others have delivered: every block's share of these rows is in this block's own memory
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        part[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (r < n_ranks)
                            part[r] = *reinterpret_cast<const float4*>(split_sums + r * rows_per * BN + col * rows_per + (row - rank * rows_per));
                    }
                    return;
                }
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
            // (a power of two: rows and columns by shift and mask, since a division is some two hundred cycles of
            // dependent instructions for a warp that has its scheduler to itself)
            const int quads = rows_per / 4, count = quads * BN, quads_shift = __ffs(quads) - 1;
            const bool swiglu = p.epilogue == EPI_SWIGLU_A;
            // 8-byte (plain, bfloat16) / 16-byte (plain, float32) / 4-byte (SwiGLU) stores need aligned rows
            const bool vec = p.stride_a == 1 && !swiglu && ((uintptr_t)out & 15) == 0 &&
                             (p.stride_b * (p.out_dtype == GK_F32 ? 4 : 2)) % 16 == 0;
            // Thread e takes the group of four rows e % quads of the columns e / quads, e / quads + 128 / quads, ...:
            // its rows, and what follows from them, are the same for all its columns.
            constexpr int U = 2;
            const int col_step = 128 >> quads_shift;  // may exceed a narrow tile's width: then some threads have no column
            const int row = rank * rows_per + 4 * (e & (quads - 1)), row_a = tile_a * BM + row;
            const int col0 = e >> quads_shift;
            const bool rows_in = row_a < p.rows_a, four_in = row_a + 3 < p.rows_a;
            (void)count;
            for (int col = col0; col < BN; col += U * col_step) {
                float4 part[U][8];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (col + u * col_step < BN) load_parts(row, col + u * col_step, part[u]);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (col + u * col_step >= BN) continue;
                    const int rb = tile_b * BN + col + u * col_step;
                    if (!rows_in || rb >= p.rows_b) continue;
                    const float4 v = add_up(part[u]);
                    const float vs[4] = {v.x, v.y, v.z, v.w};
                    if (swiglu) {
#pragma unroll
                        for (int i = 0; i < 4; i += 2) {
                            if (row_a + i + 1 < p.rows_a) {
                                const long long at = (long long)((row_a + i) >> 1) * p.stride_a + (long long)rb * p.stride_b;
                                store_out<__nv_bfloat16>(out, at, silu(vs[i]) * vs[i + 1]);
                            }
                        }
                    } else if (vec && four_in) {
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
        if (!PUSH) {
            // nobody leaves while its shared memory may still be read
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS));
    }
}

// One head of the 32 tokens of a warp: `v` holds the HD projection outputs of this lane's token in 32-bit.
// Every lane of the warp calls it (the lanes work on one another's rows); `token_ok` = the lane's row is a token.
// For a head size of 128 the lanes of a quad swap their rows' 16-column pieces first, so that lane 4j + m holds
// the columns 16m .. 16m + 15 and 64 + 16m .. 64 + 16m + 15 (the two partners of the rotation) of the four
// tokens 4j .. 4j + 3: a quad then reads a token's row of the cos and sin tables as whole lines and writes the
// token's head as whole lines, where with a row per lane every load and store of the warp touched 32 lines.
template <int HD>
__device__ __forceinline__ void qkv_head(const QkvEpilogue& e, float (&v)[HD], int token, bool token_ok, int head, int lane) {
    const bool is_q = head < e.n_q, is_k = !is_q && head < e.n_q + e.n_kv;
    if (!is_q && e.k_pages == nullptr) return;  // the same for the whole warp
    const int pos = token_ok ? e.tok_pos[token] : 0;
    __nv_bfloat16* dst = nullptr;
    if (!token_ok) {
    } else if (is_q) {
        dst = e.q_out + ((size_t)token * e.n_q + head) * HD;
    } else {
        const int hk = is_k ? head - e.n_q : head - e.n_q - e.n_kv;
        // the library's pages hold 64 positions: then by shift and mask
        const int page_index = e.page_size == 64 ? pos >> 6 : pos / e.page_size, in_page = e.page_size == 64 ? pos & 63 : pos % e.page_size;
        const int page = e.block_table[(size_t)e.slots[e.tok_seq[token]] * e.max_pages + page_index];
        const size_t at = (((size_t)page * e.n_kv + hk) * e.page_size + in_page) * HD;
        dst = (is_k ? e.k_pages : e.v_pages) + at;
    }
    const bool normed = (is_q || is_k) && e.use_norm, rotated = (is_q || is_k) && e.cos_table != nullptr;
    float inv = 1.0f;
    if (normed) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < HD; ++i) ss += v[i] * v[i];
        inv = rsqrtf(ss / (float)HD + e.eps);
    }
    const void* w = is_q ? e.wq : e.wk;
    auto weight = [&](int i) {
        return e.weights_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]) : reinterpret_cast<const float*>(w)[i];
    };
    const unsigned long long dst_bits = reinterpret_cast<unsigned long long>(dst);
    const int quad = lane & ~3, m = lane & 3;
    if constexpr (HD == 128) {
        swap_pieces<float, 16>(&v[0], lane);
        swap_pieces<float, 16>(&v[64], lane);
        // eight consecutive norm weights from index i (a multiple of 8)
        auto weights8 = [&](int i, float (&out)[8]) {
            if (e.weights_bf16) {
                const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(w) + i);
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&words[j]));
                    out[2 * j] = f.x;
                    out[2 * j + 1] = f.y;
                }
            } else {
                const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i);
                const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + i + 4);
                out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
                out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
            }
        };
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // token quad + i
            float* lo = &v[16 * i];
            float* hi = &v[64 + 16 * i];
            const float inv_i = __shfl_sync(0xffffffffu, inv, quad + i);
            const int pos_i = __shfl_sync(0xffffffffu, pos, quad + i);
            const unsigned long long to = __shfl_sync(0xffffffffu, dst_bits, quad + i);
            const float* cs = e.cos_table + (size_t)pos_i * (HD / 2) + 16 * m;
            const float* sn = e.sin_table + (size_t)pos_i * (HD / 2) + 16 * m;
#pragma unroll
            for (int j0 = 0; j0 < 16; j0 += 8) {
                if (normed) {
                    float wl[8], wh[8];
                    weights8(16 * m + j0, wl);
                    weights8(64 + 16 * m + j0, wh);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        lo[j0 + j] = (lo[j0 + j] * inv_i) * wl[j];
                        hi[j0 + j] = (hi[j0 + j] * inv_i) * wh[j];
                    }
                }
                if (rotated) {
                    float c[8], sv[8];
                    load32(cs + j0, c);
                    load32(sn + j0, sv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float a = lo[j0 + j], b = hi[j0 + j];
                        lo[j0 + j] = a * c[j] - b * sv[j];
                        hi[j0 + j] = b * c[j] + a * sv[j];
                    }
                }
            }
            uint32_t r[8];
            pack8(lo, r);
            pack8(lo + 8, r + 4);
            if (to) store32(reinterpret_cast<__nv_bfloat16*>(to) + 16 * m, r);
            pack8(hi, r);
            pack8(hi + 8, r + 4);
            if (to) store32(reinterpret_cast<__nv_bfloat16*>(to) + 64 + 16 * m, r);
        }
    } else {
        // a head of 64: the partners of the rotation are 32 apart, within a row's 64 columns, so the row is
        // finished by its own lane and only its stores go through the swap
        if (normed) {
#pragma unroll
            for (int i = 0; i < HD; ++i) v[i] = (v[i] * inv) * weight(i);
        }
        if (rotated) {
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
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) pack8(&v[8 * i], r + 4 * i);
        swap_pieces<uint32_t, 8>(r, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const unsigned long long to = __shfl_sync(0xffffffffu, dst_bits, quad + i);
            if (to) store32(reinterpret_cast<__nv_bfloat16*>(to) + 16 * m, r + 8 * i);
        }
    }
}

// The heads of one half (`half` = 0, 1) of a 256-wide tile for the token of this thread's row; `t_row`
// addresses the row's accumulator.  Every lane takes part in the tensor-memory loads; rows beyond the tokens do no more.
template <int HD, int BN>
__device__ __forceinline__ void qkv_tile(const GemmParams& p, uint32_t t_row, int row_a, bool a_ok, int tile_b, int half, int lane) {
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
        qkv_head<HD>(p.qkv, v, row_a, a_ok, head, lane);
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
                if (p.qkv.head_dim == 128) qkv_tile<128, BN>(p, t_row, row_a, a_ok, tile_b, half, lane);
                else qkv_tile<64, BN>(p, t_row, row_a, a_ok, tile_b, half, lane);
            } else {
                write_columns(p, t_row, true, row_a, a_ok, tile_b * BN, half * (BN / 2), (half + 1) * (BN / 2), lane);
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

// ---------------------------------------------------------------- two blocks on one 256 x 256 tile
// The same walk over tiles by pairs of blocks on neighbouring SMs (a cluster of two).  Each block of a pair
// loads its own 128 rows of A and HALF of the tile's 256 rows of B; one thread of the first block issues
// tcgen05.mma.cta_group::2, which multiplies in both SMs at once (M = 256: each block's 128 rows of A against
// all 256 rows of B, read from both blocks' shared memory) and leaves each block's 128 x 256 accumulator in its
// own tensor memory.  A block thus brings in 32 KB per k-block instead of 48 KB for the same 128 x 256 x 64
// product, and six stages instead of four fit in its shared memory: the k-blocks in flight cover the 1.3 us a
// TMA load takes from L2, which four stages of the one-block kernel do not (its MMA thread waits for data half
// of the time).  Loads carry no multicast.  Barriers: `full` lives in the first block and counts both blocks'
// loads; tcgen05.commit arrives on `empty` and `acc_full` in both blocks; the output warps of both blocks
// arrive on the first block's `acc_empty`.
template <int STAGES>
struct alignas(1024) PairSmem {
    __nv_bfloat16 a[STAGES][BM * BK];
    __nv_bfloat16 b[STAGES][BM * BK];  // this block's 128 of the tile's 256 rows of B
    uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t cluster_address(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// arrives on the barrier at this offset in both blocks of the pair once the MMAs issued so far have finished
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int STAGES>
__global__ void __launch_bounds__(PERSISTENT_THREADS, 1) gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                           const __grid_constant__ CUtensorMap map_b,
                                                                           const GemmParams p) {
    constexpr int BN = 256;
    extern __shared__ unsigned char smem_raw[];
    PairSmem<STAGES>& sm = *reinterpret_cast<PairSmem<STAGES>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t TMEM_COLS = 512;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tiles_a = (p.rows_a + 2 * BM - 1) / (2 * BM), tiles_b = (p.rows_b + BN - 1) / BN;  // tiles of 256 x 256
    const int n_tiles = tiles_a * tiles_b;
    const int n_kb = p.k_blocks;
    constexpr int OUTPUT_WARPS = (PERSISTENT_THREADS - 64) / 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.full[s], 2);   // one arrival (with its byte count) from each block's producer
            mbar_init(&sm.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.acc_full[b], 1);
            mbar_init(&sm.acc_empty[b], 2 * OUTPUT_WARPS);  // one arrival per output warp of both blocks
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
    }
    if (warp == 1) {  // in both blocks: the allocation spans the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // both blocks' barriers are initialised before either signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    constexpr uint32_t STAGE_BYTES = 2 * BM * BK * sizeof(__nv_bfloat16);  // what ONE block loads per k-block

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (both blocks): this block's rows of A and its half of B, signalled to the first block
            pdl_wait();
            bool ok = true;
            long long it = 0;
            for (int t = pair; t < n_tiles && ok; t += n_pairs) {
                const int tile_a = t % tiles_a, tile_b = t / tiles_a;
                for (int kb = 0; kb < n_kb && ok; ++kb, ++it) {
                    const int s = (int)(it % STAGES);
                    if (it >= STAGES) ok = mbar_wait(&sm.empty[s], (uint32_t)((it / STAGES) - 1) & 1);
                    if (!ok) break;
                    const uint32_t full = cluster_address(smem_u32(&sm.full[s]), 0);
                    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(full), "r"(STAGE_BYTES) : "memory");
                    tma_load_2d_pair(sm.a[s], &map_a, kb * BK, (tile_a * 2 + (int)rank) * BM, full);
                    tma_load_2d_pair(sm.b[s], &map_b, kb * BK, tile_b * BN + (int)rank * BM, full);
                }
            }
            if (!ok) atomicExch(p.error_flag, 31);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (first block only)
            const uint32_t idesc = umma_idesc(2 * BM, BN);
            bool ok = true;
            long long it = 0;
            int j = 0;
            for (int t = pair; t < n_tiles && ok; t += n_pairs, ++j) {
                const int buf = j & 1;
                if (j >= 2) ok = mbar_wait(&sm.acc_empty[buf], (uint32_t)((j >> 1) - 1) & 1);  // both blocks have drained it
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
                        umma_pair(acc, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc, kb > 0 || k > 0);
                    umma_commit_pair(&sm.empty[s]);
                }
                umma_commit_pair(&sm.acc_full[buf]);
            }
            if (!ok) atomicExch(p.error_flag, 32);
        }
    } else {
        // ---- output warps (both blocks), as in the one-block kernel: this block's 128 rows of the tile
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        pdl_wait();
        bool ok = true;
        int j = 0;
        for (int t = pair; t < n_tiles && ok; t += n_pairs, ++j) {
            const int tile_a = t % tiles_a, tile_b = t / tiles_a, buf = j & 1;
            const int row_a = (tile_a * 2 + (int)rank) * BM + quarter * 32 + lane;
            ok = mbar_wait(&sm.acc_full[buf], (uint32_t)(j >> 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t_row = tmem + buf * BN + ((uint32_t)(quarter * 32) << 16);
            const bool a_ok = row_a < p.rows_a;
            if (p.epilogue == EPI_QKV) {
                if (p.qkv.head_dim == 128) qkv_tile<128, BN>(p, t_row, row_a, a_ok, tile_b, half, lane);
                else qkv_tile<64, BN>(p, t_row, row_a, a_ok, tile_b, half, lane);
            } else {
                write_columns(p, t_row, true, row_a, a_ok, tile_b * BN, half * (BN / 2), (half + 1) * (BN / 2), lane);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                const uint32_t drained = cluster_address(smem_u32(&sm.acc_empty[buf]), 0);
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(drained) : "memory");
            }
        }
        if (!ok && lane == 0) atomicExch(p.error_flag, 33);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // nobody leaves while the other block may still signal it or read its shared memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
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

template <int BN, int STAGES>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    static_assert(STAGES * (BM + BN) * BK * 2 >= BM * BN * 4, "the partial tile must fit in the pipeline stages");
    constexpr size_t split_bytes = split_pushes(BN) ? (size_t)BM * BN * sizeof(float) : 0;
    const size_t smem = sizeof(GemmSmem<BN, STAGES>) + 1024 + (grid.z > 1 ? split_bytes : 0);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)(sizeof(GemmSmem<BN, STAGES>) + 1024 + split_bytes));
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(err));
        configured = true;
    }
    gk_launch_cluster(gemm_tc_kernel<BN, STAGES>, grid, dim3(THREADS), smem, stream, dim3(1, 1, grid.z), ma, mb, p);
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

int g_gemm_pairs = 2;  // 0: never, 1: always, 2: where it is the faster one (large products)

// `mb` must have boxes of 128 rows (each block loads half of a 256-row B tile).
bool use_pairs(int rows_a, int rows_b);

template <int STAGES>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
    const size_t smem = sizeof(PairSmem<STAGES>) + 1024;
    static bool configured = false;
    static int n_sms = 0;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(gemm_tc_pair_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        int device = 0;
        if (err == cudaSuccess) err = cudaGetDevice(&device);
        if (err == cudaSuccess) err = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int n_tiles = ((p.rows_a + 2 * BM - 1) / (2 * BM)) * ((p.rows_b + 255) / 256);
    const int pairs = n_tiles < n_sms / 2 ? n_tiles : n_sms / 2;
    gk_launch_cluster(gemm_tc_pair_kernel<STAGES>, dim3(2 * pairs), dim3(PERSISTENT_THREADS), smem, stream, dim3(2, 1, 1), ma, mb, p);
    GK_CHECK_LAUNCH("gemm_tc_pair");
    return GK_OK;
}

bool use_pairs(int rows_a, int rows_b) {
    if (g_gemm_pairs != 2) return g_gemm_pairs == 1;
    int device = 0, n_sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
    const long long tiles = (long long)((rows_a + 255) / 256) * ((rows_b + 255) / 256);
    return tiles >= 6LL * (n_sms / 2);
}

}  // namespace

// Whether many-token products with wide tiles run as pairs of blocks (tcgen05 cta_group::2): 0 never, 1 always,
// 2 (the default) where there are at least six 256 x 256 tiles per pair of SMs (a whole 4,096-token prompt of the
// 0.6B sizes takes 7.4 ms with single blocks and 7.6 with pairs; from 8,192 tokens on the two are level).  Measured on a B200: 1.35
// against 1.33 PFLOP/s at 8192^3, 1.36 against 1.32 at 4096^3, but 840 against 937 TFLOP/s on the gate|up
// product of a 2,048-token prompt (1.7 tiles per SM: start-up and the last tile's output stage dominate, and
// pairs make both a little longer).  Returns the old setting.
GK_EXPORT int gk_set_gemm_pairs(int mode) {
    const int before = g_gemm_pairs;
    g_gemm_pairs = mode < 0 ? 0 : mode > 2 ? 2 : mode;
    return before;
}

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
    p.rows32_ok = ((uintptr_t)out & 31) == 0 && (stride_a * 2) % 32 == 0;
    p.a_static = a_static;
    p.b_static = b_static;
    p.error_flag = error_flag;
    if (bn == 256 && splits == 1) {
        if (!use_pairs(rows_a, rows_b)) return launch_persistent<256, 4>(ma, mb, p, (cudaStream_t)stream);
        CUtensorMap mb_half;  // boxes of 128 rows: each block of a pair loads half of a B tile
        status = make_map(&mb_half, b, rows_b, k, ldb, BM);
        if (status) return status;
        return launch_pair<6>(ma, mb_half, p, (cudaStream_t)stream);
    }
    dim3 grid((rows_a + BM - 1) / BM, (rows_b + bn - 1) / bn, splits);
    GK_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm_tc: grid too large");
    cudaStream_t s = (cudaStream_t)stream;
    int device = 0, n_sms = 148;
    if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
    const bool one_wave = (long long)grid.x * grid.y * grid.z <= n_sms;
    switch (bn) {
        // skinny products are bound by memory latency: as many bytes in flight per block as fit where every block
        // has an SM of its own; where blocks follow one another on an SM (the output head: 1,187 tiles), two
        // resident blocks with half the ring each, so that one streams while the other starts up or writes out
        case 16: return launch<16, 5>(ma, mb, p, grid, s);
        case 32: return one_wave ? launch<32, 9>(ma, mb, p, grid, s) : launch<32, 5>(ma, mb, p, grid, s);
        case 64: return one_wave ? launch<64, 8>(ma, mb, p, grid, s) : launch<64, 4>(ma, mb, p, grid, s);
        case 128: {
            // one block per SM at most: a deeper ring instead of a second resident block (the k-blocks in flight
            // have to cover the 1.3 us a TMA load takes, and 3 stages of 32 KB cover 0.5 us of MMAs)
            if (one_wave) return launch<128, 6>(ma, mb, p, grid, s);
            return launch<128, 3>(ma, mb, p, grid, s);
        }
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
    GK_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w_qkv & 15) == 0 && ((uintptr_t)wq & 15) == 0 && ((uintptr_t)wk & 15) == 0,
               "gemm_tc_qkv: operands and norm weights must be 16-byte aligned");
    GK_REQUIRE(((uintptr_t)q_out & 31) == 0 && ((uintptr_t)k_pages & 31) == 0 && ((uintptr_t)v_pages & 31) == 0 &&
                   ((uintptr_t)cos_table & 31) == 0 && ((uintptr_t)sin_table & 31) == 0,
               "gemm_tc_qkv: queries, pages and rotary tables must be 32-byte aligned (they are read and written 32 bytes at a time)");
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
    if (!use_pairs(n_tokens, n)) return launch_persistent<256, 4>(ma, mb, p, (cudaStream_t)stream);
    CUtensorMap mb_half;
    status = make_map(&mb_half, w_qkv, n, k, k, BM);
    if (status) return status;
    return launch_pair<6>(ma, mb_half, p, (cudaStream_t)stream);
}
