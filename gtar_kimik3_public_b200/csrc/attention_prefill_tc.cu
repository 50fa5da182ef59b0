// Prefill attention on the 5th-generation tensor cores (head size 128).
//
// The same computation as attention_prefill.cu — causal, grouped-query, over the paged cache,
// flash-attention style with 32-bit running maxima and sums (reference: src/ops/flash_attention_2.py:24-60,
// visibility rule src/layers/attention.py:116-119) — with both matrix products on tcgen05.mma:
//
//   S = Q K^T     A = Q tile (128 rows x 128, shared memory), B = K page (64 keys x 128, shared memory)
//                 -> S in tensor memory, 128 lanes x 64 columns
//   O += P V      A = P (bfloat16, written back into tensor memory by the softmax warps)
//                 B = V page (64 keys x 128, shared memory, read with the keys as the MMA's K: "MN-major")
//                 -> O in tensor memory, 128 lanes x 128 columns
//
// A query tile is 128 rows = (token, query head of one kv group) pairs of one sequence and one kv head.  The
// accumulator is rescaled only when a row's maximum has grown by more than 2^8 since its last rescale (the
// probabilities then stay below 2^8, which bfloat16 and the 32-bit sum hold with room to spare), so most steps
// cost no pass over O.  Two kernels:
//
//   * attention_prefill_tc2_kernel, the default: 128 keys (two pages) a step, one block per SM with all 512
//     tensor-memory columns (two score buffers, so the MMA warp forms the next scores while the softmax works on
//     these; P; O), keys and values through TMA in rings of their own (three and two stages: the keys of a step
//     are wanted a step before its values), eight softmax warps with two threads a row, and a query tile a
//     block, the tiles with the most keys first in the grid (the SMs take blocks in the order of their index, so
//     the light tiles fill what the heavy ones leave); or, selectable, two query tiles per block, the c-th from
//     the end and then the c-th from the start.  Its own comment further down has the details.
//   * attention_prefill_tc_kernel: 64 keys a step, one query tile per block, four softmax warps (thread = row),
//     two blocks per SM (256 tensor-memory columns and 97 KB of shared memory each), so that one block's softmax
//     overlaps the other's products.  Kept selectable (gk_set_attention_prefill_keys(64)); it is the slower of the
//     two at every length measured.
//
// In both, warp 0 streams K and V pages with TMA (a 2-D map over the cache seen as [pages * heads * 64, 128]) and
// warp 1 issues the MMAs.
//
// Every mbarrier wait is bounded; a wait that gives up records a code in *error_flag and the block
// winds down (drains its copies, frees its tensor memory).

#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int D = 128;
constexpr int ROWS = 128;
constexpr int PAGE = 64;
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr uint32_t TMEM_COLS = 256;  // two blocks share an SM's 512 columns
constexpr uint32_t COL_S = 0, COL_P = 64, COL_O = 128;  // S: 64, P: 32 (bf16 pairs), O: 128
constexpr float RESCALE_THRESHOLD = 8.0f;               // in log2 units

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// K-major operand, rows of 128 bytes, 128-byte swizzle, groups of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand (V: the MMA's N runs along a row of 128 bytes = 64 head dims, its K over the rows =
// keys): the next 64 of N are `lbo` bytes away, the next eight of K 1024 bytes.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: f32 accumulator, bf16 inputs, A K-major, B K- or MN-major.
__device__ __forceinline__ uint32_t idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t id, bool acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(a), "l"(b), "r"(id),
        "r"((uint32_t)acc)
        : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t id, bool acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(id),
        "r"((uint32_t)acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {  // 2^x, one MUFU instruction; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two 32-bit numbers as one operand, and the instructions of this architecture that work on such pairs: the softmax
// warps' time is the length of their instruction stream, so half as many multiply-adds and additions shorten a step.
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void halves_of(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_pairs(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_pairs(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max_of_three(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

struct alignas(1024) Smem {
    __nv_bfloat16 q[2][ROWS * 64];                  // two 64-wide halves of the head dim, each [128 rows][128 bytes]
    __nv_bfloat16 k[KV_STAGES][2][PAGE * 64];       // per page: two halves, each [64 keys][128 bytes]
    __nv_bfloat16 v[KV_STAGES][2][PAGE * 64];
    uint64_t kv_full[KV_STAGES], kv_empty[KV_STAGES];
    uint64_t s_full, s_empty, p_full, o_done, q_ready;
    uint32_t tmem_base;
};

struct Params {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* cu_q;
    const int* kv_len;
    const int* slots;
    const int* block_table;
    int n_q, n_kv, max_pages;
    float sl2;
    int window;
    int* error_flag;
    int one_tile;  // tc2: a query tile a block, heaviest first (grid: kv head, sequence, tile), instead of a heavy and a light one
    int n_seqs, n_items;  // tc5: the list of tiles is n_items long: (tile counted from the end, sequence, kv head)
};

__global__ void __launch_bounds__(THREADS, 2) attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v,
                                                                          const Params p) {
    extern __shared__ unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.z, hk = blockIdx.y;
    const int group = p.n_q / p.n_kv;
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int n_rows = q_len * group;
    const int n_blocks = (n_rows + ROWS - 1) / ROWS;
    if ((int)blockIdx.x >= n_blocks) return;  // whole block, before any barrier or allocation
    const int row0 = (n_blocks - 1 - (int)blockIdx.x) * ROWS;  // heavy blocks first
    const int len = p.kv_len[seq], past = len - q_len;
    const int* pages = p.block_table + (size_t)p.slots[seq] * p.max_pages;
    const int last_row = min(row0 + ROWS, n_rows) - 1;
    const int max_pos = past + last_row / group, min_pos = past + row0 / group;
    const int lo_block = (p.window > 0 && min_pos - p.window + 1 > 0) ? min_pos - p.window + 1 : 0;
    const int p_begin = lo_block / PAGE, p_end = max_pos / PAGE + 1;
    const int n_iter = p_end - p_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&sm.kv_full[s], 1);
            mbar_init(&sm.kv_empty[s], 1);
        }
        mbar_init(&sm.s_full, 1);
        mbar_init(&sm.s_empty, 128);
        mbar_init(&sm.p_full, 128);
        mbar_init(&sm.o_done, 1);
        mbar_init(&sm.q_ready, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = sm.tmem_base;
    pdl_wait();  // queries and the new keys and values come from the kernel before

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: K and V pages, two 64-wide halves each
            bool ok = true;
            int issued = 0;
            for (int i = 0; i < n_iter && ok; ++i) {
                const int s = i % KV_STAGES;
                if (i >= KV_STAGES) ok = mbar_wait(&sm.kv_empty[s], ((i / KV_STAGES) - 1) & 1);
                if (!ok) break;
                const int page = pages[p_begin + i];
                const int y = (page * p.n_kv + hk) * PAGE;
                mbar_expect_tx(&sm.kv_full[s], 4 * PAGE * 64 * 2);
                tma_load_2d(sm.k[s][0], &map_k, 0, y, &sm.kv_full[s]);
                tma_load_2d(sm.k[s][1], &map_k, 64, y, &sm.kv_full[s]);
                tma_load_2d(sm.v[s][0], &map_v, 0, y, &sm.kv_full[s]);
                tma_load_2d(sm.v[s][1], &map_v, 64, y, &sm.kv_full[s]);
                issued = i + 1;
            }
            if (!ok) {
                atomicExch(p.error_flag, 11);
                for (int i = max(issued - KV_STAGES, 0); i < issued; ++i) mbar_wait(&sm.kv_full[i % KV_STAGES], (i / KV_STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            const uint32_t id_s = idesc(ROWS, PAGE, false), id_o = idesc(ROWS, D, true);
            bool ok = mbar_wait(&sm.q_ready, 0);
            fence_after();
            auto issue_qk = [&](int i) {
                const int s = i % KV_STAGES;
                if (ok) ok = mbar_wait(&sm.kv_full[s], (i / KV_STAGES) & 1);
                if (ok && i >= 1) ok = mbar_wait(&sm.s_empty, (i - 1) & 1);  // the softmax has taken the scores before
                if (!ok) return;
                fence_after();
#pragma unroll
                for (int k = 0; k < D / 16; ++k) {
                    const uint64_t da = desc_k_major(smem_u32(sm.q[k >> 2]) + (k & 3) * 32);
                    const uint64_t db = desc_k_major(smem_u32(sm.k[s][k >> 2]) + (k & 3) * 32);
                    umma_ss(tmem + COL_S, da, db, id_s, k > 0);
                }
                umma_commit(&sm.s_full);
            };
            if (n_iter > 0) issue_qk(0);
            for (int i = 0; i < n_iter && ok; ++i) {
                if (i + 1 < n_iter) issue_qk(i + 1);  // the next scores while the softmax works on these
                if (!ok) break;
                const int s = i % KV_STAGES;
                ok = mbar_wait(&sm.p_full, i & 1);
                if (!ok) break;
                fence_after();
#pragma unroll
                for (int j = 0; j < PAGE / 16; ++j) {
                    // keys 16j .. 16j+15 of the page: 16 rows of 128 bytes further on in both halves
                    const uint64_t db = desc_mn_major(smem_u32(sm.v[s][0]) + j * 16 * 128, PAGE * 128);
                    umma_ts(tmem + COL_O, tmem + COL_P + j * 8, db, id_o, i > 0 || j > 0);
                }
                umma_commit(&sm.kv_empty[s]);  // the page's shared memory is free once these have read it
                umma_commit(&sm.o_done);       // and the accumulator holds this page
            }
            if (!ok) atomicExch(p.error_flag, 12);
        }
    } else {
        // ---- softmax warps: thread = row
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int row = row0 + r;
        const bool row_ok = row < n_rows;
        const int tok = row_ok ? row / group : 0;
        const int head = hk * group + (row_ok ? row % group : 0);
        const int pos = past + tok;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        // Q row -> swizzled shared memory (zeros for rows beyond the sequence)
        {
            const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)(q_begin + tok) * p.n_q + head) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint4 val = row_ok ? src[c] : make_uint4(0, 0, 0, 0);
                uint4* dst = reinterpret_cast<uint4*>(sm.q[c >> 3]) + r * 8 + ((c & 7) ^ (r & 7));
                *dst = val;
            }
            fence_async_smem();
            mbar_arrive(&sm.q_ready);
        }
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_iter && ok; ++i) {
            const int s = i % KV_STAGES;
            const int key_base = (p_begin + i) * PAGE;
            ok = mbar_wait(&sm.s_full, i & 1);
            if (!ok) break;
            fence_after();
            uint32_t raw[2][32];
            tmem_ld32(tmem + lane_base + COL_S, raw[0]);
            tmem_ld32(tmem + lane_base + COL_S + 32, raw[1]);
            tmem_wait_ld();
            fence_before();
            mbar_arrive(&sm.s_empty);  // the scores are in registers: the buffer may be overwritten
            // the last page of the sequence may hold stale rows beyond its length: zero them in V, so that
            // probability 0 times whatever lies there cannot make a NaN
            const int valid = len - key_base;
            if (valid < PAGE) {
                ok = mbar_wait(&sm.kv_full[s], (i / KV_STAGES) & 1);
                if (!ok) break;
                for (int idx = r; idx < (PAGE - valid) * 16; idx += 128) {
                    const int vr = valid + idx / 16, chunk = idx % 16;
                    reinterpret_cast<uint4*>(sm.v[s][chunk >> 3])[vr * 8 + (chunk & 7)] = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
            }
            float mx = -INFINITY;
            const bool need_mask = key_base + PAGE - 1 > pos || p.window > 0;
            const int hidden_upto = p.window > 0 ? pos - p.window : -1;  // keys up to here are behind the window
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {  // selects, not branches: the rows of a warp differ in what they see
                    const int key = key_base + c;
                    const bool hidden = (key > pos) | (key <= hidden_upto);
                    raw[c >> 5][c & 31] = hidden ? 0xff800000u : raw[c >> 5][c & 31];  // -inf
                }
            }
            {   // four independent chains keep the maximum off the critical path
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < 64; ++c) m4[c & 3] = fmaxf(m4[c & 3], __uint_as_float(raw[c >> 5][c & 31]));
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            }
            const float m_new = fmaxf(m_used, mx * p.sl2);
            // rescale lazily: only when the maximum has grown by more than the threshold
            float corr = 1.0f;
            if (m_new > m_used + RESCALE_THRESHOLD || m_used == -INFINITY) {
                corr = m_used == -INFINITY ? 0.f : exp2f(m_used - m_new);
                m_used = m_new;
            }
            const float ref = m_used == -INFINITY ? 0.f : m_used;
            uint32_t packed[32];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float e0 = ex2(fmaf(__uint_as_float(raw[c >> 5][c & 31]), p.sl2, -ref));
                const float e1 = ex2(fmaf(__uint_as_float(raw[(c + 1) >> 5][(c + 1) & 31]), p.sl2, -ref));
                sum4[(c >> 1) & 3] += e0 + e1;
                __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                packed[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l = l * corr + sum;
            // the accumulator may be touched only when the product of the page before has landed in it
            if (i > 0) {
                ok = mbar_wait(&sm.o_done, (i - 1) & 1);
                if (!ok) break;
                fence_after();
            }
            if (i > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem + lane_base + COL_O + c0, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
                    tmem_st32(tmem + lane_base + COL_O + c0, o);
                }
            }
            tmem_st32(tmem + lane_base + COL_P, packed);
            tmem_wait_st();
            fence_before();
            mbar_arrive(&sm.p_full);
        }
        if (!ok && lane == 0) atomicExch(p.error_flag, 13);
        // ---- the result: O / l
        if (ok && n_iter > 0) ok = mbar_wait(&sm.o_done, (n_iter - 1) & 1);
        fence_after();
        if (ok && n_iter > 0) {
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = p.out + ((size_t)(q_begin + tok) * p.n_q + head) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem + lane_base + COL_O + c0, o);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        w.x = *reinterpret_cast<uint32_t*>(&h0);
                        w.y = *reinterpret_cast<uint32_t*>(&h1);
                        w.z = *reinterpret_cast<uint32_t*>(&h2);
                        w.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(orow + c0 + c) = w;
                    }
                }
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// ---------------------------------------------------------------- the same with 128 keys per step
// One block per SM with all 512 tensor-memory columns: two score buffers of 128 keys (two pages) each, so the
// MMA warp forms the next scores while the softmax warps work on these; P (64 columns) and O (128) beside
// them.  Eight softmax warps, two threads a row (the exponentials are what a step waits for longest).  A step of 128 keys costs as many tcgen05.mma as a step of 64 (an instruction costs about 84 cycles
// whether its N is 64 or 128), and the chain of dependent steps of a query tile is half as long.  A block
// takes one query tile (the default; heaviest tiles first in the grid) or two one after the other, the c-th from
// the end and the c-th from the start: under the causal mask their work adds up to the same for every block.
constexpr int KEYS2 = 2 * PAGE;
constexpr int K_STAGES2 = 3;
constexpr uint32_t COL2_S = 0, COL2_P = 256, COL2_O = 320;  // S: 2 x 128, P: 64 (bf16 pairs), O: 128

struct alignas(1024) Smem2 {
    __nv_bfloat16 q[2][ROWS * 64];                      // two 64-wide halves of the head dim
    // K and V have rings of their own: the keys of a step are wanted a whole step before its values (the scores
    // are formed ahead), and are free again as soon as the scores are, so three stages of keys and two of values
    // keep a TMA load's 1.3 us off the chain of steps
    __nv_bfloat16 k[K_STAGES2][2][2][PAGE * 64];        // [stage][half of the head dim][page of the step][64 keys x 128 bytes]
    __nv_bfloat16 v[KV_STAGES][2][2][PAGE * 64];        // [stage][page of the step][half of the head dim][64 keys x 128 bytes]
    uint64_t k_full[K_STAGES2], k_empty[K_STAGES2], v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], s_empty[2], p_full, o_done, q_ready;
    uint64_t max_ready[2][4], sum_ready;  // the two halves of a quarter's rows have left their maxima (a barrier per quarter of the rows: only
                                        // the two warps that share rows wait for each other) / all rows their sums
    float row_max[2][2][ROWS];  // [step parity][half of the keys][row]
    float row_sum[2][ROWS];
    uint32_t tmem_base;
};

constexpr int THREADS2 = 352;  // TMA warp, the warp that issues the score products, eight softmax warps, the warp that issues the P V products

__global__ void __launch_bounds__(THREADS2, 1) attention_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                           const __grid_constant__ CUtensorMap map_v,
                                                                           const Params p) {
    extern __shared__ unsigned char smem_raw[];
    Smem2& sm = *reinterpret_cast<Smem2*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Two ways of dealing out the query tiles.  Pairs (grid: pair, kv head, sequence): a block takes the c-th tile
    // from the end and the c-th from the start, equal work for every block, right where all blocks run at once.
    // One tile a block (grid: kv head, sequence, tile from the end): blocks are handed to the SMs in the order of
    // their index, so the heaviest tiles start first and the light ones fill what is left, which wastes less than
    // whole waves of equal pairs do where there are several blocks an SM.
    const int seq = p.one_tile ? blockIdx.y : blockIdx.z, hk = p.one_tile ? blockIdx.x : blockIdx.y;
    const int first = p.one_tile ? blockIdx.z : blockIdx.x;
    const int group = p.n_q / p.n_kv;
    // row / group and row % group by shift and mask where the group is a power of two (a division is some two hundred
    // cycles of dependent instructions, and a tile's queries and results each cost a thread four of them)
    const int group_shift = (group & (group - 1)) == 0 ? __ffs(group) - 1 : -1;
    auto over_group = [&](int x) { return group_shift >= 0 ? x >> group_shift : x / group; };
    auto in_group = [&](int x) { return group_shift >= 0 ? x & (group - 1) : x % group; };
    const int q_begin = p.cu_q[seq], q_len = p.cu_q[seq + 1] - q_begin;
    const int n_rows = q_len * group;
    const int n_blocks = (n_rows + ROWS - 1) / ROWS;
    if ((p.one_tile ? first : 2 * first) >= n_blocks) return;  // whole block, before any barrier or allocation
    // the block's query tiles: the heavy one first
    const int tile_of[2] = {n_blocks - 1 - first, p.one_tile ? -1 : first};
    const int n_tiles = tile_of[0] > tile_of[1] && !p.one_tile ? 2 : 1;
    const int len = p.kv_len[seq], past = len - q_len;
    const int* pages = p.block_table + (size_t)p.slots[seq] * p.max_pages;
    // pages [p_begin, p_end) of query tile u, in steps of two
    auto span = [&](int u, int& p_begin, int& p_end) {
        const int row0 = tile_of[u] * ROWS;
        const int last_row = min(row0 + ROWS, n_rows) - 1;
        const int max_pos = past + over_group(last_row), min_pos = past + over_group(row0);
        const int lo = (p.window > 0 && min_pos - p.window + 1 > 0) ? min_pos - p.window + 1 : 0;
        p_begin = lo / PAGE;
        p_end = max_pos / PAGE + 1;
    };

    // A softmax warp's halves of a tile's Q rows -> swizzled shared memory (zeros for rows beyond the sequence).  The four
    // lanes of a quad work on the rows of the quad together, 32 bytes of a row's 128 each, so that a load or store of
    // the warp touches eight whole lines instead of 32 partly.  (`half`: which 64 of the head's 128 elements.)
    auto query_row = [&](__nv_bfloat16* base, int tile, int rr, int half_of_head) -> __nv_bfloat16* {
        const int row_i = tile * ROWS + rr;
        if (row_i >= n_rows) return nullptr;
        return base + ((size_t)(q_begin + over_group(row_i)) * p.n_q + hk * group + in_group(row_i)) * D + half_of_head * 64 + (lane & 3) * 16;
    };
    auto load_queries = [&](int tile) {
        const int quad_row = (warp & 3) * 32 + (lane & ~3), piece = lane & 3, half_of_head = (warp - 2) >> 2;
        uint32_t val[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // all four loads on their way before the first is used
            const __nv_bfloat16* src = query_row(const_cast<__nv_bfloat16*>(p.q), tile, quad_row + i, half_of_head);
#pragma unroll
            for (int j = 0; j < 8; ++j) val[i][j] = 0u;
            if (src) load32(src, val[i]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rr = quad_row + i;
            uint4* dst = reinterpret_cast<uint4*>(sm.q[half_of_head]) + rr * 8;
            dst[(2 * piece) ^ (rr & 7)] = make_uint4(val[i][0], val[i][1], val[i][2], val[i][3]);
            dst[(2 * piece + 1) ^ (rr & 7)] = make_uint4(val[i][4], val[i][5], val[i][6], val[i][7]);
        }
        fence_async_smem();
    };
    // The block's first tile of queries comes in while thread 0 sets up the barriers and warp 1 the tensor memory.
    if (warp >= 2 && warp < 10) {
        pdl_wait();  // queries come from the kernel before
        load_queries(tile_of[0]);
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < K_STAGES2; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
        }
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.s_full[b], 1);
            mbar_init(&sm.s_empty[b], 256);
            for (int quarter = 0; quarter < 4; ++quarter) mbar_init(&sm.max_ready[b][quarter], 64);
        }
        mbar_init(&sm.p_full, 256);
        mbar_init(&sm.o_done, 1);
        mbar_init(&sm.q_ready, 256);
        mbar_init(&sm.sum_ready, 256);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = sm.tmem_base;
    pdl_wait();  // queries and the new keys and values come from the kernel before

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: per step two pages of K and of V, each in two 64-wide halves; the keys run one step
            // ahead of the values
            bool ok = true;
            auto load = [&](int g, int pg, int p_end, bool keys) {
                const int n_pages = min(2, p_end - pg);
                if (keys) {
                    const int s = g % K_STAGES2;
                    if (g >= K_STAGES2) ok = mbar_wait(&sm.k_empty[s], ((g / K_STAGES2) - 1) & 1);
                    if (!ok) return;
                    mbar_expect_tx(&sm.k_full[s], (uint32_t)n_pages * 2 * PAGE * 64 * 2);
                    for (int j = 0; j < n_pages; ++j) {
                        const int y = (pages[pg + j] * p.n_kv + hk) * PAGE;
                        tma_load_2d(sm.k[s][0][j], &map_k, 0, y, &sm.k_full[s]);
                        tma_load_2d(sm.k[s][1][j], &map_k, 64, y, &sm.k_full[s]);
                    }
                } else {
                    const int s = g % KV_STAGES;
                    if (g >= KV_STAGES) ok = mbar_wait(&sm.v_empty[s], ((g / KV_STAGES) - 1) & 1);
                    if (!ok) return;
                    mbar_expect_tx(&sm.v_full[s], (uint32_t)n_pages * 2 * PAGE * 64 * 2);
                    for (int j = 0; j < n_pages; ++j) {
                        const int y = (pages[pg + j] * p.n_kv + hk) * PAGE;
                        tma_load_2d(sm.v[s][j][0], &map_v, 0, y, &sm.v_full[s]);
                        tma_load_2d(sm.v[s][j][1], &map_v, 64, y, &sm.v_full[s]);
                    }
                }
            };
            // the steps of the block's tiles in one list: (first page, end page of the tile)
            int g_k = 0, g_v = 0;          // steps whose keys / values have been asked for
            int uk = 0, pk = 0, ek = 0;    // where the keys are: tile, next page, end page
            int uv = 0, pv = 0, ev = 0;    // where the values are
            if (n_tiles > 0) { span(0, pk, ek); pv = pk; ev = ek; }
            auto advance = [&](int& u, int& pg, int& pe) {
                pg += 2;
                if (pg >= pe && ++u < n_tiles) span(u, pg, pe);
            };
            while (ok && (uk < n_tiles || uv < n_tiles)) {
                if (uk < n_tiles && g_k <= g_v + 1) {  // keys at most two steps ahead of the values
                    load(g_k++, pk, ek, true);
                    advance(uk, pk, ek);
                } else {
                    load(g_v++, pv, ev, false);
                    advance(uv, pv, ev);
                }
            }
            if (!ok) atomicExch(p.error_flag, 41);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- issuer of the score products S = Q K^T.  It runs ahead of the softmax by one step (two score
            // buffers).  A tcgen05.mma costs its issuing thread about 100 cycles, as long as the product takes on
            // the tensor cores, so a thread that also waits on barriers between its products leaves the tensor
            // cores idle meanwhile: the two kinds of product of a step have a thread each, and one fills the
            // other's waits.
            const uint32_t id_s = idesc(ROWS, KEYS2, false);
            bool ok = true;
            int g = 0;
            for (int u = 0; u < n_tiles && ok; ++u) {
                int p_begin, p_end;
                span(u, p_begin, p_end);
                const int n_iter = (p_end - p_begin + 1) / 2;
                ok = mbar_wait(&sm.q_ready, u & 1);
                if (!ok) break;
                for (int i = 0; i < n_iter && ok; ++i, ++g) {
                    const int s = g % K_STAGES2, b = g & 1;
                    ok = mbar_wait(&sm.k_full[s], (g / K_STAGES2) & 1);
                    if (ok && g >= 2) ok = mbar_wait(&sm.s_empty[b], ((g >> 1) - 1) & 1);  // the softmax has taken what was there
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint64_t da = desc_k_major(smem_u32(sm.q[k >> 2]) + (k & 3) * 32);
                        const uint64_t db = desc_k_major(smem_u32(sm.k[s][k >> 2][0]) + (k & 3) * 32);
                        umma_ss(tmem + COL2_S + b * KEYS2, da, db, id_s, k > 0);
                    }
                    umma_commit(&sm.k_empty[s]);  // the keys' shared memory is free once the scores are formed
                    umma_commit(&sm.s_full[b]);
                }
                // the tile's queries may be overwritten once its last scores are formed: the softmax warps wait for
                // the tile's last o_done before they load the next tile's, and that product follows these scores
            }
            if (!ok) atomicExch(p.error_flag, 42);
        }
    } else if (warp == 10) {
        if (lane == 0) {
            // ---- issuer of the products O += P V
            const uint32_t id_o = idesc(ROWS, D, true);
            bool ok = true;
            int g = 0;
            for (int u = 0; u < n_tiles && ok; ++u) {
                int p_begin, p_end;
                span(u, p_begin, p_end);
                const int n_iter = (p_end - p_begin + 1) / 2;
                for (int i = 0; i < n_iter && ok; ++i, ++g) {
                    const int s = g % KV_STAGES;
                    ok = mbar_wait(&sm.p_full, g & 1);
                    if (ok) ok = mbar_wait(&sm.v_full[s], (g / KV_STAGES) & 1);
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int j = 0; j < KEYS2 / 16; ++j) {
                        // keys 16j .. 16j+15 of the step: page j / 4, 16 rows of 128 bytes further on per j in both halves
                        const uint64_t db = desc_mn_major(smem_u32(sm.v[s][j >> 2][0]) + (j & 3) * 16 * 128, PAGE * 128);
                        umma_ts(tmem + COL2_O, tmem + COL2_P + j * 8, db, id_o, i > 0 || j > 0);
                    }
                    umma_commit(&sm.v_empty[s]);  // the values' shared memory is free once these have read it
                    umma_commit(&sm.o_done);       // and the accumulator holds this step
                }
            }
            if (!ok) atomicExch(p.error_flag, 44);
        }
    } else {
        // ---- softmax warps: two threads a row.  Warps 2-5 take keys 0..63 of a step, warps 6-9 keys 64..127 (a
        // warp reaches the tensor-memory lanes of its quarter, warp % 4, whatever its columns); the halves of a
        // row exchange their maxima through shared memory, keep a sum each and add the two at the end.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        bool ok = true;
        int g = 0;
        for (int u = 0; u < n_tiles && ok; ++u) {
            int p_begin, p_end;
            span(u, p_begin, p_end);
            const int n_iter = (p_end - p_begin + 1) / 2;
            const int row = tile_of[u] * ROWS + r;
            const bool row_ok = row < n_rows;
            const int tok = row_ok ? over_group(row) : 0;
            const int pos = past + tok;
            const int quad_row = quarter * 32 + (lane & ~3);
            auto row_at = [&](__nv_bfloat16* base, int rr) -> __nv_bfloat16* { return query_row(base, tile_of[u], rr, half); };
            // the block's first tile is in shared memory already; a later one may come in now that the MMAs that read
            // the tile before have finished (its last o_done was waited for below)
            if (u > 0) load_queries(tile_of[u]);
            mbar_arrive(&sm.q_ready);
            float m_used = -INFINITY, l = 0.f;
            for (int i = 0; i < n_iter && ok; ++i, ++g) {
                const int s = g % KV_STAGES, b = g & 1;
                const int key_base = (p_begin + 2 * i) * PAGE + half * 64;  // the first key this thread looks at
                const uint32_t s_cols = tmem + lane_base + COL2_S + b * KEYS2 + half * 64;
                ok = mbar_wait(&sm.s_full[b], (g >> 1) & 1);
                if (!ok) break;
                fence_after();
                uint32_t raw[2][32];
                tmem_ld32(s_cols, raw[0]);
                tmem_ld32(s_cols + 32, raw[1]);
                tmem_wait_ld();
                fence_before();
                mbar_arrive(&sm.s_empty[b]);  // the scores are in registers: the buffer may be overwritten
                // rows of V beyond the sequence's length or beyond the pages this step loaded (a stale page end, no
                // second page): zero them, so that probability 0 times whatever lies there cannot make a NaN
                const int step_base = (p_begin + 2 * i) * PAGE;
                const int valid = min(len - step_base, min(2, p_end - (p_begin + 2 * i)) * PAGE);
                if (valid < KEYS2) {
                    ok = mbar_wait(&sm.v_full[s], (g / KV_STAGES) & 1);
                    if (!ok) break;
                    for (int idx = half * 128 + r; idx < (KEYS2 - valid) * 16; idx += 256) {
                        const int vr = valid + idx / 16, chunk = idx % 16;
                        reinterpret_cast<uint4*>(sm.v[s][vr >> 6][chunk >> 3])[(vr & 63) * 8 + (chunk & 7)] = make_uint4(0, 0, 0, 0);
                    }
                    fence_async_smem();
                }
                // scores of keys the row must not see become -inf (whatever they were: stale keys may hold anything);
                // only the steps on the diagonal, or with a window, come here
                if (key_base + 63 > pos || p.window > 0) {
                    const int hidden_upto = p.window > 0 ? pos - p.window : -1;  // keys up to here are behind the window
#pragma unroll
                    for (int c = 0; c < 64; ++c) {  // selects, not branches: the rows of a warp differ in what they see
                        const int key = key_base + c;
                        const bool hidden = (key > pos) | (key <= hidden_upto);
                        raw[c >> 5][c & 31] = hidden ? 0xff800000u : raw[c >> 5][c & 31];
                    }
                }
                float mx;
                {   // four independent chains keep the maximum off the critical path
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int c = 0; c < 64; c += 2)
                        m4[(c >> 1) & 3] = max_of_three(m4[(c >> 1) & 3], __uint_as_float(raw[c >> 5][c & 31]), __uint_as_float(raw[(c + 1) >> 5][(c + 1) & 31]));
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
                // the row's maximum over both halves
                sm.row_max[g & 1][half][r] = mx;
                mbar_arrive(&sm.max_ready[g & 1][quarter]);  // (release: the store above is visible to who sees the phase end)
                ok = mbar_wait(&sm.max_ready[g & 1][quarter], (g >> 1) & 1);
                if (!ok) break;
                mx = fmaxf(mx, sm.row_max[g & 1][half ^ 1][r]);
                const float m_new = fmaxf(m_used, mx * p.sl2);
                float corr = 1.0f;  // rescale lazily: only when the maximum has grown by more than the threshold
                if (m_new > m_used + RESCALE_THRESHOLD || m_used == -INFINITY) {
                    corr = m_used == -INFINITY ? 0.f : exp2f(m_used - m_new);
                    m_used = m_new;
                }
                const float ref = m_used == -INFINITY ? 0.f : m_used;
                uint32_t packed[32];
                const uint64_t scale2 = pair_of(p.sl2, p.sl2), shift2 = pair_of(-ref, -ref);
                uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};  // four running pairs of sums
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    float x0, x1;
                    halves_of(fma_pairs(pair_of(__uint_as_float(raw[c >> 5][c & 31]), __uint_as_float(raw[(c + 1) >> 5][(c + 1) & 31])), scale2, shift2), x0, x1);
                    const float e0 = ex2(x0), e1 = ex2(x1);
                    sums[(c >> 1) & 3] = add_pairs(sums[(c >> 1) & 3], pair_of(e0, e1));
                    __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
                    packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                }
                float sum_lo, sum_hi;
                halves_of(add_pairs(add_pairs(sums[0], sums[1]), add_pairs(sums[2], sums[3])), sum_lo, sum_hi);
                l = l * corr + (sum_lo + sum_hi);
                // P and the accumulator may be touched only when the product of the step before has finished
                if (g > 0) {
                    ok = mbar_wait(&sm.o_done, (g - 1) & 1);
                    if (!ok) break;
                    fence_after();
                }
                if (i > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {  // this thread's half of the accumulator's columns
#pragma unroll 1
                    for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem + lane_base + COL2_O + c0, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
                        tmem_st32(tmem + lane_base + COL2_O + c0, o);
                    }
                }
                tmem_st32(tmem + lane_base + COL2_P + half * 32, packed);
                tmem_wait_st();
                fence_before();
                mbar_arrive(&sm.p_full);
            }
            if (!ok) break;
            // ---- the tile's result: O / l, this thread's half of the columns; l is the sum of both halves' sums
            sm.row_sum[half][r] = l;
            mbar_arrive(&sm.sum_ready);
            ok = mbar_wait(&sm.o_done, (g - 1) & 1);
            if (ok) ok = mbar_wait(&sm.sum_ready, u & 1);
            if (!ok) break;
            fence_after();
            const float inv = 1.0f / (sm.row_sum[0][r] + sm.row_sum[1][r]);
            uint32_t packed[32];  // this thread's 64 columns of its row, then 16 columns of each row of the quad
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem + lane_base + COL2_O + half * 64 + c0, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                    packed[(c0 + c) >> 1] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            swap_pieces<uint32_t, 8>(packed, lane);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __nv_bfloat16* dst = row_at(p.out, quad_row + i);
                if (dst) store32(dst, packed + 8 * i);
            }
            fence_before();  // (row_sum is written again only after the next tile's steps, each a barrier of all rows' threads)
        }
        if (!ok && lane == 0) atomicExch(p.error_flag, 43);
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
    }
}

// ---------------------------------------------------------------- the same, with blocks that stay
// The kernel above, but a block per SM that stays and takes query tiles from the launch's list one after another (the
// list: tile counted from the end, then sequence, then kv head, so the heaviest tiles come first; block b of G takes
// entries b, 2G - 1 - b, 2G + b, ...: back and forth, so that every block gets heavy and light ones).  What a tile
// costs beside its steps (set-up of barriers and tensor memory, queries in, first scores, the next block's start:
// 3.8 us of 5.3 at 2,048 tokens) then falls under the steps of the tile before: the queries of the next tile come by
// TMA (a 3-D map over [token, head, 128]: a box of 128 / group tokens x group heads x 64 elements is a tile's 128 rows
// in the order the rows have) as soon as the last scores of the tile in hand are formed, and its first scores are
// formed while the softmax warps still write out the result.  Needs a group size that divides 128.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

struct alignas(1024) Smem5 {
    __nv_bfloat16 q[2][ROWS * 64];
    __nv_bfloat16 k[K_STAGES2][2][2][PAGE * 64];
    __nv_bfloat16 v[KV_STAGES][2][2][PAGE * 64];
    uint64_t k_full[K_STAGES2], k_empty[K_STAGES2], v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], s_empty[2], p_full, o_done;
    uint64_t q_full, q_empty, o_free;     // a tile's queries have landed / its last scores are formed / its result is read
    uint64_t max_ready[2][4], sum_ready;
    float row_max[2][2][ROWS];
    float row_sum[2][ROWS];
    uint32_t tmem_base;
};

struct Tile {
    int seq, hk, tile;         // the tile-th 128 rows of (sequence, kv head)
    int q_begin, n_rows, len, past;
    const int* pages;
    int p_begin, p_end;        // its pages, taken in steps of two
};

// Entry `item` of the launch's list; false if the sequence has no such tile.
__device__ __forceinline__ bool tile_of_item(const Params& p, int item, int group, Tile& t) {
    const int per = p.n_kv * p.n_seqs;
    const int from_end = item / per, rem = item - from_end * per;
    t.seq = rem / p.n_kv;
    t.hk = rem - t.seq * p.n_kv;
    t.q_begin = p.cu_q[t.seq];
    const int q_len = p.cu_q[t.seq + 1] - t.q_begin;
    t.n_rows = q_len * group;
    t.tile = (t.n_rows + ROWS - 1) / ROWS - 1 - from_end;
    if (t.tile < 0) return false;
    t.len = p.kv_len[t.seq];
    t.past = t.len - q_len;
    t.pages = p.block_table + (size_t)p.slots[t.seq] * p.max_pages;
    const int row0 = t.tile * ROWS, last_row = min(row0 + ROWS, t.n_rows) - 1;
    const int max_pos = t.past + last_row / group, min_pos = t.past + row0 / group;
    const int lo = (p.window > 0 && min_pos - p.window + 1 > 0) ? min_pos - p.window + 1 : 0;
    t.p_begin = lo / PAGE;
    t.p_end = max_pos / PAGE + 1;
    return true;
}

__global__ void __launch_bounds__(THREADS2, 1) attention_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                           const __grid_constant__ CUtensorMap map_v,
                                                                           const __grid_constant__ CUtensorMap map_q,
                                                                           const Params p) {
    extern __shared__ unsigned char smem_raw[];
    Smem5& sm = *reinterpret_cast<Smem5*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.n_q / p.n_kv;
    const int G = gridDim.x, me = blockIdx.x;
    // the block's next tile after round `r` of the list (r = -1: its first); false when the list is through
    auto next_tile = [&](int& r, Tile& t) -> bool {
        for (++r; r * G < p.n_items; ++r) {
            const int item = r * G + ((r & 1) ? G - 1 - me : me);
            if (item < p.n_items && tile_of_item(p, item, group, t)) return true;
        }
        return false;
    };
    auto steps_of = [](const Tile& t) { return (t.p_end - t.p_begin + 1) / 2; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < K_STAGES2; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
        }
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.s_full[b], 1);
            mbar_init(&sm.s_empty[b], 256);
            for (int quarter = 0; quarter < 4; ++quarter) mbar_init(&sm.max_ready[b][quarter], 64);
        }
        mbar_init(&sm.p_full, 256);
        mbar_init(&sm.o_done, 1);
        mbar_init(&sm.q_full, 1);
        mbar_init(&sm.q_empty, 1);
        mbar_init(&sm.o_free, 256);
        mbar_init(&sm.sum_ready, 256);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pdl_launch_dependents();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = sm.tmem_base;
    pdl_wait();  // queries and the new keys and values come from the kernel before

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: a tile's queries, then per step two pages of K and of V; the keys run ahead of the values
            bool ok = true;
            auto load = [&](int g, const Tile& t, int i, bool keys) {
                const int pg = t.p_begin + 2 * i;
                const int n_pages = min(2, t.p_end - pg);
                if (keys) {
                    const int s = g % K_STAGES2;
                    if (g >= K_STAGES2) ok = mbar_wait(&sm.k_empty[s], ((g / K_STAGES2) - 1) & 1);
                    if (!ok) return;
                    mbar_expect_tx(&sm.k_full[s], (uint32_t)n_pages * 2 * PAGE * 64 * 2);
                    for (int j = 0; j < n_pages; ++j) {
                        const int y = (t.pages[pg + j] * p.n_kv + t.hk) * PAGE;
                        tma_load_2d(sm.k[s][0][j], &map_k, 0, y, &sm.k_full[s]);
                        tma_load_2d(sm.k[s][1][j], &map_k, 64, y, &sm.k_full[s]);
                    }
                } else {
                    const int s = g % KV_STAGES;
                    if (g >= KV_STAGES) ok = mbar_wait(&sm.v_empty[s], ((g / KV_STAGES) - 1) & 1);
                    if (!ok) return;
                    mbar_expect_tx(&sm.v_full[s], (uint32_t)n_pages * 2 * PAGE * 64 * 2);
                    for (int j = 0; j < n_pages; ++j) {
                        const int y = (t.pages[pg + j] * p.n_kv + t.hk) * PAGE;
                        tma_load_2d(sm.v[s][j][0], &map_v, 0, y, &sm.v_full[s]);
                        tma_load_2d(sm.v[s][j][1], &map_v, 64, y, &sm.v_full[s]);
                    }
                }
            };
            // queries of the n-th tile of the block, once the last scores of the tile before are formed
            auto load_queries = [&](const Tile& t, int n) {
                if (n > 0) ok = mbar_wait(&sm.q_empty, (n - 1) & 1);
                if (!ok) return;
                mbar_expect_tx(&sm.q_full, (uint32_t)(2 * ROWS * 64 * 2));
                const int token = t.q_begin + t.tile * (ROWS / group);
                tma_load_3d(sm.q[0], &map_q, 0, t.hk * group, token, &sm.q_full);
                tma_load_3d(sm.q[1], &map_q, 64, t.hk * group, token, &sm.q_full);
            };
            Tile tk, tv;
            int rk = -1, rv = -1, ik = 0, iv = 0, n_k = 0;
            int g_k = 0, g_v = 0;  // steps whose keys / values have been asked for
            bool more_k = next_tile(rk, tk), more_v = next_tile(rv, tv);
            if (more_k) load_queries(tk, 0);
            while (ok && (more_k || more_v)) {
                if (more_k && g_k <= g_v + 1) {  // keys at most two steps ahead of the values
                    load(g_k++, tk, ik, true);
                    if (++ik == steps_of(tk)) {
                        ik = 0;
                        more_k = next_tile(rk, tk);
                        if (more_k && ok) load_queries(tk, ++n_k);
                    }
                } else {
                    load(g_v++, tv, iv, false);
                    if (++iv == steps_of(tv)) {
                        iv = 0;
                        more_v = next_tile(rv, tv);
                    }
                }
            }
            if (!ok) atomicExch(p.error_flag, 61);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- issuer of the score products S = Q K^T, a step ahead of the softmax (two score buffers)
            const uint32_t id_s = idesc(ROWS, KEYS2, false);
            bool ok = true;
            int g = 0, n = 0, r = -1;
            Tile t;
            while (ok && next_tile(r, t)) {
                const int n_iter = steps_of(t);
                ok = mbar_wait(&sm.q_full, n & 1);
                if (!ok) break;
                for (int i = 0; i < n_iter && ok; ++i, ++g) {
                    const int s = g % K_STAGES2, b = g & 1;
                    ok = mbar_wait(&sm.k_full[s], (g / K_STAGES2) & 1);
                    if (ok && g >= 2) ok = mbar_wait(&sm.s_empty[b], ((g >> 1) - 1) & 1);  // the softmax has taken what was there
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint64_t da = desc_k_major(smem_u32(sm.q[k >> 2]) + (k & 3) * 32);
                        const uint64_t db = desc_k_major(smem_u32(sm.k[s][k >> 2][0]) + (k & 3) * 32);
                        umma_ss(tmem + COL2_S + b * KEYS2, da, db, id_s, k > 0);
                    }
                    umma_commit(&sm.k_empty[s]);  // the keys' shared memory is free once the scores are formed
                    umma_commit(&sm.s_full[b]);
                }
                umma_commit(&sm.q_empty);  // and so are the queries', once the tile's last scores are
                ++n;
            }
            if (!ok) atomicExch(p.error_flag, 62);
        }
    } else if (warp == 10) {
        if (lane == 0) {
            // ---- issuer of the products O += P V
            const uint32_t id_o = idesc(ROWS, D, true);
            bool ok = true;
            int g = 0, n = 0, r = -1;
            Tile t;
            while (ok && next_tile(r, t)) {
                const int n_iter = steps_of(t);
                for (int i = 0; i < n_iter && ok; ++i, ++g) {
                    const int s = g % KV_STAGES;
                    ok = mbar_wait(&sm.p_full, g & 1);
                    if (ok) ok = mbar_wait(&sm.v_full[s], (g / KV_STAGES) & 1);
                    // a tile's first product overwrites the accumulator: the result of the tile before has been read
                    if (ok && i == 0 && n > 0) ok = mbar_wait(&sm.o_free, (n - 1) & 1);
                    if (!ok) break;
                    fence_after();
#pragma unroll
                    for (int j = 0; j < KEYS2 / 16; ++j) {
                        const uint64_t db = desc_mn_major(smem_u32(sm.v[s][j >> 2][0]) + (j & 3) * 16 * 128, PAGE * 128);
                        umma_ts(tmem + COL2_O, tmem + COL2_P + j * 8, db, id_o, i > 0 || j > 0);
                    }
                    umma_commit(&sm.v_empty[s]);
                    umma_commit(&sm.o_done);
                }
                ++n;
            }
            if (!ok) atomicExch(p.error_flag, 64);
        }
    } else {
        // ---- softmax warps: two threads a row, as in the kernel above
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int quad_row = quarter * 32 + (lane & ~3), piece = lane & 3;
        bool ok = true;
        int g = 0, n = 0, round = -1;
        Tile t;
        while (ok && next_tile(round, t)) {
            const int p_begin = t.p_begin, p_end = t.p_end, len = t.len;
            const int n_iter = steps_of(t);
            const int row = t.tile * ROWS + r;
            const bool row_ok = row < t.n_rows;
            const int tok = row_ok ? row / group : 0;
            const int pos = t.past + tok;
            float m_used = -INFINITY, l = 0.f;
            for (int i = 0; i < n_iter && ok; ++i, ++g) {
                const int s = g % KV_STAGES, b = g & 1;
                const int key_base = (p_begin + 2 * i) * PAGE + half * 64;  // the first key this thread looks at
                const uint32_t s_cols = tmem + lane_base + COL2_S + b * KEYS2 + half * 64;
                ok = mbar_wait(&sm.s_full[b], (g >> 1) & 1);
                if (!ok) break;
                fence_after();
                uint32_t raw[2][32];
                tmem_ld32(s_cols, raw[0]);
                tmem_ld32(s_cols + 32, raw[1]);
                tmem_wait_ld();
                fence_before();
                mbar_arrive(&sm.s_empty[b]);  // the scores are in registers: the buffer may be overwritten
                const int step_base = (p_begin + 2 * i) * PAGE;
                const int valid = min(len - step_base, min(2, p_end - (p_begin + 2 * i)) * PAGE);
                if (valid < KEYS2) {
                    ok = mbar_wait(&sm.v_full[s], (g / KV_STAGES) & 1);
                    if (!ok) break;
                    for (int idx = half * 128 + r; idx < (KEYS2 - valid) * 16; idx += 256) {
                        const int vr = valid + idx / 16, chunk = idx % 16;
                        reinterpret_cast<uint4*>(sm.v[s][vr >> 6][chunk >> 3])[(vr & 63) * 8 + (chunk & 7)] = make_uint4(0, 0, 0, 0);
                    }
                    fence_async_smem();
                }
                if (key_base + 63 > pos || p.window > 0) {
                    const int hidden_upto = p.window > 0 ? pos - p.window : -1;
#pragma unroll
                    for (int c = 0; c < 64; ++c) {
                        const int key = key_base + c;
                        const bool hidden = (key > pos) | (key <= hidden_upto);
                        raw[c >> 5][c & 31] = hidden ? 0xff800000u : raw[c >> 5][c & 31];
                    }
                }
                float mx;
                {
                    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int c = 0; c < 64; c += 2)
                        m4[(c >> 1) & 3] = max_of_three(m4[(c >> 1) & 3], __uint_as_float(raw[c >> 5][c & 31]), __uint_as_float(raw[(c + 1) >> 5][(c + 1) & 31]));
                    mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                }
                sm.row_max[g & 1][half][r] = mx;
                mbar_arrive(&sm.max_ready[g & 1][quarter]);
                ok = mbar_wait(&sm.max_ready[g & 1][quarter], (g >> 1) & 1);
                if (!ok) break;
                mx = fmaxf(mx, sm.row_max[g & 1][half ^ 1][r]);
                const float m_new = fmaxf(m_used, mx * p.sl2);
                float corr = 1.0f;
                if (m_new > m_used + RESCALE_THRESHOLD || m_used == -INFINITY) {
                    corr = m_used == -INFINITY ? 0.f : exp2f(m_used - m_new);
                    m_used = m_new;
                }
                const float ref = m_used == -INFINITY ? 0.f : m_used;
                uint32_t packed[32];
                const uint64_t scale2 = pair_of(p.sl2, p.sl2), shift2 = pair_of(-ref, -ref);
                uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};  // four running pairs of sums
#pragma unroll
                for (int c = 0; c < 64; c += 2) {
                    float x0, x1;
                    halves_of(fma_pairs(pair_of(__uint_as_float(raw[c >> 5][c & 31]), __uint_as_float(raw[(c + 1) >> 5][(c + 1) & 31])), scale2, shift2), x0, x1);
                    const float e0 = ex2(x0), e1 = ex2(x1);
                    sums[(c >> 1) & 3] = add_pairs(sums[(c >> 1) & 3], pair_of(e0, e1));
                    __nv_bfloat162 pair = __floats2bfloat162_rn(e0, e1);
                    packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
                }
                float sum_lo, sum_hi;
                halves_of(add_pairs(add_pairs(sums[0], sums[1]), add_pairs(sums[2], sums[3])), sum_lo, sum_hi);
                l = l * corr + (sum_lo + sum_hi);
                if (g > 0) {
                    ok = mbar_wait(&sm.o_done, (g - 1) & 1);
                    if (!ok) break;
                    fence_after();
                }
                if (i > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
                    for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem + lane_base + COL2_O + c0, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
                        tmem_st32(tmem + lane_base + COL2_O + c0, o);
                    }
                }
                tmem_st32(tmem + lane_base + COL2_P + half * 32, packed);
                tmem_wait_st();
                fence_before();
                mbar_arrive(&sm.p_full);
            }
            if (!ok) break;
            // ---- the tile's result: O / l, this thread's half of the columns; l is the sum of both halves' sums
            sm.row_sum[half][r] = l;
            mbar_arrive(&sm.sum_ready);
            ok = mbar_wait(&sm.o_done, (g - 1) & 1);
            if (ok) ok = mbar_wait(&sm.sum_ready, n & 1);
            if (!ok) break;
            fence_after();
            const float inv = 1.0f / (sm.row_sum[0][r] + sm.row_sum[1][r]);
            uint32_t packed[32];
#pragma unroll
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t o[32];
                tmem_ld32(tmem + lane_base + COL2_O + half * 64 + c0, o);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                    packed[(c0 + c) >> 1] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            fence_before();
            mbar_arrive(&sm.o_free);  // the accumulator is in registers: the next tile's first product may overwrite it
            swap_pieces<uint32_t, 8>(packed, lane);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row_i = t.tile * ROWS + quad_row + i;
                if (row_i < t.n_rows) {
                    __nv_bfloat16* dst = p.out + ((size_t)(t.q_begin + row_i / group) * p.n_q + t.hk * group + row_i % group) * D + half * 64 + piece * 16;
                    store32(dst, packed + 8 * i);
                }
            }
            ++n;
        }
        if (!ok && lane == 0) atomicExch(p.error_flag, 63);
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
    }
}

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

// The pages of one layer, [n_pages, n_kv, 64, 128], as a matrix of n_pages * n_kv * 64 rows of 128.
int make_page_map(CUtensorMap* map, const void* base, long long rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * sizeof(__nv_bfloat16)};
    cuuint32_t box[2] = {64, (cuuint32_t)PAGE};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return GK_OK;
}

// The queries [n_tokens, n_q, 128] as a 3-D tensor; a box is 128 / group tokens x group heads x 64 elements.
int make_query_map(CUtensorMap* map, const void* base, long long n_tokens, int n_q, int group) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: the driver does not offer cuTensorMapEncodeTiled");
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_q, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)D * sizeof(__nv_bfloat16), (cuuint64_t)n_q * D * sizeof(__nv_bfloat16)};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(ROWS / group)};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: cuTensorMapEncodeTiled (queries) failed with code %d", (int)r);
    return GK_OK;
}

int g_attention_prefill_keys = KEYS2;  // 128 (the default) or 64
int g_attention_prefill_stay = 2;      // with 128 keys a step: blocks that stay and take tiles from a list: 0 never, 1 always, 2 (default) where the tiles are more than the SMs (needs the token count and a group that divides 128)
int g_attention_prefill_one_tile = 1;  // with 128 keys a step: 1 (the default) a query tile a block, heaviest first; 0 a heavy and a light tile a block

}  // namespace

// Same arguments as gk_attention_prefill_bf16 plus the number of pages of the layer's storage and the
// device error flag of the bounded waits.  head_dim must be 128.
static int prefill_tc_entry(const void* q, const void* k_pages, const void* v_pages, void* out,
                            const int* cu_q, const int* kv_len, const int* slots, const int* block_table,
                            int n_seqs, int max_q_len, int n_q, int n_kv, int head_dim, int max_pages,
                            int page_size, long long n_pages, float scale, int window, int* error_flag,
                            void* stream, long long n_tokens) {
    GK_REQUIRE(n_seqs >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_prefill_tc: bad head counts %d/%d", n_q, n_kv);
    GK_REQUIRE(page_size == PAGE && head_dim == D, "attention_prefill_tc: needs page_size %d and head_dim %d", PAGE, D);
    GK_REQUIRE(n_kv <= 65535 && n_seqs <= 65535 && window >= 0 && max_q_len >= 0 && n_pages > 0, "attention_prefill_tc: bad sizes");
    GK_REQUIRE(((uintptr_t)k_pages & 15) == 0 && ((uintptr_t)v_pages & 15) == 0 && ((uintptr_t)q & 31) == 0 &&
                   ((uintptr_t)out & 31) == 0, "attention_prefill_tc: pages must be 16-byte, queries and output 32-byte aligned");
    GK_REQUIRE(error_flag != nullptr, "attention_prefill_tc: error_flag is required");
    if (n_seqs == 0 || max_q_len == 0) return GK_OK;
    CUtensorMap mk, mv;
    int status = make_page_map(&mk, k_pages, n_pages * n_kv * PAGE);
    if (status) return status;
    status = make_page_map(&mv, v_pages, n_pages * n_kv * PAGE);
    if (status) return status;
    const size_t smem = sizeof(Smem) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: %s", cudaGetErrorString(err));
        configured = true;
    }
    Params p;
    p.q = (const __nv_bfloat16*)q;
    p.out = (__nv_bfloat16*)out;
    p.cu_q = cu_q;
    p.kv_len = kv_len;
    p.slots = slots;
    p.block_table = block_table;
    p.n_q = n_q;
    p.n_kv = n_kv;
    p.max_pages = max_pages;
    p.sl2 = scale * 1.4426950408889634f;
    p.window = window;
    p.error_flag = error_flag;
    p.one_tile = 0;
    p.n_seqs = n_seqs;
    p.n_items = 0;
    const int group = n_q / n_kv;
    const long long blocks = ((long long)max_q_len * group + ROWS - 1) / ROWS;
    GK_REQUIRE(blocks <= 2147483647LL, "attention_prefill_tc: too many rows");
    // measured for one prompt: 42 against 58 us at 2,048 tokens, 396 against 442 us at 8,192
    static int n_sms = 0;
    if (n_sms == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) n_sms = 148;
    }
    // measured for one prompt, blocks that stay against a block a tile: 22.4 against 21.5 us at 1,024 tokens (a tile an
    // SM: nothing to put under anything), 35.0 against 37.3 at 2,048, 99 against 104 at 4,096, 322 against 328 at 8,192
    const bool stay = g_attention_prefill_stay == 1 || (g_attention_prefill_stay == 2 && blocks * n_kv * n_seqs > n_sms);
    if (g_attention_prefill_keys == KEYS2 && stay && n_tokens > 0 && ROWS % group == 0 &&
        blocks * n_kv * n_seqs < 2147483647LL) {
        CUtensorMap mq;
        status = make_query_map(&mq, q, n_tokens, n_q, group);
        if (status) return status;
        const size_t smem5 = sizeof(Smem5) + 1024;
        static bool configured5 = false;
        if (!configured5) {
            cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem5);
            if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: %s", cudaGetErrorString(err));
            configured5 = true;
        }
        p.n_seqs = n_seqs;
        p.n_items = (int)(blocks * n_kv * n_seqs);
        dim3 grid5((unsigned)(p.n_items < n_sms ? p.n_items : n_sms));
        gk_launch(attention_prefill_tc5_kernel, grid5, dim3(THREADS2), smem5, (cudaStream_t)stream, mk, mv, mq, p);
        GK_CHECK_LAUNCH("attention_prefill_tc5");
        return GK_OK;
    }
    if (g_attention_prefill_keys == KEYS2) {
        const size_t smem2 = sizeof(Smem2) + 1024;
        static bool configured2 = false;
        if (!configured2) {
            cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
            if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_prefill_tc: %s", cudaGetErrorString(err));
            configured2 = true;
        }
        // measured for one prompt, a tile a block against pairs: 35.7 against 38.8 us at 2,048 tokens, 104 against 120 at
        // 4,096, 332 against 375 at 8,192, 1,170 against 1,186 at 16,384
        p.one_tile = g_attention_prefill_one_tile && blocks <= 65535;
        dim3 grid2((unsigned)((blocks + 1) / 2), n_kv, n_seqs);
        if (p.one_tile) grid2 = dim3(n_kv, n_seqs, (unsigned)blocks);
        gk_launch(attention_prefill_tc2_kernel, grid2, dim3(THREADS2), smem2, (cudaStream_t)stream, mk, mv, p);
        GK_CHECK_LAUNCH("attention_prefill_tc2");
        return GK_OK;
    }
    dim3 grid((unsigned)blocks, n_kv, n_seqs);
    gk_launch(attention_prefill_tc_kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream, mk, mv, p);
    GK_CHECK_LAUNCH("attention_prefill_tc");
    return GK_OK;
}

GK_EXPORT int gk_attention_prefill_tc_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                           const int* cu_q, const int* kv_len, const int* slots, const int* block_table,
                                           int n_seqs, int max_q_len, int n_q, int n_kv, int head_dim, int max_pages,
                                           int page_size, long long n_pages, float scale, int window, int* error_flag,
                                           void* stream) {
    return prefill_tc_entry(q, k_pages, v_pages, out, cu_q, kv_len, slots, block_table, n_seqs, max_q_len, n_q, n_kv, head_dim,
                            max_pages, page_size, n_pages, scale, window, error_flag, stream, 0);
}

// The same with the number of tokens in `q` (its first dimension), which the kernel with blocks that stay needs for
// the tensor map of the queries.
GK_EXPORT int gk_attention_prefill_tc_tokens_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                                  const int* cu_q, const int* kv_len, const int* slots, const int* block_table,
                                                  int n_seqs, int max_q_len, int n_q, int n_kv, int head_dim, int max_pages,
                                                  int page_size, long long n_pages, float scale, int window, int* error_flag,
                                                  void* stream, long long n_tokens) {
    return prefill_tc_entry(q, k_pages, v_pages, out, cu_q, kv_len, slots, block_table, n_seqs, max_q_len, n_q, n_kv, head_dim,
                            max_pages, page_size, n_pages, scale, window, error_flag, stream, n_tokens);
}

// With 128 keys a step: blocks that stay and take query tiles from the launch's list (where the token count is given
// and the group divides 128): 1 = always, 2 (the default) = where the tiles are more than the SMs, 0 = never (a block a
// tile, or a pair of tiles).  Returns the old setting.
GK_EXPORT int gk_set_attention_prefill_stay(int mode) {
    const int before = g_attention_prefill_stay;
    g_attention_prefill_stay = mode < 0 ? 0 : mode > 2 ? 2 : mode;
    return before;
}

// Keys per step of the tcgen05 prefill attention: 128 (the default: one block per SM, two score buffers, eight
// softmax warps, pairs of query tiles) or 64 (two blocks per SM, one query tile each).  Returns the old setting.
// With 128 keys a step: 1 (the default) = a query tile a block with the heaviest first, 0 = a heavy and a light query
// tile a block.  Returns the old setting.
GK_EXPORT int gk_set_attention_prefill_one_tile(int mode) {
    const int before = g_attention_prefill_one_tile;
    g_attention_prefill_one_tile = mode ? 1 : 0;
    return before;
}

GK_EXPORT int gk_set_attention_prefill_keys(int keys) {
    const int before = g_attention_prefill_keys;
    g_attention_prefill_keys = keys == PAGE ? PAGE : KEYS2;
    return before;
}
