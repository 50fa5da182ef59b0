// Prefill attention in bfloat16: the new tokens of every sequence of a step attend, causally,
// over the sequence's keys and values in the paged cache (their own included; a sequence may
// already hold cached tokens).  Flash-attention style: the score matrix is never written out; keys
// are taken a page (64) at a time with running 32-bit maxima and sums
// (src/ops/flash_attention_2.py:24-60 is the reference's kernel of the same scheme; its rule for a
// continued sequence, key j visible to new token i iff j <= past + i, is src/layers/attention.py:116-119).
//
// The rows of a block's tile are (token, query head of one kv group) pairs, token-major, so the
// `group` query heads that share a kv head share every loaded page.  Grid (row block, kv head,
// sequence); a warp owns 16 rows; K and V pages stream through a three-stage cp.async ring.
// Scores, softmax statistics and the output accumulator are 32-bit; probabilities are rounded to
// bfloat16 for the second product (flash_attention_2.py:55).

#include "attention_mma.cuh"

namespace {

using namespace attn;

constexpr int PF_WARPS = 4;
constexpr int PF_ROWS = PF_WARPS * 16;
constexpr int PF_STAGES = 3;

template <int D>
struct PrefillSmem {
    __nv_bfloat16 k[PF_STAGES][PAGE * D];
    __nv_bfloat16 v[PF_STAGES][PAGE * D];
};

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32) attention_prefill_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q,
    const int* __restrict__ kv_len, const int* __restrict__ slots, const int* __restrict__ block_table, int n_q,
    int n_kv, int max_pages, float sl2, int window) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    PrefillSmem<D>& sm = *reinterpret_cast<PrefillSmem<D>*>(smem_raw);
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, hk = blockIdx.y;
    const int group = n_q / n_kv;
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int n_rows = q_len * group;
    // heavy blocks (late tokens, long key ranges) first
    const int n_blocks = (n_rows + PF_ROWS - 1) / PF_ROWS;
    if ((int)blockIdx.x >= n_blocks) return;
    const int row0 = (n_blocks - 1 - (int)blockIdx.x) * PF_ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int len = kv_len[seq], past = len - q_len;
    const int* pages = block_table + (size_t)slots[seq] * max_pages;

    // rows of this thread: r_lo = row0 + warp*16 + lane/4 and r_lo + 8
    const int wrow0 = row0 + warp * 16;
    int tok[2], pos[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = wrow0 + (lane >> 2) + 8 * h;
        row_ok[h] = r < n_rows;
        tok[h] = row_ok[h] ? r / group : 0;
        pos[h] = past + tok[h];
    }
    // Query fragments straight from global memory.
    uint32_t qf[D / 16][4];
    {
        const int c0 = (lane & 3) * 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = wrow0 + (lane >> 2) + 8 * h;
            const __nv_bfloat16* qrow = q + ((size_t)(q_begin + tok[h]) * n_q + (size_t)hk * group + (r % group)) * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qf[ks][h] = row_ok[h] ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + c0) : 0u;
                qf[ks][h + 2] = row_ok[h] ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + c0 + 8) : 0u;
            }
        }
    }
    // key range of the block: from the first key its first row may see to the last key its last row sees
    const int last_row = min(row0 + PF_ROWS, n_rows) - 1;
    const int max_pos = past + last_row / group;
    const int min_pos = past + row0 / group;
    const int lo_block = (window > 0 && min_pos - window + 1 > 0) ? min_pos - window + 1 : 0;
    const int p_begin = lo_block / PAGE, p_end = max_pos / PAGE + 1;
    const int n_iter = p_end - p_begin;
    // of this warp
    const int w_last_row = min(wrow0 + 16, n_rows) - 1;
    const int w_max_pos = w_last_row >= wrow0 ? past + w_last_row / group : -1;
    const int w_min_pos = past + wrow0 / group;
    const int w_lo = (window > 0 && w_min_pos - window + 1 > 0) ? w_min_pos - window + 1 : 0;

    auto issue = [&](int it) {
        if (it < n_iter) {
            const int p = p_begin + it;
            const int page = pages[p];
            const int valid = min(PAGE, len - p * PAGE);
            const size_t base = ((size_t)page * n_kv + hk) * PAGE * D;
            const int stage = it % PF_STAGES;
            load_page_async<D, PF_WARPS * 32>(sm.k[stage], k_pages + base, valid, tid);
            load_page_async<D, PF_WARPS * 32>(sm.v[stage], v_pages + base, valid, tid);
        }
        cp_async_commit();
    };

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;

#pragma unroll
    for (int st = 0; st < PF_STAGES - 1; ++st) issue(st);
    for (int it = 0; it < n_iter; ++it) {
        cp_async_wait<PF_STAGES - 2>();  // page `it` has landed
        __syncthreads();                 // for everyone; and the stage refilled next was read an iteration ago
        issue(it + PF_STAGES - 1);
        const int stage = it % PF_STAGES;
        const int key_base = (p_begin + it) * PAGE;
        if (key_base <= w_max_pos && key_base + PAGE > w_lo) {  // warp-uniform
            // groups of 16 keys beyond the warp's last position are in the future of all its rows
            const int n16 = min(PAGE / 16, (w_max_pos - key_base) / 16 + 1);
            const bool need_mask = key_base + PAGE - 1 > w_min_pos || key_base < w_lo || window > 0;
            float s[8][4];
            uint32_t p[4][4];
            if (!need_mask) {  // the common case: a page wholly in the past of all the warp's rows
                qk_page<D, true>(s, qf, sm.k[stage], 4, lane);
                softmax_page<D>(s, m, l, o, p, sl2);
                pv_page<D, true>(o, p, sm.v[stage], 4, lane);
            } else {
                qk_page<D, false>(s, qf, sm.k[stage], n16, lane);
#pragma unroll
                for (int n = 0; n < 8; ++n)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int key = key_base + n * 8 + (lane & 3) * 2 + c;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const bool hidden = key > pos[h] || (window > 0 && key <= pos[h] - window);
                            if (hidden) s[n][2 * h + c] = -INFINITY;
                        }
                    }
                softmax_page<D>(s, m, l, o, p, sl2);
                pv_page<D, false>(o, p, sm.v[stage], n16, lane);
            }
        }
    }
    cp_async_wait<0>();

    const int c0 = (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_ok[h]) continue;
        const int r = wrow0 + (lane >> 2) + 8 * h;
        const float inv = 1.0f / l[h];
        __nv_bfloat16* orow = out + ((size_t)(q_begin + tok[h]) * n_q + (size_t)hk * group + (r % group)) * D;
#pragma unroll
        for (int j = 0; j < D / 8; ++j)
            *reinterpret_cast<uint32_t*>(orow + j * 8 + c0) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
    }
}

template <int D>
int launch_prefill(const void* q, const void* k_pages, const void* v_pages, void* out, const int* cu_q, const int* kv_len,
                   const int* slots, const int* block_table, int n_seqs, int max_q_len, int n_q, int n_kv, int max_pages,
                   float scale, int window, cudaStream_t stream) {
    const size_t smem = sizeof(PrefillSmem<D>);
    static bool configured = false;
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_prefill: %s", cudaGetErrorString(err));
        configured = true;
    }
    const int group = n_q / n_kv;
    const long long blocks = ((long long)max_q_len * group + PF_ROWS - 1) / PF_ROWS;
    GK_REQUIRE(blocks <= 2147483647LL, "attention_prefill: too many rows");
    dim3 grid((unsigned)blocks, n_kv, n_seqs);
    gk_launch(attention_prefill_kernel<D>, grid, dim3(PF_WARPS * 32), smem, stream, (const __nv_bfloat16*)q,
              (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out, cu_q, kv_len, slots,
              block_table, n_q, n_kv, max_pages, scale * 1.4426950408889634f, window);
    GK_CHECK_LAUNCH("attention_prefill");
    return GK_OK;
}

}  // namespace

// q, out: [n_tokens, n_q, head_dim] packed by sequence (cu_q[i] = first token of sequence i);
// kv_len[i] counts the sequence's cached tokens including this step's; max_q_len = the longest
// sequence part of the step (sizes the grid).
GK_EXPORT int gk_attention_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                        const int* cu_q, const int* kv_len, const int* slots, const int* block_table,
                                        int n_seqs, int max_q_len, int n_q, int n_kv, int head_dim, int max_pages,
                                        int page_size, float scale, int window, void* stream) {
    GK_REQUIRE(n_seqs >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_prefill: bad head counts %d/%d", n_q, n_kv);
    GK_REQUIRE(page_size == attn::PAGE, "attention_prefill: page_size must be %d, got %d", attn::PAGE, page_size);
    GK_REQUIRE(head_dim == 64 || head_dim == 128, "attention_prefill: head_dim %d is not 64 or 128 (use the exact kernel)", head_dim);
    GK_REQUIRE(n_kv <= 65535 && n_seqs <= 65535, "attention_prefill: grid too large");
    GK_REQUIRE(window >= 0 && max_q_len >= 0, "attention_prefill: bad window or length");
    if (n_seqs == 0 || max_q_len == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64)
        return launch_prefill<64>(q, k_pages, v_pages, out, cu_q, kv_len, slots, block_table, n_seqs, max_q_len, n_q, n_kv,
                                  max_pages, scale, window, s);
    return launch_prefill<128>(q, k_pages, v_pages, out, cu_q, kv_len, slots, block_table, n_seqs, max_q_len, n_q, n_kv,
                               max_pages, scale, window, s);
}
