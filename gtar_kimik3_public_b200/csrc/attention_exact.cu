// Causal grouped-query attention over the paged cache, any head size, any dtype: the exact
// kernel.  It is the 32-bit path's attention and the fallback of the bfloat16 path for head
// sizes the tensor-core kernels do not take.
//
// For a token at position pos of its sequence, query head hq, kv head hk = hq / (n_q / n_kv):
//   s_j = (q . k_j) * scale      for the visible keys j <= pos (and j > pos - window, if a window is set)
//   o   = sum_j softmax(s)_j v_j
// which is the rule  key j visible to query i iff j <= past + i  of the reference
// (src/layers/attention.py:116-119) with consecutive query heads sharing a kv head
// (src/ops/flash_attention_2.py:33-34), scale = head_dim^-0.5 (flash_attention_2.py:216).
//
// One warp per (token, query head).  Keys are taken in blocks of 32 from key 0 upward, one key
// per lane, with a running maximum and sum (all 32-bit, expf).  The sequence of operations for
// a (token, head) depends only on its own position and keys: results are bit-equal however the
// tokens are cut into steps or batched.

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_ACC = 16;  // head_dim <= 512

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + i);
        acc = fmaf(q[i], kv.x, acc);
        acc = fmaf(q[i + 1], kv.y, acc);
        acc = fmaf(q[i + 2], kv.z, acc);
        acc = fmaf(q[i + 3], kv.w, acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q,
                                                        const __nv_bfloat16* __restrict__ k, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float2 f = __bfloat1622float2(p[c]);
            acc = fmaf(q[i + 2 * c], f.x, acc);
            acc = fmaf(q[i + 2 * c + 1], f.y, acc);
        }
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attention_exact_kernel(
    const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ out,
    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ slots,
    const int* __restrict__ block_table, int n_tokens, int n_q, int n_kv, int head_dim, int max_pages, int page_size,
    float scale, int window) {
    extern __shared__ float q_smem[];  // WARPS * head_dim
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long wid = (long long)blockIdx.x * WARPS + warp;
    if (wid >= (long long)n_tokens * n_q) return;  // whole warp leaves together; no block-wide sync below
    const int t = (int)(wid / n_q);
    const int hq = (int)(wid - (long long)t * n_q);
    const int hk = hq / (n_q / n_kv);
    const int pos = tok_pos[t];
    const int slot = slots[tok_seq[t]];
    const int* pages = block_table + (size_t)slot * max_pages;
    float* qs = q_smem + warp * head_dim;
    const T* qrow = q + ((size_t)t * n_q + hq) * head_dim;
    for (int i = lane; i < head_dim; i += 32) qs[i] = to_float(qrow[i]);
    __syncwarp();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int c = 0; c < MAX_ACC; ++c) acc[c] = 0.f;
    const int n_acc = (head_dim + 31) >> 5;

    for (int j0 = (lo >> 5) << 5; j0 <= pos; j0 += 32) {
        const int page = pages[j0 / page_size];  // page_size is a multiple of 32: one page per block
        const int in_page = j0 % page_size;
        const size_t base = (((size_t)page * n_kv + hk) * page_size + in_page) * head_dim;
        const int j = j0 + lane;
        const bool valid = j <= pos && j >= lo;
        float s = -INFINITY;
        if (valid) s = dot_row<T>(qs, k_pages + base + (size_t)lane * head_dim, head_dim) * scale;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        const int n_here = min(32, pos - j0 + 1);
#pragma unroll
        for (int c = 0; c < MAX_ACC; ++c)
            if (c < n_acc) acc[c] *= corr;
        for (int jj = 0; jj < n_here; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vrow = v_pages + base + (size_t)jj * head_dim;
#pragma unroll
            for (int c = 0; c < MAX_ACC; ++c) {
                const int dim = lane + 32 * c;
                if (c < n_acc && dim < head_dim) acc[c] = fmaf(pj, to_float(vrow[dim]), acc[c]);
            }
        }
        m = m_new;
    }
    T* orow = out + ((size_t)t * n_q + hq) * head_dim;
#pragma unroll
    for (int c = 0; c < MAX_ACC; ++c) {
        const int dim = lane + 32 * c;
        if (c < n_acc && dim < head_dim) orow[dim] = from_float<T>(acc[c] / l);
    }
}

}  // namespace

GK_EXPORT int gk_attention_exact(const void* q, const void* k_pages, const void* v_pages, void* out, int dtype,
                                 const int* tok_pos, const int* tok_seq, const int* slots, const int* block_table,
                                 int n_tokens, int n_q, int n_kv, int head_dim, int max_pages, int page_size,
                                 float scale, int window, void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "attention_exact: bad dtype %d", dtype);
    GK_REQUIRE(n_tokens >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_exact: bad head counts %d/%d", n_q,
               n_kv);
    GK_REQUIRE(head_dim > 0 && head_dim % 8 == 0 && head_dim <= 32 * MAX_ACC,
               "attention_exact: head_dim %d must be a multiple of 8 and at most %d", head_dim, 32 * MAX_ACC);
    GK_REQUIRE(page_size > 0 && page_size % 32 == 0, "attention_exact: page_size %d must be a multiple of 32",
               page_size);
    GK_REQUIRE(window >= 0, "attention_exact: window must be >= 0 (0 = none)");
    if (n_tokens == 0) return GK_OK;
    const long long warps = (long long)n_tokens * n_q;
    const long long blocks = (warps + WARPS - 1) / WARPS;
    GK_REQUIRE(blocks < 2147483647LL, "attention_exact: too many tokens");
    const size_t smem = (size_t)WARPS * head_dim * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(attention_exact_kernel<T>, dim3((unsigned)blocks), dim3(WARPS * 32), smem, s,
            (const T*)q, (const T*)k_pages, (const T*)v_pages, (T*)out, tok_pos, tok_seq, slots, block_table, n_tokens,
            n_q, n_kv, head_dim, max_pages, page_size, scale, window);
    })
    GK_CHECK_LAUNCH("attention_exact");
    return GK_OK;
}
