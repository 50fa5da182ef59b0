// Decode attention in bfloat16: one new token per sequence attends over its cached keys and
// values in the paged cache.  Memory-bound: every cached key and value is read once per step
// and is shared by all query heads of its group, which form the 16 rows of the tensor-core
// tile (the reference expands nothing either: kv head = query head / group,
// src/ops/flash_attention_2.py:33-34; visibility rule of src/layers/attention.py:116-119 with
// one query at the last position).
//
// Grid (split, kv head, sequence).  A sequence's pages are divided among `n_splits` blocks so
// that small batches still fill the GPU; each block streams its pages through a multi-stage
// cp.async pipeline, its four warps taking 16 keys of a page each, and ends with an unnormalised
// partial result (max, sum, output).  Up to eight splits form a thread-block cluster: every block sends its
// partial outputs into the shared memory of the block that merges them (each block merges a share); more
// splits leave their partial results in scratch memory and a second kernel merges them.
// Lengths come from device memory, so a captured launch stays valid as sequences grow.
//
// Softmax statistics and accumulators are 32-bit; probabilities are rounded to bfloat16 for
// the second product, as in the reference's kernel (flash_attention_2.py:55).

#include "attention_decode_fused.cuh"
#include "no_alloc.h"

namespace {

using namespace attn;

constexpr int WARPS = 4;
constexpr int STAGES = 3;

template <int D>
struct DecodeSmem {
    __nv_bfloat16 k[STAGES][PAGE * D];
    __nv_bfloat16 v[STAGES][PAGE * D];
    // what the fused input stage needs and no kernel of the step writes: the q and k norm weights and the
    // rotation of the new token's position, fetched while the kernel in front still runs
    float wq[D], wk[D], cos[D / 2], sin[D / 2];
    // Where the other blocks of a cluster leave their partial results for the outputs that this block merges
    // ([source block][this block's outputs]) and their maxima and sums ([source block][head of the group][2]): a
    // region of its own, since they arrive while this block may still be streaming pages through the stages.
    float from_o[16 * D + 8 * 32];
    float from_ml[8 * 16 * 2];
};

template <int D>
__global__ void __launch_bounds__(WARPS * 32) attention_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
    const __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
    float* __restrict__ part_ml, const int* __restrict__ kv_len, const int* __restrict__ slots,
    const int* __restrict__ block_table, int n_q, int n_kv, int max_pages, float sl2, int window, int n_splits,
    int cluster_merge, int group, const FusedQkv fused) {  // group = n_q / n_kv, divided on the host
    extern __shared__ __align__(128) unsigned char smem_raw[];
    DecodeSmem<D>& sm = *reinterpret_cast<DecodeSmem<D>*>(smem_raw);
    const int split = blockIdx.x, hk = blockIdx.y, seq = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();
    // Two trips to memory before the wait, not one after another for every item: the length, the slot and the norm
    // weights first; then, from the length and the slot, the ids of the first pages and the rotation's row.
    const int len = kv_len[seq];
    const int slot = slots[seq];
    float w_q = 1.f, w_k = 1.f;  // thread c holds element c (a head has at most as many elements as the block threads)
    if (fused.qkv && fused.use_norm && tid < D) {
        w_q = weight_at(fused.wq, fused.weights_bf16, tid);
        w_k = weight_at(fused.wk, fused.weights_bf16, tid);
    }
    const int lo = (window > 0 && len - window > 0) ? len - window : 0;  // first visible key
    const int* pages = block_table + (size_t)slot * max_pages;
    const int first_page = lo / PAGE, end_page = (len + PAGE - 1) / PAGE;
    // By shift and mask where the splits are a power of two (the host's choice always is): a division by a run-time
    // number is a chain of some thirty dependent instructions, here in front of the first page's id and, for the
    // places of the merged outputs, in the kernel's tail, where nothing hides it.
    const bool pow2 = (n_splits & (n_splits - 1)) == 0;
    const int split_shift = __ffs(n_splits) - 1;
    const int units = (group * D + 31) / 32;  // the group's outputs are dealt out for merging in units of 32
    const int cap = (pow2 ? (units + n_splits - 1) >> split_shift : (units + n_splits - 1) / n_splits) * 32;
    const int pages_here = end_page - first_page + n_splits - 1;
    const int per_split = pow2 ? pages_here >> split_shift : pages_here / n_splits;
    const int p_begin = first_page + split * per_split;
    const int p_end = min(p_begin + per_split, end_page);
    const int n_iter = max(p_end - p_begin, 0);
    const int new_page = (len - 1) / PAGE;

    auto issue_page = [&](int it, int page, int stage) {  // stage = it % STAGES, which the caller has at hand
        const int p = p_begin + it;
        const int valid = min(PAGE, len - p * PAGE);
        const size_t base = ((size_t)page * n_kv + hk) * PAGE * D;
        load_page_async<D, WARPS * 32>(sm.k[stage], k_pages + base, valid, tid);
        load_page_async<D, WARPS * 32>(sm.v[stage], v_pages + base, valid, tid);
    };
    auto issue = [&](int it, int stage) {
        if (it < n_iter) issue_page(it, pages[p_begin + it], stage);
        cp_async_commit();
    };
    // Lengths, slots and the page table are step inputs (copied in before the step's first kernel),
    // and every page but the one holding the new token was written by earlier steps: all of that may
    // be read while the kernel before this one (which writes the new token's key and value and the
    // queries) is still running.
    static_assert(STAGES == 3, "two pages are asked for ahead of the loop");
    int early = 0, early_page0 = 0, early_page1 = 0;
    if (0 < n_iter && p_begin < new_page) {
        early_page0 = pages[p_begin];
        early = 1;
        if (1 < n_iter && p_begin + 1 < new_page) {
            early_page1 = pages[p_begin + 1];
            early = 2;
        }
    }
    float cs = 1.f, sn = 0.f;
    if (fused.qkv && fused.cos_table && tid < D / 2) {
        cs = fused.cos_table[(size_t)(len - 1) * (D / 2) + tid];
        sn = fused.sin_table[(size_t)(len - 1) * (D / 2) + tid];
    }
    if (early > 0) {
        issue_page(0, early_page0, 0);
        cp_async_commit();
    }
    if (early > 1) {
        issue_page(1, early_page1, 1);
        cp_async_commit();
    }
    if (fused.qkv && tid < D) {
        sm.wq[tid] = w_q;
        sm.wk[tid] = w_k;
        if (tid < D / 2) {
            sm.cos[tid] = cs;
            sm.sin[tid] = sn;
        }
    }
    if (fused.qkv) __syncthreads();  // the constants above, for every warp: ahead of the wait, where the barrier costs nothing
    pdl_wait();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s)
        if (s >= early) issue(s, s);

    // The new token's raw key and value are asked for first (by the warp of the block that will write them), so
    // that they are on their way while the queries are prepared.
    const bool owns_new = fused.qkv != nullptr && fused.write_kv && new_page >= p_begin && new_page < p_end;
    __nv_bfloat162 k_raw[D / 64], k_new[D / 64], v_new[D / 64];  // lane l: elements 2l, 2l+1 of each 64-wide half
    if (owns_new && warp == 0) {
        const int n_heads = n_q + 2 * n_kv;
        const __nv_bfloat16* krow = fused.qkv + ((size_t)seq * n_heads + n_q + hk) * D;
        const __nv_bfloat16* vrow = fused.qkv + ((size_t)seq * n_heads + n_q + n_kv + hk) * D;
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
            k_raw[hf] = *reinterpret_cast<const __nv_bfloat162*>(krow + hf * 64 + 2 * lane);
            v_new[hf] = *reinterpret_cast<const __nv_bfloat162*>(vrow + hf * 64 + 2 * lane);
        }
    }
    // Query fragments: row r of the tile is query head hk*group + r (rows >= group are zero).
    uint32_t qf[D / 16][4];
    const int pos_new = len - 1;
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
        const int n_heads = n_q + 2 * n_kv;
        const __nv_bfloat16* qbase = fused.qkv ? fused.qkv + ((size_t)seq * n_heads + (size_t)hk * group) * D
                                               : q + ((size_t)seq * n_q + (size_t)hk * group) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = r0 + (i & 1) * 8, c = ks * 16 + c0 + (i >> 1) * 8;
                qf[ks][i] = r < group ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)r * D + c) : 0u;
            }
        }
        if (fused.qkv) {
            // A thread holds, of each of its two rows, the elements c0, c0+1, c0+8, c0+9 of every
            // 16-wide step: a quad holds a whole row, and the rotation partner of column c (c + D/2)
            // is four steps further on in the same thread.
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h * 8 >= group) continue;  // the upper eight rows of the tile hold no head of a group of up to eight
                float x[D / 16][4];
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qf[ks][h]));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qf[ks][h + 2]));
                    x[ks][0] = a.x; x[ks][1] = a.y; x[ks][2] = b.x; x[ks][3] = b.y;
                }
                if (fused.use_norm) {
                    float ss = 0.f;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
                        for (int e = 0; e < 4; ++e) ss += x[ks][e] * x[ks][e];
                    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                    const float inv = rsqrtf(ss / (float)D + fused.eps);
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = ks * 16 + c0 + (e & 1) + (e >> 1) * 8;
                            x[ks][e] = (x[ks][e] * inv) * sm.wq[c];
                        }
                }
                if (fused.cos_table) {
#pragma unroll
                    for (int ks = 0; ks < D / 32; ++ks)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int c = ks * 16 + c0 + (e & 1) + (e >> 1) * 8;  // first half of the head
                            const float cs = sm.cos[c], sn = sm.sin[c];
                            const float a = x[ks][e], b = x[ks + D / 32][e];
                            x[ks][e] = a * cs - b * sn;
                            x[ks + D / 32][e] = b * cs + a * sn;
                        }
                }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    qf[ks][h] = pack_bf16(x[ks][0], x[ks][1]);
                    qf[ks][h + 2] = pack_bf16(x[ks][2], x[ks][3]);
                }
            }
        }
    }
    // The new token's key and value, by the block that holds its page: one warp makes them, writes them
    // to the cache, and keeps them for patching the page's copy in shared memory once that has landed.
    if (owns_new && warp == 0) {
        float kx[D / 64][2];
        float ss = 0.f;
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
            const float2 f = __bfloat1622float2(k_raw[hf]);
            kx[hf][0] = f.x;
            kx[hf][1] = f.y;
            ss += f.x * f.x + f.y * f.y;
        }
        if (fused.use_norm) {
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + fused.eps);
#pragma unroll
            for (int hf = 0; hf < D / 64; ++hf)
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    kx[hf][e] = (kx[hf][e] * inv) * sm.wk[hf * 64 + 2 * lane + e];
        }
        if (fused.cos_table) {
            // partner of column c is c + D/2: for D = 128 the other half held by this lane, for D = 64 the
            // lane 16 further on
            if (D == 128) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 2 * lane + e;
                    const float cs = sm.cos[c], sn = sm.sin[c];
                    const float a = kx[0][e], b = kx[D / 64 - 1][e];
                    kx[0][e] = a * cs - b * sn;
                    kx[D / 64 - 1][e] = b * cs + a * sn;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float mine = kx[0][e];
                    const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                    const int c = (2 * lane + e) % (D / 2);
                    const float cs = sm.cos[c], sn = sm.sin[c];
                    kx[0][e] = lane < 16 ? mine * cs - other * sn : mine * cs + other * sn;
                }
            }
        }
        const size_t at = (((size_t)pages[new_page] * n_kv + hk) * PAGE + (pos_new % PAGE)) * D;
#pragma unroll
        for (int hf = 0; hf < D / 64; ++hf) {
            k_new[hf] = __floats2bfloat162_rn(kx[hf][0], kx[hf][1]);
            *reinterpret_cast<__nv_bfloat162*>(const_cast<__nv_bfloat16*>(k_pages) + at + hf * 64 + 2 * lane) = k_new[hf];
            *reinterpret_cast<__nv_bfloat162*>(const_cast<__nv_bfloat16*>(v_pages) + at + hf * 64 + 2 * lane) = v_new[hf];
        }
    }

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;

    const int key0 = warp * 16;
    const uint32_t k_offset = k_lane_offset<D>(key0, lane), v_offset = v_lane_offset<D>(key0, lane);
    const uint32_t k_tiles = smem_u32(sm.k[0]), v_tiles = smem_u32(sm.v[0]);
    constexpr uint32_t TILE_BYTES = PAGE * D * 2;
    for (int it = 0, stage = 0; it < n_iter; ++it, stage = stage + 1 == STAGES ? 0 : stage + 1) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();  // page `it` has landed for everyone; the stage issued next was consumed an iteration ago
        issue(it + STAGES - 1, stage == 0 ? STAGES - 1 : stage - 1);
        if (owns_new && p_begin + it == new_page) {  // block-uniform
            if (warp == 0) {
                const int row = pos_new % PAGE;
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf) {
                    const int col = hf * 64 + 2 * lane;  // element index; its 16-byte chunk is col / 8
                    const int word = swz<D>(row, col >> 3) * 8 + (col & 7);
                    *reinterpret_cast<__nv_bfloat162*>(sm.k[stage] + word) = k_new[hf];
                    *reinterpret_cast<__nv_bfloat162*>(sm.v[stage] + word) = v_new[hf];
                }
            }
            __syncthreads();
        }
        const int abs0 = (p_begin + it) * PAGE + key0;
        if (abs0 < len && abs0 + 16 > lo) {  // warp-uniform: skip sixteen keys that are all hidden
            float s[2][4];
            qk_16keys_at<D>(s, qf, k_tiles + stage * TILE_BYTES, k_offset);
            if (abs0 + 16 > len || abs0 < lo) {  // warp-uniform: only the sixteen keys at an edge have hidden ones
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int key = abs0 + n * 8 + (lane & 3) * 2 + c;
                        if (key >= len || key < lo) s[n][c] = s[n][2 + c] = -INFINITY;
                    }
            }
            uint32_t p[4];
            softmax_update<D>(s, m, l, o, p, sl2);
            pv_16keys_at<D>(o, p, v_tiles + stage * TILE_BYTES, v_offset);
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    // Merge the four warps through shared memory (the stages are free now).
    float* red_o = reinterpret_cast<float*>(smem_raw);          // [WARPS][16][D]
    float* red_ml = red_o + WARPS * 16 * D;                    // [WARPS][16][2]
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = r0 + 8 * h;
            if (r >= group) continue;  // rows of the tile beyond the heads of this group hold nothing
            if ((lane & 3) == 0) {
                red_ml[(warp * 16 + r) * 2] = m[h];
                red_ml[(warp * 16 + r) * 2 + 1] = l[h];
            }
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                red_o[(warp * 16 + r) * D + j * 8 + c0] = o[j][2 * h];
                red_o[(warp * 16 + r) * D + j * 8 + c0 + 1] = o[j][2 * h + 1];
            }
        }
    }
    __syncthreads();
    // With a cluster, outputs are dealt out in units of 32: unit u is merged by block u % n_splits, which holds
    // room for cap = (units a block can have) * 32 values from every block.
    auto unit_owner = [&](int unit) { return pow2 ? unit & (n_splits - 1) : unit % n_splits; };
    auto unit_place = [&](int unit) { return pow2 ? unit >> split_shift : unit / n_splits; };
    for (int idx = tid; idx < group * D; idx += WARPS * 32) {
        const int r = idx / D, c = idx % D;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, red_ml[(w * 16 + r) * 2]);
        float ll = 0.f, acc = 0.f;
        if (mm != -INFINITY) {
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float f = exp2_fast(red_ml[(w * 16 + r) * 2] - mm);
                ll += red_ml[(w * 16 + r) * 2 + 1] * f;
                acc += red_o[(w * 16 + r) * D + c] * f;
            }
        }
        const int hq = hk * group + r;
        if (n_splits == 1) {
            out[((size_t)seq * n_q + hq) * D + c] = __float2bfloat16_rn(__fdividef(acc, ll));
        } else if (cluster_merge) {
            // The splits of one (sequence, kv head) are one cluster: a block sends each of its partial outputs
            // straight into the shared memory of the block that merges that output, and its maxima and sums to
            // every block (posted stores: nobody fetches from another SM and waits), no scratch, no second kernel.
            const int unit = idx >> 5, owner = unit_owner(unit);
            const uint32_t at = smem_u32(sm.from_o + split * cap + unit_place(unit) * 32 + (idx & 31));
            uint32_t remote;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(at), "r"(owner));
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(acc) : "memory");
            if (c == 0) {
                const uint32_t ml_at = smem_u32(sm.from_ml + (split * 16 + r) * 2);
                for (int to = 0; to < n_splits; ++to) {
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(ml_at), "r"(to));
                    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote), "f"(mm), "f"(ll) : "memory");
                }
            }
        } else {
            const size_t at = ((size_t)seq * n_q + hq) * n_splits + split;
            part_o[at * D + c] = acc;
            if (c == 0) {
                part_ml[at * 2] = mm;
                part_ml[at * 2 + 1] = ll;
            }
        }
    }
    if (n_splits > 1 && cluster_merge) {
        // everything sent has arrived once every block of the cluster is here
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        // every block merges its own share of the group's outputs, in split order, from its own shared memory
        for (int unit = split + warp * n_splits; unit < units; unit += WARPS * n_splits) {
            const int idx = unit * 32 + lane;
            if (idx >= group * D) break;
            const int r = idx / D;
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                ms[sp] = -INFINITY;
                ls[sp] = os[sp] = 0.f;
                if (sp < n_splits) {
                    ms[sp] = sm.from_ml[(sp * 16 + r) * 2];
                    ls[sp] = sm.from_ml[(sp * 16 + r) * 2 + 1];
                    os[sp] = sm.from_o[sp * cap + unit_place(unit) * 32 + lane];
                }
            }
            float mm = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) mm = fmaxf(mm, ms[sp]);
            float ll = 0.f, acc = 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
                if (sp < n_splits && ms[sp] != -INFINITY) {
                    const float f = exp2_fast(ms[sp] - mm);
                    ll += ls[sp] * f;
                    acc += os[sp] * f;
                }
            out[((size_t)seq * n_q + hk * group + r) * D + (idx % D)] = __float2bfloat16_rn(__fdividef(acc, ll));
        }
    }
}

// out[seq, head, :] = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M),  M = max_s m_s
template <int D>
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              __nv_bfloat16* __restrict__ out, int n_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = blockIdx.x;  // seq * n_q + head
    const float* ml = part_ml + row * n_splits * 2;
    float mm = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, ml[2 * s]);
    float ll = 0.f;
    for (int s = 0; s < n_splits; ++s)
        if (ml[2 * s] != -INFINITY) ll += ml[2 * s + 1] * exp2f(ml[2 * s] - mm);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s)
            if (ml[2 * s] != -INFINITY) acc += part_o[(row * n_splits + s) * D + c] * exp2f(ml[2 * s] - mm);
        out[row * D + c] = __float2bfloat16_rn(__fdividef(acc, ll));
    }
}

template <int D>
int launch_decode(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o, float* part_ml,
                  const int* kv_len, const int* slots, const int* block_table, int n_seqs, int n_q, int n_kv,
                  int max_pages, float scale, int window, int n_splits, cudaStream_t stream, const FusedQkv& fused) {
    const size_t stage_bytes = sizeof(DecodeSmem<D>);
    const size_t merge_bytes = (size_t)WARPS * 16 * (D + 2) * sizeof(float);
    const size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    static bool configured = false;  // per template instance; the attribute is per device function
    if (!configured) {
        cudaError_t err = cudaFuncSetAttribute(attention_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_decode: %s", cudaGetErrorString(err));
        configured = true;
    }
    const float sl2 = scale * 1.4426950408889634f;
    dim3 grid(n_splits, n_kv, n_seqs);
    // up to eight splits without scratch: they form a cluster and merge through distributed shared memory
    const int cluster_merge = n_splits > 1 && n_splits <= 8 && part_o == nullptr;
    gk_launch_cluster(attention_decode_kernel<D>, grid, dim3(WARPS * 32), smem, stream,
        dim3(cluster_merge ? n_splits : 1, 1, 1),
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, (__nv_bfloat16*)out,
        part_o, part_ml, kv_len, slots, block_table, n_q, n_kv, max_pages, sl2, window, n_splits, cluster_merge, n_q / n_kv, fused);
    GK_CHECK_LAUNCH("attention_decode");
    if (n_splits > 1 && !cluster_merge) {
        gk_launch(attention_decode_merge_kernel<D>, dim3(n_seqs * n_q), dim3(D <= 64 ? 64 : 128), 0, stream,
                  (const float*)part_o, (const float*)part_ml, (__nv_bfloat16*)out, n_splits);
        GK_CHECK_LAUNCH("attention_decode_merge");
    }
    return GK_OK;
}

}  // namespace

// With scratch (any number of splits; a second kernel merges them):
//   part_o  float [n_seqs * n_q * n_splits * head_dim],  part_ml  float [n_seqs * n_q * n_splits * 2].
// Without scratch (null pointers; up to 8 splits): the splits of a (sequence, kv head) run as one
// thread-block cluster and merge through distributed shared memory.
static int decode_entry(const void* q, const void* k_pages, const void* v_pages, void* out, float* part_o, float* part_ml,
                        const int* kv_len, const int* slots, const int* block_table, int n_seqs, int n_q, int n_kv,
                        int head_dim, int max_pages, int page_size, float scale, int window, int n_splits, void* stream,
                        const FusedQkv& fused) {
    GK_REQUIRE(n_seqs >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_decode: bad head counts %d/%d", n_q, n_kv);
    GK_REQUIRE(n_q / n_kv <= 16, "attention_decode: groups of more than 16 query heads per kv head are not supported");
    GK_REQUIRE(page_size == attn::PAGE, "attention_decode: page_size must be %d, got %d", attn::PAGE, page_size);
    GK_REQUIRE(head_dim == 64 || head_dim == 128, "attention_decode: head_dim %d is not 64 or 128 (use the exact kernel)", head_dim);
    GK_REQUIRE(n_splits >= 1 && n_splits <= 65535 && n_kv <= 65535 && n_seqs <= 65535, "attention_decode: grid too large");
    GK_REQUIRE(n_splits <= 8 || (part_o && part_ml), "attention_decode: scratch is needed for more than eight splits");
    GK_REQUIRE((part_o == nullptr) == (part_ml == nullptr), "attention_decode: both scratch arrays or neither");
    GK_REQUIRE(window >= 0, "attention_decode: window must be >= 0");
    if (n_seqs == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 64)
        return launch_decode<64>(q, k_pages, v_pages, out, part_o, part_ml, kv_len, slots, block_table, n_seqs, n_q, n_kv,
                                 max_pages, scale, window, n_splits, s, fused);
    return launch_decode<128>(q, k_pages, v_pages, out, part_o, part_ml, kv_len, slots, block_table, n_seqs, n_q, n_kv,
                              max_pages, scale, window, n_splits, s, fused);
}

GK_EXPORT int gk_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, void* out,
                                       float* part_o, float* part_ml, const int* kv_len, const int* slots,
                                       const int* block_table, int n_seqs, int n_q, int n_kv, int head_dim,
                                       int max_pages, int page_size, float scale, int window, int n_splits,
                                       void* stream) {
    FusedQkv none = {};
    return decode_entry(q, k_pages, v_pages, out, part_o, part_ml, kv_len, slots, block_table, n_seqs, n_q, n_kv, head_dim,
                        max_pages, page_size, scale, window, n_splits, stream, none);
}

// Decode attention that also does the step before it: `qkv` is the packed projection of each sequence's
// new token, [n_seqs, (n_q + 2 n_kv) * head_dim] bfloat16.  Per-head RMSNorm of q and k (`use_norm`,
// weights of `weight_dtype`), rotation at position kv_len - 1 (tables [positions][head_dim / 2], null =
// none) and the write of the new key and value into the pages (`write_kv`) happen inside the kernel.
GK_EXPORT int gk_attention_decode_fused_bf16(const void* qkv, const void* wq, const void* wk, int weight_dtype,
                                             int use_norm, float eps, const float* cos_table, const float* sin_table,
                                             int table_positions, int max_position, int write_kv, void* k_pages,
                                             void* v_pages, void* out, float* part_o, float* part_ml,
                                             const int* kv_len, const int* slots, const int* block_table, int n_seqs,
                                             int n_q, int n_kv, int head_dim, int max_pages, int page_size,
                                             float scale, int window, int n_splits, void* stream) {
    GK_REQUIRE(qkv != nullptr, "attention_decode_fused: qkv is required");
    GK_REQUIRE(GK_VALID_DTYPE(weight_dtype), "attention_decode_fused: bad weight dtype");
    GK_REQUIRE(!use_norm || (wq && wk), "attention_decode_fused: norm weights missing");
    GK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attention_decode_fused: cos and sin tables go together");
    GK_REQUIRE(cos_table == nullptr || max_position < table_positions,
               "attention_decode_fused: position %d is beyond the rotary table (%d positions)", max_position, table_positions);
    FusedQkv fused;
    fused.qkv = (const __nv_bfloat16*)qkv;
    fused.wq = wq;
    fused.wk = wk;
    fused.weights_bf16 = weight_dtype == GK_BF16;
    fused.use_norm = use_norm;
    fused.eps = eps;
    fused.cos_table = cos_table;
    fused.sin_table = sin_table;
    fused.write_kv = write_kv;
    return decode_entry(nullptr, k_pages, v_pages, out, part_o, part_ml, kv_len, slots, block_table, n_seqs, n_q, n_kv,
                        head_dim, max_pages, page_size, scale, window, n_splits, stream, fused);
}

// ---------------------------------------------------------------- the entry point that allocates nothing
// Scratch for the partial results of the splits, owned by the library.  In host code this name is
// only a handle for cudaGetSymbolAddress; the kernels get the device address looked up below.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[GK_NO_ALLOC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_no_alloc_ptr[MAX_DEVICES] = {};  // device address of the scratch, per device, once looked up
}  // namespace

GK_EXPORT int gk_attention_decode_bf16_no_alloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                                                const int* kv_len, const int* slots, const int* block_table,
                                                int n_seqs, int n_q, int n_kv, int head_dim, int max_pages,
                                                int page_size, float scale, int window, int n_splits, void* stream) {
    GK_REQUIRE(n_seqs >= 0 && n_q > 0 && n_splits >= 1 && (head_dim == 64 || head_dim == 128),
               "attention_decode_no_alloc: bad sizes n_seqs=%d n_q=%d n_splits=%d head_dim=%d", n_seqs, n_q, n_splits, head_dim);
    const unsigned long long need = (unsigned long long)n_seqs * n_q * n_splits * (head_dim + 2) * sizeof(float);
    GK_REQUIRE(need <= GK_NO_ALLOC_SCRATCH_BYTES,
               "attention_decode_no_alloc: %d sequences x %d heads x %d splits need %llu bytes of scratch; the "
               "built-in scratch holds %u (use fewer splits, or gk_attention_decode_bf16 with scratch of your own)",
               n_seqs, n_q, n_splits, need, (unsigned)GK_NO_ALLOC_SCRATCH_BYTES);
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_decode_no_alloc: cudaGetDevice: %s", cudaGetErrorString(err));
    GK_REQUIRE(device >= 0 && device < MAX_DEVICES, "attention_decode_no_alloc: device %d is out of range", device);
    if (g_no_alloc_ptr[device] == nullptr) {
        // once per device, with that device current: the array's address on THIS device
        void* ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);
        if (err != cudaSuccess || ptr == nullptr)
            return gk_fail(GK_CUDA_ERROR, "attention_decode_no_alloc: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
        g_no_alloc_ptr[device] = static_cast<float*>(ptr);
    }
    float* part_o = g_no_alloc_ptr[device];
    float* part_ml = part_o + (size_t)n_seqs * n_q * n_splits * head_dim;
    return gk_attention_decode_bf16(q, k_pages, v_pages, out, part_o, part_ml, kv_len, slots, block_table, n_seqs, n_q,
                                    n_kv, head_dim, max_pages, page_size, scale, window, n_splits, stream);
}

// How many clusters of `cluster` blocks of the decode attention kernel the device holds at once (blocks for a cluster
// of one), or a negative CUDA error.  Clusters are placed inside a GPC, so this is less than the SMs' places divided by
// the cluster size; the host's choice of the number of splits counts waves with it.
GK_EXPORT int gk_attention_decode_resident_clusters(int head_dim, int cluster) {
    if ((head_dim != 64 && head_dim != 128) || cluster < 1 || cluster > 8) return -1;
    const size_t smem = head_dim == 64 ? sizeof(DecodeSmem<64>) : sizeof(DecodeSmem<128>);
    const void* kernel = head_dim == 64 ? (const void*)attention_decode_kernel<64> : (const void*)attention_decode_kernel<128>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return -(int)err;
    gk_prepare_kernel(kernel);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster * 1024, 1, 1);
    cfg.blockDim = dim3(WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    err = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    if (err != cudaSuccess) return -(int)err;
    return clusters;
}
