// Decode attention in bfloat16 with the pages of all sequences dealt out evenly.
//
// The kernel of attention_decode.cu gives every (sequence, kv head) pair the same number of blocks, which is right
// where that fills the device once; where it does not (a hundred pairs and more: the last wave of blocks streams at
// what a few blocks can ask for, not at what the memory gives), and where the sequences of a step differ in
// length, this kernel is used instead.  The pages that the step has to read are put in one line, pair after pair
// (sequence-major, then kv head, then page), and the line is cut into as many equal pieces as the grid has blocks.
// A block walks its piece page by page through the same cp.async ring, its four warps taking 16 keys of a page
// each; wherever a pair ends inside the piece, or the piece ends, it leaves an unnormalised partial result (max,
// sum, output) for the pair.  A pair that lies inside one piece is written out directly.  The pieces of a pair
// that is spread over several blocks go to scratch memory, and the block that finishes last (a ticket counter
// per pair decides which) merges them in the order of the pieces, so the result does not depend on who merges.
// The ticket counters are zero between launches: the merging block sets its pair's counter back.
//
// Formulas as in attention_decode.cu (src/ops/flash_attention_2.py:33-34,55; src/layers/attention.py:116-119);
// the fused input stage (per-head RMSNorm of q and k, rotation, write of the new key and value) as there, by the
// block whose piece holds the pair's last page (src/layers/rmsnorm.py:11-16, src/layers/rope.py:17-33,
// src/layers/attention.py:82-89).  Lengths come from device memory: a captured launch stays valid as sequences grow.

#include "attention_decode_fused.cuh"

namespace {

using namespace attn;

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int NST = 3;

template <int D>
struct FlatSmem {
    __nv_bfloat16 k[NST][PAGE * D];
    __nv_bfloat16 v[NST][PAGE * D];
    float wq[D], wk[D];
    int ticket[4];  // two are used; the struct's size stays a multiple of 16 bytes
};

// Where a block stands in the line of pages.
struct Cursor {
    int seq, head, page;         // the unit: page `page` of kv head `head` of sequence `seq`
    int first_page, end_page;    // the sequence's visible pages
    int len;
    const int* pages;            // the sequence's row of the page table
};

struct FlatParams {
    const __nv_bfloat16* q;          // [n_seqs, n_q, D] (unused with fused.qkv)
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    __nv_bfloat16* out;              // [n_seqs, n_q, D]
    float* part_o;                   // [ids][group][D]
    float* part_ml;                  // [ids][group][2]
    int* tickets;                    // [n_seqs * n_kv], zero between launches
    const int* kv_len;
    const int* slots;
    const int* block_table;
    int n_seqs, n_q, n_kv, max_pages, window;
    int group;                       // n_q / n_kv, divided on the host
    float sl2;
};

__device__ __forceinline__ void load_sequence(Cursor& c, const FlatParams& p) {
    c.len = p.kv_len[c.seq];
    const int lo = (p.window > 0 && c.len - p.window > 0) ? c.len - p.window : 0;
    c.first_page = lo / PAGE;
    c.end_page = (c.len + PAGE - 1) / PAGE;
    c.pages = p.block_table + (size_t)p.slots[c.seq] * p.max_pages;
}

// to the next unit of the line (the caller knows that there is one)
__device__ __forceinline__ void advance(Cursor& c, const FlatParams& p) {
    if (++c.page < c.end_page) return;
    if (++c.head < p.n_kv) {
        c.page = c.first_page;
        return;
    }
    c.head = 0;
    do {  // sequences without pages hold no unit
        ++c.seq;
        load_sequence(c, p);
    } while (c.end_page <= c.first_page && c.seq + 1 < p.n_seqs);
    c.page = c.first_page;
}

// out[pair] from its `n_parts` parts in scratch (ids b_first + pair, ...), merged in their order.  Up to four parts
// are asked for at once, so that the merge costs one trip to the L2 cache and not one per part.
template <int D>
__device__ __forceinline__ void merge_parts(const FlatParams& p, int pair, int b_first, int n_parts, int group, int tid) {
    const size_t id0 = (size_t)b_first + pair;
    const int seq = pair / p.n_kv, hk = pair % p.n_kv;
    for (int idx = tid; idx < group * D; idx += THREADS) {
        const int r = idx / D, c = idx % D;
        float mm = -INFINITY, ll = 0.f, acc = 0.f;
        if (n_parts <= 4) {
            float ms[4], ls[4], os[4];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const bool have = s < n_parts;
                ms[s] = have ? __ldcg(p.part_ml + ((id0 + s) * group + r) * 2) : -INFINITY;
                ls[s] = have ? __ldcg(p.part_ml + ((id0 + s) * group + r) * 2 + 1) : 0.f;
                os[s] = have ? __ldcg(p.part_o + ((id0 + s) * group + r) * D + c) : 0.f;
            }
#pragma unroll
            for (int s = 0; s < 4; ++s) mm = fmaxf(mm, ms[s]);
#pragma unroll
            for (int s = 0; s < 4; ++s)
                if (ms[s] != -INFINITY) {
                    const float f = exp2_fast(ms[s] - mm);
                    ll += ls[s] * f;
                    acc += os[s] * f;
                }
        } else {
            for (int s = 0; s < n_parts; ++s) mm = fmaxf(mm, __ldcg(p.part_ml + ((id0 + s) * group + r) * 2));
            for (int s = 0; s < n_parts; ++s) {
                const float ms = __ldcg(p.part_ml + ((id0 + s) * group + r) * 2);
                if (ms != -INFINITY) {
                    const float f = exp2_fast(ms - mm);
                    ll += __ldcg(p.part_ml + ((id0 + s) * group + r) * 2 + 1) * f;
                    acc += __ldcg(p.part_o + ((id0 + s) * group + r) * D + c) * f;
                }
            }
        }
        p.out[((size_t)seq * p.n_q + hk * group + r) * D + c] = __float2bfloat16_rn(__fdividef(acc, ll));
    }
}

// 16-byte pieces of a pair's record: [q: group x D bf16] and, with the fused input stage,
// [cos: D/2 f32][sin: D/2 f32][k: D bf16][v: D bf16]
template <int D>
__host__ __device__ constexpr int record_pieces(int group, bool fused) {
    return (group * D * 2 + (fused ? 4 * D * 2 : 0)) / 16;
}

template <int D>
__global__ void __launch_bounds__(THREADS) attention_decode_flat_kernel(const FlatParams p, const FusedQkv fused) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    FlatSmem<D>& sm = *reinterpret_cast<FlatSmem<D>*>(smem_raw);
    const int group = p.group;
    const int record_slots = record_pieces<D>(group, fused.qkv != nullptr);
    // two records: what the pair in hand, and the next, need at their start (see below)
    uint4* records = reinterpret_cast<uint4*>(smem_raw + sizeof(FlatSmem<D>));
    float* red_o = reinterpret_cast<float*>(records + 2 * record_slots);     // [WARPS][group][D]
    float* red_ml = red_o + WARPS * group * D;                                // [WARPS][group][2]
    int* first_unit = reinterpret_cast<int*>(red_ml + WARPS * group * 2);     // [n_seqs + 1]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_launch_dependents();

    // ---- the line of pages: lengths, slots and the page table are step inputs, readable before the kernel in
    // front has finished
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < p.n_seqs; base += 32) {
            const int seq = base + lane;
            int units = 0;
            if (seq < p.n_seqs) {
                const int len = p.kv_len[seq];
                const int lo = (p.window > 0 && len - p.window > 0) ? len - p.window : 0;
                units = max((len + PAGE - 1) / PAGE - lo / PAGE, 0) * p.n_kv;
            }
            int incl = units;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            if (seq < p.n_seqs) first_unit[seq] = carry + incl - units;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) first_unit[p.n_seqs] = carry;
    }
    if (fused.qkv) {
        for (int c = tid; c < D; c += THREADS) {
            sm.wq[c] = fused.use_norm ? weight_at(fused.wq, fused.weights_bf16, c) : 1.f;
            sm.wk[c] = fused.use_norm ? weight_at(fused.wk, fused.weights_bf16, c) : 1.f;
        }
    }
    __syncthreads();
    const int n_units = first_unit[p.n_seqs];
    const int chunk = max((n_units + (int)gridDim.x - 1) / (int)gridDim.x, 1);
    const int lo_unit = blockIdx.x * chunk;
    const int count = min(chunk, n_units - lo_unit);
    if (count <= 0) return;

    // the sequence that holds the block's first unit
    Cursor cc;
    {
        int a = 0, b = p.n_seqs;  // first_unit[a] <= lo_unit < first_unit[b]
        while (b - a > 1) {
            const int mid = (a + b) >> 1;
            if (first_unit[mid] <= lo_unit) a = mid;
            else b = mid;
        }
        // of sequences that start at the same unit (those before hold nothing) the last one holds it
        cc.seq = a;
        load_sequence(cc, p);
        const int n_pages = cc.end_page - cc.first_page;
        const int r = lo_unit - first_unit[a];
        cc.head = r / n_pages;
        cc.page = cc.first_page + r % n_pages;
    }
    Cursor ic = cc;  // the unit asked for next

    int issued = 0, issue_stage = 0;  // issue_stage = issued % NST
    auto issue = [&]() {
        if (issued < count) {
            const int page = ic.pages[ic.page];
            const int valid = min(PAGE, ic.len - ic.page * PAGE);
            const size_t base = ((size_t)page * p.n_kv + ic.head) * PAGE * D;
            load_page_async<D, THREADS>(sm.k[issue_stage], p.k_pages + base, valid, tid);
            load_page_async<D, THREADS>(sm.v[issue_stage], p.v_pages + base, valid, tid);
            ++issued;
            issue_stage = issue_stage + 1 == NST ? 0 : issue_stage + 1;
            if (issued < count) advance(ic, p);
        }
        cp_async_commit();
    };
    // Every page but a sequence's last (which gets the new token from the kernel in front, or from this one)
    // was written by earlier steps and may be asked for at once.
    int early = 0;
#pragma unroll
    for (int s = 0; s < NST - 1; ++s)
        if (early == s && s < count && ic.page != ic.end_page - 1) {
            issue();
            early = s + 1;
        }
    pdl_wait();
#pragma unroll
    for (int s = 0; s < NST - 1; ++s)
        if (s >= early) issue();

    // ---- what a pair needs at its start (its queries; with the fused input stage also the rotation of the new
    // token's position and the new key and value rows) comes through shared memory: a thread fetches 16 bytes of
    // the NEXT pair's record when a pair begins and stores them when it ends, so that only the block's first pair
    // waits for memory.  Record: [q: group x D bf16][cos: D/2 f32][sin: D/2 f32][k: D bf16][v: D bf16].
    const int n_heads = p.n_q + 2 * p.n_kv;
    const int q_bytes = group * D * 2, record_bytes = q_bytes + (fused.qkv ? 4 * D * 2 : 0);
    const bool ahead = record_slots <= THREADS;  // else the record is fetched where it is needed
    auto fetch = [&](const Cursor& c, int piece) -> uint4 {
        // 16 bytes at offset piece * 16 of the record of the pair that `c` stands in
        const int at = piece * 16;
        const char* src;
        if (at < q_bytes) {
            src = reinterpret_cast<const char*>(fused.qkv ? fused.qkv + ((size_t)c.seq * n_heads + (size_t)c.head * group) * D
                                                          : p.q + ((size_t)c.seq * p.n_q + (size_t)c.head * group) * D) + at;
        } else {
            const int which = (at - q_bytes) / (D * 2), within = (at - q_bytes) % (D * 2);
            if (which < 2) {
                if (!fused.cos_table) return make_uint4(0, 0, 0, 0);
                src = reinterpret_cast<const char*>((which == 0 ? fused.cos_table : fused.sin_table) + (size_t)(c.len - 1) * (D / 2)) + within;
            } else {
                src = reinterpret_cast<const char*>(fused.qkv + ((size_t)c.seq * n_heads + p.n_q + (which == 3 ? p.n_kv : 0) + c.head) * D) + within;
            }
        }
        return *reinterpret_cast<const uint4*>(src);
    };
    // the pair after the one `c` stands in, if this block reaches it: `left` = units of the block from c on
    auto next_pair = [&](Cursor& c, int left) -> bool {
        const int rest = c.end_page - c.page;  // units of c's pair from c on
        if (left <= rest) return false;
        c.page = c.end_page - 1;
        advance(c, p);
        return true;
    };

    uint32_t qf[D / 16][4];
    __nv_bfloat162 k_new[D / 64], v_new[D / 64];  // lane l: elements 2l, 2l+1 of each 64-wide half (warp 0)
    bool owns_new = false;
    float m[2], l[2], o[D / 8][4];
    bool fresh = true;   // the unit in hand is the first of its pair in this block
    int turn = 0;        // which of the two records the pair in hand reads
    uint4 coming = make_uint4(0, 0, 0, 0);
    bool have_coming = false;

    if (ahead && tid * 16 < record_bytes) records[tid] = fetch(cc, tid);

    const int key0 = warp * 16;
    const uint32_t k_offset = k_lane_offset<D>(key0, lane), v_offset = v_lane_offset<D>(key0, lane);
    const uint32_t k_tiles = smem_u32(sm.k[0]), v_tiles = smem_u32(sm.v[0]);
    constexpr uint32_t TILE_BYTES = PAGE * D * 2;
    for (int it = 0, stage = 0; it < count; ++it, stage = stage + 1 == NST ? 0 : stage + 1) {
        cp_async_wait<NST - 2>();
        __syncthreads();  // unit `it` has landed for everyone; the stage asked for next was used an iteration ago
        issue();
        if (fresh) {
            // ---- a pair begins: its queries, and its new key and value if its last page is in this piece
            fresh = false;
            m[0] = m[1] = -INFINITY;
            l[0] = l[1] = 0.f;
#pragma unroll
            for (int j = 0; j < D / 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
            if (!ahead) {
                for (int piece = tid; piece * 16 < record_bytes; piece += THREADS) records[turn * record_slots + piece] = fetch(cc, piece);
                __syncthreads();
            } else {
                Cursor nc = cc;
                have_coming = next_pair(nc, count - it) && tid * 16 < record_bytes;
                if (have_coming) coming = fetch(nc, tid);
            }
            const char* rec = reinterpret_cast<const char*>(records + turn * record_slots);
            const int pos_new = cc.len - 1;
            owns_new = fused.qkv != nullptr && fused.write_kv && (cc.end_page - cc.page) <= count - it;
            const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int r = r0 + (i & 1) * 8, c = ks * 16 + c0 + (i >> 1) * 8;
                    qf[ks][i] = r < group ? *reinterpret_cast<const uint32_t*>(rec + (r * D + c) * 2) : 0u;
                }
            if (fused.qkv) {
                const float* cos_row = reinterpret_cast<const float*>(rec + q_bytes);
                const float* sin_row = cos_row + D / 2;
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
                                const float cs = cos_row[c], sn = sin_row[c];
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
                if (owns_new && warp == 0) {
                    const __nv_bfloat16* krow = reinterpret_cast<const __nv_bfloat16*>(rec + q_bytes + 2 * D * 2);
                    const __nv_bfloat16* vrow = krow + D;
                    float kx[D / 64][2];
                    float ss = 0.f;
#pragma unroll
                    for (int hf = 0; hf < D / 64; ++hf) {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(krow + hf * 64 + 2 * lane));
                        v_new[hf] = *reinterpret_cast<const __nv_bfloat162*>(vrow + hf * 64 + 2 * lane);
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
                            for (int e = 0; e < 2; ++e) kx[hf][e] = (kx[hf][e] * inv) * sm.wk[hf * 64 + 2 * lane + e];
                    }
                    if (fused.cos_table) {
                        // partner of column c is c + D/2: for D = 128 the other half held by this lane, for D = 64
                        // the lane 16 further on
                        if (D == 128) {
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int c = 2 * lane + e;
                                const float cs = cos_row[c], sn = sin_row[c];
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
                                const float cs = cos_row[c], sn = sin_row[c];
                                kx[0][e] = lane < 16 ? mine * cs - other * sn : mine * cs + other * sn;
                            }
                        }
                    }
                    const size_t at = (((size_t)cc.pages[cc.end_page - 1] * p.n_kv + cc.head) * PAGE + (pos_new % PAGE)) * D;
#pragma unroll
                    for (int hf = 0; hf < D / 64; ++hf) {
                        k_new[hf] = __floats2bfloat162_rn(kx[hf][0], kx[hf][1]);
                        *reinterpret_cast<__nv_bfloat162*>(const_cast<__nv_bfloat16*>(p.k_pages) + at + hf * 64 + 2 * lane) = k_new[hf];
                        *reinterpret_cast<__nv_bfloat162*>(const_cast<__nv_bfloat16*>(p.v_pages) + at + hf * 64 + 2 * lane) = v_new[hf];
                    }
                }
            }
        }

        const bool last_page = cc.page == cc.end_page - 1;
        if (owns_new && last_page) {  // block-uniform
            if (warp == 0) {
                const int row = (cc.len - 1) % PAGE;
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
        const int lo = (p.window > 0 && cc.len - p.window > 0) ? cc.len - p.window : 0;
        const int abs0 = cc.page * PAGE + key0;
        if (abs0 < cc.len && abs0 + 16 > lo) {  // warp-uniform: skip sixteen keys that are all hidden
            float sc[2][4];
            qk_16keys_at<D>(sc, qf, k_tiles + stage * TILE_BYTES, k_offset);
            if (abs0 + 16 > cc.len || abs0 < lo) {  // warp-uniform: only the sixteen keys at an edge have hidden ones
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int key = abs0 + n * 8 + (lane & 3) * 2 + c;
                        if (key >= cc.len || key < lo) sc[n][c] = sc[n][2 + c] = -INFINITY;
                    }
            }
            uint32_t pr[4];
            softmax_update<D>(sc, m, l, o, pr, p.sl2);
            pv_16keys_at<D>(o, pr, v_tiles + stage * TILE_BYTES, v_offset);
        }

        if (last_page || it == count - 1) {
            // ---- the block's part of this pair is complete: merge the four warps, then either write the pair's
            // result (all its pages were here) or leave the part in scratch; the tickets are taken at the end
            const int pair = cc.seq * p.n_kv + cc.head;
            const int n_pages = cc.end_page - cc.first_page;
            const int pair_begin = first_unit[cc.seq] + cc.head * n_pages;
            const int b_first = pair_begin / chunk, b_last = (pair_begin + n_pages - 1) / chunk;
            const int n_parts = b_last - b_first + 1;
            {
                const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = r0 + 8 * h;
                    if (r >= group) continue;  // rows of the tile beyond the heads of this group hold nothing
                    if ((lane & 3) == 0) {
                        red_ml[(warp * group + r) * 2] = m[h];
                        red_ml[(warp * group + r) * 2 + 1] = l[h];
                    }
#pragma unroll
                    for (int j = 0; j < D / 8; ++j) {
                        red_o[(warp * group + r) * D + j * 8 + c0] = o[j][2 * h];
                        red_o[(warp * group + r) * D + j * 8 + c0 + 1] = o[j][2 * h + 1];
                    }
                }
            }
            if (have_coming) records[(turn ^ 1) * record_slots + tid] = coming;  // the next pair's record, fetched when this one began
            have_coming = false;
            turn ^= 1;
            __syncthreads();
            const size_t id = (size_t)blockIdx.x + pair;  // grows by one from part to part along the line
            for (int idx = tid; idx < group * D; idx += THREADS) {
                const int r = idx / D, c = idx % D;
                float mm = -INFINITY;
#pragma unroll
                for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, red_ml[(w * group + r) * 2]);
                float ll = 0.f, acc = 0.f;
                if (mm != -INFINITY) {
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) {
                        const float f = exp2_fast(red_ml[(w * group + r) * 2] - mm);
                        ll += red_ml[(w * group + r) * 2 + 1] * f;
                        acc += red_o[(w * group + r) * D + c] * f;
                    }
                }
                if (n_parts == 1) {
                    p.out[((size_t)cc.seq * p.n_q + cc.head * group + r) * D + c] = __float2bfloat16_rn(__fdividef(acc, ll));
                } else {
                    p.part_o[(id * group + r) * D + c] = acc;
                    if (c == 0) {
                        p.part_ml[(id * group + r) * 2] = mm;
                        p.part_ml[(id * group + r) * 2 + 1] = ll;
                    }
                }
            }
            if (n_parts > 1) {
                // a ticket for the part; who draws the pair's last ticket merges its parts, in their order
                __threadfence();  // this thread's share of the part is visible to the device before the ticket is taken
                __syncthreads();
                if (tid == 0) sm.ticket[0] = atomicAdd(p.tickets + pair, 1);
                __syncthreads();
                if (sm.ticket[0] == n_parts - 1) {
                    __threadfence();
                    merge_parts<D>(p, pair, b_first, n_parts, group, tid);
                    if (tid == 0) p.tickets[pair] = 0;
                }
            }
            fresh = true;
        }
        if (it + 1 < count) advance(cc, p);
    }
    cp_async_wait<0>();
}

// The kernel may use `smem` bytes of dynamic shared memory (the attribute only ever grows).
template <int D>
int allow_smem(size_t smem) {
    static size_t allowed = 0;  // per template instance; the attribute is per device function
    if (smem > allowed) {
        cudaError_t err = cudaFuncSetAttribute(attention_decode_flat_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "attention_decode_flat: %s", cudaGetErrorString(err));
        allowed = smem;
    }
    return GK_OK;
}

template <int D>
int launch_flat(const FlatParams& p, const FusedQkv& fused, int n_blocks, cudaStream_t stream) {
    const int group = p.group;
    const size_t smem = sizeof(FlatSmem<D>) + 2 * (size_t)record_pieces<D>(group, fused.qkv != nullptr) * 16 +
                        (size_t)WARPS * group * (D + 2) * sizeof(float) + ((size_t)p.n_seqs + 1) * sizeof(int);
    GK_REQUIRE(smem <= 227 * 1024, "attention_decode_flat: %d sequences with groups of %d heads need %zu bytes of shared memory",
               p.n_seqs, group, smem);
    int status = allow_smem<D>(smem);
    if (status != GK_OK) return status;
    gk_launch(attention_decode_flat_kernel<D>, dim3(n_blocks), dim3(THREADS), smem, stream, p, fused);
    GK_CHECK_LAUNCH("attention_decode_flat");
    return GK_OK;
}

}  // namespace

// Decode attention over `n_blocks` equal pieces of the step's pages.  `qkv` null: queries from `q`
// [n_seqs, n_q, head_dim], keys and values in the pages already; else the packed projection of each sequence's new
// token, and the kernel norms (`use_norm`, weights of `weight_dtype`), rotates (tables [positions][head_dim / 2],
// null = none) and writes the new key and value (`write_kv`) itself.  `part` holds
// (n_blocks + n_seqs * n_kv) * (n_q / n_kv) * (head_dim + 2) floats; `tickets` n_seqs * n_kv ints that are zero
// before the first launch (the kernel leaves them zero).
GK_EXPORT int gk_attention_decode_flat_bf16(const void* q, const void* qkv, const void* wq, const void* wk, int weight_dtype,
                                            int use_norm, float eps, const float* cos_table, const float* sin_table,
                                            int table_positions, int max_position, int write_kv, void* k_pages,
                                            void* v_pages, void* out, float* part, int* tickets, const int* kv_len,
                                            const int* slots, const int* block_table, int n_seqs, int n_q, int n_kv,
                                            int head_dim, int max_pages, int page_size, float scale, int window,
                                            int n_blocks, void* stream) {
    GK_REQUIRE((q != nullptr) != (qkv != nullptr), "attention_decode_flat: either q or qkv");
    GK_REQUIRE(n_seqs >= 0 && n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "attention_decode_flat: bad head counts %d/%d", n_q, n_kv);
    GK_REQUIRE(n_q / n_kv <= 16, "attention_decode_flat: groups of more than 16 query heads per kv head are not supported");
    GK_REQUIRE(page_size == attn::PAGE, "attention_decode_flat: page_size must be %d, got %d", attn::PAGE, page_size);
    GK_REQUIRE(head_dim == 64 || head_dim == 128, "attention_decode_flat: head_dim %d is not 64 or 128", head_dim);
    GK_REQUIRE(n_blocks >= 1 && part != nullptr && tickets != nullptr, "attention_decode_flat: blocks, scratch and tickets are required");
    GK_REQUIRE(window >= 0, "attention_decode_flat: window must be >= 0");
    GK_REQUIRE((long long)n_seqs * n_kv + n_blocks < (1LL << 31), "attention_decode_flat: too many parts");
    FusedQkv fused = {};
    if (qkv) {
        GK_REQUIRE(GK_VALID_DTYPE(weight_dtype), "attention_decode_flat: bad weight dtype");
        GK_REQUIRE(!use_norm || (wq && wk), "attention_decode_flat: norm weights missing");
        GK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attention_decode_flat: cos and sin tables go together");
        GK_REQUIRE(cos_table == nullptr || max_position < table_positions,
                   "attention_decode_flat: position %d is beyond the rotary table (%d positions)", max_position, table_positions);
        fused.qkv = (const __nv_bfloat16*)qkv;
        fused.wq = wq;
        fused.wk = wk;
        fused.weights_bf16 = weight_dtype == GK_BF16;
        fused.use_norm = use_norm;
        fused.eps = eps;
        fused.cos_table = cos_table;
        fused.sin_table = sin_table;
        fused.write_kv = write_kv;
    }
    if (n_seqs == 0) return GK_OK;
    const int group = n_q / n_kv;
    FlatParams p;
    p.q = (const __nv_bfloat16*)q;
    p.k_pages = (const __nv_bfloat16*)k_pages;
    p.v_pages = (const __nv_bfloat16*)v_pages;
    p.out = (__nv_bfloat16*)out;
    p.part_o = part;
    p.part_ml = part + ((size_t)n_blocks + (size_t)n_seqs * n_kv) * group * head_dim;
    p.tickets = tickets;
    p.kv_len = kv_len;
    p.slots = slots;
    p.block_table = block_table;
    p.n_seqs = n_seqs;
    p.group = group;
    p.n_q = n_q;
    p.n_kv = n_kv;
    p.max_pages = max_pages;
    p.window = window;
    p.sl2 = scale * 1.4426950408889634f;
    cudaStream_t s = (cudaStream_t)stream;
    return head_dim == 64 ? launch_flat<64>(p, fused, n_blocks, s) : launch_flat<128>(p, fused, n_blocks, s);
}

// How many blocks of the kernel above the device holds at once (for groups of up to four query heads a kv head),
// or a negative CUDA error: the host cuts the line of pages into that many pieces at most.
GK_EXPORT int gk_attention_decode_flat_resident_blocks(int head_dim) {
    if (head_dim != 64 && head_dim != 128) return -1;
    const size_t smem = (head_dim == 64 ? sizeof(FlatSmem<64>) : sizeof(FlatSmem<128>)) + 2 * (size_t)(4 + 4) * head_dim * 2 +
                        (size_t)WARPS * 4 * (head_dim + 2) * sizeof(float) + 1024;
    const void* kernel = head_dim == 64 ? (const void*)attention_decode_flat_kernel<64> : (const void*)attention_decode_flat_kernel<128>;
    if ((head_dim == 64 ? allow_smem<64>(smem) : allow_smem<128>(smem)) != GK_OK) return -1;
    gk_prepare_kernel(kernel);
    int per_sm = 0, device = 0, n_sms = 0;
    cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem);
    if (err == cudaSuccess) err = cudaGetDevice(&device);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) return -(int)err;
    return per_sm * n_sms;
}
