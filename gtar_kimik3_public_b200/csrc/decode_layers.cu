// A run of decoder layers of a decode step (one new token per sequence, up to eight sequences) as ONE persistent
// kernel: per layer  x = RMSNorm(h); q|k|v = x Wqkv^T; per-head q/k RMSNorm, rotation, cache write, attention over
// the paged cache; h += o Wo^T; y = RMSNorm(h); h += (silu(y Wg^T) * (y Wu^T)) Wd^T
// (src/models/transformer.py:47-48, src/layers/attention.py:79-121, src/layers/swiglu.py:14, src/layers/rmsnorm.py:11-16,
// src/layers/rope.py:17-33).
//
// Why one kernel.  Launched one by one, the seven kernels of a layer each move a few megabytes and last three
// microseconds, most of it the hand-over from the kernel in front and their own serial stages; the memory idles
// meanwhile.  Here one block per SM stays resident for all layers.  A layer is five stages (q|k|v product, attention,
// output product, gate|up product with SwiGLU, down product) separated by barriers over the whole grid, and what
// a warp will need in LATER stages, weights and cached keys and values, does not depend on those barriers: every
// warp owns a ring of 4 KB slots in shared memory and a fixed list of tiles to stream through it (its share of each
// product's weight rows, its share of the cached keys and values), and keeps the ring full with cp.async across
// stage and layer boundaries.  When a barrier opens, the data of the next stage is in shared memory already and
// the stage costs its arithmetic and one trip to L2 for the activations.
//
// Work split.  Products: weight rows in groups of eight (the N of mma.sync.m16n8k16; the tokens are its rows),
// group g to block (g + rotation) % grid; a group's K range is cut in `ksplit` parts that go to different warps of
// the block, whose partial sums meet in shared memory in a fixed order.  Attention: the tiles of 4 KB of keys (16
// keys of head size 128) of all (sequence, kv head) pairs form one line that is cut into equal runs, one per warp of
// the grid; a warp leaves an unnormalised partial result per pair it touches, and the warp that arrives last at a
// pair (a ticket counter) merges the pair's partial results in their order.  The new token's key and value never
// come from memory: the warp that holds a pair's last tile makes them from the q|k|v row, writes them to the cache
// and puts them into its copy of the tile.
//
// Every wait (the grid barrier) is bounded: a block that waits too long raises an abort word that ends every other
// wait at once, sets the error flag and lets the kernel run out; nothing is indexed by data that another block writes.

#include "attention_mma.cuh"

namespace {

using namespace attn;

constexpr int MK_WARPS = 8;
constexpr int MK_THREADS = MK_WARPS * 32;
constexpr int MK_SLOT = 4096;        // bytes of a ring slot: 8 weight rows x 256 k, or 16 keys x 128 (32 x 64)
constexpr int MK_TOKENS = 8;         // token rows kept in shared memory: the kernel takes up to eight sequences
constexpr int MK_TILE_K = 256;       // k of a weight tile
constexpr int MK_ATT_MIN_RUN = 4;    // fewest key tiles a warp takes in the attention stage
constexpr long long MK_WAIT_LIMIT = 1LL << 30;  // clock cycles a block waits at a barrier before it gives up

enum MkStage : int { ST_QKV = 0, ST_ATT = 1, ST_OPROJ = 2, ST_GATEUP = 3, ST_DOWN = 4, ST_COUNT = 5 };

struct MkLayer {  // one entry of the run list; mirrored by the host (96 bytes)
    const __nv_bfloat16* w_qkv;   // [(n_q + 2 n_kv) D, hidden]
    const __nv_bfloat16* w_o;     // [hidden, n_q D]
    const __nv_bfloat16* w_gu;    // [2 inter, hidden], gate and up rows interleaved
    const __nv_bfloat16* w_down;  // [hidden, inter]
    const void* norm_in;          // [hidden]
    const void* norm_post;        // [hidden]
    const void* q_norm;           // [D] or null: no per-head norm
    const void* k_norm;
    __nv_bfloat16* k_pages;       // [pages, n_kv, 64, D]
    __nv_bfloat16* v_pages;
    float eps_in, eps_post, eps_qk;
    int pad;
};

struct MkProduct {
    int n, k;            // weight rows, row length
    int ksplit;          // parts of a group's K range (warps that share a group): a power of two
    int ksplit_shift;    // its logarithm
    int part_k;          // k / ksplit
    int part_tiles;      // tiles of a part
    int rotation;        // group g goes to block (g + rotation) % grid
};

struct MkParams {
    const MkLayer* layers;
    int n_layers;
    int n_seqs, hidden, n_q, n_kv, inter;
    MkProduct prod[4];   // q|k|v, output, gate|up, down
    float* h;            // [n_seqs, hidden] the residual stream, updated in place
    __nv_bfloat16* qkv;  // [n_seqs, (n_q + 2 n_kv) D]
    __nv_bfloat16* att;  // [n_seqs, n_q D]
    __nv_bfloat16* act;  // [n_seqs, inter]
    float* part;         // attention partial results
    int part_splits;     // partial results a pair can have
    unsigned* words;     // [0] barrier count, [1] blocks that have left, [2] abort, [8 ...] a ticket per pair
    const int* kv_len;
    const int* slots;
    const int* block_table;
    int max_pages;
    const float* cos_table;   // [positions, D / 2] or null
    const float* sin_table;
    int norm_bf16, qk_bf16;   // types of the norm weights
    float sl2;                // softmax scale * log2(e)
    int x_stride;             // elements between token rows of the activations in shared memory
    int red_floats;           // floats of the partial-sum area
    int* error_flag;
    long long* stamps;        // null, or [blocks][barriers][2] nanosecond clock readings: arrival at, release from each barrier
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float weight_of(const void* w, int bf16, int i) {
    return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]) : reinterpret_cast<const float*>(w)[i];
}
__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + __expf(-g)); }

// All blocks wait here for one another.  `target` counts the arrivals that must have been seen.
__device__ __forceinline__ long long clock_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void grid_barrier(const MkParams& p, unsigned& target) {
    __syncthreads();
    const unsigned ordinal = target / gridDim.x;  // barriers passed so far
    target += gridDim.x;
    if (threadIdx.x == 0) {
        if (p.stamps) p.stamps[((size_t)blockIdx.x * (p.n_layers * ST_COUNT) + ordinal) * 2] = clock_ns();
        __threadfence();
        red_release_add(p.words, 1u);
        const long long begin = clock64();
        int spins = 0;
        while (ld_acquire(p.words) < target) {
            if ((++spins & 31) == 0) {
                if (ld_relaxed(p.words + 2) != 0u) break;
                if (clock64() - begin > MK_WAIT_LIMIT) {
                    atomicExch(p.words + 2, 1u);
                    atomicExch(p.error_flag, 7);
                    break;
                }
            }
        }
        __threadfence();
        if (p.stamps) p.stamps[((size_t)blockIdx.x * (p.n_layers * ST_COUNT) + ordinal) * 2 + 1] = clock_ns();
    }
    __syncthreads();
}

// measurements only: thread 0 of block 0 notes the time at place `k` (0..7) of stage `ordinal`, behind the barriers' stamps
__device__ __forceinline__ void note(const MkParams& p, int ordinal, int k) {
    if (p.stamps && blockIdx.x == 0 && threadIdx.x == 0)
        p.stamps[(size_t)gridDim.x * (p.n_layers * ST_COUNT) * 2 + (size_t)ordinal * 8 + k] = clock_ns();
}

// ------------------------------------------------------------------ what a warp streams through its ring
struct BlockTables {   // in shared memory: the step's sequences as every warp of the block needs them
    int tiles_of[MK_TOKENS + 1];   // tiles_of[b] = key tiles of all pairs of the sequences before b
    int pair_tiles[MK_TOKENS];     // key tiles of one (sequence, kv head) pair
    int len[MK_TOKENS];            // cached tokens including the new one
    long long table_row[MK_TOKENS];  // where the sequence's row of the page table begins
};

struct WarpPlan {
    int items[4];        // (group, part) items of this block in each product; the warp takes warp, warp + 8, ...
    int effective[4];    // (block + rotation) % grid: the block's first group in each product
    int att_begin, att_end;   // the warp's run of key tiles in the line of all pairs' tiles
    int att_seq, att_hk, att_j;  // where that run begins
};

struct Cursor {   // a position in the warp's list of tiles
    int layer, stage, item, tile;   // products: item id and tile of its part; attention: item = key tile, tile = 0 keys / 1 values
    int seq, hk, j;                 // attention: the key tile is tile j of the pair (seq, hk)
};

template <int D>
struct Geometry {
    static constexpr int KEYS = MK_SLOT / (D * 2);  // keys of a tile
};

__device__ __forceinline__ int product_of(int stage) { return stage == ST_QKV ? 0 : stage - 1; }

// Moves `c` to the first tile at or after it that exists; false when the list has ended.
__device__ __forceinline__ bool settle(const MkParams& p, const WarpPlan& plan, Cursor& c, int warp) {
    while (c.layer < p.n_layers) {
        if (c.stage == ST_ATT) {
            if (c.item < plan.att_end) return true;
        } else if (c.item < plan.items[product_of(c.stage)]) {
            return true;
        }
        ++c.stage;
        if (c.stage == ST_COUNT) {
            c.stage = 0;
            ++c.layer;
        }
        c.tile = 0;
        if (c.stage == ST_ATT) {
            c.item = plan.att_begin;
            c.seq = plan.att_seq;
            c.hk = plan.att_hk;
            c.j = plan.att_j;
        } else {
            c.item = warp;
        }
    }
    return false;
}

__device__ __forceinline__ void advance(const MkParams& p, const BlockTables& bt, Cursor& c) {
    if (c.stage == ST_ATT) {
        if (++c.tile == 2) {
            c.tile = 0;
            ++c.item;
            if (++c.j == bt.pair_tiles[c.seq]) {
                c.j = 0;
                if (++c.hk == p.n_kv) {
                    c.hk = 0;
                    ++c.seq;  // beyond the last sequence only when the run has ended
                }
            }
        }
    } else if (++c.tile == p.prod[product_of(c.stage)].part_tiles) {
        c.tile = 0;
        c.item += MK_WARPS;
    }
}

// (sequence, kv head, tile of the pair) of key tile `a` in the line of all pairs' tiles
__device__ __forceinline__ void pair_of(const MkParams& p, const BlockTables& bt, int a, int& seq, int& hk, int& j) {
    seq = 0;
    while (seq + 1 < p.n_seqs && a >= bt.tiles_of[seq + 1]) ++seq;
    const int within = a - bt.tiles_of[seq];
    hk = within / bt.pair_tiles[seq];
    j = within - hk * bt.pair_tiles[seq];
}

// Asks for the tile at `c` into `slot` (one cp.async group of the warp).
template <int D>
__device__ __forceinline__ void request_tile(const MkParams& p, const WarpPlan& plan, const BlockTables& bt, const Cursor& c,
                                             unsigned char* slot, int lane) {
    const MkLayer& layer = p.layers[c.layer];
    if (c.stage == ST_ATT) {
        constexpr int KEYS = Geometry<D>::KEYS;
        const int key0 = c.j * KEYS;
        const int page = p.block_table[bt.table_row[c.seq] + key0 / PAGE];
        const __nv_bfloat16* src = (c.tile ? layer.v_pages : layer.k_pages) + (((size_t)page * p.n_kv + c.hk) * PAGE + key0 % PAGE) * D;
        load_tile_async<D>(reinterpret_cast<__nv_bfloat16*>(slot), src, D, KEYS, min(KEYS, bt.len[c.seq] - key0), lane, 32);
    } else {
        const int which = product_of(c.stage);
        const MkProduct& pr = p.prod[which];
        const __nv_bfloat16* w = c.stage == ST_QKV ? layer.w_qkv : c.stage == ST_OPROJ ? layer.w_o : c.stage == ST_GATEUP ? layer.w_gu : layer.w_down;
        const int local_group = c.item >> pr.ksplit_shift, part = c.item & (pr.ksplit - 1);
        const int k0 = part * pr.part_k + c.tile * MK_TILE_K;
        const int chunks = min(MK_TILE_K, pr.part_k - c.tile * MK_TILE_K) / 8;  // 16-byte pieces of a row
        // lane -> weight row lane / 4 of the group, pieces lane % 4, + 4, + 8, ...
        const int row = lane >> 2;
        const __nv_bfloat16* src = w + (size_t)((plan.effective[which] + local_group * (int)gridDim.x) * 8 + row) * pr.k + k0;
        unsigned char* dst = slot + row * 512;
#pragma unroll
        for (int i = 0; i < MK_TILE_K / 32; ++i) {
            const int chunk = (lane & 3) + 4 * i;
            if (chunk < chunks) cp_async_16(dst + ((chunk ^ row) & 7 | (chunk & ~7)) * 16, src + chunk * 8, true);
        }
    }
}

template <int D, int NSLOT>
struct Ring {
    unsigned char* base;   // this warp's NSLOT slots
    Cursor ahead;          // next tile to ask for
    bool more;             // `ahead` names a tile
    int taken;             // tiles consumed so far (slot of the next one: taken % NSLOT)

    __device__ __forceinline__ void request_next(const MkParams& p, const WarpPlan& plan, const BlockTables& bt, int slot_index, int warp, int lane) {
        if (more) {
            request_tile<D>(p, plan, bt, ahead, base + slot_index * MK_SLOT, lane);
            advance(p, bt, ahead);
            more = settle(p, plan, ahead, warp);
        }
        cp_async_commit();  // an empty group keeps the count of groups in flight fixed
    }
    // The next tile of the warp's list has landed: returns its slot.
    __device__ __forceinline__ unsigned char* acquire() {
        cp_async_wait<NSLOT - 1>();
        __syncwarp();
        return base + (taken % NSLOT) * MK_SLOT;
    }
    // The slot returned by the last acquire() is free again: ask for the tile NSLOT further on into it.
    __device__ __forceinline__ void release(const MkParams& p, const WarpPlan& plan, const BlockTables& bt, int warp, int lane) {
        __syncwarp();
        request_next(p, plan, bt, taken % NSLOT, warp, lane);
        ++taken;
    }
};

// ------------------------------------------------------------------ activations into shared memory
// Warp w brings token w: RMSNorm of the stream's row (32-bit, rounded to bfloat16 as the product's operand).  The
// norm's weights do not depend on the barrier in front of the stage, so a lane fetches its share of them before it
// waits there (fetch_norm_weights) and they arrive meanwhile; layers have weights of their own, so these come from
// memory every time.
constexpr int NORM_KEEP = 8;  // float4 a lane keeps: rows of up to 1,024 elements; longer rows fetch the rest late

struct NormWeights {
    float4 w[NORM_KEEP];
};

__device__ __forceinline__ float4 norm_weight4(const void* weight, int bf16, int i) {
    if (bf16) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(weight) + i));
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(weight) + i));
}

__device__ __forceinline__ void fetch_norm_weights(const MkParams& p, NormWeights& nw, const void* weight, int warp, int lane) {
    if (warp >= p.n_seqs) return;
#pragma unroll
    for (int it = 0; it < NORM_KEEP; ++it) {
        const int i = lane * 4 + it * 128;
        if (i < p.hidden) nw.w[it] = norm_weight4(weight, p.norm_bf16, i);
    }
}

__device__ __forceinline__ void load_normed(const MkParams& p, __nv_bfloat16* x, const NormWeights& nw, const void* weight, float eps,
                                            int warp, int lane) {
    if (warp >= p.n_seqs) return;
    const float* row = p.h + (size_t)warp * p.hidden;
    __nv_bfloat16* dst = x + (size_t)warp * p.x_stride;
    float4 kept[NORM_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NORM_KEEP; ++it) {
        const int i = lane * 4 + it * 128;
        kept[it] = i < p.hidden ? __ldcg(reinterpret_cast<const float4*>(row + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int it = 0; it < NORM_KEEP; ++it) ss += kept[it].x * kept[it].x + kept[it].y * kept[it].y + kept[it].z * kept[it].z + kept[it].w * kept[it].w;
    for (int i = lane * 4 + NORM_KEEP * 128; i < p.hidden; i += 128) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(row + i));
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)p.hidden + eps);
    auto put = [&](int i, const float4& v, const float4& w) {
        uint2 packed;
        packed.x = pack_bf16((v.x * inv) * w.x, (v.y * inv) * w.y);
        packed.y = pack_bf16((v.z * inv) * w.z, (v.w * inv) * w.w);
        *reinterpret_cast<uint2*>(dst + i) = packed;
    };
#pragma unroll
    for (int it = 0; it < NORM_KEEP; ++it) {
        const int i = lane * 4 + it * 128;
        if (i < p.hidden) put(i, kept[it], nw.w[it]);
    }
    for (int i = lane * 4 + NORM_KEEP * 128; i < p.hidden; i += 128)
        put(i, __ldcg(reinterpret_cast<const float4*>(row + i)), norm_weight4(weight, p.norm_bf16, i));
}

// ... or copies its row of a bfloat16 buffer [n_seqs, k].
__device__ __forceinline__ void load_plain(const MkParams& p, __nv_bfloat16* x, const __nv_bfloat16* src, int k, int warp, int lane) {
    if (warp >= p.n_seqs) return;
    const uint4* row = reinterpret_cast<const uint4*>(src + (size_t)warp * k);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)warp * p.x_stride);
    for (int i = lane; i < k / 8; i += 32) dst[i] = __ldcg(row + i);
}

// ------------------------------------------------------------------ a product stage
// OUT[token, n] = sum_k X[token, k] W[n, k] for this block's groups of eight weight rows; X is in shared memory.
template <int D, int NSLOT>
__device__ __forceinline__ void product_stage(const MkParams& p, const WarpPlan& plan, const BlockTables& bt, Ring<D, NSLOT>& ring, int stage,
                                              const MkLayer& layer, const __nv_bfloat16* x, float* red, int warp, int lane, int ordinal) {
    const MkProduct& pr = p.prod[product_of(stage)];
    const int my_items = plan.items[product_of(stage)];
    note(p, ordinal, 2);
    for (int item = warp; item < my_items; item += MK_WARPS) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of MMAs, added at the end
        const int part = item & (pr.ksplit - 1);
        const int b_row = lane & 7, piece = lane >> 3;
        for (int tile = 0; tile < pr.part_tiles; ++tile) {
            const unsigned char* slot = ring.acquire();
            const int k0 = part * pr.part_k + tile * MK_TILE_K;
            const int steps32 = min(MK_TILE_K, pr.part_k - tile * MK_TILE_K) / 32;
            // A: tokens 0..7 on rows 0..7 of the MMA (rows 8..15 are zero); lane -> row lane & 7, 16-byte piece lane >> 3
            const __nv_bfloat16* a_row = x + (size_t)b_row * p.x_stride + k0 + piece * 8;
            const unsigned char* b_base = slot + b_row * 512;
            if (steps32 == MK_TILE_K / 32) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {  // four steps' operands asked for together, then their MMAs
                    uint32_t a[4][4], b[4][4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int st = half * 4 + i;
                        ldmatrix_x4(a[i], a_row + st * 32);
                        const int chunk = st * 4 + piece;
                        ldmatrix_x4(b[i], b_base + ((chunk ^ b_row) & 7 | (chunk & ~7)) * 16);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t a_lo[4] = {a[i][0], 0u, a[i][1], 0u}, a_hi[4] = {a[i][2], 0u, a[i][3], 0u};
                        mma_16816(acc, a_lo, b[i][0], b[i][1]);
                        mma_16816(acc2, a_hi, b[i][2], b[i][3]);
                    }
                }
            } else {
                for (int st = 0; st < steps32; ++st) {
                    uint32_t a[4], b[4];
                    ldmatrix_x4(a, a_row + st * 32);
                    const int chunk = st * 4 + piece;
                    ldmatrix_x4(b, b_base + ((chunk ^ b_row) & 7 | (chunk & ~7)) * 16);
                    const uint32_t a_lo[4] = {a[0], 0u, a[1], 0u}, a_hi[4] = {a[2], 0u, a[3], 0u};
                    mma_16816(acc, a_lo, b[0], b[1]);
                    mma_16816(acc2, a_hi, b[2], b[3]);
                }
            }
            ring.release(p, plan, bt, warp, lane);
        }
        // lane holds token lane / 4, weight rows 2 (lane % 4) and + 1 of the group
        *reinterpret_cast<float2*>(red + (size_t)item * 64 + (lane >> 2) * 8 + (lane & 3) * 2) = make_float2(acc[0] + acc2[0], acc[1] + acc2[1]);
    }
    note(p, ordinal, 3);
    __syncthreads();
    note(p, ordinal, 4);
    // the parts of a group summed in their order, then the output stage
    const int items_block = my_items;  // the same for every warp of the block
    const int groups_block = items_block >> pr.ksplit_shift;
    const int effective = plan.effective[product_of(stage)];
    for (int idx = threadIdx.x; idx < groups_block * 64; idx += MK_THREADS) {
        const int local_group = idx >> 6, token = (idx >> 3) & 7, col = idx & 7;
        if (token >= p.n_seqs) continue;
        if (stage == ST_GATEUP && (col & 1)) continue;
        const float* src = red + (size_t)local_group * pr.ksplit * 64 + token * 8 + col;
        float sum = 0.f, sum_up = 0.f;
        for (int part = 0; part < pr.ksplit; ++part) {
            sum += src[part * 64];
            if (stage == ST_GATEUP) sum_up += src[part * 64 + 1];
        }
        const int n = (effective + local_group * (int)gridDim.x) * 8 + col;
        if (stage == ST_QKV) {
            p.qkv[(size_t)token * pr.n + n] = __float2bfloat16_rn(sum);
        } else if (stage == ST_GATEUP) {
            p.act[(size_t)token * p.inter + (n >> 1)] = __float2bfloat16_rn(silu_f(sum) * sum_up);
        } else {
            float* dst = p.h + (size_t)token * p.hidden + n;
            // the branch's output is a bfloat16 projection added to the 32-bit stream (transformer.py:47-48)
            __stcg(dst, __ldcg(dst) + __bfloat162float(__float2bfloat16_rn(sum)));
        }
    }
    note(p, ordinal, 5);
}

// ------------------------------------------------------------------ the attention stage
template <int D, int NSLOT>
__device__ __forceinline__ void attention_stage(const MkParams& p, const WarpPlan& plan, const BlockTables& bt, Ring<D, NSLOT>& ring,
                                                const MkLayer& layer, int run, int warp, int lane) {
    constexpr int KEYS = Geometry<D>::KEYS;
    const int group = p.n_q / p.n_kv;
    const int n_heads = p.n_q + 2 * p.n_kv;
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    int a = plan.att_begin;
    int seq = plan.att_seq, hk = plan.att_hk, j0 = plan.att_j;
    while (a < plan.att_end) {
        const int pair_tiles = bt.pair_tiles[seq];
        const int j_end = min(pair_tiles, j0 + (plan.att_end - a));
        const int len = bt.len[seq];
        const int pos_new = len - 1;
        const bool owns_new = j_end == pair_tiles;  // the pair's last tile holds the new token's place
        const __nv_bfloat16* row_base = p.qkv + (size_t)seq * n_heads * D;

        // The new token's raw key and value, asked for first.
        __nv_bfloat162 k_raw[D / 64], k_new[D / 64], v_new[D / 64];  // lane l: elements 2l, 2l+1 of each 64-wide half
        if (owns_new) {
#pragma unroll
            for (int hf = 0; hf < D / 64; ++hf) {
                k_raw[hf] = __ldcg(reinterpret_cast<const __nv_bfloat162*>(row_base + (size_t)(p.n_q + hk) * D + hf * 64 + 2 * lane));
                v_new[hf] = __ldcg(reinterpret_cast<const __nv_bfloat162*>(row_base + (size_t)(p.n_q + p.n_kv + hk) * D + hf * 64 + 2 * lane));
            }
        }
        // Query fragments: row r of the tile is query head hk * group + r (rows >= group are zero; group <= 8).
        uint32_t qf[D / 16][4];
        {
            const __nv_bfloat16* qbase = row_base + (size_t)hk * group * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qf[ks][0] = r0 < group ? __ldcg(reinterpret_cast<const unsigned*>(qbase + (size_t)r0 * D + ks * 16 + c0)) : 0u;
                qf[ks][2] = r0 < group ? __ldcg(reinterpret_cast<const unsigned*>(qbase + (size_t)r0 * D + ks * 16 + c0 + 8)) : 0u;
                qf[ks][1] = 0u;
                qf[ks][3] = 0u;
            }
            float x[D / 16][4];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qf[ks][0]));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&qf[ks][2]));
                x[ks][0] = lo.x; x[ks][1] = lo.y; x[ks][2] = hi.x; x[ks][3] = hi.y;
            }
            if (layer.q_norm) {
                float ss = 0.f;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
                    for (int e = 0; e < 4; ++e) ss += x[ks][e] * x[ks][e];
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                const float inv = 1.0f / sqrtf(ss / (float)D + layer.eps_qk);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = ks * 16 + c0 + (e & 1) + (e >> 1) * 8;
                        x[ks][e] = (x[ks][e] * inv) * weight_of(layer.q_norm, p.qk_bf16, c);
                    }
            }
            if (p.cos_table) {
                const float* cs_row = p.cos_table + (size_t)pos_new * (D / 2);
                const float* sn_row = p.sin_table + (size_t)pos_new * (D / 2);
#pragma unroll
                for (int ks = 0; ks < D / 32; ++ks)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int c = ks * 16 + c0 + (e & 1) + (e >> 1) * 8;  // first half of the head
                        const float cs = cs_row[c], sn = sn_row[c];
                        const float u = x[ks][e], v = x[ks + D / 32][e];
                        x[ks][e] = u * cs - v * sn;
                        x[ks + D / 32][e] = v * cs + u * sn;
                    }
            }
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qf[ks][0] = pack_bf16(x[ks][0], x[ks][1]);
                qf[ks][2] = pack_bf16(x[ks][2], x[ks][3]);
            }
        }
        if (owns_new) {
            float kx[D / 64][2];
            float ss = 0.f;
#pragma unroll
            for (int hf = 0; hf < D / 64; ++hf) {
                const float2 f = __bfloat1622float2(k_raw[hf]);
                kx[hf][0] = f.x;
                kx[hf][1] = f.y;
                ss += f.x * f.x + f.y * f.y;
            }
            if (layer.k_norm) {
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss / (float)D + layer.eps_qk);
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf)
#pragma unroll
                    for (int e = 0; e < 2; ++e) kx[hf][e] = (kx[hf][e] * inv) * weight_of(layer.k_norm, p.qk_bf16, hf * 64 + 2 * lane + e);
            }
            if (p.cos_table) {
                const float* cs_row = p.cos_table + (size_t)pos_new * (D / 2);
                const float* sn_row = p.sin_table + (size_t)pos_new * (D / 2);
                if (D == 128) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = 2 * lane + e;
                        const float cs = cs_row[c], sn = sn_row[c];
                        const float u = kx[0][e], v = kx[D / 64 - 1][e];
                        kx[0][e] = u * cs - v * sn;
                        kx[D / 64 - 1][e] = v * cs + u * sn;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float mine = kx[0][e];
                        const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                        const int c = (2 * lane + e) % (D / 2);
                        const float cs = cs_row[c], sn = sn_row[c];
                        kx[0][e] = lane < 16 ? mine * cs - other * sn : mine * cs + other * sn;
                    }
                }
            }
            const int page = p.block_table[bt.table_row[seq] + pos_new / PAGE];
            const size_t at = (((size_t)page * p.n_kv + hk) * PAGE + (pos_new % PAGE)) * D;
#pragma unroll
            for (int hf = 0; hf < D / 64; ++hf) {
                k_new[hf] = __floats2bfloat162_rn(kx[hf][0], kx[hf][1]);
                *reinterpret_cast<__nv_bfloat162*>(layer.k_pages + at + hf * 64 + 2 * lane) = k_new[hf];
                *reinterpret_cast<__nv_bfloat162*>(layer.v_pages + at + hf * 64 + 2 * lane) = v_new[hf];
            }
        }

        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[D / 8][4];
#pragma unroll
        for (int jj = 0; jj < D / 8; ++jj)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[jj][i] = 0.f;

        for (int j = j0; j < j_end; ++j) {
            __nv_bfloat16* k_tile = reinterpret_cast<__nv_bfloat16*>(ring.acquire());
            const bool patch = owns_new && j == pair_tiles - 1;
            if (patch) {
                const int row = pos_new % KEYS;
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf) {
                    const int col = hf * 64 + 2 * lane;
                    *reinterpret_cast<__nv_bfloat162*>(k_tile + swz<D>(row, col >> 3) * 8 + (col & 7)) = k_new[hf];
                }
                __syncwarp();
            }
            float s[KEYS / 8][4];
#pragma unroll
            for (int sub = 0; sub < KEYS / 16; ++sub) {
                float s2[2][4];
                qk_16keys<D>(s2, qf, k_tile, sub * 16, lane);
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s[sub * 2 + n][i] = s2[n][i];
            }
            ring.release(p, plan, bt, warp, lane);
            __nv_bfloat16* v_tile = reinterpret_cast<__nv_bfloat16*>(ring.acquire());
            if (patch) {
                const int row = pos_new % KEYS;
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf) {
                    const int col = hf * 64 + 2 * lane;
                    *reinterpret_cast<__nv_bfloat162*>(v_tile + swz<D>(row, col >> 3) * 8 + (col & 7)) = v_new[hf];
                }
                __syncwarp();
            }
#pragma unroll
            for (int sub = 0; sub < KEYS / 16; ++sub) {
                const int abs0 = j * KEYS + sub * 16;
                if (abs0 < len) {  // warp-uniform
                    float s2[2][4];
#pragma unroll
                    for (int n = 0; n < 2; ++n)
#pragma unroll
                        for (int i = 0; i < 4; ++i) s2[n][i] = s[sub * 2 + n][i];
#pragma unroll
                    for (int n = 0; n < 2; ++n)
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int key = abs0 + n * 8 + c0 + c;
                            if (key >= len) s2[n][c] = s2[n][2 + c] = -INFINITY;
                        }
                    uint32_t pf[4];
                    softmax_update<D>(s2, m, l, o, pf, p.sl2);
                    pv_16keys<D>(o, pf, v_tile, sub * 16, lane);
                }
            }
            ring.release(p, plan, bt, warp, lane);
        }

        // This warp's partial result of the pair, and a ticket: the last warp of the pair merges.
        const int pair = seq * p.n_kv + hk;
        const int pair_start = bt.tiles_of[seq] + hk * pair_tiles;        // the pair's first tile in the line
        const int first_warp = pair_start / run, last_warp = (pair_start + pair_tiles - 1) / run;
        const int n_splits = last_warp - first_warp + 1;
        const int split = a / run - first_warp;
        const int stride = group * (D + 2);
        float* mine = p.part + ((size_t)pair * p.part_splits + split) * stride;
        if (r0 < group) {
            if ((lane & 3) == 0) {
                mine[r0 * (D + 2) + D] = m[0];
                mine[r0 * (D + 2) + D + 1] = l[0];
            }
#pragma unroll
            for (int jj = 0; jj < D / 8; ++jj)
                *reinterpret_cast<float2*>(mine + r0 * (D + 2) + jj * 8 + c0) = make_float2(o[jj][0], o[jj][1]);
        }
        __threadfence();
        __syncwarp();
        unsigned ticket = 0;
        if (lane == 0) ticket = atomicAdd(p.words + 8 + pair, 1u);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        if (ticket == (unsigned)(n_splits - 1)) {
            if (lane == 0) atomicExch(p.words + 8 + pair, 0u);
            __threadfence();
            const float* all = p.part + (size_t)pair * p.part_splits * stride;
            for (int r = 0; r < group; ++r) {
                float top = -INFINITY;
                for (int sp = 0; sp < n_splits; ++sp) top = fmaxf(top, __ldcg(all + (size_t)sp * stride + r * (D + 2) + D));
                float denom = 0.f;
                float num[D / 32];
#pragma unroll
                for (int e = 0; e < D / 32; ++e) num[e] = 0.f;
                if (top != -INFINITY) {
                    for (int sp = 0; sp < n_splits; ++sp) {
                        const float* src = all + (size_t)sp * stride + r * (D + 2);
                        const float ms = __ldcg(src + D);
                        const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - top);
                        denom += __ldcg(src + D + 1) * wgt;
#pragma unroll
                        for (int e = 0; e < D / 32; ++e) num[e] += __ldcg(src + e * 32 + lane) * wgt;
                    }
                }
                __nv_bfloat16* dst = p.att + ((size_t)seq * p.n_q + (size_t)hk * group + r) * D;
#pragma unroll
                for (int e = 0; e < D / 32; ++e) dst[e * 32 + lane] = __float2bfloat16_rn(denom > 0.f ? num[e] / denom : 0.f);
            }
        }
        a += j_end - j0;
        j0 = 0;  // the run goes on with the next pair's first tile
        if (++hk == p.n_kv) {
            hk = 0;
            ++seq;
        }
    }
}

// ------------------------------------------------------------------ the kernel
template <int D, int NSLOT>
__global__ void __launch_bounds__(MK_THREADS, 1) decode_layers_kernel(const MkParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ BlockTables bt;
    __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(smem);
    float* red = reinterpret_cast<float*>(smem + (size_t)MK_TOKENS * p.x_stride * 2);
    unsigned char* rings = reinterpret_cast<unsigned char*>(red) + (size_t)p.red_floats * 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int KEYS = Geometry<D>::KEYS;

    // The step's sequences: lengths, slots and the page table are step inputs, in place before the step's first kernel.
    if (threadIdx.x == 0) {
        bt.tiles_of[0] = 0;
        for (int b = 0; b < MK_TOKENS; ++b) {
            const int len = b < p.n_seqs ? p.kv_len[b] : 0;
            bt.len[b] = len;
            bt.pair_tiles[b] = (len + KEYS - 1) / KEYS;
            bt.tiles_of[b + 1] = bt.tiles_of[b] + bt.pair_tiles[b] * p.n_kv;
            bt.table_row[b] = b < p.n_seqs ? (long long)p.slots[b] * p.max_pages : 0;
        }
    }
    // rows of tokens that do not exist stay zero for the whole kernel
    for (int i = threadIdx.x; i < MK_TOKENS * p.x_stride / 2; i += MK_THREADS) reinterpret_cast<uint32_t*>(x)[i] = 0u;
    __syncthreads();

    WarpPlan plan;
    const int all_tiles = bt.tiles_of[MK_TOKENS];
    const int grid_warps = (int)gridDim.x * MK_WARPS;
    const int run = max(MK_ATT_MIN_RUN, (all_tiles + grid_warps - 1) / grid_warps);
    const int grid_warp = warp * (int)gridDim.x + (int)blockIdx.x;  // neighbours in the line sit on different SMs
    plan.att_begin = min(all_tiles, grid_warp * run);
    plan.att_end = min(all_tiles, plan.att_begin + run);
    plan.att_seq = plan.att_hk = plan.att_j = 0;
    if (plan.att_begin < plan.att_end) pair_of(p, bt, plan.att_begin, plan.att_seq, plan.att_hk, plan.att_j);
    for (int i = 0; i < 4; ++i) {
        const MkProduct& pr = p.prod[i];
        const int groups = pr.n / 8;
        const int effective = ((int)blockIdx.x + pr.rotation) % (int)gridDim.x;
        const int mine = effective < groups ? (groups - effective + (int)gridDim.x - 1) / (int)gridDim.x : 0;
        plan.effective[i] = effective;
        plan.items[i] = mine << pr.ksplit_shift;
    }

    Ring<D, NSLOT> ring;
    ring.base = rings + (size_t)warp * NSLOT * MK_SLOT;
    ring.taken = 0;
    ring.ahead = Cursor{0, 0, warp, 0, 0, 0, 0};
    ring.more = settle(p, plan, ring.ahead, warp);
    // Weights do not depend on the kernel in front.  The first NSLOT tiles are weights of the first product unless
    // the warp has fewer: then keys and values would come next, and those wait for the kernel in front.
    int early = 0;
    for (; early < NSLOT && ring.more && ring.ahead.layer == 0 && ring.ahead.stage == ST_QKV; ++early) ring.request_next(p, plan, bt, early, warp, lane);
    NormWeights nw;
    fetch_norm_weights(p, nw, p.layers[0].norm_in, warp, lane);
    pdl_wait();
    for (; early < NSLOT; ++early) ring.request_next(p, plan, bt, early, warp, lane);

    unsigned target = 0;
    for (int l = 0; l < p.n_layers; ++l) {
        const MkLayer& layer = p.layers[l];
        note(p, l * ST_COUNT + ST_QKV, 0);
        load_normed(p, x, nw, layer.norm_in, layer.eps_in, warp, lane);
        __syncthreads();
        note(p, l * ST_COUNT + ST_QKV, 1);
        product_stage<D, NSLOT>(p, plan, bt, ring, ST_QKV, layer, x, red, warp, lane, l * ST_COUNT + ST_QKV);
        grid_barrier(p, target);
        attention_stage<D, NSLOT>(p, plan, bt, ring, layer, run, warp, lane);
        grid_barrier(p, target);
        note(p, l * ST_COUNT + ST_OPROJ, 0);
        load_plain(p, x, p.att, p.n_q * D, warp, lane);
        __syncthreads();
        note(p, l * ST_COUNT + ST_OPROJ, 1);
        product_stage<D, NSLOT>(p, plan, bt, ring, ST_OPROJ, layer, x, red, warp, lane, l * ST_COUNT + ST_OPROJ);
        fetch_norm_weights(p, nw, layer.norm_post, warp, lane);  // on their way while the block waits
        grid_barrier(p, target);
        note(p, l * ST_COUNT + ST_GATEUP, 0);
        load_normed(p, x, nw, layer.norm_post, layer.eps_post, warp, lane);
        __syncthreads();
        note(p, l * ST_COUNT + ST_GATEUP, 1);
        product_stage<D, NSLOT>(p, plan, bt, ring, ST_GATEUP, layer, x, red, warp, lane, l * ST_COUNT + ST_GATEUP);
        grid_barrier(p, target);
        note(p, l * ST_COUNT + ST_DOWN, 0);
        load_plain(p, x, p.act, p.inter, warp, lane);
        __syncthreads();
        note(p, l * ST_COUNT + ST_DOWN, 1);
        product_stage<D, NSLOT>(p, plan, bt, ring, ST_DOWN, layer, x, red, warp, lane, l * ST_COUNT + ST_DOWN);
        if (l + 1 < p.n_layers) {
            fetch_norm_weights(p, nw, p.layers[l + 1].norm_in, warp, lane);
            grid_barrier(p, target);
        }
    }
    cp_async_wait<0>();
    // The block that leaves last puts the words back to zero for the next launch (every block has then passed
    // every barrier, aborted or not).
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.words + 1, 1u) == gridDim.x - 1) {
            const int pairs = p.n_seqs * p.n_kv;
            for (int i = 0; i < 8 + pairs; ++i) p.words[i] = 0u;
            __threadfence();
        }
    }
    pdl_launch_dependents();
}

template <int D>
cudaError_t launch_for_slots(int n_slots, int grid, size_t smem, cudaStream_t stream, const MkParams& p) {
    auto go = [&](auto kernel) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return err;
        return gk_launch(kernel, dim3(grid), dim3(MK_THREADS), smem, stream, p);
    };
    // two ring depths are compiled (each is a copy of the whole kernel): five slots a warp where they fit, else three
    if (n_slots >= 5) return go(decode_layers_kernel<D, 5>);
    return go(decode_layers_kernel<D, 3>);
}

int pow2_at_least(int v) {
    int r = 1;
    while (r < v) r <<= 1;
    return r;
}

}  // namespace

// Bytes of the work areas that gk_decode_layers needs for `n_seqs` sequences of up to `max_kv_len` tokens:
// out[0] = floats of the attention partial results, out[1] = 32-bit words of counters.  Also the check whether the
// kernel takes these sizes at all: returns GK_UNSUPPORTED (with the reason as the last error) if not.
GK_EXPORT int gk_decode_layers_plan(int n_seqs, int hidden, int n_q, int n_kv, int head_dim, int inter, int max_kv_len,
                                    int page_size, long long* out) {
    if (n_seqs < 1 || n_seqs > MK_TOKENS) return gk_fail(GK_UNSUPPORTED, "decode_layers: takes 1 to %d sequences, got %d", MK_TOKENS, n_seqs);
    if (head_dim != 64 && head_dim != 128) return gk_fail(GK_UNSUPPORTED, "decode_layers: head size %d (64 or 128)", head_dim);
    if (page_size != PAGE) return gk_fail(GK_UNSUPPORTED, "decode_layers: pages of %d positions (64)", page_size);
    if (n_kv < 1 || n_q % n_kv || n_q / n_kv > 8) return gk_fail(GK_UNSUPPORTED, "decode_layers: %d query heads on %d kv heads (groups of up to 8)", n_q, n_kv);
    if (hidden % 128 || inter % 32 || (n_q * head_dim) % 32) return gk_fail(GK_UNSUPPORTED, "decode_layers: widths %d / %d / %d", hidden, inter, n_q * head_dim);
    const int keys = MK_SLOT / (head_dim * 2);
    const int pair_tiles = (max_kv_len + keys - 1) / keys;
    out[0] = (long long)n_seqs * n_kv * ((pair_tiles + MK_ATT_MIN_RUN - 1) / MK_ATT_MIN_RUN + 1) * (n_q / n_kv) * (head_dim + 2);
    out[1] = 8 + (long long)n_seqs * n_kv;
    return GK_OK;
}

GK_EXPORT int gk_decode_layers(const void* layers, int n_layers, int n_seqs, int hidden, int n_q, int n_kv, int head_dim,
                               int inter, float* h, void* qkv, void* att, void* act, float* part, long long part_floats,
                               unsigned* words, const int* kv_len, const int* slots, const int* block_table, int max_pages,
                               int max_kv_len, const float* cos_table, const float* sin_table, int table_positions,
                               int norm_bf16, int qk_bf16, float scale, int* error_flag, long long* stamps, void* stream) {
    long long need[2];
    const int status = gk_decode_layers_plan(n_seqs, hidden, n_q, n_kv, head_dim, inter, max_kv_len, PAGE, need);
    if (status != GK_OK) return status;
    GK_REQUIRE(n_layers >= 1, "decode_layers: no layers");
    GK_REQUIRE(part_floats >= need[0], "decode_layers: %lld floats of partial results, %lld needed", part_floats, need[0]);
    GK_REQUIRE(cos_table == nullptr || table_positions >= max_kv_len, "decode_layers: rotary tables hold %d positions, %d needed", table_positions, max_kv_len);
    int device = 0, sms = 0, smem_max = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);

    MkParams p = {};
    p.layers = (const MkLayer*)layers;
    p.n_layers = n_layers;
    p.n_seqs = n_seqs; p.hidden = hidden; p.n_q = n_q; p.n_kv = n_kv; p.inter = inter;
    const int widths[4][2] = {{(n_q + 2 * n_kv) * head_dim, hidden}, {hidden, n_q * head_dim}, {2 * inter, hidden}, {hidden, inter}};
    int k_max = 0, red_floats = 0;
    for (int i = 0; i < 4; ++i) {
        MkProduct& pr = p.prod[i];
        pr.n = widths[i][0];
        pr.k = widths[i][1];
        GK_REQUIRE(pr.n % 8 == 0, "decode_layers: %d weight rows are no multiple of 8", pr.n);
        const int groups = pr.n / 8;
        const int per_block = (groups + sms - 1) / sms;
        int ksplit = pow2_at_least((16 + per_block - 1) / per_block);
        if (ksplit > 8) ksplit = 8;
        while (ksplit > 1 && (pr.k % (32 * ksplit) != 0 || pr.k / ksplit < 64)) ksplit >>= 1;
        GK_REQUIRE(pr.k % 32 == 0, "decode_layers: rows of %d are no multiple of 32", pr.k);
        pr.ksplit = ksplit;
        pr.ksplit_shift = 0;
        while ((1 << pr.ksplit_shift) < ksplit) ++pr.ksplit_shift;
        pr.part_k = pr.k / ksplit;
        pr.part_tiles = (pr.part_k + MK_TILE_K - 1) / MK_TILE_K;
        pr.rotation = (i * 37) % sms;
        if (pr.k > k_max) k_max = pr.k;
        if (per_block * ksplit * 64 > red_floats) red_floats = per_block * ksplit * 64;
    }
    p.h = h; p.qkv = (__nv_bfloat16*)qkv; p.att = (__nv_bfloat16*)att; p.act = (__nv_bfloat16*)act;
    p.part = part;
    const int keys = MK_SLOT / (head_dim * 2);
    p.part_splits = (((max_kv_len + keys - 1) / keys) + MK_ATT_MIN_RUN - 1) / MK_ATT_MIN_RUN + 1;
    p.words = words;
    p.kv_len = kv_len; p.slots = slots; p.block_table = block_table; p.max_pages = max_pages;
    p.cos_table = cos_table; p.sin_table = sin_table;
    p.norm_bf16 = norm_bf16; p.qk_bf16 = qk_bf16;
    p.sl2 = scale * 1.4426950408889634f;
    p.x_stride = k_max + 8;
    p.error_flag = error_flag;
    p.stamps = stamps;
    red_floats = (red_floats + 31) / 32 * 32;
    while (((size_t)MK_TOKENS * p.x_stride * 2 + (size_t)red_floats * 4) % 128) red_floats += 4;  // the rings start on a 128-byte line
    p.red_floats = red_floats;
    const size_t fixed = (size_t)MK_TOKENS * p.x_stride * 2 + (size_t)red_floats * 4;
    int n_slots = (int)(((size_t)smem_max - fixed) / ((size_t)MK_WARPS * MK_SLOT));
    if ((size_t)smem_max < fixed || n_slots < 3)
        return gk_fail(GK_UNSUPPORTED, "decode_layers: rows of %d elements leave no room for the rings in shared memory", k_max);
    n_slots = n_slots >= 5 ? 5 : 3;
    const size_t smem = fixed + (size_t)n_slots * MK_WARPS * MK_SLOT;
    cudaError_t err = head_dim == 128 ? launch_for_slots<128>(n_slots, sms, smem, (cudaStream_t)stream, p)
                                      : launch_for_slots<64>(n_slots, sms, smem, (cudaStream_t)stream, p);
    if (err != cudaSuccess) return gk_fail(GK_CUDA_ERROR, "decode_layers: launch failed: %s", cudaGetErrorString(err));
    GK_CHECK_LAUNCH("decode_layers");
    return GK_OK;
}
