// Product of a few tokens with a weight matrix,  OUT[t, n] = sum_k X[t, k] * W[n, k]  for up to 16 tokens (32 for short K)
// (every projection of a decode step: src/layers/attention.py:62-65, src/layers/swiglu.py:9-14), built for
// latency rather than arithmetic: with so few tokens the time goes to getting the weights in, not to the
// multiplications.
//
// The weight rows are taken in groups of eight.  There is one block of eight warps per SM at most, and it is
// small in registers and threads, so that the blocks of the next kernel in the stream are resident beside it
// (programmatic dependent launch).  A block takes every grid-th group; within a group its warps take the
// 32-wide k-chunks in turn.  A thread is responsible for 16 bytes of one weight row per chunk, and it asks for
// all of them, for all its chunks, with cp.async into shared memory before the kernel has waited for the
// kernel in front of it: weights do not depend on that kernel, so by the time that kernel has finished the
// block's whole share of the matrix is in shared memory or on its way.  Once it has waited, it fetches the
// tokens' activations (one trip to L2): for K up to 1024 a warp sees the same four chunks in every group, so a
// thread keeps its 16 bytes of each in registers; for longer K the block copies all of them into shared
// memory.  Per chunk a thread then takes its own 16 bytes of weights back out of shared memory (nobody else
// reads them), and two mma.sync.m16n8k16 (tokens on the 16 rows, the eight weight rows on the 8 columns,
// 32-bit accumulation) finish the chunk.  Shared-memory bandwidth is what this part costs: every weight byte
// is read from it once, and nothing else.  Which k goes to which slot of the instruction
// is the same for both operands and otherwise of no consequence for a sum, so both are read as plain
// contiguous 16-byte pieces.  The warps' partial sums of a group meet in shared memory (in the place of a
// weight piece the thread has used up) and are added in the order of the warps by one warp, which writes the
// group's result.
//
// Output stages: plain store (bfloat16 or float32) and SwiGLU over row pairs (gate and up rows interleaved,
// even = gate, odd = up: both of a channel end up in the same thread).

#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int ROWS = 8;          // weight rows of a group = the N of the MMA
constexpr int CHUNK = 32;        // k of one 16-byte piece per thread and row: 4 threads x 8 elements
constexpr int MAX_GROUPS = 8;    // groups a block can take (its partial sums stay in shared memory)
constexpr int X_REGS = 4;        // chunks per warp and group up to which the activations stay in registers
constexpr int X_REGS_LONG = 12;  // the same for up to eight tokens (one set of rows): rows of up to 3,072 elements
constexpr int ROUND_ITEMS = 24;  // chunks per thread whose weights fit in shared memory at once (96 KB a block)

struct GemvParams {
    const __nv_bfloat16* w;   // [n][ldw]
    const __nv_bfloat16* x;   // [tokens][ldx]
    void* out;                // [tokens][n] (or [tokens][n / 2] with SwiGLU)
    int n, k, tokens;
    long long ldw, ldx, ldo;
    int out_f32, swiglu;
    // Optional: the activations are the RMSNorm of the rows of a 32-bit stream, formed here (`norm_h` set, `x` unused):
    //   x[t, k] = bfloat16((h[t, k] * rsqrt(mean_k h[t, k]^2 + eps)) * norm_w[k])       (src/layers/rmsnorm.py:11-16)
    // every block holds whole rows of its tokens (its threads' pieces of a row are the row), so it forms the row's
    // sum of squares itself; the norm's weights are fetched before the wait for the kernel in front.
    const float* norm_h;      // [tokens][ldh]
    const void* norm_w;       // [k]
    int norm_w_bf16;
    float norm_eps;
    long long ldh;
    // Optional: the result is added to a 32-bit stream instead of stored (`resid` set, `out` unused):
    //   resid[t, n] += bfloat16(sum)   (the projection's output is bfloat16, the stream 32-bit: src/models/transformer.py:47-48)
    float* resid;             // [tokens][ldr]
    long long ldr;
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16 bytes from global to shared memory without passing through registers; `bytes` = 0 writes zeros
__device__ __forceinline__ void copy16_async(void* smem_dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ float silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// ROW_SETS: sets of eight tokens, 1, 2 or 4.  An MMA takes two sets on its rows 0..7 and 8..15 (with one set the
// upper rows are zero); with four sets (17 to 32 tokens) every weight piece goes through two MMAs' worth of
// tokens, with the activations of all of them in registers: short K only (a warp has at most four chunks), all
// weights in one round, and two partial sums a thread where the group's first two weight pieces were.
// Shared memory: [item of the round][thread] 16-byte weight pieces; the tokens' activations, a row every
// `x_stride` bytes (the rows of two tokens a quarter-warp reads together lie in different banks); and, when the
// weights come in more than one round, [group of the block][thread] partial sums (with one round a thread
// leaves its partial sum where the group's first weight piece was).
// XR: chunks per warp and group up to which the activations stay in registers (X_REGS; 12 for up to eight tokens of
// up to 3,072 elements: every thread fetches its own pieces straight from memory, no staging by the block, and all
// SMs take part where the staged path would use fewer, fatter blocks).
template <int ROW_SETS, bool NORM = false, int XR = X_REGS>
__global__ void __launch_bounds__(THREADS, NORM || XR > X_REGS ? 2 : ROW_SETS == 4 ? 2 : 3) gemv_mma_kernel(const GemvParams p, int round_items, int x_stride) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float row_ss[WARPS][16];  // NORM: the warps' parts of each token's sum of squares
    constexpr bool TWO_ROWS = ROW_SETS >= 2;
    constexpr int TILES = (ROW_SETS + 1) / 2;  // MMAs' worth of tokens
    constexpr int X_ROWS = 8 * ROW_SETS;
    uint4* pieces = reinterpret_cast<uint4*>(smem);
    unsigned char* xs = smem + (size_t)round_items * THREADS * 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = lane >> 2, piece = lane & 3;  // group: weight row (B) and token (A); piece: 8 of the chunk's 32 k
    if (threadIdx.x == 0) pdl_launch_dependents();

    const int n_groups = (p.n + ROWS - 1) / ROWS;
    const int my_groups = ((int)blockIdx.x < n_groups) ? (n_groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int n_chunks = (p.k + CHUNK - 1) / CHUNK;
    const int cpw = (n_chunks + WARPS - 1) / WARPS;  // chunks of a group per warp: warp, warp + 8, ...
    const int n_items = my_groups * cpw;             // item i: group i / cpw of the block, chunk warp + (i % cpw) * 8
    const bool one_round = n_items <= round_items;
    float4* partial = one_round ? reinterpret_cast<float4*>(pieces) : reinterpret_cast<float4*>(xs + (size_t)X_ROWS * x_stride);
    const int partial_step = one_round ? cpw * THREADS : THREADS;  // from one group's partial sums to the next group's

    // The weights of items first .. first + round_items - 1 (item = group of the block * cpw + chunk of the warp),
    // on their way to shared memory.
    auto request_into = [&](int first, int count, uint4* dst) {
        int g = first / cpw, j = first % cpw;
        dst += threadIdx.x;
        for (int item = first; item < first + count && item < n_items; ++item) {
            const int row = ((int)blockIdx.x + g * (int)gridDim.x) * ROWS + group;
            const int k = (warp + j * WARPS) * CHUNK + piece * 8;
            const bool in = row < p.n && k < p.k;
            copy16_async(dst, in ? p.w + (size_t)row * p.ldw + k : p.w, in ? 16 : 0);
            dst += THREADS;
            if (++j == cpw) {
                j = 0;
                ++g;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // A block whose share exceeds shared memory takes it in rounds of half the space: two rounds are on their way
    // while a third is multiplied (a thread reads only the pieces it asked for itself, so it may ask for the round
    // after next into the half it has just finished with, without a barrier).
    const int half_items = round_items / 2;

    // With the residual output stage, the stream's old values of the outputs this thread will write (warp g of the
    // block finishes the block's g-th group) are asked for as soon as the kernel in front has finished, long before
    // the sums are there.
    float2 old[TILES][TWO_ROWS ? 2 : 1];
    auto fetch_old = [&]() {
        if (p.resid == nullptr || warp >= my_groups) return;
        const int col = ((int)blockIdx.x + warp * (int)gridDim.x) * ROWS + 2 * piece;
#pragma unroll
        for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
            for (int half = 0; half < (TWO_ROWS ? 2 : 1); ++half) {
                const int token = 16 * tile + group + 8 * half;
                old[tile][half] = make_float2(0.f, 0.f);
                if (token < p.tokens && col + 1 < p.n) old[tile][half] = *reinterpret_cast<const float2*>(p.resid + (size_t)token * p.ldr + col);
                else if (token < p.tokens && col < p.n) old[tile][half].x = p.resid[(size_t)token * p.ldr + col];
            }
    };

    // after the block's barrier: warp g of the block finishes the block's g-th group
    auto finish = [&]() {
        if (warp >= my_groups) return;
        const int col = ((int)blockIdx.x + warp * (int)gridDim.x) * ROWS + 2 * piece;
#pragma unroll
        for (int tile = 0; tile < TILES; ++tile) {
        // the warps' sums in their order (a tile's partial sums lie THREADS pieces after the tile before)
        const float4* slots = partial + (size_t)warp * partial_step + tile * THREADS + lane;
        float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float4 v = slots[w * 32];
            sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
        }
        // sum[0], sum[1]: token `group` of the tile, weight rows col and col + 1;  sum[2], sum[3]: token group + 8
#pragma unroll
        for (int half = 0; half < (TWO_ROWS ? 2 : 1); ++half) {
            const int token = 16 * tile + group + 8 * half;
            if (token >= p.tokens) continue;
            const float a = sum[2 * half], b = sum[2 * half + 1];
            if (p.resid) {
                float* o = p.resid + (size_t)token * p.ldr + col;
                const float na = old[tile][half].x + __bfloat162float(__float2bfloat16(a));
                const float nb = old[tile][half].y + __bfloat162float(__float2bfloat16(b));
                if (col + 1 < p.n) *reinterpret_cast<float2*>(o) = make_float2(na, nb);
                else if (col < p.n) o[0] = na;
            } else if (p.swiglu) {
                if (col + 1 < p.n)
                    reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)token * p.ldo + (col >> 1)] = __float2bfloat16(silu(a) * b);
            } else if (p.out_f32) {
                float* o = reinterpret_cast<float*>(p.out) + (size_t)token * p.ldo + col;
                if (col < p.n) o[0] = a;
                if (col + 1 < p.n) o[1] = b;
            } else {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)token * p.ldo + col;
                if (col + 1 < p.n && ((p.ldo & 1) == 0)) {
                    *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(a, b);
                } else {
                    if (col < p.n) o[0] = __float2bfloat16(a);
                    if (col + 1 < p.n) o[1] = __float2bfloat16(b);
                }
            }
        }
        }
    };

    // before the kernel in front has finished
    if (one_round) {
        request_into(0, round_items, pieces);
    } else {
        request_into(0, half_items, pieces);
        request_into(half_items, half_items, pieces + (size_t)half_items * THREADS);
    }
    // NORM: this thread's pieces of the norm's weights (the same for every token), also before the wait
    float nw[NORM ? XR : 1][8];
    if (NORM) {
#pragma unroll
        for (int j = 0; j < XR; ++j) {
            const int k = (warp + j * WARPS) * CHUNK + piece * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) nw[NORM ? j : 0][e] = 0.f;
            if (j < cpw && k < p.k) {
                if (p.norm_w_bf16) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.norm_w) + k);
                    const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r[e]));
                        nw[NORM ? j : 0][2 * e] = f.x;
                        nw[NORM ? j : 0][2 * e + 1] = f.y;
                    }
                } else {
                    const float4 lo = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm_w) + k);
                    const float4 hi = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm_w) + k + 4);
                    nw[NORM ? j : 0][0] = lo.x; nw[NORM ? j : 0][1] = lo.y; nw[NORM ? j : 0][2] = lo.z; nw[NORM ? j : 0][3] = lo.w;
                    nw[NORM ? j : 0][4] = hi.x; nw[NORM ? j : 0][5] = hi.y; nw[NORM ? j : 0][6] = hi.z; nw[NORM ? j : 0][7] = hi.w;
                }
            }
        }
    }
    pdl_wait();
    fetch_old();
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4* wp = pieces + threadIdx.x;
    if (cpw <= XR && one_round) {
        // short K: the thread's pieces of the activations straight from memory into registers, no staging
        uint4 xr[TILES][XR], xr2[TILES][XR];
        if (NORM) {
            // the rows of the stream: 32 bytes a piece, their squares summed over the block, then scaled and rounded
            static_assert(!NORM || TILES == 1, "the norm on load is built for up to 16 tokens");
            float hv[XR][8], hv2[TWO_ROWS ? XR : 1][8];
            float ss = 0.f, ss2 = 0.f;
#pragma unroll
            for (int j = 0; j < XR; ++j) {
                const int k = (warp + j * WARPS) * CHUNK + piece * 8;
                const bool in = j < cpw && k < p.k;
                const bool in1 = in && group < p.tokens, in2 = TWO_ROWS && in && group + 8 < p.tokens;
                const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 a = in1 ? *reinterpret_cast<const float4*>(p.norm_h + (size_t)group * p.ldh + k) : z;
                const float4 b = in1 ? *reinterpret_cast<const float4*>(p.norm_h + (size_t)group * p.ldh + k + 4) : z;
                hv[j][0] = a.x; hv[j][1] = a.y; hv[j][2] = a.z; hv[j][3] = a.w; hv[j][4] = b.x; hv[j][5] = b.y; hv[j][6] = b.z; hv[j][7] = b.w;
                if (TWO_ROWS) {
                    const float4 c = in2 ? *reinterpret_cast<const float4*>(p.norm_h + (size_t)(group + 8) * p.ldh + k) : z;
                    const float4 d = in2 ? *reinterpret_cast<const float4*>(p.norm_h + (size_t)(group + 8) * p.ldh + k + 4) : z;
                    hv2[TWO_ROWS ? j : 0][0] = c.x; hv2[TWO_ROWS ? j : 0][1] = c.y; hv2[TWO_ROWS ? j : 0][2] = c.z; hv2[TWO_ROWS ? j : 0][3] = c.w;
                    hv2[TWO_ROWS ? j : 0][4] = d.x; hv2[TWO_ROWS ? j : 0][5] = d.y; hv2[TWO_ROWS ? j : 0][6] = d.z; hv2[TWO_ROWS ? j : 0][7] = d.w;
                }
            }
#pragma unroll
            for (int j = 0; j < XR; ++j)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    ss += hv[j][e] * hv[j][e];
                    if (TWO_ROWS) ss2 += hv2[TWO_ROWS ? j : 0][e] * hv2[TWO_ROWS ? j : 0][e];
                }
            // the four lanes that share a token, then the warps in their order
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            if (TWO_ROWS) {
                ss2 += __shfl_xor_sync(0xffffffffu, ss2, 1);
                ss2 += __shfl_xor_sync(0xffffffffu, ss2, 2);
            }
            if (piece == 0) {
                row_ss[warp][group] = ss;
                row_ss[warp][group + 8] = ss2;
            }
            __syncthreads();
            float total = 0.f, total2 = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                total += row_ss[w][group];
                total2 += row_ss[w][group + 8];
            }
            const float inv = rsqrtf(total / (float)p.k + p.norm_eps);
            const float inv2 = rsqrtf(total2 / (float)p.k + p.norm_eps);
            auto pack2 = [](float lo, float hi) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                return *reinterpret_cast<uint32_t*>(&v);
            };
#pragma unroll
            for (int j = 0; j < XR; ++j) {
                const float* w8 = nw[NORM ? j : 0];
                xr[0][j] = make_uint4(pack2((hv[j][0] * inv) * w8[0], (hv[j][1] * inv) * w8[1]), pack2((hv[j][2] * inv) * w8[2], (hv[j][3] * inv) * w8[3]),
                                      pack2((hv[j][4] * inv) * w8[4], (hv[j][5] * inv) * w8[5]), pack2((hv[j][6] * inv) * w8[6], (hv[j][7] * inv) * w8[7]));
                if (TWO_ROWS) {
                    const float* h2 = hv2[TWO_ROWS ? j : 0];
                    xr2[0][j] = make_uint4(pack2((h2[0] * inv2) * w8[0], (h2[1] * inv2) * w8[1]), pack2((h2[2] * inv2) * w8[2], (h2[3] * inv2) * w8[3]),
                                           pack2((h2[4] * inv2) * w8[4], (h2[5] * inv2) * w8[5]), pack2((h2[6] * inv2) * w8[6], (h2[7] * inv2) * w8[7]));
                } else {
                    xr2[0][j] = zero;
                }
            }
        } else {
#pragma unroll
        for (int tile = 0; tile < TILES; ++tile) {
#pragma unroll
            for (int j = 0; j < XR; ++j) {
                const int k = (warp + j * WARPS) * CHUNK + piece * 8;
                const bool in = j < cpw && k < p.k;
                const int token = 16 * tile + group;
                xr[tile][j] = in && token < p.tokens ? *reinterpret_cast<const uint4*>(p.x + (size_t)token * p.ldx + k) : zero;
                xr2[tile][j] = TWO_ROWS && in && token + 8 < p.tokens ? *reinterpret_cast<const uint4*>(p.x + (size_t)(token + 8) * p.ldx + k) : zero;
            }
        }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        for (int g = 0; g < my_groups; ++g) {
            float acc0[TILES][4], acc1[TILES][4];
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile) {
#pragma unroll
                for (int i = 0; i < 4; ++i) acc0[tile][i] = acc1[tile][i] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < XR; ++j) {
                if (j < cpw) {
                    const uint4 wv = *wp;
                    wp += THREADS;
#pragma unroll
                    for (int tile = 0; tile < TILES; ++tile) {
                        mma_bf16(acc0[tile], xr[tile][j].x, xr2[tile][j].x, xr[tile][j].y, xr2[tile][j].y, wv.x, wv.y);
                        mma_bf16(acc1[tile], xr[tile][j].z, xr2[tile][j].z, xr[tile][j].w, xr2[tile][j].w, wv.z, wv.w);
                    }
                }
            }
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile)
                partial[(size_t)g * partial_step + tile * THREADS + threadIdx.x] =
                    make_float4(acc0[tile][0] + acc1[tile][0], acc0[tile][1] + acc1[tile][1], acc0[tile][2] + acc1[tile][2],
                                acc0[tile][3] + acc1[tile][3]);
        }
        __syncthreads();
        finish();
        return;
    }
    if (ROW_SETS == 4 || NORM) return;  // (the host sends 17 to 32 tokens, and the norm on load, here only where the path above applies)
    // the activations of all tokens into shared memory; zeros for the rows that are no token and from K up to
    // the end of the last chunk any warp looks at
    const int x_pieces = cpw * WARPS * 4;  // 16-byte pieces of a row
    // a thread takes the same piece of every row: no division by a run-time number behind the wait
    for (int piece_at = threadIdx.x; piece_at < x_pieces; piece_at += THREADS) {
        const int at = piece_at * 8;
#pragma unroll 4
        for (int row = 0; row < X_ROWS; ++row) {
            const bool in = row < p.tokens && at < p.k;
            copy16_async(xs + (size_t)row * x_stride + at * 2, in ? p.x + (size_t)row * p.ldx + at : p.x, in ? 16 : 0);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    const unsigned char* xa_first = xs + (size_t)group * x_stride + (warp * CHUNK + piece * 8) * 2;
    // one chunk: the thread's weights, the token's activations (zeros beyond K, see above), two MMAs into two
    // accumulators that do not wait for one another
    auto chunk = [&](const uint4 wv, const unsigned char* xa_at, float (&acc0)[4], float (&acc1)[4]) {
        const uint4 xa = *reinterpret_cast<const uint4*>(xa_at);
        const uint4 xb = TWO_ROWS ? *reinterpret_cast<const uint4*>(xa_at + 8 * (size_t)x_stride) : zero;
        mma_bf16(acc0, xa.x, xb.x, xa.y, xb.y, wv.x, wv.y);
        mma_bf16(acc1, xa.z, xb.z, xa.w, xb.w, wv.z, wv.w);
    };
    if (one_round) {
        for (int g = 0; g < my_groups; ++g) {
            float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
            const unsigned char* xa_at = xa_first;
#pragma unroll 4
            for (int j = 0; j < cpw; ++j) {
                chunk(*wp, xa_at, acc0, acc1);
                wp += THREADS;
                xa_at += WARPS * CHUNK * 2;
            }
            partial[(size_t)g * partial_step + threadIdx.x] =
                make_float4(acc0[0] + acc1[0], acc0[1] + acc1[1], acc0[2] + acc1[2], acc0[3] + acc1[3]);
        }
    } else {
        // a block's share exceeds shared memory: the weights come in rounds of half the space
        int in_round = half_items, round = -1;
        for (int g = 0; g < my_groups; ++g) {
            float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
            const unsigned char* xa_at = xa_first;
            for (int j = 0; j < cpw; ++j) {
                if (in_round == half_items) {
                    ++round;
                    // the half just finished with takes the round after next (rounds 0 and 1 were asked for above)
                    if (round >= 1) request_into((round + 1) * half_items, half_items, pieces + (size_t)((round + 1) & 1) * half_items * THREADS);
                    asm volatile("cp.async.wait_group 1;" ::: "memory");  // all but the newest: this round's pieces are here
                    wp = pieces + (size_t)(round & 1) * half_items * THREADS + threadIdx.x;
                    in_round = 0;
                }
                chunk(*wp, xa_at, acc0, acc1);
                wp += THREADS;
                xa_at += WARPS * CHUNK * 2;
                ++in_round;
            }
            partial[(size_t)g * partial_step + threadIdx.x] =
                make_float4(acc0[0] + acc1[0], acc0[1] + acc1[1], acc0[2] + acc1[2], acc0[3] + acc1[3]);
        }
    }
    __syncthreads();
    finish();
}

}  // namespace

namespace {

int launch_gemv(GemvParams& p, cudaStream_t stream) {
    static int n_sms = 0;
    constexpr size_t SMEM_MAX = 200 * 1024;
    if (n_sms == 0) {
        int device = 0;
        cudaError_t err = cudaGetDevice(&device);
        if (err == cudaSuccess) err = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(gemv_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(gemv_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(gemv_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(gemv_mma_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(gemv_mma_kernel<1, false, X_REGS_LONG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (err == cudaSuccess) err = cudaFuncSetAttribute(gemv_mma_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (err != cudaSuccess) { n_sms = 0; return gk_fail(GK_CUDA_ERROR, "gemv: %s", cudaGetErrorString(err)); }
    }
    const int n_groups = (p.n + ROWS - 1) / ROWS;
    GK_REQUIRE(n_groups <= n_sms * MAX_GROUPS, "gemv: takes up to %d weight rows on this device, got %d", n_sms * MAX_GROUPS * ROWS, p.n);
    const int n_chunks = (p.k + CHUNK - 1) / CHUNK;
    int blocks = n_groups < n_sms ? n_groups : n_sms;
    // up to eight tokens, no norm on load: rows of up to 3,072 elements stay in registers too (if the block's weights
    // come in one round)
    const int cpw_all = (n_chunks + WARPS - 1) / WARPS;
    const bool long_registers = p.tokens <= 8 && p.norm_h == nullptr && cpw_all > X_REGS && cpw_all <= X_REGS_LONG &&
                                ((n_groups + blocks - 1) / blocks) * cpw_all <= ROUND_ITEMS;
    if (cpw_all > X_REGS && !long_registers) {
        // long K: every block copies all activations from L2, so fewer blocks with more groups each (as many
        // as fit in one round of weights) cost less there than they lose in the multiplications
        const int fit = ROUND_ITEMS / ((n_chunks + WARPS - 1) / WARPS);
        const int per_block = fit < 1 ? 1 : fit > MAX_GROUPS ? MAX_GROUPS : fit;
        const int fewer = (n_groups + per_block - 1) / per_block;
        if (fewer < blocks) blocks = fewer;
    }
    dim3 grid(blocks);
    const int groups_per_block = (n_groups + grid.x - 1) / grid.x;
    const int cpw = (n_chunks + WARPS - 1) / WARPS;
    const int items = groups_per_block * cpw;
    // rows of the activations in shared memory: the same number of chunks for every warp, and an odd multiple
    // of 64 bytes apart (none when they stay in registers: short K and all weights in one round)
    int x_stride = cpw * WARPS * CHUNK * 2;
    if (x_stride % 128 == 0) x_stride += 64;
    const bool x_in_registers = (cpw <= X_REGS || long_registers) && items <= ROUND_ITEMS;
    const size_t x_bytes = x_in_registers ? 0 : (size_t)(p.tokens > 8 ? 16 : 8) * x_stride;
    // weight pieces of as many chunks as fit beside them (a block whose share does not fit takes it in rounds and
    // keeps its partial sums in a buffer of their own)
    int round_items = items < ROUND_ITEMS ? items : ROUND_ITEMS;
    const size_t partial_bytes = (size_t)groups_per_block * THREADS * 16;
    if ((size_t)round_items * THREADS * 16 + x_bytes + (items > round_items ? partial_bytes : 0) > SMEM_MAX) {
        const size_t fixed = x_bytes + partial_bytes;
        GK_REQUIRE(fixed + THREADS * 16 <= SMEM_MAX, "gemv: k = %d with %d tokens needs %zu bytes of shared memory for the activations alone, more than %zu",
                   p.k, p.tokens, fixed, SMEM_MAX);
        round_items = (int)((SMEM_MAX - fixed) / (THREADS * 16));
    }
    if (items > round_items) {
        // in rounds anyway: as many pieces on their way as the block's shared memory holds
        const int most = (int)((SMEM_MAX - x_bytes - partial_bytes) / (THREADS * 16));
        round_items = items < most ? items : most;
    }
    const size_t smem = (size_t)round_items * THREADS * 16 + x_bytes + (items > round_items ? partial_bytes : 0);
    if (p.norm_h) {
        GK_REQUIRE(p.tokens <= 16 && x_in_registers, "gemv: the norm on load takes up to 16 tokens, k <= 1024 and a block's weights in one round; got %d tokens, k = %d, %d pieces a thread",
                   p.tokens, p.k, items);
        if (p.tokens > 8) gk_launch(gemv_mma_kernel<2, true>, grid, dim3(THREADS), smem, stream, p, round_items, x_stride);
        else gk_launch(gemv_mma_kernel<1, true>, grid, dim3(THREADS), smem, stream, p, round_items, x_stride);
        GK_CHECK_LAUNCH("gemv");
        return GK_OK;
    }
    if (p.tokens > 16) {
        GK_REQUIRE(x_in_registers && cpw >= 2, "gemv: 17 to 32 tokens need 257 <= k <= 1024 and a block's weights in one round; got k = %d, %d pieces a thread",
                   p.k, items);
        gk_launch(gemv_mma_kernel<4>, grid, dim3(THREADS), smem, stream, p, round_items, x_stride);
    } else if (p.tokens > 8) {
        gk_launch(gemv_mma_kernel<2>, grid, dim3(THREADS), smem, stream, p, round_items, x_stride);
    } else if (long_registers) {
        gk_launch(gemv_mma_kernel<1, false, X_REGS_LONG>, grid, dim3(THREADS), smem, stream, p, round_items, x_stride);
    } else {
        gk_launch(gemv_mma_kernel<1>, grid, dim3(THREADS), smem, stream, p, round_items, x_stride);
    }
    GK_CHECK_LAUNCH("gemv");
    return GK_OK;
}

}  // namespace

// OUT[t, :] = x[t, :] @ w^T for 1 to 16 tokens (17 to 32 where 257 <= k <= 1024) and up to 64 weight rows per SM; `w` [n, k] and `x` [tokens, k]
// bfloat16 with rows in steps of 8 elements (16 bytes); OUT bfloat16 or float32, [tokens, n], or with `swiglu`
// [tokens, n / 2] bfloat16 = silu(even rows) * odd rows.
GK_EXPORT int gk_gemv_bf16(const void* w, int n, int k, long long ldw, const void* x, int tokens, long long ldx, void* out,
                           int out_dtype, int swiglu, void* stream) {
    GK_REQUIRE(n > 0 && k > 0 && tokens > 0 && tokens <= 32, "gemv: takes 1 to 32 tokens and positive sizes; got %d tokens, n=%d k=%d",
               tokens, n, k);
    GK_REQUIRE(k % 8 == 0 && ldw % 8 == 0 && ldx % 8 == 0, "gemv: k and the row strides must be multiples of 8 elements; got k=%d ldw=%lld ldx=%lld",
               k, ldw, ldx);
    GK_REQUIRE(((uintptr_t)w & 15) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 3) == 0, "gemv: operands must be 16-byte aligned");
    GK_REQUIRE(GK_VALID_DTYPE(out_dtype), "gemv: bad output dtype");
    GK_REQUIRE(!swiglu || (n % 2 == 0 && out_dtype == GK_BF16), "gemv: the SwiGLU output stage needs an even number of rows and writes bfloat16");
    GemvParams p = {};
    p.w = (const __nv_bfloat16*)w;
    p.x = (const __nv_bfloat16*)x;
    p.out = out;
    p.n = n;
    p.k = k;
    p.tokens = tokens;
    p.ldw = ldw;
    p.ldx = ldx;
    p.ldo = swiglu ? n / 2 : n;
    p.out_f32 = out_dtype == GK_F32;
    p.swiglu = swiglu;
    return launch_gemv(p, (cudaStream_t)stream);
}

// The same product with the activations formed here as the RMSNorm of a 32-bit stream's rows (`norm_h` [tokens, k] with
// rows `ldh` apart, `norm_w` [k] float32 or bfloat16; up to 16 tokens, k <= 1024 and a block's weights in one round), and /
// or with the result added to a 32-bit stream (`resid` [tokens, n], rows `ldr` apart) instead of stored.  Either pointer
// may be null; with `norm_h` set `x` is not read, with `resid` set `out` is not written.
GK_EXPORT int gk_gemv_bf16_stream(const void* w, int n, int k, long long ldw, const void* x, int tokens, long long ldx, void* out,
                                  int out_dtype, int swiglu, const float* norm_h, long long ldh, const void* norm_w, int norm_w_bf16,
                                  float norm_eps, float* resid, long long ldr, void* stream) {
    GK_REQUIRE(n > 0 && k > 0 && tokens > 0 && tokens <= 32, "gemv: takes 1 to 32 tokens and positive sizes; got %d tokens, n=%d k=%d",
               tokens, n, k);
    GK_REQUIRE(k % 8 == 0 && ldw % 8 == 0, "gemv: k and the weights' row stride must be multiples of 8 elements; got k=%d ldw=%lld", k, ldw);
    GK_REQUIRE(((uintptr_t)w & 15) == 0, "gemv: the weights must be 16-byte aligned");
    GK_REQUIRE(norm_h != nullptr || (x != nullptr && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0), "gemv: activations must be 16-byte aligned rows");
    GK_REQUIRE(norm_h == nullptr || (norm_w != nullptr && ldh % 4 == 0 && ((uintptr_t)norm_h & 15) == 0 && ((uintptr_t)norm_w & 15) == 0 && norm_eps > 0.f),
               "gemv: the norm on load needs 16-byte aligned rows and weights and a positive eps");
    GK_REQUIRE(resid == nullptr || (!swiglu && ldr % 2 == 0 && ((uintptr_t)resid & 7) == 0), "gemv: the residual output stage needs 8-byte aligned rows and no SwiGLU");
    GK_REQUIRE(resid != nullptr || (out != nullptr && GK_VALID_DTYPE(out_dtype) && ((uintptr_t)out & 3) == 0), "gemv: bad output");
    GK_REQUIRE(!swiglu || (n % 2 == 0 && out_dtype == GK_BF16), "gemv: the SwiGLU output stage needs an even number of rows and writes bfloat16");
    GemvParams p = {};
    p.w = (const __nv_bfloat16*)w;
    p.x = (const __nv_bfloat16*)x;
    p.out = out;
    p.n = n;
    p.k = k;
    p.tokens = tokens;
    p.ldw = ldw;
    p.ldx = ldx;
    p.ldo = swiglu ? n / 2 : n;
    p.out_f32 = out_dtype == GK_F32;
    p.swiglu = swiglu;
    p.norm_h = norm_h;
    p.norm_w = norm_w;
    p.norm_w_bf16 = norm_w_bf16;
    p.norm_eps = norm_eps;
    p.ldh = ldh;
    p.resid = resid;
    p.ldr = ldr;
    return launch_gemv(p, (cudaStream_t)stream);
}
