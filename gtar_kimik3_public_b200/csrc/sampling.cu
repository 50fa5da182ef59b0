// Token choice from 32-bit logits: greedy argmax, and temperature (+ top-k) sampling.
//
// The reference samples with  logits / temperature -> optional top-k mask (values below the
// k-th largest become -inf, ties at the threshold survive) -> softmax -> multinomial
// (src/engine.py:5-12).  Here the multinomial draw is done with the Gumbel-max rule, which
// draws from exactly the same distribution: token = argmax_i (logit_i / T + g_i),
// g_i = -log(-log(u_i)), u_i uniform in (0,1).  u_i comes from a counter-based generator keyed by
// (seed, request, step, i), so a request's tokens do not depend on what else is in the batch
// and a host implementation can reproduce them.
//
// Ties go to the lowest index in both kernels.

#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30;
    x *= 0xBF58476D1CE4E5B9ULL;
    x ^= x >> 27;
    x *= 0x94D049BB133111EBULL;
    x ^= x >> 31;
    return x;
}

__device__ __forceinline__ float uniform_open(unsigned long long seed, unsigned long long request,
                                              unsigned long long step, unsigned long long index) {
    unsigned long long x = seed * 0x9E3779B97F4A7C15ULL + request * 0xBF58476D1CE4E5B9ULL +
                           step * 0x94D049BB133111EBULL + index;
    x = mix64(x);
    return ((float)(x >> 41) + 0.5f) * (1.0f / 8388608.0f);
}

// Order-preserving map float -> uint32 (larger float, larger key).
__device__ __forceinline__ unsigned int float_key(float f) {
    unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct Best {
    float value;
    int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}

__device__ __forceinline__ Best block_best(Best mine, Best* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.value = __shfl_xor_sync(0xffffffffu, mine.value, o);
        other.index = __shfl_xor_sync(0xffffffffu, mine.index, o);
        mine = better(mine, other);
    }
    if (lane == 0) scratch[warp] = mine;
    __syncthreads();
    if (warp == 0) {
        Best t = lane < n_warps ? scratch[lane] : Best{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.value = __shfl_xor_sync(0xffffffffu, t.value, o);
            other.index = __shfl_xor_sync(0xffffffffu, t.index, o);
            t = better(t, other);
        }
        if (lane == 0) scratch[0] = t;
    }
    __syncthreads();
    return scratch[0];
}

// Every element of row[begin .. end) goes to `visit(value, index)`: the elements up to the first 16-byte
// boundary one by one, then four at a time with several loads of a thread in flight (a thread that waits for
// each element before it asks for the next scans at a few GB/s), then the rest.
template <typename Visit>
__device__ __forceinline__ void scan_slice(const float* __restrict__ row, int begin, int end, Visit visit) {
    const int lead = min((int)((16 - ((uintptr_t)(row + begin) & 15)) & 15) / 4, max(end - begin, 0));
    if ((int)threadIdx.x < lead) visit(row[begin + threadIdx.x], begin + (int)threadIdx.x);
    const int vec_begin = begin + lead, n_vec = max(end - vec_begin, 0) / 4;
    const float4* vec = reinterpret_cast<const float4*>(row + vec_begin);
    constexpr int IN_FLIGHT = 4;
    for (int v0 = threadIdx.x; v0 < n_vec; v0 += blockDim.x * IN_FLIGHT) {
        float4 got[IN_FLIGHT];
#pragma unroll
        for (int u = 0; u < IN_FLIGHT; ++u) {
            const int v = v0 + u * (int)blockDim.x;
            if (v < n_vec) got[u] = vec[v];
        }
#pragma unroll
        for (int u = 0; u < IN_FLIGHT; ++u) {
            const int v = v0 + u * (int)blockDim.x;
            if (v < n_vec) {
                const int i = vec_begin + 4 * v;
                visit(got[u].x, i);
                visit(got[u].y, i + 1);
                visit(got[u].z, i + 2);
                visit(got[u].w, i + 3);
            }
        }
    }
    for (int i = vec_begin + 4 * n_vec + threadIdx.x; i < end; i += blockDim.x) visit(row[i], i);
}

// Grid (parts, rows): block (p, r) scans its slice of row r and leaves its best (value, index) in
// `partial[r * parts + p]`; with one part it writes the answer itself.
__global__ void argmax_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                              int* __restrict__ out, Best* __restrict__ partial) {
    __shared__ Best scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int parts = gridDim.x, part = blockIdx.x, r = blockIdx.y;
    const float* row = logits + (size_t)r * row_stride;
    const int per = (vocab + parts - 1) / parts;
    const int begin = part * per, end = min(begin + per, vocab);
    Best mine{-INFINITY, 0x7fffffff};
    scan_slice(row, begin, end, [&](float x, int i) { mine = better(mine, Best{x, i}); });
    Best b = block_best(mine, scratch);
    if (threadIdx.x == 0) {
        if (parts == 1) out[r] = b.index == 0x7fffffff ? 0 : b.index;
        else partial[(size_t)r * parts + part] = b;
    }
}

// One warp per row picks among the parts' results; `steps` (sampling only) is advanced here, once per row.
__global__ void best_merge_kernel(const Best* __restrict__ partial, int parts, int* __restrict__ out, int* __restrict__ steps) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    Best mine{-INFINITY, 0x7fffffff};
    for (int p = threadIdx.x; p < parts; p += 32) mine = better(mine, partial[(size_t)r * parts + p]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.value = __shfl_xor_sync(0xffffffffu, mine.value, o);
        other.index = __shfl_xor_sync(0xffffffffu, mine.index, o);
        mine = better(mine, other);
    }
    if (threadIdx.x == 0) {
        out[r] = mine.index == 0x7fffffff ? 0 : mine.index;
        if (steps) steps[r] += 1;
    }
}

// The key of the row's k-th largest logit: a radix select over the order-preserving keys, eight bits a pass, each
// pass a scan of the row.  A cluster of up to SELECT_BLOCKS blocks shares a row: every block counts its slice into a
// histogram in its own shared memory, and after a cluster barrier every block adds up all of them through
// distributed shared memory and comes to the same bin.  Two histograms in turn, so that a block may clear the next
// one while others still read this one.  Lanes that meet in a bin add to it once.
constexpr int SELECT_BLOCKS = 8;

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(1024, 1) top_k_threshold_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                                                                  int top_k, unsigned int* __restrict__ threshold) {
    __shared__ unsigned int hist[2][256];
    __shared__ unsigned int total[256];
    __shared__ unsigned int sel_prefix, sel_remaining;
    pdl_launch_dependents();
    pdl_wait();
    uint32_t n_ranks;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n_ranks));
    const int r = blockIdx.x / (int)n_ranks, rank = blockIdx.x % (int)n_ranks;  // the cluster's blocks are consecutive
    const float* row = logits + (size_t)r * row_stride;
    const int per = (vocab + (int)n_ranks - 1) / (int)n_ranks;
    const int begin = rank * per, end = min(begin + per, vocab);
    const int lane = threadIdx.x & 31;
    unsigned int prefix = 0, mask = 0;
    if (threadIdx.x == 0) sel_remaining = (unsigned)top_k;
    if (threadIdx.x < 256) hist[0][threadIdx.x] = 0;
    __syncthreads();
    int pass = 0;
    for (int shift = 24; shift >= 0; shift -= 8, ++pass) {
        unsigned int* mine = hist[pass & 1];
        scan_slice(row, begin, end, [&](float x, int) {
            const unsigned int key = float_key(x);
            if ((key & mask) == prefix) {
                const unsigned int bin = (key >> shift) & 255u;
                const unsigned int same = __match_any_sync(__activemask(), bin);
                if (lane == __ffs(same) - 1) atomicAdd(&mine[bin], (unsigned)__popc(same));
            }
        });
        cluster_barrier();  // every block's counts of this pass are complete
        if (threadIdx.x < 256) {
            const uint32_t local = (uint32_t)__cvta_generic_to_shared(&mine[threadIdx.x]);
            unsigned int sum = 0;
#pragma unroll
            for (int b = 0; b < SELECT_BLOCKS; ++b) {
                if (b < (int)n_ranks) {
                    uint32_t remote;
                    unsigned int v;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(b));
                    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
                    sum += v;
                }
            }
            total[threadIdx.x] = sum;
            hist[(pass + 1) & 1][threadIdx.x] = 0;  // last read a pass ago, before the barrier above
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // from the highest bin down: lane l sums bins 255 - 8l .. 248 - 8l, the warp finds the lane in whose
            // bins the count reaches what is still wanted, and that lane finds the bin
            const unsigned int remaining = sel_remaining;
            unsigned int own = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) own += total[255 - 8 * lane - j];
            unsigned int upto = own;  // inclusive sum over lanes 0 .. lane
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int other = __shfl_up_sync(0xffffffffu, upto, o);
                if (lane >= o) upto += other;
            }
            const unsigned int reached = __ballot_sync(0xffffffffu, upto >= remaining);
            const int owner = reached ? __ffs(reached) - 1 : 31;
            if (lane == owner) {
                unsigned int cum = upto - own;
                int chosen = 248 - 8 * lane;
                for (int j = 0; j < 8; ++j) {
                    const int b = 255 - 8 * lane - j;
                    if (cum + total[b] >= remaining) {
                        chosen = b;
                        break;
                    }
                    cum += total[b];
                }
                sel_remaining = remaining - cum;
                sel_prefix = prefix | ((unsigned)chosen << shift);
            }
        }
        __syncthreads();
        prefix = sel_prefix;
        mask |= 255u << shift;
    }
    if (threadIdx.x == 0 && rank == 0) threshold[r] = prefix;
    cluster_barrier();  // nobody leaves while its histogram may still be read
}

// Grid (parts, rows): the best of  logit / T + Gumbel noise  over the block's slice of the row, among the logits
// whose key reaches the row's threshold (`threshold` null: all).
__global__ void sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, float temperature,
                              const unsigned int* __restrict__ threshold, unsigned long long seed,
                              const int* __restrict__ request_ids, int* __restrict__ steps, int advance_steps,
                              int* __restrict__ out, Best* __restrict__ partial) {
    __shared__ Best scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int parts = gridDim.x, part = blockIdx.x, r = blockIdx.y;
    const float* row = logits + (size_t)r * row_stride;
    const int per = (vocab + parts - 1) / parts;
    const int begin = part * per, end = min(begin + per, vocab);
    const unsigned int threshold_key = threshold ? threshold[r] : 0u;
    const unsigned long long request = (unsigned long long)(unsigned int)request_ids[r];
    const unsigned long long step = (unsigned long long)(unsigned int)steps[r];
    Best mine{-INFINITY, 0x7fffffff};
    scan_slice(row, begin, end, [&](float x, int i) {
        if (float_key(x) < threshold_key) return;
        const float u = uniform_open(seed, request, step, (unsigned long long)i);
        const float g = -logf(-logf(u));
        mine = better(mine, Best{x / temperature + g, i});
    });
    Best b = block_best(mine, scratch);
    if (threadIdx.x == 0) {
        if (parts == 1) {
            out[r] = b.index == 0x7fffffff ? 0 : b.index;
            if (advance_steps) steps[r] = (int)step + 1;
        } else {
            partial[(size_t)r * parts + part] = b;
        }
    }
}

}  // namespace

// `scratch` (8 bytes * n_rows * parts) is needed when `parts` > 1: a row is then scanned by that many
// blocks and a second kernel picks among their results (ties still go to the lowest index).
GK_EXPORT int gk_argmax(const float* logits, long long row_stride, int n_rows, int vocab, int* out, int parts,
                        void* scratch, void* stream) {
    GK_REQUIRE(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "argmax: bad sizes rows=%d vocab=%d", n_rows, vocab);
    GK_REQUIRE(parts >= 1 && parts <= 1024 && n_rows <= 65535, "argmax: bad split %d of %d rows", parts, n_rows);
    GK_REQUIRE(parts == 1 || scratch, "argmax: scratch is needed when a row is split");
    if (n_rows == 0) return GK_OK;
    gk_launch(argmax_kernel, dim3(parts, n_rows), dim3(parts == 1 ? 1024 : 256), 0, (cudaStream_t)stream, logits,
              row_stride, vocab, out, (Best*)scratch);
    GK_CHECK_LAUNCH("argmax");
    if (parts > 1) {
        gk_launch(best_merge_kernel, dim3(n_rows), dim3(32), 0, (cudaStream_t)stream, (const Best*)scratch, parts, out, (int*)nullptr);
        GK_CHECK_LAUNCH("argmax_merge");
    }
    return GK_OK;
}

// `scratch`: 4 bytes * n_rows for the top-k thresholds, then 8 bytes * n_rows * parts for the parts' results.
GK_EXPORT int gk_sample(const float* logits, long long row_stride, int n_rows, int vocab, float temperature, int top_k,
                        unsigned long long seed, const int* request_ids, int* steps, int advance_steps, int* out,
                        int parts, void* scratch, void* stream) {
    GK_REQUIRE(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
    GK_REQUIRE(temperature > 0.f, "sample: temperature must be positive (0 means greedy: call argmax)");
    GK_REQUIRE(top_k >= 0, "sample: top_k must be >= 0 (0 = off)");
    GK_REQUIRE(parts >= 1 && parts <= 1024 && n_rows <= 65535, "sample: bad split %d of %d rows", parts, n_rows);
    const bool select = top_k > 0 && top_k < vocab;
    GK_REQUIRE((parts == 1 && !select) || scratch, "sample: scratch is needed for top-k and when a row is split");
    if (n_rows == 0) return GK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    unsigned int* threshold = select ? (unsigned int*)scratch : nullptr;
    Best* partial = (Best*)((char*)scratch + 8 * (((size_t)n_rows + 1) / 2));  // 8-byte aligned, after the thresholds
    if (select) {
        // as many blocks a row as leaves all of them on the GPU at once (two of 1,024 threads fit an SM)
        static int n_sms = 0;
        if (n_sms == 0) {
            int device = 0;
            if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) n_sms = 148;
        }
        int blocks = SELECT_BLOCKS;
        while (blocks > 1 && (long long)n_rows * blocks > 2LL * n_sms) blocks /= 2;
        gk_launch_cluster(top_k_threshold_kernel, dim3(n_rows * blocks), dim3(1024), 0, s, dim3(blocks, 1, 1), logits, row_stride,
                          vocab, top_k, threshold);
        GK_CHECK_LAUNCH("top_k_threshold");
    }
    gk_launch(sample_kernel, dim3(parts, n_rows), dim3(256), 0, s, logits, row_stride, vocab, temperature,
              (const unsigned int*)threshold, seed, request_ids, steps, advance_steps, out, partial);
    GK_CHECK_LAUNCH("sample");
    if (parts > 1) {
        gk_launch(best_merge_kernel, dim3(n_rows), dim3(32), 0, s, (const Best*)partial, parts, out, advance_steps ? steps : (int*)nullptr);
        GK_CHECK_LAUNCH("sample_merge");
    }
    return GK_OK;
}
