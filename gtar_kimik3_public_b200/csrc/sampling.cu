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
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) mine = better(mine, Best{row[i], i});
    Best b = block_best(mine, scratch);
    if (threadIdx.x == 0) {
        if (parts == 1) out[r] = b.index == 0x7fffffff ? 0 : b.index;
        else partial[(size_t)r * parts + part] = b;
    }
}

__global__ void argmax_merge_kernel(const Best* __restrict__ partial, int parts, int* __restrict__ out) {
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
    if (threadIdx.x == 0) out[r] = mine.index == 0x7fffffff ? 0 : mine.index;
}

__global__ void sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab, float temperature,
                              int top_k, unsigned long long seed, const int* __restrict__ request_ids,
                              int* __restrict__ steps, int advance_steps, int* __restrict__ out) {
    __shared__ Best scratch[32];
    __shared__ unsigned int hist[256];
    __shared__ unsigned int sel_prefix, sel_remaining;
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * row_stride;

    unsigned int threshold_key = 0;  // keep everything
    if (top_k > 0 && top_k < vocab) {
        unsigned int prefix = 0, mask = 0;
        if (threadIdx.x == 0) sel_remaining = (unsigned)top_k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
                const unsigned int key = float_key(row[i]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                unsigned int remaining = sel_remaining, cum = 0;
                int chosen = 0;
                for (int b = 255; b >= 0; --b) {
                    if (cum + hist[b] >= remaining) {
                        chosen = b;
                        break;
                    }
                    cum += hist[b];
                }
                sel_remaining = remaining - cum;
                sel_prefix = prefix | ((unsigned)chosen << shift);
            }
            __syncthreads();
            prefix = sel_prefix;
            mask |= 255u << shift;
        }
        threshold_key = prefix;
    }

    const unsigned long long request = (unsigned long long)(unsigned int)request_ids[blockIdx.x];
    const unsigned long long step = (unsigned long long)(unsigned int)steps[blockIdx.x];
    Best mine{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (float_key(x) < threshold_key) continue;
        const float u = uniform_open(seed, request, step, (unsigned long long)i);
        const float g = -logf(-logf(u));
        mine = better(mine, Best{x / temperature + g, i});
    }
    Best b = block_best(mine, scratch);
    if (threadIdx.x == 0) {
        out[blockIdx.x] = b.index == 0x7fffffff ? 0 : b.index;
        if (advance_steps) steps[blockIdx.x] = (int)step + 1;
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
        gk_launch(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, (cudaStream_t)stream, (const Best*)scratch, parts, out);
        GK_CHECK_LAUNCH("argmax_merge");
    }
    return GK_OK;
}

GK_EXPORT int gk_sample(const float* logits, long long row_stride, int n_rows, int vocab, float temperature, int top_k,
                        unsigned long long seed, const int* request_ids, int* steps, int advance_steps, int* out,
                        void* stream) {
    GK_REQUIRE(n_rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", n_rows, vocab);
    GK_REQUIRE(temperature > 0.f, "sample: temperature must be positive (0 means greedy: call argmax)");
    GK_REQUIRE(top_k >= 0, "sample: top_k must be >= 0 (0 = off)");
    if (n_rows == 0) return GK_OK;
    gk_launch(sample_kernel, dim3(n_rows), dim3(1024), 0, (cudaStream_t)stream, logits, row_stride, vocab, temperature,
              top_k, seed, request_ids, steps, advance_steps, out);
    GK_CHECK_LAUNCH("sample");
    return GK_OK;
}
