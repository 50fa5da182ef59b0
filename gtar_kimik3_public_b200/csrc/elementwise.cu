// Token-wise kernels: embedding gather, residual add + RMSNorm, SwiGLU, and per-head
// q/k RMSNorm + rotary position encoding fused with the write of K and V into the paged cache.
//
// Formulas (reference): RMSNorm  w * (x * rsqrt(mean(x^2) + eps))   src/layers/rmsnorm.py:11-16
//                       rotary   x*cos + rotate_half(x)*sin         src/layers/rope.py:17-33
//                       SwiGLU   silu(gate) * up                    src/layers/swiglu.py:14
// All arithmetic is 32-bit; inputs and outputs may be bfloat16.

#include "common.cuh"

// ---------------------------------------------------------------- embedding gather
template <typename TT>
__global__ void embed_rows_kernel(const TT* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                  int hidden) {
    pdl_launch_dependents();  // the next kernel may take its place on the SMs and fetch what does not depend on this one
    pdl_wait();
    const int t = blockIdx.x;
    const TT* row = table + (size_t)ids[t] * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(row[i]);
}

GK_EXPORT int gk_embed_rows(const void* table, int table_dtype, const int* ids, float* out, int n_tokens, int hidden,
                            void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(table_dtype), "embed_rows: bad table dtype %d", table_dtype);
    GK_REQUIRE(n_tokens >= 0 && hidden > 0, "embed_rows: bad sizes n_tokens=%d hidden=%d", n_tokens, hidden);
    if (n_tokens == 0) return GK_OK;
    const int threads = hidden >= 1024 ? 256 : 128;
    GK_DISPATCH_DTYPE(table_dtype, TT, {
        gk_launch(embed_rows_kernel<TT>, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)stream, (const TT*)table, ids, out,
                  hidden);
    })
    GK_CHECK_LAUNCH("embed_rows");
    return GK_OK;
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row.  h (32-bit residual stream) gets `delta` added in place when
// `rows` is null; with `rows`, only the listed rows are read and h is left as it is (the
// last norm of a step, taken at the wanted positions only).
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T>
__device__ __forceinline__ void load2(const T* p, float (&v)[2]);
template <>
__device__ __forceinline__ void load2<float>(const float* p, float (&v)[2]) {
    const float2 f = *reinterpret_cast<const float2*>(p);
    v[0] = f.x; v[1] = f.y;
}
template <>
__device__ __forceinline__ void load2<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[2]) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    v[0] = f.x; v[1] = f.y;
}
template <typename T>
__device__ __forceinline__ void store2(T* p, const float (&v)[2]);
template <>
__device__ __forceinline__ void store2<float>(float* p, const float (&v)[2]) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
}
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[2]) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v[0], v[1]);
}

// VEC = 4: rows are read and written four elements at a time (hidden a multiple of 4, aligned rows).
// The sum of squares is formed element by element in the same order either way.
// KEEP > 0 (with VEC = 4): a thread keeps its KEEP groups of four elements of the row in registers between the sum of
// squares and the scaling (rows of up to 1024 * KEEP elements), and has fetched its share of the norm's weights
// before it waits for the kernel in front: those do not depend on it, and in a decode step this kernel is one link
// of a chain in which every trip to memory behind the wait counts.  The sum of squares is formed in the same order.
template <typename TD, typename TW, typename TO, int VEC, int KEEP = 0>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta, const TW* __restrict__ w,
                                   TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();  // the next kernel may take its place on the SMs and fetch what does not depend on this one
    if (KEEP > 0) {
        float wv[KEEP > 0 ? KEEP : 1][4];
#pragma unroll
        for (int it = 0; it < KEEP; ++it) {
            const int i = (threadIdx.x + it * blockDim.x) * 4;
            if (i < hidden) load4(w + i, wv[it]);
        }
        pdl_wait();
        const int src = rows ? rows[blockIdx.x] : blockIdx.x;
        float* hrow = h + (size_t)src * hidden;
        const bool has_delta = delta != nullptr;
        const TD* drow = delta + (size_t)src * hidden;
        TO* orow = out + (size_t)blockIdx.x * hidden;
        const bool write_back = (rows == nullptr) && has_delta;
        float v[KEEP > 0 ? KEEP : 1][4];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < KEEP; ++it) {
            const int i = (threadIdx.x + it * blockDim.x) * 4;
            if (i < hidden) {
                load4(hrow + i, v[it]);
                if (has_delta) {
                    float d[4];
                    load4(drow + i, d);
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[it][j] += d[j];
                }
                if (write_back) store4(hrow + i, v[it]);
#pragma unroll
                for (int j = 0; j < 4; ++j) ss += v[it][j] * v[it][j];
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
        for (int it = 0; it < KEEP; ++it) {
            const int i = (threadIdx.x + it * blockDim.x) * 4;
            if (i < hidden) {
                float o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = (v[it][j] * inv) * wv[it][j];
                store4(orow + i, o);
            }
        }
        return;
    }
    pdl_wait();
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* hrow = h + (size_t)src * hidden;
    const bool has_delta = delta != nullptr;
    const TD* drow = delta + (size_t)src * hidden;
    TO* orow = out + (size_t)blockIdx.x * hidden;
    const bool write_back = (rows == nullptr) && has_delta;
    float ss = 0.f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float v[4], d[4];
            load4(hrow + i, v);
            if (has_delta) {
                load4(drow + i, d);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] += d[j];
            }
            if (write_back) store4(hrow + i, v);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss += v[j] * v[j];
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = hrow[i];
            if (has_delta) v += to_float(drow[i]);
            if (write_back) hrow[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
            float v[4], d[4], wv[4];
            load4(hrow + i, v);
            if (has_delta && !write_back) {
                load4(drow + i, d);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] += d[j];
            }
            load4(w + i, wv);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = (v[j] * inv) * wv[j];
            store4(orow + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            float v = hrow[i];
            if (has_delta && !write_back) v += to_float(drow[i]);
            orow[i] = from_float<TO>((v * inv) * to_float(w[i]));
        }
    }
}

// A warp per row, for many rows of up to 1,024 elements.  Lane l stands for the threads l, 32 + l, ..., 224 + l of the
// block-per-row kernel above (KEEP = 1, 256 threads): the same four elements each, the same partial sums in the same
// order, the same butterfly over each group of 32 and then over the eight groups' sums.  A row's result is therefore
// bit for bit the same whichever of the two kernels the number of rows selects.  What it saves: three block barriers a
// row, and a lane has sixteen loads in flight where a thread of the other kernel has two.
template <typename TD, typename TW, typename TO>
__global__ void __launch_bounds__(256) add_rmsnorm_warp_rows_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                                                    const TW* __restrict__ w, TO* __restrict__ out,
                                                                    const int* __restrict__ rows, int n_rows, int hidden,
                                                                    float eps) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, row = blockIdx.x * 8 + (threadIdx.x >> 5);
    float wv[8][4];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int i = (32 * g + lane) * 4;
        if (i < hidden) load4(w + i, wv[g]);
    }
    pdl_wait();
    if (row >= n_rows) return;
    const int src = rows ? rows[row] : row;
    float* hrow = h + (size_t)src * hidden;
    const bool has_delta = delta != nullptr;
    const TD* drow = delta + (size_t)src * hidden;
    TO* orow = out + (size_t)row * hidden;
    const bool write_back = (rows == nullptr) && has_delta;
    float v[8][4], d[8][4];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int i = (32 * g + lane) * 4;
        if (i < hidden) {
            load4(hrow + i, v[g]);
            if (has_delta) load4(drow + i, d[g]);
        }
    }
    float sums[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int i = (32 * g + lane) * 4;
        float ss = 0.f;
        if (i < hidden) {
            if (has_delta) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[g][j] += d[g][j];
            }
            if (write_back) store4(hrow + i, v[g]);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss += v[g][j] * v[g][j];
        }
        sums[g] = ss;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int g = 0; g < 8; ++g) sums[g] += __shfl_xor_sync(0xffffffffu, sums[g], o);
    }
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) t = lane == g ? sums[g] : t;
    t = warp_sum(t);
    const float inv = 1.0f / sqrtf(t / (float)hidden + eps);
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const int i = (32 * g + lane) * 4;
        if (i < hidden) {
            float o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = (v[g][j] * inv) * wv[g][j];
            store4(orow + i, o);
        }
    }
}

GK_EXPORT int gk_add_rmsnorm(float* h, const void* delta, int delta_dtype, const void* weight, int weight_dtype,
                             void* out, int out_dtype, const int* rows, int n_out_rows, int hidden, float eps,
                             void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(delta_dtype) && GK_VALID_DTYPE(weight_dtype) && GK_VALID_DTYPE(out_dtype),
               "add_rmsnorm: bad dtype code");
    GK_REQUIRE(n_out_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", n_out_rows, hidden);
    GK_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
    if (n_out_rows == 0) return GK_OK;
    // A fixed block size: the order of the sum of squares must not depend on anything but the row.
    const int threads = 256;
    const bool vec = hidden % 4 == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)delta & 15) == 0 &&
                     ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0;
    cudaStream_t s = (cudaStream_t)stream;
    GK_DISPATCH_DTYPE(delta_dtype, TD, {
        GK_DISPATCH_DTYPE(weight_dtype, TW, {
            GK_DISPATCH_DTYPE(out_dtype, TO, {
                if (vec && hidden <= threads * 4 && n_out_rows >= 512)
                    gk_launch(add_rmsnorm_warp_rows_kernel<TD, TW, TO>, dim3((n_out_rows + 7) / 8), dim3(threads), 0, s, h,
                              (const TD*)delta, (const TW*)weight, (TO*)out, rows, n_out_rows, hidden, eps);
                else if (vec && hidden <= threads * 4)
                    gk_launch(add_rmsnorm_kernel<TD, TW, TO, 4, 1>, dim3(n_out_rows), dim3(threads), 0, s, h, (const TD*)delta,
                              (const TW*)weight, (TO*)out, rows, hidden, eps);
                else if (vec && hidden <= threads * 8)
                    gk_launch(add_rmsnorm_kernel<TD, TW, TO, 4, 2>, dim3(n_out_rows), dim3(threads), 0, s, h, (const TD*)delta,
                              (const TW*)weight, (TO*)out, rows, hidden, eps);
                else if (vec && hidden <= threads * 16)
                    gk_launch(add_rmsnorm_kernel<TD, TW, TO, 4, 4>, dim3(n_out_rows), dim3(threads), 0, s, h, (const TD*)delta,
                              (const TW*)weight, (TO*)out, rows, hidden, eps);
                else if (vec)
                    gk_launch(add_rmsnorm_kernel<TD, TW, TO, 4>, dim3(n_out_rows), dim3(threads), 0, s, h, (const TD*)delta,
                              (const TW*)weight, (TO*)out, rows, hidden, eps);
                else
                    gk_launch(add_rmsnorm_kernel<TD, TW, TO, 1>, dim3(n_out_rows), dim3(threads), 0, s, h, (const TD*)delta,
                              (const TW*)weight, (TO*)out, rows, hidden, eps);
            })
        })
    })
    GK_CHECK_LAUNCH("add_rmsnorm");
    return GK_OK;
}

// ---------------------------------------------------------------- SwiGLU on a packed row
// interleaved = 0: rows are [gate (I) | up (I)];  1: gate and up alternate (g0 u0 g1 u1 ...).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, long long total,
                              int interleaved) {
    pdl_launch_dependents();  // the next kernel may take its place on the SMs and fetch what does not depend on this one
    pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long t = idx / inter;
    const int i = (int)(idx - t * inter);
    const T* row = gate_up + t * 2 * inter;
    const float g = to_float(interleaved ? row[2 * i] : row[i]);
    const float u = to_float(interleaved ? row[2 * i + 1] : row[inter + i]);
    const float act = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(act * u);
}

GK_EXPORT int gk_swiglu(const void* gate_up, void* out, int dtype, int n_tokens, int inter, int interleaved,
                        void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype), "swiglu: bad dtype %d", dtype);
    GK_REQUIRE(n_tokens >= 0 && inter > 0, "swiglu: bad sizes");
    const long long total = (long long)n_tokens * inter;
    if (total == 0) return GK_OK;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    GK_REQUIRE(blocks < 2147483647LL, "swiglu: too many elements");
    GK_DISPATCH_DTYPE(dtype, T, {
        gk_launch(swiglu_kernel<T>, dim3((unsigned)blocks), dim3(threads), 0, (cudaStream_t)stream, (const T*)gate_up,
                  (T*)out, inter, total, interleaved);
    })
    GK_CHECK_LAUNCH("swiglu");
    return GK_OK;
}

// ---------------------------------------------------------------- q/k norm + rotary + cache write
// One warp per (token, head) of the packed projection row [q heads | k heads | v heads].
//   q head: normalise, rotate, store to q_out[token, head, :]
//   k head: normalise, rotate, store to the token's place in the K pages
//   v head: copy to the token's place in the V pages
// Page of token: block_table[slot, pos / page_size]; place in page: pos % page_size.
// Pages are laid out [page, kv_head, page_size, head_dim].
// `use_norm` = 0 skips the normalisation, `cos_table` = null skips the rotation, so that the
// same kernel serves a mixer without q/k norm or without positions; `k_pages` = null writes no
// keys and values (a layer that reads the storage another layer fills).
template <typename T, typename TW>
__global__ void qk_norm_rope_write_kernel(const T* __restrict__ qkv, const TW* __restrict__ wq, const TW* __restrict__ wk,
                                          const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                          const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                          const int* __restrict__ slots, const int* __restrict__ block_table,
                                          T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                          int n_tokens, int n_q, int n_kv, int head_dim, int max_pages, int page_size,
                                          float eps, int use_norm) {
    pdl_launch_dependents();  // the next kernel may take its place on the SMs and fetch what does not depend on this one
    pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const long long wid = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int n_heads = n_q + 2 * n_kv;
    if (wid >= (long long)n_tokens * n_heads) return;
    const int t = (int)(wid / n_heads);
    const int head = (int)(wid - (long long)t * n_heads);
    const size_t src = ((size_t)t * n_heads + head) * head_dim;
    const int pos = tok_pos[t];
    T* dst;
    const TW* w = nullptr;
    bool rotate = true;
    if (head < n_q) {
        dst = q_out + ((size_t)t * n_q + head) * head_dim;
        w = wq;
    } else {
        if (k_pages == nullptr) return;  // this layer reads another layer's keys and values
        const int hk = head < n_q + n_kv ? head - n_q : head - n_q - n_kv;
        const int slot = slots[tok_seq[t]];
        const int page = block_table[(size_t)slot * max_pages + pos / page_size];
        const size_t at = (((size_t)page * n_kv + hk) * page_size + (pos % page_size)) * head_dim;
        if (head < n_q + n_kv) {
            dst = k_pages + at;
            w = wk;
        } else {
            dst = v_pages + at;
            rotate = false;
        }
    }
    const T* in = qkv + src;
    if (!rotate) {
        if (head_dim % 4 == 0) {  // rows start on 8-byte boundaries (head_dim even, so offsets are multiples of it)
            for (int i = lane * 4; i < head_dim; i += 128) {
                float v[4];
                load4(in + i, v);
                store4(dst + i, v);
            }
        } else {
            for (int i = lane; i < head_dim; i += 32) dst[i] = in[i];
        }
        return;
    }
    const int half = head_dim >> 1;
    if (half % 2 == 0) {
        // two neighbouring pairs (p, p + half), (p + 1, p + 1 + half) per lane and iteration
        float inv = 1.0f;
        if (use_norm) {
            float ss = 0.f;
            for (int p = lane * 2; p < half; p += 64) {
                float a[2], b[2];
                load2(in + p, a);
                load2(in + p + half, b);
                ss += a[0] * a[0] + b[0] * b[0];
                ss += a[1] * a[1] + b[1] * b[1];
            }
            ss = warp_sum(ss);
            inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
        }
        for (int p = lane * 2; p < half; p += 64) {
            float a[2], b[2], ra[2], rb[2];
            load2(in + p, a);
            load2(in + p + half, b);
            if (use_norm) {
                float wa[2], wb[2];
                load2(w + p, wa);
                load2(w + p + half, wb);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    a[j] = (a[j] * inv) * wa[j];
                    b[j] = (b[j] * inv) * wb[j];
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                ra[j] = a[j];
                rb[j] = b[j];
            }
            if (cos_table) {
                float c[2], sn[2];
                load2(cos_table + (size_t)pos * half + p, c);
                load2(sin_table + (size_t)pos * half + p, sn);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    ra[j] = a[j] * c[j] - b[j] * sn[j];
                    rb[j] = b[j] * c[j] + a[j] * sn[j];
                }
            }
            store2(dst + p, ra);
            store2(dst + p + half, rb);
        }
        return;
    }
    float inv = 1.0f;
    if (use_norm) {
        float ss = 0.f;
        for (int p = lane; p < half; p += 32) {
            const float a = to_float(in[p]), b = to_float(in[p + half]);
            ss += a * a + b * b;
        }
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)head_dim + eps);
    }
    for (int p = lane; p < half; p += 32) {
        float a = to_float(in[p]), b = to_float(in[p + half]);
        if (use_norm) {
            a = (a * inv) * to_float(w[p]);
            b = (b * inv) * to_float(w[p + half]);
        }
        float ra = a, rb = b;
        if (cos_table) {
            const float c = cos_table[(size_t)pos * half + p], s = sin_table[(size_t)pos * half + p];
            ra = a * c - b * s;
            rb = b * c + a * s;
        }
        dst[p] = from_float<T>(ra);
        dst[p + half] = from_float<T>(rb);
    }
}

// E (a multiple of 4) consecutive elements, four at a time
template <int E, typename T>
__device__ __forceinline__ void load_run(const T* p, float (&v)[E]) {
#pragma unroll
    for (int i = 0; i < E; i += 4) {
        float part[4];
        load4(p + i, part);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i + j] = part[j];
    }
}
template <int E, typename T>
__device__ __forceinline__ void store_run(T* p, const float (&v)[E]) {
#pragma unroll
    for (int i = 0; i < E; i += 4) {
        const float part[4] = {v[i], v[i + 1], v[i + 2], v[i + 3]};
        store4(p + i, part);
    }
}

// The same for bfloat16 rows and head sizes 64 and 128 with eight lanes per (token, head): a lane takes HD / 16
// neighbouring elements of the row's first half and their partners of the rotation in the second half, everything
// it needs (the row, the norm weights, the token's row of the cos and sin tables) is asked for at once, and the
// row stays in registers between the sum of squares and the scaling.  With a warp per (token, head) and four
// bytes a lane and load, 2,048 tokens x 32 heads were seven rounds of warps, each a chain of five trips to memory.
template <int HD, typename TW>
__global__ void __launch_bounds__(256) qk_norm_rope_write_wide_kernel(
    const __nv_bfloat16* __restrict__ qkv, const TW* __restrict__ wq, const TW* __restrict__ wk,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ slots, const int* __restrict__ block_table,
    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
    int n_tokens, int n_q, int n_kv, int max_pages, int page_size, float eps, int use_norm) {
    constexpr int E = HD / 16, HALF = HD / 2;  // elements a lane takes of each half of the row
    pdl_launch_dependents();
    pdl_wait();
    const int n_heads = n_q + 2 * n_kv;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 3) + (threadIdx.x >> 3);
    const int sub = threadIdx.x & 7;
    const bool valid = item < (long long)n_tokens * n_heads;  // every lane stays for the shuffles
    const int t = valid ? (int)(item / n_heads) : 0;
    const int head = valid ? (int)(item - (long long)t * n_heads) : 0;
    const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
    const int pos = tok_pos[t];
    __nv_bfloat16* dst = nullptr;
    if (!valid) {
    } else if (is_q) {
        dst = q_out + ((size_t)t * n_q + head) * HD;
    } else if (k_pages != nullptr) {
        const int hk = is_k ? head - n_q : head - n_q - n_kv;
        const int page = block_table[(size_t)slots[tok_seq[t]] * max_pages + pos / page_size];
        dst = (is_k ? k_pages : v_pages) + (((size_t)page * n_kv + hk) * page_size + (pos % page_size)) * HD;
    }
    const __nv_bfloat16* in = qkv + ((size_t)t * n_heads + head) * HD + sub * E;
    float a[E], b[E];
    load_run<E>(in, a);
    load_run<E>(in + HALF, b);
    if (is_q || is_k) {
        float wa[E], wb[E], c[E], sn[E];
        const TW* w = is_q ? wq : wk;
        if (use_norm) {
            load_run<E>(w + sub * E, wa);
            load_run<E>(w + HALF + sub * E, wb);
        }
        if (cos_table) {
            load_run<E>(cos_table + (size_t)pos * HALF + sub * E, c);
            load_run<E>(sin_table + (size_t)pos * HALF + sub * E, sn);
        }
        if (use_norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < E; ++i) ss += a[i] * a[i] + b[i] * b[i];
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
            for (int i = 0; i < E; ++i) {
                a[i] = (a[i] * inv) * wa[i];
                b[i] = (b[i] * inv) * wb[i];
            }
        }
        if (cos_table) {
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const float x = a[i], y = b[i];
                a[i] = x * c[i] - y * sn[i];
                b[i] = y * c[i] + x * sn[i];
            }
        }
    }
    if (dst) {
        store_run<E>(dst + sub * E, a);
        store_run<E>(dst + HALF + sub * E, b);
    }
}

GK_EXPORT int gk_qk_norm_rope_write(const void* qkv, int dtype,
                                    const void* wq, const void* wk, int weight_dtype, const float* cos_table,
                                    const float* sin_table, int table_positions, const int* tok_pos,
                                    const int* tok_seq, const int* slots, const int* block_table, void* q_out,
                                    void* k_pages, void* v_pages, int n_tokens, int n_q, int n_kv, int head_dim,
                                    int max_pages, int page_size, float eps, int use_norm, int max_position,
                                    void* stream) {
    GK_REQUIRE(GK_VALID_DTYPE(dtype) && GK_VALID_DTYPE(weight_dtype), "qk_norm_rope_write: bad dtype code");
    GK_REQUIRE(n_tokens >= 0 && n_q > 0 && n_kv > 0 && head_dim > 0 && head_dim % 2 == 0,
               "qk_norm_rope_write: bad sizes n_q=%d n_kv=%d head_dim=%d", n_q, n_kv, head_dim);
    GK_REQUIRE(page_size > 0 && max_pages > 0, "qk_norm_rope_write: bad page geometry");
    GK_REQUIRE(!use_norm || (wq && wk), "qk_norm_rope_write: norm weights missing");
    GK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "qk_norm_rope_write: cos and sin tables go together");
    GK_REQUIRE(cos_table == nullptr || max_position < table_positions,
               "qk_norm_rope_write: position %d is beyond the rotary table (%d positions)", max_position,
               table_positions);
    if (n_tokens == 0) return GK_OK;
    const int threads = 128;
    const long long warps = (long long)n_tokens * (n_q + 2 * n_kv);
    const long long blocks = (warps + 3) / 4;
    GK_REQUIRE(blocks < 2147483647LL, "qk_norm_rope_write: too many tokens");
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)k_pages & 15) == 0 &&
                         ((uintptr_t)v_pages & 15) == 0 && ((uintptr_t)wq & 15) == 0 && ((uintptr_t)wk & 15) == 0 &&
                         ((uintptr_t)cos_table & 15) == 0 && ((uintptr_t)sin_table & 15) == 0;
    if (dtype == GK_BF16 && (head_dim == 64 || head_dim == 128) && aligned) {
        const long long wide_blocks = (warps + 31) / 32;  // 32 (token, head) items per block of 256 threads
        GK_DISPATCH_DTYPE(weight_dtype, TW, {
            if (head_dim == 128)
                gk_launch(qk_norm_rope_write_wide_kernel<128, TW>, dim3((unsigned)wide_blocks), dim3(256), 0, s,
                          (const __nv_bfloat16*)qkv, (const TW*)wq, (const TW*)wk, cos_table, sin_table, tok_pos, tok_seq, slots,
                          block_table, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, n_tokens, n_q,
                          n_kv, max_pages, page_size, eps, use_norm);
            else
                gk_launch(qk_norm_rope_write_wide_kernel<64, TW>, dim3((unsigned)wide_blocks), dim3(256), 0, s,
                          (const __nv_bfloat16*)qkv, (const TW*)wq, (const TW*)wk, cos_table, sin_table, tok_pos, tok_seq, slots,
                          block_table, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, n_tokens, n_q,
                          n_kv, max_pages, page_size, eps, use_norm);
        })
        GK_CHECK_LAUNCH("qk_norm_rope_write");
        return GK_OK;
    }
    GK_DISPATCH_DTYPE(dtype, T, {
        GK_DISPATCH_DTYPE(weight_dtype, TW, {
            gk_launch(qk_norm_rope_write_kernel<T, TW>, dim3((unsigned)blocks), dim3(threads), 0, s, (const T*)qkv,
                      (const TW*)wq, (const TW*)wk, cos_table, sin_table, tok_pos, tok_seq, slots, block_table, (T*)q_out,
                      (T*)k_pages, (T*)v_pages, n_tokens, n_q, n_kv, head_dim, max_pages, page_size, eps, use_norm);
        })
    })
    GK_CHECK_LAUNCH("qk_norm_rope_write");
    return GK_OK;
}
