// What the decode attention kernels share: the description of the step they may do themselves before attending.
#pragma once

#include "attention_mma.cuh"

namespace attn {

// Optional fusion of the step before attention: with `qkv` set, the kernel takes the packed
// projection row of each sequence's new token [q heads | k heads | v heads], applies the per-head
// RMSNorm (weights `wq`, `wk`, float32 or bfloat16) and the rotation (tables [position][D/2]) itself,
// uses the result as its queries, and — unless `write_kv` is 0 — writes the new token's key and
// value into the page that holds it (and patches the copy of that page it has in shared memory).
// Formulas: src/layers/rmsnorm.py:11-16, src/layers/rope.py:17-33, order src/layers/attention.py:82-89.
struct FusedQkv {
    const __nv_bfloat16* qkv;   // null: queries come from `q`, keys and values are in the cache already
    const void* wq;
    const void* wk;
    int weights_bf16;           // dtype of wq / wk
    int use_norm;
    float eps;
    const float* cos_table;     // null: no rotation
    const float* sin_table;
    int write_kv;
};

__device__ __forceinline__ float weight_at(const void* w, int bf16, int i) {
    return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]) : reinterpret_cast<const float*>(w)[i];
}

}  // namespace attn
