// Kernel parameter blocks, filled by api.cu.
#pragma once
#include "common.cuh"

namespace fa {

constexpr int kAttnThreads = 384;  // 3 warpgroups: two compute groups, one producer / MMA group
constexpr int kFwdThreads = kAttnThreads;

struct FwdParams {
    float* lse;  // [B, H, Mpad], log2 domain
    MaskArgs mask;
    int H, B, G;
    int gh;            // heads per scheduling group
    int by_length;     // take the blocks of a head in the plan's sorted order (few items per CTA)
    float scale_log2;  // sm_scale * log2(e)
    int* status;
    long long wait_limit;  // SM clocks a bounded wait may last
};

struct DeltaParams {
    OutTensor o, d_o;
    float* delta;  // [B, H, Mpad]
    int B, H, M, D;
    int64_t Mpad;
    bool bf16;
};

struct DkdvParams {
    const float* lse;    // [B, H, Mpad]
    const float* delta;  // [B, H, Mpad]
    MaskArgs mask;
    int B, H, Hk, G;
    int gh;  // kv heads per scheduling group
    int by_length;  // take the blocks of a head in the plan's sorted order (few items per CTA)
    float scale_log2, sm_scale;
    int* status;
    long long wait_limit;  // SM clocks a bounded wait may last
};

struct DqParams {
    const float* lse;
    const float* delta;
    MaskArgs mask;
    int B, H, G;
    int gh;  // heads per scheduling group
    int by_length;  // take the blocks of a head in the plan's sorted order (few items per CTA)
    float scale_log2, sm_scale;
    int* status;
    long long wait_limit;  // SM clocks a bounded wait may last
};

// fp32 kernels (attn_f32.cu): plain pointers and element strides, no tensor maps
struct F32Tensor {
    float* ptr;
    int64_t sb, sh, sl;  // element strides; the D stride is 1
};

struct F32Params {
    F32Tensor q, k, v, o, d_o, dq, dk, dv;
    float* lse;    // [B, H, Mpad], natural log-sum-exp of the scaled scores; -inf for a row without keys
    float* delta;  // [B, H, Mpad]
    MaskArgs mask;
    int B, H, Hk, G;
    float scale;
};

// Ordered compaction of per-tile flags (list[i] = flags of tile lo+i) into the visited list:
// entry = (i) | flags << 10. One warp; returns the number of visited tiles.
__device__ __forceinline__ int compact_visit_list(uint16_t* list, int n, int lane) {
    int T = 0;
    for (int base = 0; base < n; base += 32) {
        const int i = base + lane;
        const uint32_t f = (i < n) ? list[i] : 0u;
        const uint32_t m = __ballot_sync(0xffffffffu, (f & TILE_VISIT) != 0);
        __syncwarp();
        if (f & TILE_VISIT) list[T + __popc(m & ((1u << lane) - 1u))] = uint16_t(uint32_t(i) | (f << 10));
        T += __popc(m);
        __syncwarp();
    }
    return T;
}

}  // namespace fa
