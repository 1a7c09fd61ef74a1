// Mask plan: 32-bit id codes, per-block id min/max, per-block visit ranges; and the debug
// kernel that materialises keep / tile-class decisions with the attention kernels' own
// predicate. The reference has no counterpart (it evaluates every tile inside the causal
// bound, flash_triton.py:94-129); the rule encoded is flash_triton.py:114.
#include "common.cuh"

namespace fa {

struct IdsView {
    const void* ptr;
    int64_t sb, sh, sl;
    int is64;
};

__device__ __forceinline__ long long load_id(const IdsView& v, int b, int h, int l) {
    const int64_t off = int64_t(b) * v.sb + int64_t(h) * v.sh + int64_t(l) * v.sl;
    return v.is64 ? static_cast<const long long*>(v.ptr)[off]
                  : static_cast<long long>(static_cast<const int*>(v.ptr)[off]);
}

__device__ __forceinline__ int block_reduce_min(int v, int* scratch) {
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    int r = scratch[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) r = min(r, scratch[w]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ int block_reduce_max(int v, int* scratch) {
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    int r = scratch[0];
    for (int w = 1; w < (blockDim.x >> 5); ++w) r = max(r, scratch[w]);
    __syncthreads();
    return r;
}

// grid (nQ + nK, He, B), 128 threads: one block of 128 queries or 128 keys.
__global__ void __launch_bounds__(128) plan_codes_kernel(IdsView eq, IdsView ek, int32_t* plan, PlanLayout L,
                                                         int* status) {
    __shared__ int scratch[4];
    const int he = blockIdx.y, b = blockIdx.z;
    const int64_t bh = int64_t(b) * L.He + he;
    const bool is_q = int(blockIdx.x) < L.nQ;
    const int blk = is_q ? blockIdx.x : blockIdx.x - L.nQ;
    const int l = blk * kBlk + threadIdx.x;
    const int len = is_q ? L.M : L.N;
    const bool valid = l < len;
    int code;
    if (is_q) {
        code = kCodeAny;
        if (valid) {
            const long long id = load_id(eq, b, he, l);
            if (id >= 0) {
                code = kCodeAny;
            } else if (id >= -2147483648LL) {
                code = int(id);
            } else {
                code = int(-2147483647 - 1);
                atomicCAS(status, 0, ST_ID_RANGE);
            }
        }
        plan[L.off_qc + bh * L.Mpad + l] = code;
    } else {
        code = 0;
        if (valid) {
            const long long id = load_id(ek, b, he, l);
            code = (id < 0 && id >= -2147483648LL) ? int(id) : 0;
        }
        plan[L.off_kc + bh * L.Npad + l] = code;
    }
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) plan[L.off_ctr + threadIdx.x] = 0;
    const int mn = block_reduce_min(valid ? code : 0x7fffffff, scratch);
    const int mx = block_reduce_max(valid ? code : int(-2147483647 - 1), scratch);
    // monotone within the block: no rise or no fall between neighbours. The padding entries of a ragged
    // last block count too (with the codes stored for them): the kernels' chunk tests read them.
    __shared__ int codes[kBlk];
    codes[threadIdx.x] = code;
    __syncthreads();
    int rise = 0, fall = 0;
    if (threadIdx.x > 0) {
        rise = code > codes[threadIdx.x - 1];
        fall = code < codes[threadIdx.x - 1];
    }
    const int any_rise = block_reduce_max(rise, scratch);
    const int any_fall = block_reduce_max(fall, scratch);
    const int mono = !(any_rise && any_fall);
    if (threadIdx.x == 0) {
        plan[(is_q ? L.off_qmono + bh * L.nQ : L.off_kmono + bh * L.nK) + blk] = mono;
        if (is_q) {
            plan[L.off_qmin + bh * L.nQ + blk] = mn;
            plan[L.off_qmax + bh * L.nQ + blk] = mx;
        } else {
            plan[L.off_kmin + bh * L.nK + blk] = mn;
            plan[L.off_kmax + bh * L.nK + blk] = mx;
        }
    }
}

// grid (nQ + nK, He, B), 128 threads: visit range of one query block over key blocks, or of
// one key block over query blocks.
__global__ void __launch_bounds__(128) plan_ranges_kernel(int32_t* plan, PlanLayout L, int gap, int causal) {
    __shared__ int scratch[4];
    const int he = blockIdx.y, b = blockIdx.z;
    const int64_t bh = int64_t(b) * L.He + he;
    const bool is_q = int(blockIdx.x) < L.nQ;
    const int blk = is_q ? blockIdx.x : blockIdx.x - L.nQ;
    const int32_t* qmin = plan + L.off_qmin + bh * L.nQ;
    const int32_t* qmax = plan + L.off_qmax + bh * L.nQ;
    const int32_t* kmin = plan + L.off_kmin + bh * L.nK;
    const int32_t* kmax = plan + L.off_kmax + bh * L.nK;
    const int n_other = is_q ? L.nK : L.nQ;
    int lo = 0x7fffffff, hi = 0;
    for (int o = threadIdx.x; o < n_other; o += blockDim.x) {
        const int qb = is_q ? blk : o, kb = is_q ? o : blk;
        const uint32_t f = classify_tile(qb, kb, L.M, L.N, gap, causal, 1, qmin[qb], qmax[qb], kmin[kb], kmax[kb]);
        if (f & TILE_VISIT) {
            lo = min(lo, o);
            hi = max(hi, o + 1);
        }
    }
    lo = block_reduce_min(lo, scratch);
    hi = block_reduce_max(hi, scratch);
    if (hi == 0) lo = 0;
    if (threadIdx.x == 0) {
        if (is_q) {
            plan[L.off_kvlo + bh * L.nQ + blk] = lo;
            plan[L.off_kvhi + bh * L.nQ + blk] = hi;
        } else {
            plan[L.off_qlo + bh * L.nK + blk] = lo;
            plan[L.off_qhi + bh * L.nK + blk] = hi;
        }
    }
}

// grid (2, He, B), 1024 threads: the blocks of one head sorted by the length of their visit range,
// longest first; equal lengths keep the order "from the long end" (last query block first, first key
// block first). Rank by counting: block i goes to the position given by the number of blocks that
// come before it.
__global__ void __launch_bounds__(1024) plan_order_kernel(int32_t* plan, PlanLayout L) {
    __shared__ int len[kListCap];
    const bool is_q = blockIdx.x == 0;
    const int he = blockIdx.y, b = blockIdx.z;
    const int64_t bh = int64_t(b) * L.He + he;
    const int n = is_q ? L.nQ : L.nK;
    const int32_t* lo = plan + (is_q ? L.off_kvlo : L.off_qlo) + bh * n;
    const int32_t* hi = plan + (is_q ? L.off_kvhi : L.off_qhi) + bh * n;
    int32_t* ord = plan + (is_q ? L.off_ordq : L.off_ordk) + bh * n;
    // natural position i: query block nQ-1-i, key block i
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int blk = is_q ? n - 1 - i : i;
        len[i] = hi[blk] - lo[blk];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int li = len[i];
        int rank = 0;
        for (int j = 0; j < n; ++j) rank += (len[j] > li) || (len[j] == li && j < i);
        ord[rank] = is_q ? n - 1 - i : i;
    }
}

// grid (nK, nQ, B*He), 128 threads: one tile. A tile that the plan does not visit reports
// keep = 0 everywhere, a tile without a flagged check reports keep = 1 for the entries that
// check covers: exactly what the attention kernels assume.
__global__ void __launch_bounds__(128) debug_mask_kernel(MaskArgs a, uint8_t* keep, uint8_t* tile_class) {
    const int kb = blockIdx.x, qb = blockIdx.y;
    const int b = blockIdx.z / a.He, he = blockIdx.z % a.He;
    const int64_t bh = int64_t(b) * a.He + he;
    int lo, hi;
    kv_range(a, b, he, qb, lo, hi);
    int qlo, qhi;
    q_range(a, b, he, kb, qlo, qhi);
    uint32_t f = classify_from_plan(a, b, he, qb, kb);
    const bool in_range = (kb >= lo && kb < hi) && (qb >= qlo && qb < qhi);
    if (!in_range) f = 0;
    if (tile_class && threadIdx.x == 0) tile_class[(bh * a.L.nQ + qb) * a.L.nK + kb] = uint8_t(f);
    if (!keep) return;
    const int i = qb * kBlk + threadIdx.x;
    if (i >= a.M) return;
    const int qc = (a.mode == 1) ? a.plan[a.L.off_qc + bh * a.L.Mpad + i] : 0;
    for (int c = 0; c < kBlk; ++c) {
        const int j = kb * kBlk + c;
        if (j >= a.N) break;
        bool kp = false;
        if (f & TILE_VISIT) {
            kp = true;
            const int kc = (f & TILE_DOC) ? a.plan[a.L.off_kc + bh * a.L.Npad + j] : 0;
            if (f & TILE_BOUND) kp = kp && keep_entry(i, j, 0, 0, a.N, a.gap, a.causal, 0);
            if (f & TILE_DOC) kp = kp && ((qc >= 0) || (qc == kc));
        }
        keep[(bh * a.M + i) * int64_t(a.N) + j] = kp ? 1 : 0;
    }
}

// ---- host launchers (called from api.cu) ------------------------------------------------
cudaError_t launch_plan_build(const void* eq_ptr, const int64_t* eq_stride, int eq64, const void* ek_ptr,
                              const int64_t* ek_stride, int ek64, int32_t* plan, const PlanLayout& L, int gap,
                              int causal, int* status, cudaStream_t stream) {
    IdsView q{eq_ptr, eq_stride[0], eq_stride[1], eq_stride[2], eq64};
    IdsView k{ek_ptr, ek_stride[0], ek_stride[1], ek_stride[2], ek64};
    dim3 grid(L.nQ + L.nK, L.He, L.B);
    plan_codes_kernel<<<grid, 128, 0, stream>>>(q, k, plan, L, status);
    plan_ranges_kernel<<<grid, 128, 0, stream>>>(plan, L, gap, causal);
    plan_order_kernel<<<dim3(2, L.He, L.B), 1024, 0, stream>>>(plan, L);
    return cudaGetLastError();
}

cudaError_t launch_debug_mask(const MaskArgs& a, uint8_t* keep, uint8_t* tile_class, cudaStream_t stream) {
    dim3 grid(a.L.nK, a.L.nQ, a.L.B * a.He);
    debug_mask_kernel<<<grid, 128, 0, stream>>>(a, keep, tile_class);
    return cudaGetLastError();
}

}  // namespace fa
