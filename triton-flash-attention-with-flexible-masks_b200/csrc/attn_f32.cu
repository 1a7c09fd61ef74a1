// fp32 inputs (flash_triton.py:512 accepts any float dtype; testing.py:158 lists fp32). The tensor-core
// kernels of this library work on 16-bit operands; a 16-bit product cannot meet the 1e-4 tolerance
// asked of fp32 results, so fp32 tensors take the kernels below: the same flash-attention recurrence
// (flash_triton.py:94-133 forward, :250-311 dK/dV, :387-423 dQ), the same mask plan, tile
// classification and per-entry predicate as the 16-bit kernels, but all arithmetic in fp32 FMAs.
// They cover every head dim the reference accepts (16, 32, 64, 128) and are meant for checks and
// small problems, not for speed.
//
// One CTA = 128 threads = 4 warps works on 32 "rows" (queries in the forward and dQ kernels, keys
// in the dK/dV kernel) against tiles of 32 "columns"; warp w owns rows 8w..8w+7, lane = column.
// Two building blocks on shared-memory tiles with rows padded to D + 4 floats:
//   rows_dot_cols: s[r] = sum_d A[row r][d] * B[col lane][d]   (A broadcast, B one row per lane)
//   rows_acc:      acc[r][k] += sum_c P[row r][c] * V[c][lane + 32 k]
#include "../../include/fa_b200.h"
#include "common.cuh"
#include "params.cuh"

namespace fa {

constexpr int kT = 32;  // rows per CTA and columns per tile

template <int D>
struct F32Smem {
    static constexpr int LD = D + 4;
    static constexpr int tile = kT * LD;  // floats
};

// loads rows [r0, r0 + 32) of a [L, D] slice into a padded tile; rows >= L are zero
template <int D>
__device__ __forceinline__ void load_tile(float* dst, const float* src, int64_t sl, int r0, int L) {
    constexpr int LD = F32Smem<D>::LD;
    for (int i = threadIdx.x; i < kT * (D / 4); i += blockDim.x) {
        const int r = i / (D / 4), c4 = i % (D / 4);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r0 + r < L) {
            const float* p = src + int64_t(r0 + r) * sl + 4 * c4;
            if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) v = *reinterpret_cast<const float4*>(p);
            else v = make_float4(p[0], p[1], p[2], p[3]);
        }
        *reinterpret_cast<float4*>(dst + r * LD + 4 * c4) = v;
    }
}

template <int D>
__device__ __forceinline__ void rows_dot_cols(const float* A, const float* Bt, int warp, int lane, float (&s)[8]) {
    constexpr int LD = F32Smem<D>::LD;
#pragma unroll
    for (int r = 0; r < 8; ++r) s[r] = 0.f;
#pragma unroll 4
    for (int d4 = 0; d4 < D / 4; ++d4) {
        const float4 b = *reinterpret_cast<const float4*>(Bt + lane * LD + 4 * d4);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float4 a = *reinterpret_cast<const float4*>(A + (8 * warp + r) * LD + 4 * d4);
            s[r] = fmaf(a.x, b.x, s[r]);
            s[r] = fmaf(a.y, b.y, s[r]);
            s[r] = fmaf(a.z, b.z, s[r]);
            s[r] = fmaf(a.w, b.w, s[r]);
        }
    }
}

template <int D>
__device__ __forceinline__ void rows_acc(const float* P, const float* V, int warp, int lane, float (&acc)[8][(D + 31) / 32]) {
    constexpr int LD = F32Smem<D>::LD;
    constexpr int NK = (D + 31) / 32;
#pragma unroll 4
    for (int c = 0; c < kT; ++c) {
        float v[NK];
#pragma unroll
        for (int k = 0; k < NK; ++k) v[k] = (lane + 32 * k < D) ? V[c * LD + lane + 32 * k] : 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float p = P[(8 * warp + r) * kT + c];
#pragma unroll
            for (int k = 0; k < NK; ++k) acc[r][k] = fmaf(p, v[k], acc[r][k]);
        }
    }
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// does the 128 x 128 block that holds rows i0.. and columns j0.. contain an unmasked entry at all?
__device__ __forceinline__ bool block_visited(const MaskArgs& mk, int b, int he, int i0, int j0) {
    return (classify_from_plan(mk, b, he, i0 / kBlk, j0 / kBlk) & TILE_VISIT) != 0;
}

__device__ __forceinline__ int code_q(const MaskArgs& mk, int b, int he, int i) {
    return (mk.mode == 1 && i < mk.M) ? mk.plan[mk.L.off_qc + (int64_t(b) * mk.He + he) * mk.L.Mpad + i] : 0;
}
__device__ __forceinline__ int code_k(const MaskArgs& mk, int b, int he, int j) {
    return (mk.mode == 1 && j < mk.N) ? mk.plan[mk.L.off_kc + (int64_t(b) * mk.He + he) * mk.L.Npad + j] : 0;
}

// ---------------------------------------------------------------------------------------------
// forward: grid (ceil(M / 32), H, B)
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) f32_fwd_kernel(const F32Params p) {
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;
    float* Ks = Qs + F32Smem<D>::tile;
    float* Vs = Ks + F32Smem<D>::tile;
    float* Ps = Vs + F32Smem<D>::tile;  // [32][32]
    constexpr int NK = (D + 31) / 32;
    const MaskArgs& mk = p.mask;
    const int i0 = blockIdx.x * kT, h = blockIdx.y, b = blockIdx.z, hk = h / p.G;
    const int he = (mk.He == 1) ? 0 : h;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    load_tile<D>(Qs, p.q.ptr + int64_t(b) * p.q.sb + int64_t(h) * p.q.sh, p.q.sl, i0, mk.M);
    float m[8], l[8], acc[8][NK];
    int qc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.f;
        qc[r] = code_q(mk, b, he, i0 + 8 * warp + r);
#pragma unroll
        for (int k = 0; k < NK; ++k) acc[r][k] = 0.f;
    }
    const int hi = mk.causal ? min(mk.N, i0 + kT + mk.gap) : mk.N;  // keys beyond the last row's causal bound
    const float* kbase = p.k.ptr + int64_t(b) * p.k.sb + int64_t(hk) * p.k.sh;
    const float* vbase = p.v.ptr + int64_t(b) * p.v.sb + int64_t(hk) * p.v.sh;
    for (int j0 = 0; j0 < hi; j0 += kT) {
        if (!block_visited(mk, b, he, i0, j0)) continue;  // uniform for the CTA
        __syncthreads();
        load_tile<D>(Ks, kbase, p.k.sl, j0, mk.N);
        load_tile<D>(Vs, vbase, p.v.sl, j0, mk.N);
        __syncthreads();
        const int j = j0 + lane;
        const int kc = code_k(mk, b, he, j);
        float s[8];
        rows_dot_cols<D>(Qs, Ks, warp, lane, s);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int i = i0 + 8 * warp + r;
            const bool keep = keep_entry(i, j, qc[r], kc, mk.N, mk.gap, mk.causal, mk.mode);
            const float sv = keep ? s[r] * p.scale : -INFINITY;
            const float mn = fmaxf(m[r], warp_max(sv));
            const float alpha = (m[r] == -INFINITY) ? 0.f : expf(m[r] - mn);
            const float pe = (sv == -INFINITY) ? 0.f : expf(sv - mn);
            l[r] = l[r] * alpha + warp_sum(pe);
            m[r] = mn;
#pragma unroll
            for (int k = 0; k < NK; ++k) acc[r][k] *= alpha;
            Ps[(8 * warp + r) * kT + lane] = pe;
        }
        __syncwarp();
        rows_acc<D>(Ps, Vs, warp, lane, acc);
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int i = i0 + 8 * warp + r;
        if (i >= mk.M) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
        float* po = p.o.ptr + int64_t(b) * p.o.sb + int64_t(h) * p.o.sh + int64_t(i) * p.o.sl;
#pragma unroll
        for (int k = 0; k < NK; ++k)
            if (lane + 32 * k < D) po[lane + 32 * k] = acc[r][k] * inv;
        if (lane == 0) p.lse[(int64_t(b) * p.H + h) * mk.L.Mpad + i] = l[r] > 0.f ? m[r] + logf(l[r]) : -INFINITY;
    }
}

// delta = rowsum(o * dO) (flash_triton.py:161-165): grid (ceil(M / 4), H, B), one warp per row
template <int D>
__global__ void __launch_bounds__(128) f32_delta_kernel(const F32Params p) {
    const int i = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int h = blockIdx.y, b = blockIdx.z;
    if (i >= p.mask.L.Mpad) return;
    float a = 0.f;
    if (i < p.mask.M) {
        const float* po = p.o.ptr + int64_t(b) * p.o.sb + int64_t(h) * p.o.sh + int64_t(i) * p.o.sl;
        const float* pd = p.d_o.ptr + int64_t(b) * p.d_o.sb + int64_t(h) * p.d_o.sh + int64_t(i) * p.d_o.sl;
        for (int d = lane; d < D; d += 32) a = fmaf(po[d], pd[d], a);
    }
    a = warp_sum(a);
    if (lane == 0) p.delta[(int64_t(b) * p.H + h) * p.mask.L.Mpad + i] = a;
}

// ---------------------------------------------------------------------------------------------
// dQ: grid (ceil(M / 32), H, B). rows = queries, columns = keys
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) f32_bwd_dq_kernel(const F32Params p) {
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;
    float* dOs = Qs + F32Smem<D>::tile;
    float* Ks = dOs + F32Smem<D>::tile;
    float* Vs = Ks + F32Smem<D>::tile;
    float* Ps = Vs + F32Smem<D>::tile;
    constexpr int NK = (D + 31) / 32;
    const MaskArgs& mk = p.mask;
    const int i0 = blockIdx.x * kT, h = blockIdx.y, b = blockIdx.z, hk = h / p.G;
    const int he = (mk.He == 1) ? 0 : h;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    load_tile<D>(Qs, p.q.ptr + int64_t(b) * p.q.sb + int64_t(h) * p.q.sh, p.q.sl, i0, mk.M);
    load_tile<D>(dOs, p.d_o.ptr + int64_t(b) * p.d_o.sb + int64_t(h) * p.d_o.sh, p.d_o.sl, i0, mk.M);
    float acc[8][NK], lse[8], dl[8];
    int qc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int i = i0 + 8 * warp + r;
        const int64_t ro = (int64_t(b) * p.H + h) * mk.L.Mpad + i;
        lse[r] = (i < mk.M) ? p.lse[ro] : -INFINITY;
        dl[r] = (i < mk.M) ? p.delta[ro] : 0.f;
        qc[r] = code_q(mk, b, he, i);
#pragma unroll
        for (int k = 0; k < NK; ++k) acc[r][k] = 0.f;
    }
    const int hi = mk.causal ? min(mk.N, i0 + kT + mk.gap) : mk.N;
    const float* kbase = p.k.ptr + int64_t(b) * p.k.sb + int64_t(hk) * p.k.sh;
    const float* vbase = p.v.ptr + int64_t(b) * p.v.sb + int64_t(hk) * p.v.sh;
    for (int j0 = 0; j0 < hi; j0 += kT) {
        if (!block_visited(mk, b, he, i0, j0)) continue;
        __syncthreads();
        load_tile<D>(Ks, kbase, p.k.sl, j0, mk.N);
        load_tile<D>(Vs, vbase, p.v.sl, j0, mk.N);
        __syncthreads();
        const int j = j0 + lane;
        const int kc = code_k(mk, b, he, j);
        float s[8], dp[8];
        rows_dot_cols<D>(Qs, Ks, warp, lane, s);
        rows_dot_cols<D>(dOs, Vs, warp, lane, dp);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int i = i0 + 8 * warp + r;
            const bool keep = (i < mk.M) && keep_entry(i, j, qc[r], kc, mk.N, mk.gap, mk.causal, mk.mode);
            const float pe = keep ? expf(s[r] * p.scale - lse[r]) : 0.f;  // a kept entry has a finite lse
            Ps[(8 * warp + r) * kT + lane] = pe * (dp[r] - dl[r]);       // dS (flash_triton.py:301)
        }
        __syncwarp();
        rows_acc<D>(Ps, Ks, warp, lane, acc);  // dQ += dS K (flash_triton.py:420)
        __syncwarp();
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int i = i0 + 8 * warp + r;
        if (i >= mk.M) continue;
        float* pq = p.dq.ptr + int64_t(b) * p.dq.sb + int64_t(h) * p.dq.sh + int64_t(i) * p.dq.sl;
#pragma unroll
        for (int k = 0; k < NK; ++k)
            if (lane + 32 * k < D) pq[lane + 32 * k] = acc[r][k] * p.scale;  // flash_triton.py:425
    }
}

// ---------------------------------------------------------------------------------------------
// dK, dV: grid (ceil(N / 32), Hk, B). rows = keys, columns = queries; the query heads of the group
// are walked one after the other, so the group sum (flash_triton.py:635-637) needs no second pass
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128) f32_bwd_dkdv_kernel(const F32Params p) {
    extern __shared__ __align__(16) float sm[];
    float* Ks = sm;
    float* Vs = Ks + F32Smem<D>::tile;
    float* Qs = Vs + F32Smem<D>::tile;
    float* dOs = Qs + F32Smem<D>::tile;
    float* Ps = dOs + F32Smem<D>::tile;
    constexpr int NK = (D + 31) / 32;
    const MaskArgs& mk = p.mask;
    const int j0 = blockIdx.x * kT, hk = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    load_tile<D>(Ks, p.k.ptr + int64_t(b) * p.k.sb + int64_t(hk) * p.k.sh, p.k.sl, j0, mk.N);
    load_tile<D>(Vs, p.v.ptr + int64_t(b) * p.v.sb + int64_t(hk) * p.v.sh, p.v.sl, j0, mk.N);
    float dk[8][NK], dv[8][NK];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int k = 0; k < NK; ++k) dk[r][k] = dv[r][k] = 0.f;
    // first query row that can see key j0 under the causal mask (flash_triton.py:214-218)
    const int lo = mk.causal ? max(0, j0 - mk.gap) / kT * kT : 0;
    for (int g = 0; g < p.G; ++g) {
        const int h = hk * p.G + g;
        const int he = (mk.He == 1) ? 0 : h;
        int kc[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) kc[r] = code_k(mk, b, he, j0 + 8 * warp + r);
        const float* qbase = p.q.ptr + int64_t(b) * p.q.sb + int64_t(h) * p.q.sh;
        const float* dobase = p.d_o.ptr + int64_t(b) * p.d_o.sb + int64_t(h) * p.d_o.sh;
        for (int i0 = lo; i0 < mk.M; i0 += kT) {
            if (!block_visited(mk, b, he, i0, j0)) continue;
            __syncthreads();
            load_tile<D>(Qs, qbase, p.q.sl, i0, mk.M);
            load_tile<D>(dOs, dobase, p.d_o.sl, i0, mk.M);
            __syncthreads();
            const int i = i0 + lane;
            const int64_t ro = (int64_t(b) * p.H + h) * mk.L.Mpad + i;
            const float lse = (i < mk.M) ? p.lse[ro] : -INFINITY;
            const float dl = (i < mk.M) ? p.delta[ro] : 0.f;
            const int qc = code_q(mk, b, he, i);
            float s[8], dp[8];
            rows_dot_cols<D>(Ks, Qs, warp, lane, s);    // S^T
            rows_dot_cols<D>(Vs, dOs, warp, lane, dp);  // dP^T
            float pe[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int j = j0 + 8 * warp + r;
                const bool keep = (i < mk.M) && keep_entry(i, j, qc, kc[r], mk.N, mk.gap, mk.causal, mk.mode);
                pe[r] = keep ? expf(s[r] * p.scale - lse) : 0.f;
                Ps[(8 * warp + r) * kT + lane] = pe[r];
            }
            __syncwarp();
            rows_acc<D>(Ps, dOs, warp, lane, dv);  // dV += P^T dO (flash_triton.py:291)
            __syncwarp();
#pragma unroll
            for (int r = 0; r < 8; ++r) Ps[(8 * warp + r) * kT + lane] = pe[r] * (dp[r] - dl);
            __syncwarp();
            rows_acc<D>(Ps, Qs, warp, lane, dk);   // dK += dS^T Q (flash_triton.py:308)
            __syncwarp();
        }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const int j = j0 + 8 * warp + r;
        if (j >= mk.N) continue;
        float* pk = p.dk.ptr + int64_t(b) * p.dk.sb + int64_t(hk) * p.dk.sh + int64_t(j) * p.dk.sl;
        float* pv = p.dv.ptr + int64_t(b) * p.dv.sb + int64_t(hk) * p.dv.sh + int64_t(j) * p.dv.sl;
#pragma unroll
        for (int k = 0; k < NK; ++k)
            if (lane + 32 * k < D) {
                pk[lane + 32 * k] = dk[r][k] * p.scale;  // flash_triton.py:313
                pv[lane + 32 * k] = dv[r][k];
            }
    }
}

// ---------------------------------------------------------------------------------------------
template <int D>
static cudaError_t launch_f32_t(int which, const F32Params& p, cudaStream_t stream) {
    const MaskArgs& mk = p.mask;
    constexpr int tile = F32Smem<D>::tile;
    cudaError_t e = cudaSuccess;
    if (which == 0) {
        const int smem = (3 * tile + kT * kT) * 4;
        e = cudaFuncSetAttribute(f32_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        f32_fwd_kernel<D><<<dim3(cdiv(mk.M, kT), p.H, p.B), 128, smem, stream>>>(p);
    } else if (which == 1) {
        f32_delta_kernel<D><<<dim3(unsigned(mk.L.Mpad / 4), p.H, p.B), 128, 0, stream>>>(p);
    } else if (which == 2) {
        const int smem = (4 * tile + kT * kT) * 4;
        e = cudaFuncSetAttribute(f32_bwd_dkdv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        f32_bwd_dkdv_kernel<D><<<dim3(cdiv(mk.N, kT), p.Hk, p.B), 128, smem, stream>>>(p);
    } else {
        const int smem = (4 * tile + kT * kT) * 4;
        e = cudaFuncSetAttribute(f32_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        f32_bwd_dq_kernel<D><<<dim3(cdiv(mk.M, kT), p.H, p.B), 128, smem, stream>>>(p);
    }
    return cudaGetLastError();
}

// which: 0 forward, 1 delta, 2 dK / dV, 3 dQ
cudaError_t launch_f32(int which, int D, const F32Params& p, cudaStream_t stream) {
    switch (D) {
        case 16: return launch_f32_t<16>(which, p, stream);
        case 32: return launch_f32_t<32>(which, p, stream);
        case 64: return launch_f32_t<64>(which, p, stream);
        case 128: return launch_f32_t<128>(which, p, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace fa
