// Shared between the host API and all kernels: the mask-plan layout, the tile
// classification and the per-entry keep predicate.
//
// Mask rule of the reference (flash_triton.py:103-116, :254, :270-282, :401-416):
//   keep(i,j) = [j < N] & [!causal | (gap + i >= j)] & [mode != 1 | eq_i >= 0 | eq_i == ek_j]
// with gap = max(0, N - M).
#pragma once
#include <stdint.h>
#include "ptx.cuh"

namespace fa {

constexpr int kBlk = 128;  // rows of a query block = keys of a key block, for every kernel
constexpr int kListCap = 1024;  // blocks per sequence (per-item tile lists live in shared memory)

// Query code of an id >= 0 ("attends to everything"). Key codes are never positive.
constexpr int32_t kCodeAny = 0x7fffffff;

__host__ __device__ inline int cdiv(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t pad128(int64_t x) { return (x + 127) / 128 * 128; }

// Mask plan: one int32 array, sections in this order (all extents known from the problem).
//   qc   [B, He, Mpad]  query codes: kCodeAny if eq >= 0, else eq itself (must fit in int32)
//   kc   [B, He, Npad]  key codes: ek if -2^31 <= ek < 0, else 0 (can never equal a query code < 0)
//   qmin, qmax [B, He, nQ]   min / max query code per block of 128 queries (valid rows only)
//   kmin, kmax [B, He, nK]   min / max key code per block of 128 keys
//   kv_lo, kv_hi [B, He, nQ] range of key blocks with an unmasked entry, per query block
//   q_lo, q_hi   [B, He, nK] range of query blocks with an unmasked entry, per key block
//   qmono [B, He, nQ], kmono [B, He, nK]  1 if the codes of the block (all 128 stored codes, padding of a
//                ragged last block included) are monotone (non-decreasing or non-increasing), i.e. equal
//                codes are adjacent: the usual packed-documents layout
//   ord_q [B, He, nQ], ord_k [B, He, nK]  the blocks of a head sorted by the length of their visit range,
//                longest first (ties: from the long end of a causal head)
//   ctr [128]    work counters of the persistent kernels (item counter, finished-CTA counter per kernel);
//                zero between launches: the plan build clears them and every kernel clears its pair
//                when its last CTA leaves, so a plan serves one launch of each kernel at a time
struct PlanLayout {
    int B, He, M, N, nQ, nK;
    int64_t Mpad, Npad;
    int64_t off_qc, off_kc, off_qmin, off_qmax, off_kmin, off_kmax, off_kvlo, off_kvhi, off_qlo, off_qhi, off_qmono, off_kmono, off_ordq, off_ordk, off_ctr;
    int64_t total;  // int32 elements

    __host__ __device__ PlanLayout() {}
    __host__ __device__ PlanLayout(int B_, int He_, int M_, int N_) {
        B = B_; He = He_; M = M_; N = N_;
        nQ = cdiv(M, kBlk); nK = cdiv(N, kBlk);
        Mpad = pad128(M); Npad = pad128(N);
        int64_t bh = int64_t(B) * He;
        int64_t o = 0;
        off_qc = o;   o += bh * Mpad;
        off_kc = o;   o += bh * Npad;
        off_qmin = o; o += pad128(bh * nQ);
        off_qmax = o; o += pad128(bh * nQ);
        off_kmin = o; o += pad128(bh * nK);
        off_kmax = o; o += pad128(bh * nK);
        off_kvlo = o; o += pad128(bh * nQ);
        off_kvhi = o; o += pad128(bh * nQ);
        off_qlo = o;  o += pad128(bh * nK);
        off_qhi = o;  o += pad128(bh * nK);
        off_qmono = o; o += pad128(bh * nQ);
        off_kmono = o; o += pad128(bh * nK);
        off_ordq = o;  o += pad128(bh * nQ);
        off_ordk = o;  o += pad128(bh * nK);
        off_ctr = o;   o += 128;
        total = o;
    }
};

// What every attention kernel needs to evaluate the mask.
struct MaskArgs {
    const int32_t* plan;  // null when mode == 0
    unsigned int* ctr;    // work counters (CTR_* pairs), or null: the persistent kernels then share out items statically
    PlanLayout L;
    int M, N, gap, causal, mode;
    int He;               // 1 or H
    int debug;            // DBG_* bits (0 in normal use)
};

// Debug switches that change which tiles are visited and how they are evaluated, never the result:
// they exist to show that skipping tiles and the per-chunk shortcuts are exact.
enum : int {
    DBG_NO_SKIP = 1,      // visit every tile inside the causal / length bound, also those the ids mask entirely
    DBG_ALL_PARTIAL = 2,  // evaluate the bound and the id rule entry by entry on every visited tile
};

enum { CTR_FWD = 0, CTR_DKDV = 2, CTR_DQ = 4 };  // pairs {next item, CTAs finished} inside the plan's ctr section

enum : uint32_t {
    TILE_VISIT = 1u,   // at least one entry may be unmasked
    TILE_BOUND = 2u,   // needs the per-entry j < N / causal check
    TILE_DOC = 4u,     // needs the per-entry id check
    TILE_QTAIL = 8u,   // holds rows >= M (matters to the backward kernels only)
    TILE_KMONO = 16u,  // key codes of the block are monotone: a 32-key chunk is uniform iff its ends are equal
    TILE_QMONO = 32u,  // same for the query codes of the block
};

// Classification of tile (qb, kb) from the block statistics. Conservative: a tile is skipped
// only when every entry is masked, and declared free of a check only when every entry passes it.
__host__ __device__ inline uint32_t classify_tile(int qb, int kb, int M, int N, int gap, int causal,
                                                  int mode, int qmin, int qmax, int kmin, int kmax) {
    const int q0 = qb * kBlk, k0 = kb * kBlk;
    const int q1 = (q0 + kBlk < M) ? q0 + kBlk : M;  // exclusive
    const int k1 = (k0 + kBlk < N) ? k0 + kBlk : N;
    uint32_t f = TILE_VISIT;
    if (k0 + kBlk > N) f |= TILE_BOUND;
    if (q0 + kBlk > M) f |= TILE_QTAIL;
    if (causal) {
        if (k0 > q1 - 1 + gap) return 0;
        if (k1 - 1 > q0 + gap) f |= TILE_BOUND;
    }
    if (mode == 1) {
        if (qmax < 0 && (kmax < qmin || kmin > qmax)) return 0;
        const bool all_any = (qmin >= 0);
        const bool one_doc = (qmin == qmax) && (kmin == kmax) && (qmin == kmin);
        if (!all_any && !one_doc) f |= TILE_DOC;
    }
    return f;
}

__device__ __forceinline__ uint32_t classify_from_plan(const MaskArgs& a, int b, int he, int qb, int kb) {
    int qmin = 0, qmax = 0, kmin = 0, kmax = 0;
    if (a.mode == 1) {
        const int64_t bh = int64_t(b) * a.He + he;
        qmin = a.plan[a.L.off_qmin + bh * a.L.nQ + qb];
        qmax = a.plan[a.L.off_qmax + bh * a.L.nQ + qb];
        kmin = a.plan[a.L.off_kmin + bh * a.L.nK + kb];
        kmax = a.plan[a.L.off_kmax + bh * a.L.nK + kb];
    }
    uint32_t f = classify_tile(qb, kb, a.M, a.N, a.gap, a.causal, a.mode, qmin, qmax, kmin, kmax);
    if (a.debug) {
        if ((a.debug & DBG_NO_SKIP) && f == 0 && a.mode == 1) {
            f = classify_tile(qb, kb, a.M, a.N, a.gap, a.causal, 0, 0, 0, 0, 0);  // the bounds alone
            if (f) f |= TILE_DOC;                                                // the ids mask every entry
        }
        if ((a.debug & DBG_ALL_PARTIAL) && f) return f | TILE_BOUND | (a.mode == 1 ? TILE_DOC : 0u);
    }
    if (a.mode == 1 && (f & TILE_DOC)) {
        const int64_t bh = int64_t(b) * a.He + he;
        if (a.plan[a.L.off_kmono + bh * a.L.nK + kb]) f |= TILE_KMONO;
        if (a.plan[a.L.off_qmono + bh * a.L.nQ + qb]) f |= TILE_QMONO;
    }
    return f;
}

// Key-block range [lo, hi) a query block has to walk.
__device__ __forceinline__ void kv_range(const MaskArgs& a, int b, int he, int qb, int& lo, int& hi) {
    if (a.mode == 1 && !(a.debug & DBG_NO_SKIP)) {
        const int64_t bh = int64_t(b) * a.He + he;
        lo = a.plan[a.L.off_kvlo + bh * a.L.nQ + qb];
        hi = a.plan[a.L.off_kvhi + bh * a.L.nQ + qb];
    } else {
        lo = 0;
        hi = a.L.nK;
        if (a.causal) {
            const int q1 = min(qb * kBlk + kBlk, a.M);
            hi = min(a.L.nK, (q1 - 1 + a.gap) / kBlk + 1);
        }
    }
}
// Query-block range [lo, hi) a key block has to walk.
__device__ __forceinline__ void q_range(const MaskArgs& a, int b, int he, int kb, int& lo, int& hi) {
    if (a.mode == 1 && !(a.debug & DBG_NO_SKIP)) {
        const int64_t bh = int64_t(b) * a.He + he;
        lo = a.plan[a.L.off_qlo + bh * a.L.nK + kb];
        hi = a.plan[a.L.off_qhi + bh * a.L.nK + kb];
    } else {
        lo = 0;
        hi = a.L.nQ;
        if (a.causal) {
            const int first = kb * kBlk - a.gap;  // first query row that sees key k0
            lo = first > 0 ? first / kBlk : 0;
            if (lo > hi) lo = hi;
        }
    }
}

// The per-entry predicate on codes. Identical to the reference's rule on the original ids:
// qc >= 0 <=> eq >= 0; for eq < 0, qc == eq and kc == ek whenever ek is a negative int32,
// and kc == 0 != qc otherwise.
__device__ __forceinline__ bool keep_entry(int i, int j, int qc, int kc, int N, int gap, int causal, int mode) {
    bool keep = j < N;
    if (causal) keep = keep && (gap + i >= j);
    if (mode == 1) keep = keep && ((qc >= 0) || (qc == kc));
    return keep;
}

// A launch that finds the device's status word set by an earlier time-out computes nothing. It fills
// its outputs with NaN (0xFFFF is a NaN in bf16 and in fp16), so that what it leaves behind cannot be
// mistaken for a result. Called by all threads of the CTA; `tile` is nbox * 16 KB of shared memory,
// 1024-byte aligned; m1 may be null. Tiles are [128 rows, 64 * nbox columns] of a [B, H, L, D] tensor.
__device__ __forceinline__ void nan_fill_outputs(uint8_t* tile, int nbox, const CUtensorMap* m0, const CUtensorMap* m1,
                                                 int n_blk, int n_h, int n_b) {
    constexpr int kBox = kBlk * 64 * 2;
    for (int i = threadIdx.x; i < nbox * kBox / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(tile)[i] = make_uint4(~0u, ~0u, ~0u, ~0u);
    fence_proxy_async();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t src = smem_u32(tile);
        const int n = n_blk * n_h * n_b;
        for (int j = blockIdx.x; j < n; j += gridDim.x) {
            const int blk = j % n_blk, h = (j / n_blk) % n_h, b = j / (n_blk * n_h);
            for (int x = 0; x < nbox; ++x) {
                tma_store_4d(m0, src + x * kBox, x * 64, blk * kBlk, h, b);
                if (m1) tma_store_4d(m1, src + x * kBox, x * 64, blk * kBlk, h, b);
            }
            tma_store_commit();
        }
        tma_store_wait_all();
    }
}

// Device-side view of a [B, H, L, D] tensor for plain (non-TMA) stores.
struct OutTensor {
    void* ptr;
    int64_t sb, sh, sl;  // element strides; the D stride is 1
};

}  // namespace fa
