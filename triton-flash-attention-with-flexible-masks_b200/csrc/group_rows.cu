// fa_group_rows / fa_permute_rows: grouping of the queries by document id for calls without a
// causal mask.
//
// Without a causal mask the order of the query rows is free: row i of the output depends on query
// i, its id and all keys, not on its position. When the query ids are scattered (every block of 128
// queries holds every document) no tile can be skipped and every tile needs the entry-by-entry id
// check; after a stable sort of the rows by id the blocks are (nearly) uniform, the mask plan skips
// the tiles of other documents, and the few mixed blocks are the only ones that pay for the check.
// The reference has no counterpart: it evaluates every tile whatever the ids (flash_triton.py:94-129).
//
//  - fa_group_rows sorts each id row [M] of eq by the 32-bit code the mask plan uses for it
//    (ids >= 0, "attend to all", share one code that sorts last; flash_triton.py:114), keeping the
//    caller's order inside a document (stable; rows that are grouped already keep their places), and
//    writes the permutation, its inverse and the ids in the new order;
//  - fa_permute_rows moves the rows of a [B, H, M, D] tensor through such an index:
//    dst[b, h, i, :] = src[b, h, index[b, he, i], :]. With the permutation it gathers q (and dO) into
//    the grouped order; with the inverse it puts o (and dQ) back into the caller's order. It is plain
//    HBM traffic: every row is read once and written once, 16 bytes per thread.
//
// One CTA sorts one row in shared memory: a bitonic network over 64-bit keys (code, position), which
// are all distinct, so the order is the stable one whatever the network does with equal codes.
#include "../../include/fa_b200.h"
#include "common.cuh"

namespace {

struct IdRows {
    const void* ptr;
    int64_t sb, sh, sl;
    int is64;
};

constexpr int kSortThreads = 1024;

// grid (He, B). P = M rounded up to a power of two; dynamic shared memory = P * 8 bytes.
__global__ void __launch_bounds__(kSortThreads) group_rows_kernel(IdRows eq, int M, int P, int He, int32_t* order,
                                                                  int32_t* inverse, int32_t* grouped, int* status) {
    extern __shared__ __align__(16) unsigned long long keys[];
    const int he = blockIdx.x, b = blockIdx.y;
    const int64_t row = (int64_t(b) * He + he) * M;
    for (int i = threadIdx.x; i < P; i += kSortThreads) {
        unsigned long long key = ~0ull;  // padding sorts behind every row
        if (i < M) {
            const int64_t off = int64_t(b) * eq.sb + int64_t(he) * eq.sh + int64_t(i) * eq.sl;
            const long long id = eq.is64 ? static_cast<const long long*>(eq.ptr)[off]
                                         : static_cast<long long>(static_cast<const int*>(eq.ptr)[off]);
            int code = fa::kCodeAny;
            if (id < 0) {
                if (id >= -2147483648LL) {
                    code = int(id);
                } else {  // same rule and status code as the mask plan
                    code = int(-2147483647 - 1);
                    atomicCAS(status, 0, fa::ST_ID_RANGE);
                }
            }
            key = (static_cast<unsigned long long>(uint32_t(code) ^ 0x80000000u) << 32) | uint32_t(i);
        }
        keys[i] = key;
    }
    __syncthreads();
    for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (P >> 1); t += kSortThreads) {
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int l = i | j;
                const bool up = (i & k) == 0;
                const unsigned long long a = keys[i], c = keys[l];
                if ((a > c) == up) {
                    keys[i] = c;
                    keys[l] = a;
                }
            }
            __syncthreads();
        }
    }
    for (int i = threadIdx.x; i < M; i += kSortThreads) {
        const unsigned long long key = keys[i];
        const int src = int(uint32_t(key));
        order[row + i] = src;
        inverse[row + src] = i;
        grouped[row + i] = int(uint32_t(key >> 32) ^ 0x80000000u);
    }
}

struct RowTensor {
    const uint4* src;
    uint4* dst;
    int64_t s_sb, s_sh, s_sl;  // strides in 16-byte units
    int64_t d_sb, d_sh, d_sl;
};

// One thread per 16 bytes of a destination row; consecutive threads share a row, so a warp reads and
// writes whole 128-byte (or longer) stretches.
__global__ void __launch_bounds__(256) permute_rows_kernel(RowTensor t, const int32_t* index, int M, int H, int He,
                                                           int vec, int64_t total) {
    const int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= total) return;
    const int c = int(g % vec);
    const int64_t r = g / vec;
    const int i = int(r % M);
    const int64_t bh = r / M;
    const int h = int(bh % H);
    const int b = int(bh / H);
    const int he = (He == 1) ? 0 : h;
    const int s = index[(int64_t(b) * He + he) * M + i];
    t.dst[b * t.d_sb + h * t.d_sh + i * t.d_sl + c] = t.src[b * t.s_sb + h * t.s_sh + int64_t(s) * t.s_sl + c];
}

int elt_bytes(int dtype) { return dtype == FA_FP32 ? 4 : 2; }

// Base 16-byte aligned, last stride 1, the other strides of extents > 1 positive and whole 16-byte units.
int check_rows(const fa_tensor* t, int B, int H, int M, int per16) {
    if (!t || !t->ptr) return FA_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(t->ptr) % 16 != 0 || t->stride[3] != 1) return FA_ERR_ALIGNMENT;
    const int ext[3] = {B, H, M};
    for (int i = 0; i < 3; ++i)
        if (ext[i] > 1 && (t->stride[i] <= 0 || t->stride[i] % per16 != 0)) return FA_ERR_ALIGNMENT;
    return FA_OK;
}

}  // namespace

extern "C" int fa_group_rows(const fa_problem* p, const fa_ids* eq, int32_t* order, int32_t* inverse,
                             int32_t* grouped_ids, int32_t* status, void* stream) {
    size_t bytes = 0;
    const int rc = fa_plan_bytes(p, &bytes);  // validates the problem as every other entry point does
    if (rc) return rc;
    if (p->mode != FA_MODE1_DOC || !eq || !eq->ptr || !order || !inverse || !grouped_ids || !status) return FA_ERR_BAD_ARG;
    if (eq->dtype != FA_ID_INT32 && eq->dtype != FA_ID_INT64) return FA_ERR_BAD_ARG;
    if (p->M > FA_GROUP_MAX_ROWS) return FA_ERR_UNSUPPORTED;
    int P = 1;
    while (P < p->M) P <<= 1;
    const size_t smem = size_t(P) * sizeof(unsigned long long);
    // the attribute belongs to the device: set it once per device (always the same value, so a race between two
    // first calls is harmless)
    static bool attr_set[64] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FA_ERR_LAUNCH;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(group_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 int(FA_GROUP_MAX_ROWS * sizeof(unsigned long long))) != cudaSuccess)
            return FA_ERR_LAUNCH;
        attr_set[dev] = true;
    }
    const IdRows rows{eq->ptr, eq->stride[0], eq->stride[1], eq->stride[2], eq->dtype == FA_ID_INT64};
    group_rows_kernel<<<dim3(p->id_heads, p->B), kSortThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        rows, p->M, P, p->id_heads, order, inverse, grouped_ids, status);
    return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

extern "C" int fa_permute_rows(const fa_problem* p, const fa_tensor* src, const fa_tensor* dst, const int32_t* index,
                               void* stream) {
    size_t bytes = 0;
    int rc = fa_plan_bytes(p, &bytes);
    if (rc) return rc;
    if (!index) return FA_ERR_BAD_ARG;
    const int per16 = 16 / elt_bytes(p->dtype);  // elements per 16 bytes
    if (p->D % per16 != 0) return FA_ERR_UNSUPPORTED;
    if ((rc = check_rows(src, p->B, p->H, p->M, per16))) return rc;
    if ((rc = check_rows(dst, p->B, p->H, p->M, per16))) return rc;
    const int vec = p->D / per16;
    RowTensor t;
    t.src = static_cast<const uint4*>(src->ptr);
    t.dst = static_cast<uint4*>(dst->ptr);
    t.s_sb = src->stride[0] / per16; t.s_sh = src->stride[1] / per16; t.s_sl = src->stride[2] / per16;
    t.d_sb = dst->stride[0] / per16; t.d_sh = dst->stride[1] / per16; t.d_sl = dst->stride[2] / per16;
    // strides of extent-1 dimensions are never multiplied by anything but 0
    const int64_t total = int64_t(p->B) * p->H * p->M * vec;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return FA_ERR_UNSUPPORTED;
    const int He = (p->mode == FA_MODE1_DOC) ? p->id_heads : 1;
    permute_rows_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(t, index, p->M, p->H, He, vec,
                                                                                         total);
    return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}
