/*
 * C ABI of the B200 (sm_100a) document-masked flash-attention library.
 *
 * The library replaces the four Triton launches of the reference operator
 * (flash_triton.py:541 `_fwd_kernel`, :585 `_bwd_preprocess`, :596 `_bwd_kv_kernel`,
 * :617 `_bwd_q_kernel`) and adds the mask plan (per-block id ranges, no counterpart in the
 * reference: README.md:18 lists block sparsity as not implemented).
 *
 * Conventions
 *  - every pointer is a device pointer of the current CUDA device unless stated otherwise;
 *  - tensors are [B, H, L, D] with ELEMENT strides; the last stride must be 1, the other
 *    strides multiples of 8 elements and the base 16-byte aligned (TMA rules);
 *  - lse, delta and plan buffers must be 16-byte aligned (the kernels read them with bulk copies
 *    and 16-byte loads); a misaligned buffer is refused with FA_ERR_ALIGNMENT;
 *  - the caller owns every buffer;
 *  - every function enqueues on `stream` and returns without synchronising;
 *  - return value 0 = ok, otherwise an FA_ERR_* code (fa_error_string() describes it);
 *  - `status` is one int32 in device memory, zeroed by the caller. Kernels write a non-zero
 *    code there when a bounded wait ran out (100..199) or an id was out of range (200); the
 *    first code wins. A time-out code is sticky: while the word holds one, every later
 *    fa_fwd / fa_bwd_dkdv / fa_bwd_dq launch given that word computes nothing and fills its
 *    outputs (o; dk, dv; dq) with NaN, until the host has read the word and set it back to 0.
 *    The outputs of the launch in which the wait ran out are undefined. Code 200 only concerns
 *    the call that passed the id (its result may mask that query wrongly); later calls run.
 *  - one bounded wait lasts at most 5e8 SM clocks (about 0.25 s); the environment variable
 *    FA_B200_WAIT_LIMIT_CLOCKS (>= 10000), read when the library is first used, replaces the limit,
 *    e.g. on hosts where several contexts time-share the GPU.
 */
#ifndef FA_B200_H_
#define FA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_VERSION 1

/* Head dims 16, 32, 64 and 128 (flash_triton.py:512). FA_BF16 / FA_FP16 run on tensor-core kernels built for 64
 * and 128 columns; with head dims 16 and 32 the 64-wide kernels read the tensors through TMA maps of the real
 * head dim, which fill the missing columns with zeros and never write them (no padded copies anywhere).
 * FA_FP32 tensors (4-byte aligned base, last stride 1, any positive other strides) take fp32 FMA kernels
 * (testing.py:158): exact to fp32 rounding, not fast. */
enum fa_dtype { FA_BF16 = 0, FA_FP16 = 1, FA_FP32 = 2 };
enum fa_id_dtype { FA_ID_NONE = 0, FA_ID_INT32 = 1, FA_ID_INT64 = 2 };
/* score_func_mode of the reference (flash_triton.py:20-22) */
enum fa_mode { FA_MODE0_NOPE = 0, FA_MODE1_DOC = 1 };

enum fa_error {
    FA_OK = 0,
    FA_ERR_BAD_ARG = 1,      /* null pointer, non-positive size, unknown enum */
    FA_ERR_UNSUPPORTED = 2,  /* head dim not in {16,32,64,128}, unknown dtype, sm_scale <= 0 */
    FA_ERR_ALIGNMENT = 3,    /* a base address or stride breaks the TMA 16-byte rules */
    FA_ERR_TENSORMAP = 4,    /* the driver refused to encode a tensor map */
    FA_ERR_LAUNCH = 5,       /* kernel launch failed (cudaGetLastError) */
    FA_ERR_PLAN_SIZE = 6,    /* plan buffer too small / missing for FA_MODE1_DOC */
    FA_ERR_NO_DRIVER = 7,    /* cuTensorMapEncodeTiled could not be resolved */
    FA_ERR_SCRATCH_LIMIT = 8 /* fa_fwd_static_plan: the plan does not fit in FA_STATIC_PLAN_BYTES */
};

typedef struct fa_problem {
    int32_t B, H, Hk; /* batch, query heads, key/value heads (H % Hk == 0) */
    int32_t M, N, D;  /* query length, key length, head dim */
    int32_t dtype;    /* enum fa_dtype, of q/k/v/o and all gradients */
    int32_t causal;   /* bottom-right aligned: query i sees key j iff j <= i + max(0, N-M) */
    int32_t mode;     /* enum fa_mode */
    int32_t id_heads; /* head extent of the id tensors as stored in the plan: 1 (broadcast) or H */
    float sm_scale;   /* > 0 */
} fa_problem;

typedef struct fa_tensor {
    void* ptr;
    int64_t stride[4]; /* elements, order [B, H, L, D] */
} fa_tensor;

typedef struct fa_ids {
    const void* ptr;
    int64_t stride[3]; /* elements, order [B, H, L]; any value incl. 0 */
    int32_t dtype;     /* enum fa_id_dtype */
} fa_ids;

int fa_version(void);
const char* fa_error_string(int code);

/* Rows of the internal per-row fp32 buffers (log-sum-exp, delta): M rounded up to 128. */
int64_t fa_padded_rows(int32_t M);

/* Size in bytes of the mask plan for this problem (when mode == FA_MODE0_NOPE: 512 bytes, the work
 * counters of the attention kernels only; such a plan is optional). */
int fa_plan_bytes(const fa_problem* p, size_t* bytes);

/* Builds the mask plan from eq [B,H,M] / ek [B,H,N]: 32-bit id codes, per-128-block id
 * min/max, per-block ranges of blocks that hold at least one unmasked entry, and a few work
 * counters through which the CTAs of fa_fwd / fa_bwd_dkdv / fa_bwd_dq share out their work.
 * The attention kernels update those counters (although they take the plan as `const void*`) and
 * leave them zero, so a plan can be used any number of times, but only by one launch of each of
 * the three at a time.
 * Mask rule (flash_triton.py:114, README.md:16): keep = (eq >= 0) | (eq == ek). */
int fa_plan_build(const fa_problem* p, const fa_ids* eq, const fa_ids* ek, void* plan, size_t plan_bytes,
                  int32_t* status, void* stream);

/* Forward (replaces flash_triton.py:541). o has q's shape; lse is [B, H, fa_padded_rows(M)] fp32,
 * log2-domain log-sum-exp of the scaled scores (flash_triton.py:133), -inf for a row with no
 * unmasked key (whose output row is 0). plan may be NULL when mode == FA_MODE0_NOPE (here and in
 * the backward entry points): the CTAs then share out their work in a fixed order instead of through
 * the plan's counters, which costs a few percent when the work per block is uneven. */
int fa_fwd(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v,
           const fa_tensor* o, float* lse, const void* plan, int32_t* status, void* stream);

/* delta[b,h,i] = sum_d o*do in fp32 (replaces flash_triton.py:585); delta is
 * [B, H, fa_padded_rows(M)], padding rows are written as 0. */
int fa_bwd_delta(const fa_problem* p, const fa_tensor* o, const fa_tensor* d_o, float* delta, void* stream);

/* dK, dV [B, Hk, N, D] (replaces flash_triton.py:596 and the group sum at :635-637; the sum
 * over the query heads of a group is accumulated in fp32 inside the kernel). */
int fa_bwd_dkdv(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v,
                const fa_tensor* d_o, const float* lse, const float* delta, const fa_tensor* dk,
                const fa_tensor* dv, const void* plan, int32_t* status, void* stream);

/* dQ [B, H, M, D] (replaces flash_triton.py:617). */
int fa_bwd_dq(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v,
              const fa_tensor* d_o, const float* lse, const float* delta, const fa_tensor* dq,
              const void* plan, int32_t* status, void* stream);

/* Debug: materialise the kernels' decisions. keep is [B, id_heads, M, N] bytes (1 = unmasked),
 * produced by the same device predicate the attention kernels use; tile_class is
 * [B, id_heads, ceil(M/128), ceil(N/128)] bytes: bit0 visited, bit1 bound/causal check,
 * bit2 id check, bit3 query tail, bit4 / bit5 key / query codes of the block are monotone.
 * Either pointer may be NULL. */
int fa_debug_mask(const fa_problem* p, const void* plan, uint8_t* keep, uint8_t* tile_class, void* stream);

/* Size of the plan array built into the library for fa_fwd_static_plan (1 MiB per GPU). It holds
 * the plan of, e.g., one 32768-token sequence with head-broadcast ids (0.27 MB) or a batch of
 * 12 such 4096-token sequences; fa_plan_bytes() tells the size for any problem. */
#define FA_STATIC_PLAN_BYTES (1u << 20)

/* Forward for callers that cannot allocate device memory (no counterpart in the reference, whose
 * launcher allocates with torch, flash_triton.py:539-540). Same result as fa_plan_build + fa_fwd,
 * but the mask plan is built in a fixed FA_STATIC_PLAN_BYTES array inside the library instead of
 * a caller-allocated buffer, and the call allocates nothing. q, k, v, o, lse, eq, ek, status are
 * passed as for the other entry points (eq / ek may be NULL when mode == FA_MODE0_NOPE).
 * Returns FA_ERR_SCRATCH_LIMIT when the plan would not fit. The array is shared by all calls on a
 * GPU: it keeps the previous call's contents (every element read is overwritten first, nothing
 * needs clearing) and calls that overlap on the same GPU race. The first call on a device looks
 * up the array's address; make it before any stream capture on that device. */
int fa_fwd_static_plan(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v,
                       const fa_tensor* o, float* lse, const fa_ids* eq, const fa_ids* ek, int32_t* status,
                       void* stream);

/* Largest query length fa_group_rows sorts (one CTA sorts a row in shared memory). */
#define FA_GROUP_MAX_ROWS 16384

/* Grouping of the queries by id for calls WITHOUT a causal mask, where the order of the query rows is
 * free (no counterpart in the reference, which evaluates every tile whatever the ids,
 * flash_triton.py:94-129). Sorts each id row of eq [B, id_heads, M] by the 32-bit code the mask plan
 * uses for it (ids >= 0 share one code, which sorts last), stable, so rows that are grouped already keep
 * their places. Writes three int32 arrays [B, id_heads, M], contiguous: `order` (grouped position ->
 * caller's position), `inverse` (caller's position -> grouped position) and `grouped_ids` (the ids in
 * grouped order; pass them as the eq of fa_plan_build). p->M <= FA_GROUP_MAX_ROWS, else
 * FA_ERR_UNSUPPORTED. An id below -2^31 sets status 200 as in fa_plan_build. */
int fa_group_rows(const fa_problem* p, const fa_ids* eq, int32_t* order, int32_t* inverse, int32_t* grouped_ids,
                  int32_t* status, void* stream);

/* dst[b, h, i, :] = src[b, h, index[b, he, i], :] for [B, H, M, D] tensors of p->dtype (he = h, or 0 when
 * p->id_heads == 1); index is [B, id_heads, M] int32 with values in [0, M). With `order` it gathers q or dO
 * into the grouped order, with `inverse` it puts o or dQ back. src and dst must not overlap; both need a
 * 16-byte aligned base, last stride 1 and other strides that are whole 16-byte units. */
int fa_permute_rows(const fa_problem* p, const fa_tensor* src, const fa_tensor* dst, const int32_t* index,
                    void* stream);

/* Test hook for the failure path (no counterpart in the reference, which has no failure handling):
 * one warp waits on a barrier nobody arrives at, with the kernels' own bounded wait and a limit of
 * `limit_clocks` SM clocks. The wait gives up, the kernel returns normally and `*status` holds
 * 100 + role (role in 0..97). With a few thousand clocks this takes microseconds; nothing faults,
 * traps or hangs. */
int fa_debug_wait_timeout(int32_t* status, int64_t limit_clocks, int32_t role, void* stream);

/* Host-only helper, no GPU involved: the tile classification the kernels apply to tile
 * (qb, kb) given the id-code min/max of its query block and key block. Returns the tile_class
 * bits of fa_debug_mask. Exposed so that the block-skipping rule can be tested on a CPU
 * (no counterpart in the reference, which never skips a tile). */
uint32_t fa_classify_tile(int32_t M, int32_t N, int32_t causal, int32_t mode, int32_t qb, int32_t kb,
                          int32_t qmin, int32_t qmax, int32_t kmin, int32_t kmax);

#ifdef __cplusplus
}
#endif
#endif /* FA_B200_H_ */
