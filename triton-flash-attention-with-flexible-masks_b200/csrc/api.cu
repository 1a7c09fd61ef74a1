// extern "C" surface of the library (declared in include/fa_b200.h): argument checks, TMA
// tensor-map encoding, parameter packing and launches. Nothing here allocates or synchronises.
#include <cstdlib>
#include <mutex>
#include "../../include/fa_b200.h"
#include "common.cuh"
#include "params.cuh"

namespace fa {
cudaError_t launch_plan_build(const void*, const int64_t*, int, const void*, const int64_t*, int, int32_t*,
                              const PlanLayout&, int, int, int*, cudaStream_t);
cudaError_t launch_debug_mask(const MaskArgs&, uint8_t*, uint8_t*, cudaStream_t);
cudaError_t launch_fwd(int, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                       const FwdParams&, int, cudaStream_t);
cudaError_t launch_bwd_delta(const DeltaParams&, cudaStream_t);
cudaError_t launch_bwd_dkdv(int, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                            const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const DkdvParams&, int,
                            cudaStream_t);
cudaError_t launch_bwd_dq(int, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                          const CUtensorMap&, const CUtensorMap&, const DqParams&, int, cudaStream_t);

// fp32 path (attn_f32.cu)
cudaError_t launch_f32(int which, int D, const F32Params& p, cudaStream_t stream);
}  // namespace fa

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime so that the library has no link-time
// dependency on libcuda (it must load, and list its symbols, on a machine without a driver).
EncodeFn encode_fn() {
    static EncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(p);
    });
    return fn;
}

int check_problem(const fa_problem* p) {
    if (!p) return FA_ERR_BAD_ARG;
    if (p->B <= 0 || p->H <= 0 || p->Hk <= 0 || p->M <= 0 || p->N <= 0) return FA_ERR_BAD_ARG;
    if (p->H % p->Hk != 0) return FA_ERR_BAD_ARG;
    if (p->mode != FA_MODE0_NOPE && p->mode != FA_MODE1_DOC) return FA_ERR_BAD_ARG;
    if (p->id_heads != 1 && p->id_heads != p->H) return FA_ERR_BAD_ARG;
    if (p->causal && p->N < p->M) return FA_ERR_BAD_ARG;  // flash_triton.py:520
    if (p->dtype == FA_FP32) {  // fp32 FMA kernels: every head dim of the reference (flash_triton.py:512)
        if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128) return FA_ERR_UNSUPPORTED;
    } else {
        // Head dims 16 and 32 run on the 64-wide tensor-core kernels: their tensor maps cover the real head
        // dim, so the TMA loads fill the missing columns of each 64-column box with zeros (they add nothing
        // to Q K^T and give zero output columns) and the TMA stores write the real columns only.
        if (p->D != 16 && p->D != 32 && p->D != 64 && p->D != 128) return FA_ERR_UNSUPPORTED;
        if (p->dtype != FA_BF16 && p->dtype != FA_FP16) return FA_ERR_UNSUPPORTED;
    }
    if (!(p->sm_scale > 0.f)) return FA_ERR_UNSUPPORTED;
    if (fa::cdiv(p->N, fa::kBlk) > fa::kListCap || fa::cdiv(p->M, fa::kBlk) > fa::kListCap)
        return FA_ERR_UNSUPPORTED;  // at most 1024 blocks (131072 tokens) per sequence
    if (p->H > 65535 || p->B > 65535) return FA_ERR_UNSUPPORTED;
    return FA_OK;
}

int check_tensor(const fa_tensor* t, int B, int H, int L) {
    if (!t || !t->ptr) return FA_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(t->ptr) % 16 != 0) return FA_ERR_ALIGNMENT;
    if (t->stride[3] != 1) return FA_ERR_ALIGNMENT;
    const int ext[3] = {B, H, L};
    for (int i = 0; i < 3; ++i) {
        if (ext[i] > 1 && (t->stride[i] <= 0 || t->stride[i] % 8 != 0)) return FA_ERR_ALIGNMENT;
    }
    return FA_OK;
}

// fp32 tensors are read and written with plain loads and stores: 4-byte aligned base, last stride 1
int check_tensor_f32(const fa_tensor* t, int B, int H, int L) {
    if (!t || !t->ptr) return FA_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(t->ptr) % 4 != 0) return FA_ERR_ALIGNMENT;
    if (t->stride[3] != 1) return FA_ERR_ALIGNMENT;
    const int ext[3] = {B, H, L};
    for (int i = 0; i < 3; ++i) {
        if (ext[i] > 1 && t->stride[i] <= 0) return FA_ERR_ALIGNMENT;
    }
    return FA_OK;
}

fa::F32Tensor f32_view(const fa_tensor* t) {
    return fa::F32Tensor{static_cast<float*>(t->ptr), t->stride[0], t->stride[1], t->stride[2]};
}

// 4-D map over [B, H, L, D]; box = 64 elements of D x 128 rows of L; 128-byte swizzle; rows
// outside [0, L) and (head dims 16 and 32) columns outside [0, D) read as zero and are not written.
int make_map(CUtensorMap* out, const fa_tensor* t, int dtype, int B, int H, int L, int D) {
    EncodeFn fn = encode_fn();
    if (!fn) return FA_ERR_NO_DRIVER;
    const cuuint64_t dims[4] = {cuuint64_t(D), cuuint64_t(L), cuuint64_t(H), cuuint64_t(B)};
    // extent-1 dimensions may carry any stride in the caller's view; give the driver a sane one
    const int64_t sl = (L > 1) ? t->stride[2] : D;
    const int64_t sh = (H > 1) ? t->stride[1] : sl * L;
    const int64_t sb = (B > 1) ? t->stride[0] : sh * H;
    const cuuint64_t strides[3] = {cuuint64_t(sl) * 2, cuuint64_t(sh) * 2, cuuint64_t(sb) * 2};
    const cuuint32_t box[4] = {64, cuuint32_t(fa::kBlk), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r =
        fn(out, dtype == FA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, t->ptr,
           dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FA_OK : FA_ERR_TENSORMAP;
}

constexpr size_t kCtrWords = 128;  // size of the plan's counter section (PlanLayout::off_ctr)

// Debug switches, read from the environment at every call so that a test can flip them:
// FA_B200_NO_SKIP=1 visits every tile inside the causal / length bound, FA_B200_ALL_PARTIAL=1 evaluates
// the mask entry by entry on every visited tile. Results do not change (the forward's last bits can, with
// FA_B200_NO_SKIP, because tiles are dealt to its two accumulation chains by their position in the walk).
int debug_flags() {
    auto on = [](const char* name) {
        const char* e = getenv(name);
        return e && e[0] != '\0' && !(e[0] == '0' && e[1] == '\0');
    };
    return (on("FA_B200_NO_SKIP") ? fa::DBG_NO_SKIP : 0) | (on("FA_B200_ALL_PARTIAL") ? fa::DBG_ALL_PARTIAL : 0);
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int make_mask(fa::MaskArgs* m, const fa_problem* p, const void* plan) {
    if (p->mode == FA_MODE1_DOC && !plan) return FA_ERR_PLAN_SIZE;
    if (!aligned16(plan)) return FA_ERR_ALIGNMENT;  // the kernels read it with 16-byte and bulk loads
    m->plan = (p->mode == FA_MODE1_DOC) ? static_cast<const int32_t*>(plan) : nullptr;
    m->He = (p->mode == FA_MODE1_DOC) ? p->id_heads : 1;
    m->L = fa::PlanLayout(p->B, m->He, p->M, p->N);
    // the kernels count in the plan although the entry points take it as const: see fa_plan_build in the header
    unsigned int* words = static_cast<unsigned int*>(const_cast<void*>(plan));
    m->ctr = !plan ? nullptr : (p->mode == FA_MODE1_DOC) ? words + m->L.off_ctr : words;
    m->M = p->M;
    m->N = p->N;
    m->gap = p->N > p->M ? p->N - p->M : 0;  // flash_triton.py:521
    m->causal = p->causal ? 1 : 0;
    m->mode = p->mode;
    m->debug = debug_flags();
    return FA_OK;
}

fa::OutTensor out_view(const fa_tensor* t) { return fa::OutTensor{t->ptr, t->stride[0], t->stride[1], t->stride[2]}; }

constexpr float kLog2e = 1.4426950408889634f;

// Limit of one bounded wait inside the kernels, in SM clocks: FA_B200_WAIT_LIMIT_CLOCKS if set to a
// number >= 10000 when the library is first used, else the built-in default.
long long wait_limit_clocks() {
    static const long long v = [] {
        const char* e = getenv("FA_B200_WAIT_LIMIT_CLOCKS");
        if (e) {
            const long long x = atoll(e);
            if (x >= 10000) return x;
        }
        return fa::kWaitLimitClocks;
    }();
    return v;
}

// Number of SMs of the current device (persistent kernels launch one CTA per SM); cached per device.
// Heads per scheduling group of the persistent kernels (see their `decode`): as many heads as
// stream through L2 side by side without evicting each other. Measured on B200 (126 MB L2):
//  - document masks (32 heads x 32768 tokens, 64 documents): a CTA only streams the blocks of its own
//    document, and interleaving all 32 heads is fastest (groups of 1 head: 8 % slower, all CTAs pull
//    the same lines at once);
//  - no id mask, 512 heads x 8192 tokens, D = 128: groups of 8 heads (32 MB of K + V) are 14 % faster
//    than groups of 32 and draw less power; hundreds of 2048-token heads in one group: 30 % slower.
int head_group(const fa_problem* p, int heads_total) {
    int gh = 32;
    if (p->mode == FA_MODE0_NOPE) {
        const int64_t per_head = int64_t(p->M > p->N ? p->M : p->N) * p->D * 2 * 2;  // two streamed tensors
        const int64_t fit = (int64_t(32) << 20) / (per_head > 0 ? per_head : 1);
        gh = fit < 1 ? 1 : fit > 32 ? 32 : int(fit);
    }
    return gh < heads_total ? gh : heads_total;
}

int sm_count() {
    static std::mutex mu;
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return -1;
        cached[dev] = n;
    }
    return cached[dev];
}

// fp32 inputs: which = 0 forward, 1 delta, 2 dK / dV, 3 dQ; absent tensors are null
int run_f32(int which, const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v, const fa_tensor* o,
            const fa_tensor* d_o, const fa_tensor* dq, const fa_tensor* dk, const fa_tensor* dv, float* lse, float* delta,
            const void* plan, void* stream) {
    int rc;
    fa::F32Params fp{};
    const struct { const fa_tensor* t; fa::F32Tensor* dst; int H, L; } all[8] = {
        {q, &fp.q, p->H, p->M}, {k, &fp.k, p->Hk, p->N}, {v, &fp.v, p->Hk, p->N}, {o, &fp.o, p->H, p->M},
        {d_o, &fp.d_o, p->H, p->M}, {dq, &fp.dq, p->H, p->M}, {dk, &fp.dk, p->Hk, p->N}, {dv, &fp.dv, p->Hk, p->N}};
    for (const auto& a : all) {
        if (!a.t) continue;
        if ((rc = check_tensor_f32(a.t, p->B, a.H, a.L))) return rc;
        *a.dst = f32_view(a.t);
    }
    fa_problem pm = *p;
    if (which == 1) pm.mode = FA_MODE0_NOPE;  // the row sums do not depend on the mask (and take no plan)
    if ((rc = make_mask(&fp.mask, &pm, plan))) return rc;
    fp.lse = lse;
    fp.delta = delta;
    fp.B = p->B; fp.H = p->H; fp.Hk = p->Hk; fp.G = p->H / p->Hk;
    fp.scale = p->sm_scale;
    return fa::launch_f32(which, p->D, fp, static_cast<cudaStream_t>(stream)) == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

}  // namespace

extern "C" {

int fa_version(void) { return FA_VERSION; }

const char* fa_error_string(int code) {
    switch (code) {
        case FA_OK: return "ok";
        case FA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size, H % Hk != 0, causal with N < M)";
        case FA_ERR_UNSUPPORTED:
            return "unsupported problem (head dim must be 16, 32, 64 or 128, dtype bf16, fp16 or fp32, sm_scale > 0, "
                   "at most 131072 tokens per sequence)";
        case FA_ERR_ALIGNMENT:
            return "a buffer breaks the alignment rules (tensors: 16-byte aligned base, last stride 1, other strides "
                   "multiples of 8; lse, delta and plan: 16-byte aligned)";
        case FA_ERR_TENSORMAP: return "cuTensorMapEncodeTiled failed";
        case FA_ERR_LAUNCH: return "kernel launch failed";
        case FA_ERR_PLAN_SIZE: return "mask plan missing or too small";
        case FA_ERR_NO_DRIVER: return "CUDA driver entry point cuTensorMapEncodeTiled not available";
        case FA_ERR_SCRATCH_LIMIT: return "mask plan larger than the library's built-in FA_STATIC_PLAN_BYTES array";
        default: return "unknown error";
    }
}

int64_t fa_padded_rows(int32_t M) { return fa::pad128(M); }

int fa_plan_bytes(const fa_problem* p, size_t* bytes) {
    if (!bytes) return FA_ERR_BAD_ARG;
    const int rc = check_problem(p);
    if (rc) return rc;
    if (p->mode == FA_MODE0_NOPE) {
        *bytes = kCtrWords * sizeof(int32_t);  // the work counters only
        return FA_OK;
    }
    fa::PlanLayout L(p->B, p->id_heads, p->M, p->N);
    *bytes = size_t(L.total) * sizeof(int32_t);
    return FA_OK;
}

int fa_plan_build(const fa_problem* p, const fa_ids* eq, const fa_ids* ek, void* plan, size_t plan_bytes,
                  int32_t* status, void* stream) {
    const int rc = check_problem(p);
    if (rc) return rc;
    if (p->mode != FA_MODE1_DOC) {  // no mask data: the plan is the work counters, cleared here
        if (!plan) return FA_OK;
        if (reinterpret_cast<uintptr_t>(plan) % 16 != 0) return FA_ERR_ALIGNMENT;
        if (plan_bytes < kCtrWords * sizeof(int32_t)) return FA_ERR_PLAN_SIZE;
        return cudaMemsetAsync(plan, 0, kCtrWords * sizeof(int32_t), static_cast<cudaStream_t>(stream)) == cudaSuccess
                   ? FA_OK : FA_ERR_LAUNCH;
    }
    if (!eq || !ek || !eq->ptr || !ek->ptr || !plan || !status) return FA_ERR_BAD_ARG;
    if ((eq->dtype != FA_ID_INT32 && eq->dtype != FA_ID_INT64) || (ek->dtype != FA_ID_INT32 && ek->dtype != FA_ID_INT64))
        return FA_ERR_BAD_ARG;
    if (reinterpret_cast<uintptr_t>(plan) % 16 != 0) return FA_ERR_ALIGNMENT;
    fa::PlanLayout L(p->B, p->id_heads, p->M, p->N);
    if (plan_bytes < size_t(L.total) * sizeof(int32_t)) return FA_ERR_PLAN_SIZE;
    const int gap = p->N > p->M ? p->N - p->M : 0;
    const cudaError_t e = fa::launch_plan_build(eq->ptr, eq->stride, eq->dtype == FA_ID_INT64, ek->ptr, ek->stride,
                                                ek->dtype == FA_ID_INT64, static_cast<int32_t*>(plan), L, gap,
                                                p->causal ? 1 : 0, status, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

int fa_fwd(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v, const fa_tensor* o,
           float* lse, const void* plan, int32_t* status, void* stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    if (!lse || !status) return FA_ERR_BAD_ARG;
    if (!aligned16(lse)) return FA_ERR_ALIGNMENT;
    if (p->dtype == FA_FP32) return run_f32(0, p, q, k, v, o, nullptr, nullptr, nullptr, nullptr, lse, nullptr, plan, stream);
    if ((rc = check_tensor(q, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(k, p->B, p->Hk, p->N))) return rc;
    if ((rc = check_tensor(v, p->B, p->Hk, p->N))) return rc;
    if ((rc = check_tensor(o, p->B, p->H, p->M))) return rc;
    fa::FwdParams fp;
    if ((rc = make_mask(&fp.mask, p, plan))) return rc;
    CUtensorMap tq, tk, tv, to;
    if ((rc = make_map(&tq, q, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    if ((rc = make_map(&tk, k, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    if ((rc = make_map(&tv, v, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    if ((rc = make_map(&to, o, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    const int sms = sm_count();
    if (sms <= 0) return FA_ERR_LAUNCH;
    fp.lse = lse;
    fp.H = p->H;
    fp.B = p->B;
    fp.G = p->H / p->Hk;
    fp.gh = head_group(p, p->H * p->B);
    fp.by_length = (p->mode == FA_MODE1_DOC && int64_t(fa::cdiv(p->M, fa::kBlk) * p->H * p->B) < 32 * int64_t(sms)) ? 1 : 0;
    fp.scale_log2 = p->sm_scale * kLog2e;
    fp.status = status;
    fp.wait_limit = wait_limit_clocks();
    const cudaError_t e =
        fa::launch_fwd(p->D, p->dtype == FA_BF16, tq, tk, tv, to, fp, sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

int fa_bwd_delta(const fa_problem* p, const fa_tensor* o, const fa_tensor* d_o, float* delta, void* stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    if (!delta) return FA_ERR_BAD_ARG;
    if (!aligned16(delta)) return FA_ERR_ALIGNMENT;
    if (p->dtype == FA_FP32)
        return run_f32(1, p, nullptr, nullptr, nullptr, o, d_o, nullptr, nullptr, nullptr, nullptr, delta, nullptr, stream);
    if ((rc = check_tensor(o, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(d_o, p->B, p->H, p->M))) return rc;
    fa::DeltaParams dp;
    dp.o = out_view(o);
    dp.d_o = out_view(d_o);
    dp.delta = delta;
    dp.B = p->B; dp.H = p->H; dp.M = p->M; dp.D = p->D;
    dp.Mpad = fa::pad128(p->M);
    dp.bf16 = p->dtype == FA_BF16;
    const cudaError_t e = fa::launch_bwd_delta(dp, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

int fa_bwd_dkdv(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v,
                const fa_tensor* d_o, const float* lse, const float* delta, const fa_tensor* dk, const fa_tensor* dv,
                const void* plan, int32_t* status, void* stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    if (!lse || !delta || !status) return FA_ERR_BAD_ARG;
    if (!aligned16(lse) || !aligned16(delta)) return FA_ERR_ALIGNMENT;  // read with bulk copies
    if (p->dtype == FA_FP32)
        return run_f32(2, p, q, k, v, nullptr, d_o, nullptr, dk, dv, const_cast<float*>(lse), const_cast<float*>(delta), plan, stream);
    if ((rc = check_tensor(q, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(d_o, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(k, p->B, p->Hk, p->N))) return rc;
    if ((rc = check_tensor(v, p->B, p->Hk, p->N))) return rc;
    if ((rc = check_tensor(dk, p->B, p->Hk, p->N))) return rc;
    if ((rc = check_tensor(dv, p->B, p->Hk, p->N))) return rc;
    fa::DkdvParams kp;
    if ((rc = make_mask(&kp.mask, p, plan))) return rc;
    CUtensorMap tq, tk, tv, tdo;
    if ((rc = make_map(&tq, q, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    if ((rc = make_map(&tdo, d_o, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    if ((rc = make_map(&tk, k, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    if ((rc = make_map(&tv, v, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    CUtensorMap tdk, tdv;
    if ((rc = make_map(&tdk, dk, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    if ((rc = make_map(&tdv, dv, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    const int sms = sm_count();
    if (sms <= 0) return FA_ERR_LAUNCH;
    kp.lse = lse;
    kp.delta = delta;
    kp.B = p->B;
    kp.H = p->H;
    kp.Hk = p->Hk;
    kp.G = p->H / p->Hk;
    kp.gh = head_group(p, p->Hk * p->B);
    kp.by_length = (p->mode == FA_MODE1_DOC && int64_t(fa::cdiv(p->N, fa::kBlk) * p->Hk * p->B) < 32 * int64_t(sms)) ? 1 : 0;
    kp.scale_log2 = p->sm_scale * kLog2e;
    kp.sm_scale = p->sm_scale;
    kp.status = status;
    kp.wait_limit = wait_limit_clocks();
    const cudaError_t e =
        fa::launch_bwd_dkdv(p->D, p->dtype == FA_BF16, tq, tk, tv, tdo, tdk, tdv, kp, sms,
                            static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

int fa_bwd_dq(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v, const fa_tensor* d_o,
              const float* lse, const float* delta, const fa_tensor* dq, const void* plan, int32_t* status,
              void* stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    if (!lse || !delta || !status) return FA_ERR_BAD_ARG;
    if (!aligned16(lse) || !aligned16(delta)) return FA_ERR_ALIGNMENT;  // read with bulk copies
    if (p->dtype == FA_FP32)
        return run_f32(3, p, q, k, v, nullptr, d_o, dq, nullptr, nullptr, const_cast<float*>(lse), const_cast<float*>(delta), plan, stream);
    if ((rc = check_tensor(q, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(d_o, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(dq, p->B, p->H, p->M))) return rc;
    if ((rc = check_tensor(k, p->B, p->Hk, p->N))) return rc;
    if ((rc = check_tensor(v, p->B, p->Hk, p->N))) return rc;
    fa::DqParams qp;
    if ((rc = make_mask(&qp.mask, p, plan))) return rc;
    CUtensorMap tq, tk, tv, tdo;
    if ((rc = make_map(&tq, q, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    if ((rc = make_map(&tdo, d_o, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    if ((rc = make_map(&tk, k, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    if ((rc = make_map(&tv, v, p->dtype, p->B, p->Hk, p->N, p->D))) return rc;
    CUtensorMap tdq;
    if ((rc = make_map(&tdq, dq, p->dtype, p->B, p->H, p->M, p->D))) return rc;
    const int sms = sm_count();
    if (sms <= 0) return FA_ERR_LAUNCH;
    qp.lse = lse;
    qp.delta = delta;
    qp.B = p->B;
    qp.H = p->H;
    qp.G = p->H / p->Hk;
    qp.gh = head_group(p, p->H * p->B);
    qp.by_length = (p->mode == FA_MODE1_DOC && int64_t(fa::cdiv(p->M, fa::kBlk) * p->H * p->B) < 32 * int64_t(sms)) ? 1 : 0;
    qp.scale_log2 = p->sm_scale * kLog2e;
    qp.sm_scale = p->sm_scale;
    qp.status = status;
    qp.wait_limit = wait_limit_clocks();
    const cudaError_t e =
        fa::launch_bwd_dq(p->D, p->dtype == FA_BF16, tq, tk, tv, tdo, tdq, qp, sms, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

uint32_t fa_classify_tile(int32_t M, int32_t N, int32_t causal, int32_t mode, int32_t qb, int32_t kb, int32_t qmin,
                          int32_t qmax, int32_t kmin, int32_t kmax) {
    const int gap = N > M ? N - M : 0;
    return fa::classify_tile(qb, kb, M, N, gap, causal ? 1 : 0, mode, qmin, qmax, kmin, kmax);
}

int fa_debug_mask(const fa_problem* p, const void* plan, uint8_t* keep, uint8_t* tile_class, void* stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    fa::MaskArgs m;
    if ((rc = make_mask(&m, p, plan))) return rc;
    const cudaError_t e = fa::launch_debug_mask(m, keep, tile_class, static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}

}  // extern "C"
