// fa_fwd_static_plan: the forward pass for callers that cannot allocate device memory.
//
// Everywhere else in this library the caller sizes the mask plan with fa_plan_bytes(), allocates
// it, and hands it to fa_plan_build() and fa_fwd(). Some hosts have no allocator to do that with:
// a plugin inside a serving process whose memory was carved up once at start-up and which forbids
// cudaMalloc afterwards (cudaMalloc synchronises the whole device and can fail or fragment a pool
// that was sized to the last megabyte), or a plain C host that links this library without torch or
// any caching allocator of its own. For them the plan lives in the fixed array below, which is part
// of the library image: every GPU that loads the library holds FA_STATIC_PLAN_BYTES of it until
// the process exits, whether or not this entry point is ever called.
//
// Rules that follow from sharing one array:
//  - problems whose plan is larger than FA_STATIC_PLAN_BYTES are refused with FA_ERR_SCRATCH_LIMIT;
//  - the array keeps whatever the previous call left in it. Nothing in it has to start at zero:
//    the plan kernels (or, without ids, one 512-byte memset of the work counters) overwrite every
//    element the forward kernel reads, so no other clearing is done;
//  - two calls that are in flight on the same GPU at the same time (different streams) write and
//    read the same array and race. Serialise them on one stream or with events;
//  - the plan is not returned, so the backward entry points (which want the plan again) need a
//    caller-owned plan buffer; this entry point serves forward-only use.
//  - the first call on each device looks up the array's device address (see below); make that
//    first call before starting any stream capture on that device.
//
// The call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
#include <mutex>
#include "../../include/fa_b200.h"
#include <cuda_runtime.h>

// In host code this name is only a handle for the runtime, not a device address: a kernel given
// `g_static_plan` directly would read the wrong memory. The address kernels may use comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) int32_t g_static_plan[FA_STATIC_PLAN_BYTES / sizeof(int32_t)];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int32_t* g_plan_addr[kMaxDevices] = {};

// Device address of the static plan on the current device, or null with an error code.
int static_plan_address(int32_t** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FA_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_plan_addr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_plan);
        if (e != cudaSuccess || !p) return FA_ERR_LAUNCH;
        g_plan_addr[dev] = static_cast<int32_t*>(p);
    }
    *out = g_plan_addr[dev];
    return FA_OK;
}

}  // namespace

extern "C" int fa_fwd_static_plan(const fa_problem* p, const fa_tensor* q, const fa_tensor* k, const fa_tensor* v,
                                  const fa_tensor* o, float* lse, const fa_ids* eq, const fa_ids* ek,
                                  int32_t* status, void* stream) {
    size_t bytes = 0;
    int rc = fa_plan_bytes(p, &bytes);  // validates the problem as every other entry point does
    if (rc) return rc;
    if (bytes > FA_STATIC_PLAN_BYTES) return FA_ERR_SCRATCH_LIMIT;
    int32_t* plan = nullptr;
    if (bytes > 0) {
        if ((rc = static_plan_address(&plan))) return rc;
        if ((rc = fa_plan_build(p, eq, ek, plan, FA_STATIC_PLAN_BYTES, status, stream))) return rc;
    }
    return fa_fwd(p, q, k, v, o, lse, plan, status, stream);
}
