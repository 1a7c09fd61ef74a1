// fa_debug_wait_timeout: a test hook for the failure path of the attention kernels.
//
// Every mbarrier wait in the kernels is bounded (ptx.cuh `mbar_wait`): when the limit runs out the
// waiter raises the CTA's abort flag, records 100 + role in the device status word and returns, and
// the host finds the code with its next status check. Nothing in a healthy run ever takes that
// branch, and provoking it in a real kernel would need a GPU fault. This kernel runs the branch in
// the open: one warp waits, with a limit the caller chooses, on a barrier that nobody arrives at;
// the wait gives up after that many clocks (microseconds for a few thousand), the kernel returns
// normally, and the status word holds 100 + `role`. It touches no other memory.
#include "../../include/fa_b200.h"
#include "ptx.cuh"

namespace fa {

__global__ void __launch_bounds__(32) debug_wait_kernel(int* status, long long limit, int role) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int flag;
    if (threadIdx.x == 0) {
        flag = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncwarp();
    Abort ab{&flag, status, limit};
    // phase 0 of a barrier that expects one arrival which never comes
    const bool ok = mbar_wait(smem_u32(&bar), 0, ab, ST_WAIT_TIMEOUT + role);
    // a wait that did not time out would be a defect of the test hook itself: report it distinctly
    if (ok && threadIdx.x == 0) atomicCAS(status, 0, ST_WAIT_TIMEOUT + 98);
}

}  // namespace fa

extern "C" int fa_debug_wait_timeout(int32_t* status, int64_t limit_clocks, int32_t role, void* stream) {
    if (!status || limit_clocks < 1 || role < 0 || role > 97) return FA_ERR_BAD_ARG;
    fa::debug_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_clocks, role);
    return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_LAUNCH;
}
