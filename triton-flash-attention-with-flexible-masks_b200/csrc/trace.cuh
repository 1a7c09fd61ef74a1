// Optional in-kernel timeline for tuning: compiled in only with -DFA_TRACE (never in the shipped
// library). CTA (0,0,0) records (SM clock, event id) pairs per role; fa_trace_dump() copies them out.
#pragma once
#include <cuda_runtime.h>

#ifdef FA_TRACE
namespace fa {
constexpr int kTraceRoles = 4;   // 0: compute group 0, 1: compute group 1, 2: MMA issuer, 3: producer
constexpr int kTraceCap = 1024;
__device__ unsigned long long g_trace[kTraceRoles][kTraceCap];
__device__ int g_trace_n[kTraceRoles];
// The slot counter lives in a register of the (single) recording thread of each role, so that an
// event costs one fire-and-forget global store and does not stall the recorder.
__device__ __forceinline__ void trace_event(int role, int ev, int& n) {
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        if (n < kTraceCap) g_trace[role][n] = (static_cast<unsigned long long>(clock64()) << 8) | unsigned(ev & 255);
        ++n;
        g_trace_n[role] = n;
    }
}
}  // namespace fa
#define FA_TRACE_DECL int fa_trace_n = 0;
#define FA_TRACE_EV(role, ev) ::fa::trace_event(role, ev, fa_trace_n)
#define FA_TRACE_DUMP_FN(name)                                                                     \
    extern "C" int name(unsigned long long* host_events, int* host_counts) {                       \
        cudaMemcpyFromSymbol(host_events, ::fa::g_trace, sizeof(::fa::g_trace));                   \
        cudaMemcpyFromSymbol(host_counts, ::fa::g_trace_n, sizeof(::fa::g_trace_n));               \
        int zero[::fa::kTraceRoles] = {};                                                           \
        cudaMemcpyToSymbol(::fa::g_trace_n, zero, sizeof(zero));                                    \
        return 0;                                                                                  \
    }
#else
#define FA_TRACE_DECL
#define FA_TRACE_EV(role, ev) ((void)0)
#define FA_TRACE_DUMP_FN(name)
#endif
