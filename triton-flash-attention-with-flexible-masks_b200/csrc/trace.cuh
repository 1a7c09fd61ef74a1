// Optional in-kernel timeline for tuning: compiled in only with -DFA_TRACE (never in the shipped
// library). CTA (0,0,0) records (event id, 32-bit SM clock) pairs per role; the dump function copies
// them out and clears the buffer. An event is one clock read and one fire-and-forget store.
#pragma once
#include <cuda_runtime.h>

#ifdef FA_TRACE
namespace fa {
constexpr int kTraceRoles = 6;   // 0/1: compute groups, 2/3: MMA issuers, 4: producer, 5: scheduler
constexpr int kTraceCap = 2048;
__device__ unsigned long long g_trace[kTraceRoles][kTraceCap];
__device__ __forceinline__ void trace_event(bool on, int role, int ev, int& n) {
    if (on) {
        unsigned c;
        asm volatile("mov.u32 %0, %%clock;" : "=r"(c));
        if (n < kTraceCap) g_trace[role][n] = (static_cast<unsigned long long>(ev + 1) << 32) | c;
        ++n;
    }
}
}  // namespace fa
#define FA_TRACE_DECL int fa_trace_n = 0; const bool fa_trace_on = (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0);
#define FA_TRACE_EV(role, ev) ::fa::trace_event(fa_trace_on, role, ev, fa_trace_n)
#define FA_TRACE_DUMP_FN(name)                                                                     \
    extern "C" int name(unsigned long long* host_events) {                                         \
        cudaMemcpyFromSymbol(host_events, ::fa::g_trace, sizeof(::fa::g_trace));                   \
        void* sym = nullptr;                                                                       \
        cudaGetSymbolAddress(&sym, ::fa::g_trace);                                                 \
        cudaMemset(sym, 0, sizeof(::fa::g_trace));                                                 \
        return ::fa::kTraceRoles * ::fa::kTraceCap;                                                \
    }
#else
#define FA_TRACE_DECL
#define FA_TRACE_EV(role, ev) ((void)0)
#define FA_TRACE_DUMP_FN(name)
#endif
