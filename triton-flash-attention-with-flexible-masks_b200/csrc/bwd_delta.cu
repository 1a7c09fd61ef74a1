// delta[b,h,i] = sum_d O[b,h,i,d] * dO[b,h,i,d] in fp32. Replaces `_bwd_preprocess`
// (flash_triton.py:143-173). HBM-bound: reads O and dO once, writes one float per row.
// The output is padded to a multiple of 128 rows per (b,h); padding rows are written as 0 so
// that the backward kernels can bulk-copy whole 128-row slices.
#include <cuda_fp16.h>
#include "common.cuh"
#include "params.cuh"

namespace fa {

// 8 threads per row, 16 rows per CTA of 128 threads; each thread reads D/8 contiguous elements (at least 8:
// with head dims 16 and 32 only the first 2 or 4 threads of a row have any).
template <int D, bool BF16>
__global__ void __launch_bounds__(128) bwd_delta_kernel(const DeltaParams p) {
    const int h = blockIdx.y, b = blockIdx.z;
    const int row = blockIdx.x * 16 + (threadIdx.x >> 3);
    const int part = threadIdx.x & 7;
    constexpr int PER = (D >= 64) ? D / 8 : 8;  // elements per thread: 16 (D=128) or 8
    float acc = 0.f;
    if (row < p.M && part * PER < D) {
        const uint8_t* po = static_cast<const uint8_t*>(p.o.ptr) +
                            2 * (int64_t(b) * p.o.sb + int64_t(h) * p.o.sh + int64_t(row) * p.o.sl + part * PER);
        const uint8_t* pd = static_cast<const uint8_t*>(p.d_o.ptr) +
                            2 * (int64_t(b) * p.d_o.sb + int64_t(h) * p.d_o.sh + int64_t(row) * p.d_o.sl + part * PER);
#pragma unroll
        for (int v = 0; v < PER / 8; ++v) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(po) + v);
            const uint4 g = __ldg(reinterpret_cast<const uint4*>(pd) + v);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a0, a1, g0, g1;
                if constexpr (BF16) {
                    a0 = __uint_as_float(aw[k] << 16); a1 = __uint_as_float(aw[k] & 0xffff0000u);
                    g0 = __uint_as_float(gw[k] << 16); g1 = __uint_as_float(gw[k] & 0xffff0000u);
                } else {
                    const __half2 ah = *reinterpret_cast<const __half2*>(&aw[k]);
                    const __half2 gh = *reinterpret_cast<const __half2*>(&gw[k]);
                    a0 = __low2float(ah); a1 = __high2float(ah);
                    g0 = __low2float(gh); g1 = __high2float(gh);
                }
                acc = fmaf(a0, g0, acc);
                acc = fmaf(a1, g1, acc);
            }
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (part == 0 && row < p.Mpad) p.delta[(int64_t(b) * p.H + h) * p.Mpad + row] = acc;
}

cudaError_t launch_bwd_delta(const DeltaParams& p, cudaStream_t stream) {
    dim3 grid(unsigned(p.Mpad / 16), p.H, p.B);
    if (p.D == 128) {
        if (p.bf16) bwd_delta_kernel<128, true><<<grid, 128, 0, stream>>>(p);
        else bwd_delta_kernel<128, false><<<grid, 128, 0, stream>>>(p);
    } else if (p.D == 32) {
        if (p.bf16) bwd_delta_kernel<32, true><<<grid, 128, 0, stream>>>(p);
        else bwd_delta_kernel<32, false><<<grid, 128, 0, stream>>>(p);
    } else if (p.D == 16) {
        if (p.bf16) bwd_delta_kernel<16, true><<<grid, 128, 0, stream>>>(p);
        else bwd_delta_kernel<16, false><<<grid, 128, 0, stream>>>(p);
    } else {
        if (p.bf16) bwd_delta_kernel<64, true><<<grid, 128, 0, stream>>>(p);
        else bwd_delta_kernel<64, false><<<grid, 128, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace fa
