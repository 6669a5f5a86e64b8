// Measurement helper: an FFMA-only kernel that fills every SM, so that the roofline of the step
// kernels can be quoted against a measured FP32 pipe rate instead of the nominal one
// (148 SMs x 128 lanes x 2 FLOP x clock). It is not on any product path.
#include "common.cuh"
#include "kernels.h"

namespace gn {

__global__ void __launch_bounds__(256) ffma_probe_k(float *sink, int iters)
{
    float a[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) a[k] = 1.0f + 1e-3f * (float)(threadIdx.x + k);
    const float m = 0.99999994f, c = 1e-7f;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int k = 0; k < 16; ++k) a[k] = fmaf(a[k], m, c);
    }
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; ++k) sum += a[k];
    if (sum == 123.456f) sink[0] = sum;  // keeps the chains alive; practically never true
}

int launch_ffma_probe(float *sink, int iters, long long *fma_count, cudaStream_t st)
{
    const int ctas = sm_count() * 8;  // 2048 threads per SM: every scheduler has warps to pick from
    ffma_probe_k<<<ctas, 256, 0, st>>>(sink, iters);
    if (fma_count) *fma_count = (long long)ctas * 256 * 16 * iters;
    return check_launch("ffma_probe");
}

}  // namespace gn
