// Shared device helpers: activations, reductions, launch bookkeeping.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gridnet_b200.h"

#ifndef GN_ACCURATE_SIGMOID
#define GN_ACCURATE_SIGMOID 0
#endif

namespace gn {

constexpr int kNumSMs = 148;  // B200; only the fallback where the device cannot be asked
int sm_count();                // multiprocessor count of the current device (status.cu)

// Set by every launcher that sees a CUDA error; read by gn_last_cuda_error().
void record_cuda_error(cudaError_t e, const char *where);
int check_launch(const char *where);

// ---------------------------------------------------------------- activations
// exp(x) for float: ex2.approx on a product whose rounding error is fed back,
// so the relative error stays at a few ulp for every |x| (a plain
// __expf(x) loses |x| * 2^-24 in the product).
__device__ __forceinline__ float exp_f32(float x)
{
    const float l2e_hi = 1.4426950216293335f;   // float(log2(e))
    const float l2e_lo = 1.9259629911266175e-8f; // log2(e) - l2e_hi
    float t = x * l2e_hi;
    float r = fmaf(x, l2e_hi, -t);
    r = fmaf(x, l2e_lo, r);
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(t));
    return fmaf(p, r * 0.6931471805599453f, p);
}

__device__ __forceinline__ float sigmoid_(float x)
{
#if GN_ACCURATE_SIGMOID
    // 1 / (1 + exp(-x)). The exponent is capped at 87 so that exp stays finite (an overflowed
    // ex2 would turn the error-feedback term of exp_f32 into inf - inf); sigmoid(-87) = 1.6e-38.
    return __fdividef(1.0f, 1.0f + exp_f32(fminf(-x, 87.0f)));
#else
    // 1 / (1 + 2^(-x * log2 e)) in six instructions: FMUL, FMNMX, MUFU.EX2, FADD, MUFU.RCP
    // (+ the caller's multiply). The exponent is capped at 126 so that 1 + 2^t stays finite.
    // Relative error about |x| * 6e-8 from the rounded product plus 2 ulp from each MUFU.
    const float t = fminf(x * -1.4426950408889634f, 126.0f);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
#endif
}
__device__ __forceinline__ double sigmoid_(double x) { return 1.0 / (1.0 + exp(-x)); }

__device__ __forceinline__ float tanh_(float x) { return tanhf(x); }
__device__ __forceinline__ double tanh_(double x) { return tanh(x); }

// Forward value and derivative of the four activations of src/activations.h:51-138.
// The derivative at exactly 0 follows torch (relu'(0) = 0, leaky_relu'(0) = slope),
// because gridnet/backend_torch.py under autograd is the behaviour to match.
template <int ACT, typename R>
struct Act {
    static __device__ __forceinline__ R fwd(R h)
    {
        if (ACT == GN_ACT_RELU) return h > R(0) ? h : R(0);
        if (ACT == GN_ACT_LEAKY_RELU) return h > R(0) ? h : R(0.01) * h;
        if (ACT == GN_ACT_SILU) return h * sigmoid_(h);
        return tanh_(h);
    }
    // fwd and derivative together (they share the transcendental)
    static __device__ __forceinline__ void both(R h, R &f, R &d)
    {
        if (ACT == GN_ACT_RELU) {
            f = h > R(0) ? h : R(0);
            d = h > R(0) ? R(1) : R(0);
        } else if (ACT == GN_ACT_LEAKY_RELU) {
            f = h > R(0) ? h : R(0.01) * h;
            d = h > R(0) ? R(1) : R(0.01);
        } else if (ACT == GN_ACT_SILU) {
            R sg = sigmoid_(h);
            f = h * sg;
            d = sg * (R(1) + h * (R(1) - sg));
        } else {
            R th = tanh_(h);
            f = th;
            d = R(1) - th * th;
        }
    }
};

// ------------------------------------------------------------------ reductions
template <typename R>
__device__ __forceinline__ R warp_sum(R v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the whole CTA, result in every thread. `buf` needs 33 entries.
// Deterministic: fixed shuffle tree, then warp 0 adds the per-warp sums in order.
template <typename R>
__device__ __forceinline__ R block_sum(R v, R *buf)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // buf may still be read from a previous call
    if (lane == 0) buf[wid] = v;
    __syncthreads();
    if (wid == 0) {
        R t = lane < nw ? buf[lane] : R(0);
        t = warp_sum(t);
        if (lane == 0) buf[32] = t;
    }
    __syncthreads();
    return buf[32];
}

template <typename R>
__device__ __forceinline__ R sqrt_(R v);
template <>
__device__ __forceinline__ float sqrt_<float>(float v) { return sqrtf(v); }
template <>
__device__ __forceinline__ double sqrt_<double>(double v) { return sqrt(v); }

// Global loads that stay where they are written: the compiler may sink an ordinary read-only
// load past barriers down to its first use, which would put the whole memory latency back on
// the critical path of the stage the load was issued ahead of.
__device__ __forceinline__ float ld_pinned(const float *ptr)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ float2 ld_pinned2(const float *ptr)  // 8-byte aligned
{
    float2 v;
    asm volatile("ld.global.nc.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(ptr) : "memory");
    return v;
}

// How many ways to split the batch across CTAs so that the grid fills the GPU.
inline int pick_batch_chunks(long long grid_blocks, int B, int ctas_per_sm, int min_samples_per_cta = 1)
{
    long long want = 2LL * sm_count() * ctas_per_sm;  // about two waves
    long long c = (want + grid_blocks - 1) / grid_blocks;
    long long cmax = B / min_samples_per_cta;
    if (cmax < 1) cmax = 1;
    if (c > cmax) c = cmax;
    if (c < 1) c = 1;
    if (c > 65535) c = 65535;
    return (int)c;
}

// Splits the batch into chunks so that the CTAs finish in few, evenly filled rounds. The cost of a
// split is rounds * (samples per chunk + overhead), where a round is one CTA on every resident
// slot and the overhead is a CTA's fixed work (parameter loads, epilogue) in units of one sample.
inline int pick_batch_chunks_balanced(long long grid_blocks, int B, int ctas_per_sm, double overhead_samples,
                                      int max_chunks)
{
    const long long slots = (long long)sm_count() * ctas_per_sm;
    int best = 1;
    double best_cost = 1e300;
    for (int c = 1; c <= max_chunks && c <= B; ++c) {
        const int spc = (B + c - 1) / c;
        const int chunks = (B + spc - 1) / spc;
        const long long rounds = (grid_blocks * chunks + slots - 1) / slots;
        const double cost = (double)rounds * (spc + overhead_samples);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = chunks;
        }
    }
    return best;
}

}  // namespace gn
