// Whole-grid normalisation between outer steps: per sample over P = M*N*K values,
// y = (x - mean) / sqrt(var + eps) * gamma + beta with the biased variance — what
// torch.nn.LayerNorm((M,N,K)) computes in the reference's models
// (gridnet/scripts/train_mnist.py:54,62-64; gridnet/scripts/train_imagenet.py:67,85-86).
//
// All reductions are two-stage and deterministic: fixed-shape partial sums in
// double precision, then one CTA per sample adds the partials in a fixed order.
// HBM-bound; float4 accesses when the pointers and P allow.
#include "common.cuh"
#include "kernels.h"

namespace gn {

static __device__ __forceinline__ bool aligned16(const void *p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// grid B * parts (one dimension: the batch is not limited by the 65535 of gridDim.y); slice length is a multiple
// of 4 so that slices stay float4-aligned
__global__ void __launch_bounds__(256) norm_partial_stats_k(const float *__restrict__ x,
                                                            double2 *__restrict__ partials, long long P,
                                                            long long slice, int parts)
{
    __shared__ double red[33];
    const int b = blockIdx.x / parts, part = blockIdx.x - b * parts;
    const float *xs = x + (size_t)b * P;
    const long long lo = (long long)part * slice;
    const long long hi = min(P, lo + slice);
    double s = 0.0, q = 0.0;
    if (aligned16(xs) && (P & 3) == 0) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xs);
        for (long long i = lo / 4 + threadIdx.x; i < hi / 4; i += blockDim.x) {
            const float4 v = x4[i];
            // float adds inside one vector, double across vectors
            const float ls = (v.x + v.y) + (v.z + v.w);
            const float lq = fmaf(v.x, v.x, v.y * v.y) + fmaf(v.z, v.z, v.w * v.w);
            s += (double)ls;
            q += (double)lq;
        }
    } else {
        for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const double v = (double)xs[i];
            s += v;
            q = fma(v, v, q);
        }
    }
    s = block_sum(s, red);
    q = block_sum(q, red);
    if (threadIdx.x == 0) partials[(size_t)b * parts + part] = make_double2(s, q);
}

// grid B; adds nparts partials in a fixed order
__global__ void __launch_bounds__(256) norm_finalize_k(const double2 *__restrict__ partials, int nparts,
                                                       float2 *__restrict__ stats, long long P, float eps)
{
    __shared__ double red[33];
    const int b = blockIdx.x;
    const double2 *ps = partials + (size_t)b * nparts;
    double s = 0.0, q = 0.0;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) {
        const double2 v = ps[i];
        s += v.x;
        q += v.y;
    }
    s = block_sum(s, red);
    q = block_sum(q, red);
    if (threadIdx.x == 0) {
        const double mean = s / (double)P;
        double var = q / (double)P - mean * mean;
        if (var < 0.0) var = 0.0;
        stats[b] = make_float2((float)mean, (float)(1.0 / sqrt(var + (double)eps)));
    }
}

// grid B * ceil(P / 1024), one dimension
__global__ void __launch_bounds__(256) norm_apply_k(const float *__restrict__ x, const float *__restrict__ gamma,
                                                    const float *__restrict__ beta,
                                                    const float2 *__restrict__ stats, float *__restrict__ y,
                                                    long long P, unsigned chunks)
{
    const int b = blockIdx.x / chunks;
    const unsigned chunk = blockIdx.x - (unsigned)b * chunks;
    const float2 mr = stats[b];
    const float *xs = x + (size_t)b * P;
    float *ys = y + (size_t)b * P;
    const long long i0 = ((long long)chunk * blockDim.x + threadIdx.x) * 4;
    if (i0 >= P) return;
    if ((P & 3) == 0 && aligned16(xs) && aligned16(ys) && aligned16(gamma) && aligned16(beta)) {
        const float4 v = *reinterpret_cast<const float4 *>(xs + i0);
        const float4 g = *reinterpret_cast<const float4 *>(gamma + i0);
        const float4 c = *reinterpret_cast<const float4 *>(beta + i0);
        float4 o;
        o.x = fmaf((v.x - mr.x) * mr.y, g.x, c.x);
        o.y = fmaf((v.y - mr.x) * mr.y, g.y, c.y);
        o.z = fmaf((v.z - mr.x) * mr.y, g.z, c.z);
        o.w = fmaf((v.w - mr.x) * mr.y, g.w, c.w);
        *reinterpret_cast<float4 *>(ys + i0) = o;
    } else {
        for (long long i = i0; i < min(P, i0 + 4); ++i) ys[i] = fmaf((xs[i] - mr.x) * mr.y, gamma[i], beta[i]);
    }
}

// The residual form of the model loop (gridnet/scripts/train_imagenet.py:81-83): n = LayerNorm(h);
// h' = h + (net(n) - n). Given h, y = net(n) and the statistics of h, writes h' (out may be h or y) and the
// per-sample partial sums of h' for the next step's statistics. grid B * parts, slices as in norm_partial_stats_k.
__global__ void __launch_bounds__(256) norm_residual_combine_k(const float *__restrict__ h, const float *__restrict__ y,
                                                               const float *__restrict__ gamma,
                                                               const float *__restrict__ beta,
                                                               const float2 *__restrict__ stats, float *out,
                                                               double2 *__restrict__ partials, long long P,
                                                               long long slice, int parts)
{
    __shared__ double red[33];
    const int b = blockIdx.x / parts, part = blockIdx.x - b * parts;
    const float2 mr = stats[b];
    const float *hs = h + (size_t)b * P;
    const float *ys = y + (size_t)b * P;
    float *os = out + (size_t)b * P;
    const long long lo = (long long)part * slice;
    const long long hi = min(P, lo + slice);
    double s = 0.0, q = 0.0;
    if ((P & 3) == 0 && aligned16(hs) && aligned16(ys) && aligned16(os) && aligned16(gamma) && aligned16(beta)) {
        for (long long i = lo / 4 + threadIdx.x; i < hi / 4; i += blockDim.x) {
            const float4 a = reinterpret_cast<const float4 *>(hs)[i];
            const float4 v = reinterpret_cast<const float4 *>(ys)[i];
            const float4 g = reinterpret_cast<const float4 *>(gamma)[i];
            const float4 c = reinterpret_cast<const float4 *>(beta)[i];
            float4 o;
            o.x = a.x + (v.x - fmaf((a.x - mr.x) * mr.y, g.x, c.x));
            o.y = a.y + (v.y - fmaf((a.y - mr.x) * mr.y, g.y, c.y));
            o.z = a.z + (v.z - fmaf((a.z - mr.x) * mr.y, g.z, c.z));
            o.w = a.w + (v.w - fmaf((a.w - mr.x) * mr.y, g.w, c.w));
            reinterpret_cast<float4 *>(os)[i] = o;
            const float ls = (o.x + o.y) + (o.z + o.w);
            const float lq = fmaf(o.x, o.x, o.y * o.y) + fmaf(o.z, o.z, o.w * o.w);
            s += (double)ls;
            q += (double)lq;
        }
    } else {
        for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float a = hs[i];
            const float o = a + (ys[i] - fmaf((a - mr.x) * mr.y, gamma[i], beta[i]));
            os[i] = o;
            s += (double)o;
            q = fma((double)o, (double)o, q);
        }
    }
    s = block_sum(s, red);
    q = block_sum(q, red);
    if (threadIdx.x == 0) partials[(size_t)b * parts + part] = make_double2(s, q);
}

// per-sample partial sums of a = sum(gy * gamma) and c = sum(gy * gamma * xhat); grid B * parts
__global__ void __launch_bounds__(256) norm_bwd_partial_k(const float *__restrict__ x,
                                                          const float *__restrict__ gamma,
                                                          const float *__restrict__ gy,
                                                          const float2 *__restrict__ stats,
                                                          double2 *__restrict__ partials, long long P,
                                                          long long slice, int parts)
{
    __shared__ double red[33];
    const int b = blockIdx.x / parts, part = blockIdx.x - b * parts;
    const float2 mr = stats[b];
    const float *xs = x + (size_t)b * P;
    const float *gs = gy + (size_t)b * P;
    const long long lo = (long long)part * slice;
    const long long hi = min(P, lo + slice);
    double a = 0.0, c = 0.0;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float gg = gs[i] * gamma[i];
        const float xh = (xs[i] - mr.x) * mr.y;
        a += (double)gg;
        c += (double)(gg * xh);
    }
    a = block_sum(a, red);
    c = block_sum(c, red);
    if (threadIdx.x == 0) partials[(size_t)b * parts + part] = make_double2(a, c);
}

// grid B: ac[b] = (a / P, c / P)
__global__ void __launch_bounds__(64) norm_bwd_finalize_k(const double2 *__restrict__ partials, int nparts,
                                                          float2 *__restrict__ ac, long long P)
{
    if (threadIdx.x != 0) return;
    const double2 *ps = partials + (size_t)blockIdx.x * nparts;
    double a = 0.0, c = 0.0;
    for (int i = 0; i < nparts; ++i) {
        a += ps[i].x;
        c += ps[i].y;
    }
    ac[blockIdx.x] = make_float2((float)(a / (double)P), (float)(c / (double)P));
}

// one thread per grid position i; walks the batch, so grad_gamma / grad_beta need no atomics
__global__ void __launch_bounds__(256) norm_bwd_apply_k(const float *__restrict__ x, const float *__restrict__ gamma,
                                                        const float *__restrict__ gy,
                                                        const float2 *__restrict__ stats,
                                                        const float2 *__restrict__ ac, float *__restrict__ gx,
                                                        float *__restrict__ ggamma, float *__restrict__ gbeta,
                                                        int B, long long P)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= P) return;
    const float gm = gamma[i];
    float dg = 0.0f, dbt = 0.0f;
    for (int b = 0; b < B; ++b) {
        const float2 mr = __ldg(&stats[b]);
        const float2 acb = __ldg(&ac[b]);
        const size_t o = (size_t)b * P + i;
        const float g = gy[o];
        const float xh = (x[o] - mr.x) * mr.y;
        gx[o] = mr.y * (g * gm - acb.x - xh * acb.y);
        dg = fmaf(g, xh, dg);
        dbt += g;
    }
    ggamma[i] = dg;
    gbeta[i] = dbt;
}

// grid B: sums[b] = sum over the nparts partials of sample b, in a fixed order (one thread per sample is plenty)
__global__ void __launch_bounds__(64) norm_sum_partials_k(const double2 *__restrict__ partials, int nparts,
                                                          double2 *__restrict__ sums)
{
    if (threadIdx.x != 0) return;
    const double2 *ps = partials + (size_t)blockIdx.x * nparts;
    double a = 0.0, c = 0.0;
    for (int i = 0; i < nparts; ++i) {
        a += ps[i].x;
        c += ps[i].y;
    }
    sums[blockIdx.x] = make_double2(a, c);
}

// grid B: ac[b] = sums[b] / P (the sums may come from an all-reduce over the ranks that share a grid)
__global__ void __launch_bounds__(64) norm_scale_sums_k(const double2 *__restrict__ sums, float2 *__restrict__ ac,
                                                        long long P)
{
    if (threadIdx.x != 0) return;
    const double2 v = sums[blockIdx.x];
    ac[blockIdx.x] = make_float2((float)(v.x / (double)P), (float)(v.y / (double)P));
}

// ------------------------------------------------------------------ launchers
int norm_pick_parts(long long P)
{
    long long parts = P / 8192;
    if (parts < 1) parts = 1;
    if (parts > kNormMaxParts) parts = kNormMaxParts;
    return (int)parts;
}

static long long slice_len(long long P, int parts)
{
    long long s = (P + parts - 1) / parts;
    return (s + 3) & ~3LL;
}

int launch_norm_partial_stats(const float *x, double2 *partials, int B, long long P, int parts, cudaStream_t st)
{
    norm_partial_stats_k<<<(unsigned)B * (unsigned)parts, 256, 0, st>>>(x, partials, P, slice_len(P, parts), parts);
    return check_launch("norm_partial_stats");
}

int launch_norm_finalize(const double2 *partials, int nparts, float2 *stats, int B, long long P, float eps,
                         cudaStream_t st)
{
    norm_finalize_k<<<B, 256, 0, st>>>(partials, nparts, stats, P, eps);
    return check_launch("norm_finalize");
}

int launch_norm_apply(const float *x, const float *gamma, const float *beta, const float2 *stats, float *y,
                      int B, long long P, cudaStream_t st)
{
    const unsigned chunks = (unsigned)((P + 1023) / 1024);
    norm_apply_k<<<(unsigned)B * chunks, 256, 0, st>>>(x, gamma, beta, stats, y, P, chunks);
    return check_launch("norm_apply");
}

int launch_norm_residual_combine(const float *h, const float *y, const float *gamma, const float *beta,
                                 const float2 *stats, float *out, double2 *partials, int B, long long P, int parts,
                                 cudaStream_t st)
{
    norm_residual_combine_k<<<(unsigned)B * (unsigned)parts, 256, 0, st>>>(h, y, gamma, beta, stats, out, partials, P,
                                                                          slice_len(P, parts), parts);
    return check_launch("norm_residual_combine");
}

int launch_norm_local_sums(const float *x, double2 *partials, double2 *sums, int B, long long P, int parts,
                           cudaStream_t st)
{
    norm_partial_stats_k<<<(unsigned)B * (unsigned)parts, 256, 0, st>>>(x, partials, P, slice_len(P, parts), parts);
    norm_sum_partials_k<<<B, 64, 0, st>>>(partials, parts, sums);
    return check_launch("norm_local_sums");
}

int launch_norm_backward_local_sums(const float *x, const float *gamma, const float *gy, const float2 *stats,
                                    double2 *partials, double2 *sums, int B, long long P, int parts, cudaStream_t st)
{
    norm_bwd_partial_k<<<(unsigned)B * (unsigned)parts, 256, 0, st>>>(x, gamma, gy, stats, partials, P, slice_len(P, parts),
                                                                     parts);
    norm_sum_partials_k<<<B, 64, 0, st>>>(partials, parts, sums);
    return check_launch("norm_backward_local_sums");
}

int launch_norm_backward_apply(const float *x, const float *gamma, const float *gy, const float2 *stats,
                               const double2 *sums, long long P_total, float2 *ac, float *gx, float *ggamma, float *gbeta,
                               int B, long long P, cudaStream_t st)
{
    norm_scale_sums_k<<<B, 64, 0, st>>>(sums, ac, P_total);
    norm_bwd_apply_k<<<(unsigned)((P + 255) / 256), 256, 0, st>>>(x, gamma, gy, stats, ac, gx, ggamma, gbeta, B, P);
    return check_launch("norm_backward_apply");
}

int launch_norm_backward(const float *x, const float *gamma, const float *gy, const float2 *stats,
                         double2 *partials, float2 *ac, float *gx, float *ggamma, float *gbeta, int B,
                         long long P, int parts, cudaStream_t st)
{
    norm_bwd_partial_k<<<(unsigned)B * (unsigned)parts, 256, 0, st>>>(x, gamma, gy, stats, partials, P, slice_len(P, parts),
                                                                     parts);
    norm_bwd_finalize_k<<<B, 64, 0, st>>>(partials, parts, ac, P);
    norm_bwd_apply_k<<<(unsigned)((P + 255) / 256), 256, 0, st>>>(x, gamma, gy, stats, ac, gx, ggamma, gbeta, B, P);
    return check_launch("norm_backward");
}

}  // namespace gn
