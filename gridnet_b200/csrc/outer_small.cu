// The whole fused model loop as ONE persistent kernel, for problems so small that launches are what they cost
// (the reference's MNIST configuration: 32^3 grid, batch 8, 2 inner x 8 outer iterations is 17 launches of a few
// microseconds each when every outer step is a kernel of its own).
//
//   for o in range(outer): h = layer_norm(gridnet_step(h))          gridnet/scripts/train_mnist.py:62-64
//
// One CTA of 128 threads owns one 8x8x8 block and a few samples for all outer steps. It keeps its 4 x 27 weights
// per thread in registers from start to end (register-patch mapping of step_fast.cu: a thread owns a 1x2x2 patch,
// the sample's 10^3 tile sits in shared memory with rows of 12 floats, two tiles ping-pong over the inner
// iterations). Between outer steps the CTAs meet at a grid-wide barrier: the step's output is in global memory
// (the neighbours' halos are read from there), the per-sample statistics partials too; after the barrier every
// CTA adds up the partials of its own samples (all CTAs of a sample in the same order, hence the same bits) and
// normalises the next step's tile cells while loading them. The last step's output is normalised in place of a
// separate pass: each thread re-reads the four values it wrote.
//
// The barrier is a counter in global memory with a bounded wait: the launch is cooperative, so all CTAs are
// resident and it cannot deadlock; should a wait run out all the same, the kernel sets the error flag and goes on.
#include "common.cuh"
#include "kernels.h"
#include "patch_geo.cuh"

namespace gn {

namespace small8 {
constexpr int THREADS = 128;
constexpr int MAX_SPC = 2;                    // samples per CTA at most: both tiles are fetched up front
constexpr unsigned kSpinLimit = 1u << 22;     // polls of the grid barrier, ~50 ns apart
}  // namespace small8

struct OuterSmallParams {
    const float *w, *b, *s, *gamma, *beta, *x;
    float *y;
    float *buf[2];        // raw step outputs, ping-pong
    double2 *partials;    // [B][nparts]
    unsigned *barrier;    // zeroed before the launch
    int *error_flag;
    int nparts, nblocks;
    int B, M, N, K, inner, outer, spc;
    float eps;
};

template <int ACT>
__global__ void __launch_bounds__(small8::THREADS, 2) outer_small_k(const OuterSmallParams p)
{
    using namespace small8;
    using Geo = PatchGeo<8>;
    constexpr int RS = Geo::RS, PS = Geo::PS, TS = Geo::TS;
    __shared__ __align__(16) float tiles[MAX_SPC][2][TS];  // [sample of the CTA][ping-pong]
    __shared__ float2 gbtab[Geo::CELLS];
    __shared__ float2 mstats[MAX_SPC];
    __shared__ double2 wsum[MAX_SPC][4];   // per-warp (sum, sum of squares) of the CTA's outputs of this step
    __shared__ double2 rsum[4][MAX_SPC];   // per-warp sums of the samples' partials after the barrier

    const int tid = threadIdx.x;
    const int xp = tid & 3, yp = (tid >> 2) & 3, z = tid >> 4;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const int blk = blockIdx.x % p.nblocks, chunk = blockIdx.x / p.nblocks;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g00 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + 2 * yp)) * K + (bx * 8 + 2 * xp);
    const long long origin = ((long long)(bz * 8 - 1) * p.N + (by * 8 - 1)) * K + (bx * 8 - 1);
    const int s0 = chunk * p.spc, s1 = min(p.B, s0 + p.spc);

    // tile cells this thread fetches for every sample: tile offset, offset from the tile's origin (or -1 outside)
    int soff[Geo::SLOTS], rel[Geo::SLOTS];
    bool halo[Geo::SLOTS];
#pragma unroll
    for (int j = 0; j < Geo::SLOTS; ++j) {
        const int i = tid + j * THREADS;
        soff[j] = -1;
        rel[j] = -1;
        halo[j] = false;
        if (i < Geo::CELLS) {
            int cz, cy, cx;
            Geo::cell(i, soff[j], cz, cy, cx, halo[j]);
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gx = bx * 8 + cx - 1;
            const bool inside = gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < K;
            float2 gb = make_float2(0.0f, 0.0f);
            if (inside) {
                rel[j] = (cz * p.N + cy) * K + cx;
                gb = make_float2(p.gamma[origin + rel[j]], p.beta[origin + rel[j]]);
            }
            gbtab[i] = gb;
        }
    }
    float w[27][2][2];
#pragma unroll
    for (int t = 0; t < 27; ++t)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 v = *reinterpret_cast<const float2 *>(p.w + (size_t)t * P + g00 + (size_t)j * K);
            w[t][j][0] = v.x;
            w[t][j][1] = v.y;
        }
    float bias[2][2], scl[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float2 vb = *reinterpret_cast<const float2 *>(p.b + g00 + (size_t)j * K);
        const float2 vs = *reinterpret_cast<const float2 *>(p.s + g00 + (size_t)j * K);
        bias[j][0] = vb.x;
        bias[j][1] = vb.y;
        scl[j][0] = vs.x;
        scl[j][1] = vs.y;
    }
    const int toff = Geo::window_origin(xp, yp, z);
    __syncthreads();

    for (int o = 0; o < p.outer; ++o) {
        const float *src = o == 0 ? p.x : p.buf[(o - 1) & 1];
        float *dst = p.buf[o & 1];
        // fetch the tiles of all of this CTA's samples first: the loads of the second overlap the first one's arithmetic
#pragma unroll
        for (int q = 0; q < MAX_SPC; ++q) {
            const int smp = s0 + q;
            if (smp < s1) {
                const float2 mr = o > 0 ? mstats[q] : make_float2(0.0f, 1.0f);
                const float *xs = src + (size_t)smp * P + origin;
                float v[Geo::SLOTS];
#pragma unroll
                for (int j = 0; j < Geo::SLOTS; ++j)  // __ldcg: the neighbours' blocks were written by other CTAs
                    v[j] = (soff[j] >= 0 && rel[j] >= 0) ? __ldcg(xs + rel[j]) : 0.0f;
#pragma unroll
                for (int j = 0; j < Geo::SLOTS; ++j) {
                    if (soff[j] >= 0) {
                        float u = v[j];
                        if (o > 0) {
                            const float2 gb = gbtab[tid + j * THREADS];
                            u = fmaf((u - mr.x) * mr.y, gb.x, gb.y);
                        }
                        tiles[q][0][soff[j]] = u;
                        if (halo[j]) tiles[q][1][soff[j]] = u;
                    }
                }
            }
        }
        __syncthreads();
        for (int smp = s0; smp < s1; ++smp) {
            float(*tl2)[TS] = tiles[smp - s0];
            for (int it = 0; it < p.inner; ++it) {
                const bool last = it + 1 == p.inner;
                const int cur = it & 1;
                const float *tl = tl2[cur] + toff;
                float acc[2][2] = {{bias[0][0], bias[0][1]}, {bias[1][0], bias[1][1]}};
                float old[2][2];
#pragma unroll
                for (int a = 0; a < 3; ++a)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                        const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                        const float v[4] = {v01.x, v01.y, v23.x, v23.y};
                        if (a == 1 && (r == 1 || r == 2)) {
                            old[r - 1][0] = v[1];
                            old[r - 1][1] = v[2];
                        }
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int bb = r - j;
                            if (bb >= 0 && bb <= 2) {
#pragma unroll
                                for (int c = 0; c < 3; ++c) {
                                    acc[j][0] = fmaf(w[a * 9 + bb * 3 + c][j][0], v[c], acc[j][0]);
                                    acc[j][1] = fmaf(w[a * 9 + bb * 3 + c][j][1], v[c + 1], acc[j][1]);
                                }
                            }
                        }
                    }
                float nv[2][2];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) nv[j][i] = fmaf(Act<ACT, float>::fwd(acc[j][i]), scl[j][i], old[j][i]);
                if (!last) {
                    float *to = tl2[cur ^ 1] + toff + PS + RS + 1;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        to[j * RS] = nv[j][0];
                        to[j * RS + 1] = nv[j][1];
                    }
                    __syncthreads();
                } else {
                    float *ys = dst + (size_t)smp * P + g00;
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        __stcg(reinterpret_cast<float2 *>(ys + (size_t)j * K), make_float2(nv[j][0], nv[j][1]));
                    // a warp's 128 values in float (ten shuffles, not twenty), doubles above the warp
                    float sm = (nv[0][0] + nv[0][1]) + (nv[1][0] + nv[1][1]);
                    float sq = fmaf(nv[0][0], nv[0][0], nv[0][1] * nv[0][1]) + fmaf(nv[1][0], nv[1][0], nv[1][1] * nv[1][1]);
                    sm = warp_sum(sm);
                    sq = warp_sum(sq);
                    if ((tid & 31) == 0) wsum[smp - s0][tid >> 5] = make_double2((double)sm, (double)sq);
                }
            }
        }

        // ---- grid-wide barrier: every CTA's outputs and partials of step o are in global memory
        __syncthreads();
        if (tid < s1 - s0) {  // one partial per block and sample: the four warps' sums in warp order
            double sm = 0.0, sq = 0.0;
#pragma unroll
            for (int wq = 0; wq < 4; ++wq) {
                sm += wsum[tid][wq].x;
                sq += wsum[tid][wq].y;
            }
            __stcg(&p.partials[(size_t)(s0 + tid) * p.nparts + (size_t)blk * 4], make_double2(sm, sq));
        }
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            atomicAdd(p.barrier, 1u);
            const unsigned target = (unsigned)(o + 1) * gridDim.x;
            unsigned spins = 0, seen;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.barrier) : "memory");
                if (seen >= target) break;
                if (++spins > kSpinLimit) {
                    if (p.error_flag) *p.error_flag = 1;
                    break;
                }
                if (spins > 64) __nanosleep(40);
            }
        }
        __syncthreads();

        // ---- statistics of this CTA's samples: one reduction for all of them (every CTA of a sample adds the
        // same partials, one per block, in the same order)
        {
            double acc[MAX_SPC][2];
#pragma unroll
            for (int q = 0; q < MAX_SPC; ++q) {
                acc[q][0] = acc[q][1] = 0.0;
                if (s0 + q < s1) {
                    const double2 *ps = p.partials + (size_t)(s0 + q) * p.nparts;
                    for (int i = tid; i < p.nblocks; i += THREADS) {
                        const double2 v = __ldcg(ps + (size_t)i * 4);
                        acc[q][0] += v.x;
                        acc[q][1] += v.y;
                    }
                }
                acc[q][0] = warp_sum(acc[q][0]);
                acc[q][1] = warp_sum(acc[q][1]);
                if ((tid & 31) == 0) rsum[tid >> 5][q] = make_double2(acc[q][0], acc[q][1]);
            }
            __syncthreads();
            if (tid < s1 - s0) {
                double sm = 0.0, sq = 0.0;
#pragma unroll
                for (int wq = 0; wq < 4; ++wq) {
                    sm += rsum[wq][tid].x;
                    sq += rsum[wq][tid].y;
                }
                const double mean = sm / (double)P;
                double var = sq / (double)P - mean * mean;
                if (var < 0.0) var = 0.0;
                mstats[tid] = make_float2((float)mean, (float)(1.0 / sqrt(var + (double)p.eps)));
            }
        }
        __syncthreads();
    }

    // ---- the last normalisation, on the four values this thread wrote itself
    const float *lastbuf = p.buf[(p.outer - 1) & 1];
    float2 gm[2], bt[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        gm[j] = *reinterpret_cast<const float2 *>(p.gamma + g00 + (size_t)j * K);
        bt[j] = *reinterpret_cast<const float2 *>(p.beta + g00 + (size_t)j * K);
    }
    for (int smp = s0; smp < s1; ++smp) {
        const float2 mr = mstats[smp - s0];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 v = __ldcg(reinterpret_cast<const float2 *>(lastbuf + (size_t)smp * P + g00 + (size_t)j * K));
            *reinterpret_cast<float2 *>(p.y + (size_t)smp * P + g00 + (size_t)j * K) =
                make_float2(fmaf((v.x - mr.x) * mr.y, gm[j].x, bt[j].x), fmaf((v.y - mr.x) * mr.y, gm[j].y, bt[j].y));
        }
    }
}

template <int ACT>
static int launch_one(const OuterSmallParams &p, int ctas, cudaStream_t st)
{
    void *args[] = {const_cast<OuterSmallParams *>(&p)};
    const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(outer_small_k<ACT>), dim3(ctas),
                                                      dim3(small8::THREADS), args, 0, st);
    if (e != cudaSuccess) {
        record_cuda_error(e, "cudaLaunchCooperativeKernel(outer_small_k)");
        (void)cudaGetLastError();
        return GN_ERR_CUDA;
    }
    return GN_OK;
}

// How many samples per CTA the persistent kernel would use for this problem, or 0 if it does not apply: block 8,
// at least one outer step, all CTAs resident at once, at most MAX_SPC samples per CTA, and little enough work per
// outer step (B * P * inner neuron updates) that launches, not arithmetic, are what the step-by-step loop costs.
int outer_small_spc(int B, int M, int N, int K, int block, int inner, int outer, const void *w, const void *b, const void *s,
                    const void *gamma, const void *beta, const void *x, const void *y)
{
    if (block != 8 || inner < 1 || outer < 1 || B < 1 || M % 8 || N % 8 || K % 8) return 0;
    const long long P = (long long)M * N * K;
    if (P >= (1LL << 31) || (long long)B * P * inner > (1LL << 21)) return 0;
    auto al8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; };
    if (!(al8(w) && al8(b) && al8(s) && al8(gamma) && al8(beta) && al8(y)) || (reinterpret_cast<uintptr_t>(x) & 3)) return 0;
    int dev = 0, coop = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, outer_small_k<GN_ACT_SILU>, small8::THREADS, 0) != cudaSuccess ||
        per_sm < 1)
        return 0;
    const long long capacity = (long long)per_sm * sm_count();
    const long long nblocks = (long long)(M / 8) * (N / 8) * (K / 8);
    if (nblocks > capacity) return 0;
    long long chunks = capacity / nblocks;
    if (chunks > B) chunks = B;
    const int spc = (int)((B + chunks - 1) / chunks);
    return spc <= small8::MAX_SPC ? spc : 0;
}

int launch_outer_small(const float *w, const float *b, const float *s, const float *gamma, const float *beta, const float *x,
                       float *y, float *buf0, float *buf1, double2 *partials, unsigned *barrier, int *error_flag, int B, int M,
                       int N, int K, int inner, int outer, int spc, float eps, int act, cudaStream_t st)
{
    OuterSmallParams p{};
    p.w = w; p.b = b; p.s = s; p.gamma = gamma; p.beta = beta; p.x = x; p.y = y;
    p.buf[0] = buf0; p.buf[1] = buf1; p.partials = partials; p.barrier = barrier; p.error_flag = error_flag;
    p.nblocks = (M / 8) * (N / 8) * (K / 8);
    p.nparts = p.nblocks * 4;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.outer = outer; p.spc = spc; p.eps = eps;
    const int ctas = p.nblocks * ((B + spc - 1) / spc);
    switch (act) {
    case GN_ACT_RELU: return launch_one<GN_ACT_RELU>(p, ctas, st);
    case GN_ACT_LEAKY_RELU: return launch_one<GN_ACT_LEAKY_RELU>(p, ctas, st);
    case GN_ACT_SILU: return launch_one<GN_ACT_SILU>(p, ctas, st);
    default: return launch_one<GN_ACT_TANH>(p, ctas, st);
    }
}

}  // namespace gn
