// Tuned float forward kernel of the gated grid update (block size 8):
//   gate = sigmoid(sum_t x[n + o_t] * w[t][1][n] + b[1][n])
//   x[n] <- gate * x[n] + (1 - gate) * act(sum_t x[n + o_t] * w[t][0][n] + b[0][n])
// (gridnet/backend_torch.py:145-267; the kernel it stands in for is the gated forward kernel of
// src/gridnet_cuda_kernels.cu:452-560).
//
// Same construction as step_fast.cu: one CTA owns one 8 x 8 x 8 block and a range of samples, the
// 10 x 10 x 10 tile of a sample sits in shared memory with rows of 12 floats, two tiles per sample
// (ping-pong, one barrier per inner iteration), tiles arrive by bulk tensor copy two samples ahead.
// A gated neuron has 54 weights, so a thread owns a 1 x 1 x 2 patch (two neurons along x; 108
// weights in registers) and the CTA has 256 threads; a thread reads a 3 x 3 x 4 window (18 64-bit
// loads) for its 108 FMAs. The thread-to-row map puts the rows y = 0, 2, 4, 6 in one half-warp and
// y = 1, 3, 5, 7 in the other, which makes the 64-bit loads of a half-warp hit every bank once.
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace gn {

namespace gated8 {
constexpr int RS = 12, PS = 120, TS = 1200;
constexpr int THREADS = 256;
constexpr int SLOTS = 4;           // ceil(1000 / 256) tile cells per thread
constexpr int STG = 10 * 10 * 16;  // floats of one bulk-copied neighbourhood (x from 8 bx - 4)
constexpr unsigned kSpinLimit = 1u << 18;
}  // namespace gated8

struct GatedFastParams {
    const float *w, *b, *x;
    float *y;
    int B, M, N, K, inner, spc;
    int *error_flag;  // optional: set to 1 if a bounded wait on a bulk copy gave up
    // Replay mode of the backward pass: every iteration's two pre-activations ([inner][B][M,N,K] each) and the
    // activations after iterations 1 .. inner-1 ([inner-1][B][M,N,K]); y may then be nullptr.
    float *save_hv, *save_hg, *save_x;
};

template <int ACT>
__global__ void __launch_bounds__(gated8::THREADS, 1)
    gated_fwd_fast8(const __grid_constant__ CUtensorMap x_map, const GatedFastParams p)
{
    using namespace gated8;
    __shared__ __align__(16) float tiles[2][2][TS];  // [sample parity][ping-pong]
    __shared__ __align__(128) float staging[2][STG];
    __shared__ __align__(8) unsigned long long bars[2];

    const int tid = threadIdx.x;
    const int xp = tid & 3, y = 2 * ((tid >> 2) & 3) + ((tid >> 4) & 1), z = tid >> 5;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const size_t g0 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + y)) * p.K + (bx * 8 + 2 * xp);

    // tile cells this thread copies out of the staging buffer: bits 0..10 tile offset, bit 11 halo
    // (kept in both ping-pong tiles), bits 12.. staging offset
    unsigned cinfo[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        const int i = tid + j * THREADS;
        unsigned ci = 0xffffffffu;
        if (i < 1000) {
            const int cx = i % 10, cy = (i / 10) % 10, cz = i / 100;
            const bool halo = cx == 0 || cx == 9 || cy == 0 || cy == 9 || cz == 0 || cz == 9;
            ci = (unsigned)(cz * PS + cy * RS + cx) | (halo ? 0x800u : 0u) | ((unsigned)((cz * 10 + cy) * 16 + cx + 3) << 12);
        }
        cinfo[j] = ci;
    }

    float wv[27][2], wg[27][2];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        const float2 a = *reinterpret_cast<const float2 *>(p.w + (size_t)(2 * t) * P + g0);
        const float2 g = *reinterpret_cast<const float2 *>(p.w + (size_t)(2 * t + 1) * P + g0);
        wv[t][0] = a.x; wv[t][1] = a.y;
        wg[t][0] = g.x; wg[t][1] = g.y;
    }
    const float2 bv = *reinterpret_cast<const float2 *>(p.b + g0);
    const float2 bg = *reinterpret_cast<const float2 *>(p.b + P + g0);

    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    const int toff = z * PS + y * RS + 2 * xp;  // window origin of this thread inside a tile
    const unsigned bar_base = smem_u32(bars);
    auto prefetch = [&](int smp) {  // bulk copy of one sample's neighbourhood into the staging ring
        if (smp < s1 && tid == 0) {
            const int par = (smp - s0) & 1;
            mbar_expect_tx(bar_base + 8 * par, STG * 4);
            tma_load_4d(smem_u32(staging[par]), &x_map, bar_base + 8 * par, bx * 8 - 4, by * 8 - 1, bz * 8 - 1, smp);
        }
    };
    auto commit = [&](int smp, int set) {  // staging -> tile set
        if (smp < s1) {
            const int par = (smp - s0) & 1;
            if (!mbar_wait_bounded(bar_base + 8 * par, ((smp - s0) >> 1) & 1, kSpinLimit) && p.error_flag) *p.error_flag = 1;
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                const unsigned ci = cinfo[j];
                if (ci != 0xffffffffu) {
                    const float v = staging[par][ci >> 12];
                    tiles[set][0][ci & 0x7ff] = v;
                    if (ci & 0x800) tiles[set][1][ci & 0x7ff] = v;
                }
            }
        }
    };

    if (tid == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    __syncthreads();
    prefetch(s0);
    prefetch(s0 + 1);
    commit(s0, 0);
    __syncthreads();

    for (int smp = s0; smp < s1; ++smp) {
        const int set = (smp - s0) & 1;
        prefetch(smp + 2);  // the staging buffer of this sample was consumed a whole sample ago
        commit(smp + 1, set ^ 1);
        for (int it = 0; it < p.inner; ++it) {
            const bool last = it + 1 == p.inner;
            const int cur = it & 1;
            const float *tl = tiles[set][cur] + toff;
            float av[2] = {bv.x, bv.y}, ag[2] = {bg.x, bg.y}, old[2];
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    const float v[4] = {v01.x, v01.y, v23.x, v23.y};
                    if (a == 1 && r == 1) {
                        old[0] = v[1];
                        old[1] = v[2];
                    }
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + r * 3 + c;
                        av[0] = fmaf(wv[t][0], v[c], av[0]);
                        av[1] = fmaf(wv[t][1], v[c + 1], av[1]);
                        ag[0] = fmaf(wg[t][0], v[c], ag[0]);
                        ag[1] = fmaf(wg[t][1], v[c + 1], ag[1]);
                    }
                }
            float nv[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float gate = sigmoid_(ag[i]);
                nv[i] = gate * old[i] + (1.0f - gate) * Act<ACT, float>::fwd(av[i]);
            }
            if (p.save_hv) {
                const size_t o = ((size_t)it * p.B + smp) * P + g0;
                *reinterpret_cast<float2 *>(p.save_hv + o) = make_float2(av[0], av[1]);
                *reinterpret_cast<float2 *>(p.save_hg + o) = make_float2(ag[0], ag[1]);
                if (!last) *reinterpret_cast<float2 *>(p.save_x + o) = make_float2(nv[0], nv[1]);
            }
            if (!last) {
                float *to = tiles[set][cur ^ 1] + toff + PS + RS + 1;
                to[0] = nv[0];
                to[1] = nv[1];
                __syncthreads();  // the other tile is complete; this one may be overwritten next
            } else {
                if (p.y) *reinterpret_cast<float2 *>(p.y + (size_t)smp * P + g0) = make_float2(nv[0], nv[1]);
            }
        }
        __syncthreads();  // next sample's tiles are complete; this sample's tiles are free
    }
}

bool gated_fast8_applicable(const float *w, const float *b, const float *x, const float *y, int M, int N, int K, int block,
                            int inner)
{
    if (block != 8 || inner < 1 || M % 8 || N % 8 || K % 8) return false;
    if (!encode_tiled_fn()) return false;
    auto al = [](const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
    return al(w, 8) && al(b, 8) && al(y, 8) && al(x, 16);
}

int launch_gated_fwd_fast8(const float *w, const float *b, const float *x, float *y, int B, int M, int N, int K, int inner,
                           int act, cudaStream_t st, float *save_hv, float *save_hg, float *save_x, int *error_flag)
{
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    if (!fast8_make_tile_map(&map, x, B, M, N, K)) return GN_ERR_UNSUPPORTED;
    const long long nb = (long long)(M / 8) * (N / 8) * (K / 8);
    GatedFastParams p{};
    p.w = w; p.b = b; p.x = x; p.y = y;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner;
    p.save_hv = save_hv; p.save_hg = save_hg; p.save_x = save_x;
    // the forward entry point has no workspace: it reports to the library's status word
    p.error_flag = error_flag ? error_flag : device_status_ptr();
    const int chunks = pick_batch_chunks_balanced(nb, B, 1, 1.5, B < 64 ? B : 64);
    p.spc = (B + chunks - 1) / chunks;
    dim3 grid((unsigned)nb, (unsigned)((B + p.spc - 1) / p.spc));
    switch (act) {
    case GN_ACT_RELU: gated_fwd_fast8<GN_ACT_RELU><<<grid, gated8::THREADS, 0, st>>>(map, p); break;
    case GN_ACT_LEAKY_RELU: gated_fwd_fast8<GN_ACT_LEAKY_RELU><<<grid, gated8::THREADS, 0, st>>>(map, p); break;
    case GN_ACT_SILU: gated_fwd_fast8<GN_ACT_SILU><<<grid, gated8::THREADS, 0, st>>>(map, p); break;
    default: gated_fwd_fast8<GN_ACT_TANH><<<grid, gated8::THREADS, 0, st>>>(map, p); break;
    }
    return check_launch("gated_fwd_fast8");
}

}  // namespace gn
