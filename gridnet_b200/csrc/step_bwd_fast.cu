// Tuned float backward of the block-local grid update (block 8 or 4, per-block normalisation
// off), split into four kernels so that every stencil runs with the register-patch mapping of
// the forward kernel (a thread owns a 1x2x2 patch and keeps 4 x 27 values in registers):
//
//   replay   step_fwd_fast8 (step_fast.cu) in replay mode: runs the inner iterations once and
//            stores every iteration's pre-activation h_t and the activations x_t in between —
//            the inner iterations are recomputed here, never kept from the forward pass;
//   reverse  bwd_reverse8: walks the iterations backwards. delta_t = act'(h_t) * g * scale, and
//            the gradient flowing back inside the block is a 27-tap stencil over the delta tile
//            with TRANSPOSED weights (cell c receives w[n][t] * delta[n] from the neuron
//            n = c + o through its tap pointing back at c; the kernel reads them straight from
//            the weight tensor), so it is a gather, with no atomics;
//   wgrad    bwd_wgrad8: dW[n][t] += x_t[n + offset(t)] * delta_t[n], accumulated in registers
//            over samples and iterations, plus dB and dS;
//   halo     bwd_halo8: the part of dX that crosses block borders. A halo cell never feeds back
//            into its block, so its gradient only needs the per-neuron SUM of deltas:
//            dX[c] += sum over neurons n of other blocks with c = n + offset(t) of w[n][t] * Dsum[n].
//
// Everything is deterministic: there are no floating-point atomics. When wgrad splits a block's
// batch over several CTAs for occupancy, those CTAs form a thread-block cluster and combine
// their partial sums through distributed shared memory in a fixed order. The input tiles of
// wgrad arrive by bulk tensor copy like in the forward kernel; its bounded waits report through
// the int at the end of the workspace (cleared when the pass starts).
//
// Reference semantics: the gradient of gridnet/backend_torch.py:61-142 with normalize=False;
// the kernel this stands in for is gridnet_cuda_backward_kernel, src/gridnet_cuda_kernels.cu:202-450.
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "patch_geo.cuh"
#include "tma.cuh"

namespace gn {
namespace cg = cooperative_groups;

namespace bwd8 {
constexpr int THREADS = 128;
constexpr int STG = 10 * 10 * 16;  // floats of one bulk-copied tile
constexpr unsigned kSpinLimit = 1u << 18;
constexpr int RED_UNITS = 58;  // float2 partial sums per thread: 27 taps x 2 rows, bias x 2, scale x 2
}  // namespace bwd8

struct BwdParams {
    const float *w, *s, *x, *gy;
    const float *save_h, *save_x;  // from the replay
    float *delta;                  // [inner][B][P]
    float *dsum;                   // [B][P] sum of deltas over the iterations
    float *dsb;                    // [B][P] per-sample gradient of the residual scale
    float *gw, *gb, *gs, *gx;
    int B, M, N, K, inner, spc;
    int *error_flag;     // set to 1 if a bounded wait on a bulk copy gave up
    int cluster_reduce;  // wgrad: the batch chunks of a block are one cluster and reduce through shared memory
    // Per-block normalisation (block 8): the bias, the replay's per-tile statistics [inner][B][regions]
    // (mean, 1 / (std + eps), std, std + eps), and per sample and region the two sums that every cell of the
    // region's tile owes to the statistics ([B][regions] (F, E): grad_x[c] -= F + x[c] * E).
    const float *b;
    const float4 *tile_stats;
    float2 *hterm;
    // The step input given as the RAW output of the step before plus its whole-grid statistics: the
    // weight-gradient kernel (and the replay) normalise it while loading, (x - mean) * rstd * gamma + beta.
    const float2 *in_stats;  // [B] (mean, rstd); nullptr: x is used as it is
    const float *gamma, *beta;
};

// ---------------------------------------------------------------------------- reverse sweep
// INNER_T > 0: the inner iteration count is a compile-time constant (loop unrolled); 0: from the parameters.
//
// NORM (per-block normalisation, gridnet/backend_torch.py:92-97): the stencil input of iteration t was
// in = (tile - mean_t) * inv_t with inv_t = 1 / (std_t + eps) over all 1000 tile cells. With Gin[c] the gradient
// of the stencil inputs, the tile gradient is inv Gin[c] - P1 - P2 (x[c] - mean), P1 = inv sum(Gin) / 1000,
// P2 = inv sum(Gin in) / (1000 std). Both sums are sums over the block's NEURONS, no halo gradient needed:
// sum(Gin) = sum_n delta[n] W[n] (W = the neuron's 27 weights added up) and sum(Gin in) = sum_n delta[n] (h[n] -
// bias[n]). So the kernel scales delta by inv (tile, stored deltas and their sum: the other kernels then see
// inv Gin), reduces the two sums over the CTA while the gather runs (per-thread partial sums published by the
// barrier that publishes the delta tile; every warp adds the 128 of them between its first stencil rows), and
// subtracts P1 + P2 (x_t[n] - mean) from its own cells. What the halo cells owe, F = sum_t (P1 - P2 mean) and
// E = sum_t P2, goes to hterm for the cross-block kernel.
template <int SUB, int ACT, int INNER_T, bool NORM = false>
__global__ void __launch_bounds__(bwd8::THREADS, 3) bwd_reverse8(const BwdParams p)
{
    using namespace bwd8;
    using Geo = PatchGeo<SUB>;
    constexpr int RS = Geo::RS, PS = Geo::PS, TS = Geo::TS;
    static_assert(!NORM || SUB == 8, "per-block normalisation: block 8");
    __shared__ __align__(16) float D[2][TS];
    __shared__ __align__(16) float2 part_sums[2][NORM ? THREADS : 1];
    __shared__ float4 tconst[3][NORM ? THREADS : 1];  // bias, weight sum, scale of the thread's four neurons
    const int tid = threadIdx.x;
    const int xp = tid & 3, yp = (tid >> 2) & 3, z = tid >> 4;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g00 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + 2 * yp)) * K + (bx * 8 + 2 * xp);

    // Transposed weights: cell c receives w[n][26 - t] * delta[n] from its neighbour n = c + offset(t)
    // (n reads c through the tap that points back), if n is a neuron of c's own block; otherwise 0.
    float wt[27][2][2];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
        const int lz = (z & (SUB - 1)) + dz;
        const float *wp = p.w + (size_t)(26 - t) * P + g00 + ((long long)dz * p.N + dy) * K + dx;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int ly = ((2 * yp + j) & (SUB - 1)) + dy;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int lx = ((2 * xp + i) & (SUB - 1)) + dx;
                const bool same = lz >= 0 && lz < SUB && ly >= 0 && ly < SUB && lx >= 0 && lx < SUB;
                wt[t][j][i] = same ? __ldg(wp + (size_t)j * K + i) : 0.0f;
            }
        }
    }
    float scl[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float2 v = *reinterpret_cast<const float2 *>(p.s + g00 + (size_t)j * K);
        scl[j][0] = v.x;
        scl[j][1] = v.y;
    }
    if (NORM) {
        float ws[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
        for (int t = 0; t < 27; ++t)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float2 v = *reinterpret_cast<const float2 *>(p.w + (size_t)t * P + g00 + (size_t)j * K);
                ws[j][0] += v.x;
                ws[j][1] += v.y;
            }
        const float2 b0 = *reinterpret_cast<const float2 *>(p.b + g00), b1 = *reinterpret_cast<const float2 *>(p.b + g00 + K);
        tconst[0][tid] = make_float4(b0.x, b0.y, b1.x, b1.y);
        tconst[1][tid] = make_float4(ws[0][0], ws[0][1], ws[1][0], ws[1][1]);
        tconst[2][tid] = make_float4(scl[0][0], scl[0][1], scl[1][0], scl[1][1]);
    }
    for (int i = tid; i < 2 * TS; i += THREADS) (&D[0][0])[i] = 0.0f;  // the halo of both tiles stays zero
    __syncthreads();

    const int toff = Geo::window_origin(xp, yp, z);
    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    unsigned step = 0;  // picks the delta tile: consecutive iterations (also across samples) alternate
    // pre-activations of the iteration handled next and the next sample's output gradient are
    // fetched one iteration early
    float2 hn[2], gn[2];
    // NORM: the tile statistics and this thread's activations x_t of the iteration handled next
    float4 tsn = make_float4(0.0f, 1.0f, 1.0f, 1.0f);
    float2 xn[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
    auto fetch_norm = [&](int smp, int it) {
        if (NORM) {
            tsn = p.tile_stats[((size_t)it * p.B + smp) * gridDim.x + blk];
            const float *src = it > 0 ? p.save_x + ((size_t)(it - 1) * p.B + smp) * P : p.x + (size_t)smp * P;
#pragma unroll
            for (int j = 0; j < 2; ++j) xn[j] = ld_pinned2(src + g00 + (size_t)j * K);
        }
    };
    if (s0 < s1) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            hn[j] = ld_pinned2(p.save_h + ((size_t)((INNER_T > 0 ? INNER_T : p.inner) - 1) * p.B + s0) * P + g00 + (size_t)j * K);
            gn[j] = ld_pinned2(p.gy + (size_t)s0 * P + g00 + (size_t)j * K);
        }
        fetch_norm(s0, (INNER_T > 0 ? INNER_T : p.inner) - 1);
    }
    for (int smp = s0; smp < s1; ++smp) {
        const size_t so = (size_t)smp * P + g00;
        float g[2][2], dsum[2][2], dsacc[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            g[j][0] = gn[j].x;
            g[j][1] = gn[j].y;
            dsum[j][0] = dsum[j][1] = dsacc[j][0] = dsacc[j][1] = 0.0f;
        }
        float hF = 0.0f, hE = 0.0f;  // NORM: what every cell of the tile owes to the statistics, summed over t
        const int inner = INNER_T > 0 ? INNER_T : p.inner;
#pragma unroll
        for (int it = (INNER_T > 0 ? INNER_T : inner) - 1; it >= 0; --it, ++step) {
            const size_t ho = ((size_t)it * p.B + smp) * P + g00;
            float *Dt = D[step & 1];
            float dl[2][2];
            const float2 hc[2] = {hn[0], hn[1]};
            const float4 ts = tsn;
            const float2 xc[2] = {xn[0], xn[1]};
            if (it > 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    hn[j] = ld_pinned2(p.save_h + ho - (size_t)p.B * P + (size_t)j * K);
                fetch_norm(smp, it - 1);
            } else if (smp + 1 < s1) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    hn[j] = ld_pinned2(p.save_h + ((size_t)(inner - 1) * p.B + smp + 1) * P + g00 + (size_t)j * K);
                    gn[j] = ld_pinned2(p.gy + so + P + (size_t)j * K);
                }
                fetch_norm(smp + 1, inner - 1);
            }
            if (NORM) {
                const float4 cb = tconst[0][tid], cw = tconst[1][tid], cs = tconst[2][tid];
                const float bb[2][2] = {{cb.x, cb.y}, {cb.z, cb.w}}, ww[2][2] = {{cw.x, cw.y}, {cw.z, cw.w}};
                const float ss[2][2] = {{cs.x, cs.y}, {cs.z, cs.w}};
                float pa = 0.0f, pc = 0.0f;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float hv[2] = {hc[j].x, hc[j].y};
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        float f, d;
                        Act<ACT, float>::both(hv[i], f, d);
                        dsacc[j][i] = fmaf(f, g[j][i], dsacc[j][i]);
                        const float raw = d * g[j][i] * ss[j][i];
                        pa = fmaf(raw, ww[j][i], pa);
                        pc = fmaf(raw, hv[i] - bb[j][i], pc);
                        dl[j][i] = raw * ts.y;  // everything downstream sees delta / (std + eps)
                        dsum[j][i] += dl[j][i];
                    }
                    *reinterpret_cast<float2 *>(p.delta + ho + (size_t)j * K) = make_float2(dl[j][0], dl[j][1]);
                }
                part_sums[step & 1][tid] = make_float2(pa, pc);
            } else {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const float2 h = hc[j];
                    float f0, d0, f1, d1;
                    Act<ACT, float>::both(h.x, f0, d0);
                    Act<ACT, float>::both(h.y, f1, d1);
                    dsacc[j][0] = fmaf(f0, g[j][0], dsacc[j][0]);
                    dsacc[j][1] = fmaf(f1, g[j][1], dsacc[j][1]);
                    dl[j][0] = d0 * g[j][0] * scl[j][0];
                    dl[j][1] = d1 * g[j][1] * scl[j][1];
                    dsum[j][0] += dl[j][0];
                    dsum[j][1] += dl[j][1];
                    *reinterpret_cast<float2 *>(p.delta + ho + (size_t)j * K) = make_float2(dl[j][0], dl[j][1]);
                }
            }
            {
                float *to = Dt + toff + PS + RS + 1 + (z & 1);
                const int stp = 1 - 2 * (z & 1);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    to[j * RS] = (z & 1) ? dl[j][1] : dl[j][0];
                    to[j * RS + stp] = (z & 1) ? dl[j][0] : dl[j][1];
                }
            }
            __syncthreads();
            float red_a = 0.0f, red_c = 0.0f;  // NORM: this lane's share of the 128 partial sums
            if (NORM) {
                const float4 a = *reinterpret_cast<const float4 *>(&part_sums[step & 1][(tid & 31) * 4]);
                const float4 c = *reinterpret_cast<const float4 *>(&part_sums[step & 1][(tid & 31) * 4 + 2]);
                red_a = (a.x + a.z) + (c.x + c.z);
                red_c = (a.y + a.w) + (c.y + c.w);
            }
            const float *tl = Dt + toff;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    const float v[4] = {v01.x, v01.y, v23.x, v23.y};
                    if (NORM && a * 4 + r < 5) {  // one shuffle round per row (uniform: every lane takes part)
                        red_a += __shfl_xor_sync(0xffffffffu, red_a, 16 >> (a * 4 + r));
                        red_c += __shfl_xor_sync(0xffffffffu, red_c, 16 >> (a * 4 + r));
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int bb = r - j;
                        if (bb >= 0 && bb <= 2) {
#pragma unroll
                            for (int c = 0; c < 3; ++c) {
                                g[j][0] = fmaf(wt[a * 9 + bb * 3 + c][j][0], v[c], g[j][0]);
                                g[j][1] = fmaf(wt[a * 9 + bb * 3 + c][j][1], v[c + 1], g[j][1]);
                            }
                        }
                    }
                }
            if (NORM) {
                const float p1 = ts.y * red_a * (1.0f / Geo::CELLS);
                const float p2 = red_c * ts.y / ((float)Geo::CELLS * ts.z);
                hF += fmaf(-p2, ts.x, p1);
                hE += p2;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    g[j][0] -= fmaf(p2, xc[j].x - ts.x, p1);
                    g[j][1] -= fmaf(p2, xc[j].y - ts.x, p1);
                }
            }
        }
        if (NORM && tid == 0) p.hterm[(size_t)smp * gridDim.x + blk] = make_float2(hF, hE);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            *reinterpret_cast<float2 *>(p.gx + so + (size_t)j * K) = make_float2(g[j][0], g[j][1]);
            *reinterpret_cast<float2 *>(p.dsum + so + (size_t)j * K) = make_float2(dsum[j][0], dsum[j][1]);
            *reinterpret_cast<float2 *>(p.dsb + so + (size_t)j * K) = make_float2(dsacc[j][0], dsacc[j][1]);
        }
    }
}

// ------------------------------------------------------------------------- weight gradients
// NORM (per-block normalisation): the stencil input was (tile - mean_t) / (std_t + eps) and the stored deltas
// are already divided by (std_t + eps), so the tile mean is subtracted from each window value and the bias
// gradient multiplies the stored delta by (std_t + eps) again.
// FUSE_IN: x is a raw step output; its tile cells are normalised with the sample's whole-grid statistics on their
// way from the staging buffer into the tile (as in step_fwd_fast8), so the normalised tensor is never stored.
template <int SUB, bool USE_TMA, bool NORM = false, bool FUSE_IN = false>
__global__ void __launch_bounds__(bwd8::THREADS, 3) bwd_wgrad8(const __grid_constant__ CUtensorMap x_map, const BwdParams p)
{
    using namespace bwd8;
    using Geo = PatchGeo<SUB>;
    constexpr int RS = Geo::RS, PS = Geo::PS, TS = Geo::TS, SLOTS = Geo::SLOTS;
    constexpr unsigned SOFF_MASK = (1u << Geo::SOFF_BITS) - 1, HALO_BIT = 1u << Geo::SOFF_BITS;
    constexpr int SRC_SHIFT = Geo::SOFF_BITS + 1;
    constexpr bool CI_SMEM = SUB == 4;  // 14 cell descriptors per thread do not fit beside 108 accumulators
    static_assert(SUB == 8 || USE_TMA, "block 4 tiles are fetched by bulk tensor copy only");
    // One pool: the staging ring (USE_TMA: raw 10 x 10 rows of 16 floats, x from 8 bx - 4, of the step
    // input, two samples deep), then the two tiles. The cluster reduction at the end reuses all of it.
    constexpr int STGF = USE_TMA ? 2 * STG : 4;
    constexpr int POOL = STGF + 2 * TS;
    __shared__ __align__(128) float pool[POOL];
    float(*staging)[USE_TMA ? STG : 4] = reinterpret_cast<float(*)[USE_TMA ? STG : 4]>(pool);
    float(*tiles)[TS] = reinterpret_cast<float(*)[TS]>(pool + STGF);
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ unsigned ctab[CI_SMEM ? SLOTS * THREADS : 1];
    static_assert(!FUSE_IN || (SUB == 8 && USE_TMA), "normalise-on-load: block 8 with bulk tensor copies");
    __shared__ float2 gbtab[FUSE_IN ? SLOTS * THREADS : 1];  // (gamma, beta) per tile cell; 0 outside the grid
    const int tid = threadIdx.x;
    const int xp = tid & 3, yp = (tid >> 2) & 3, z = tid >> 4;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g00 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + 2 * yp)) * K + (bx * 8 + 2 * xp);
    const long long origin = ((long long)(bz * 8 - 1) * p.N + (by * 8 - 1)) * K + (bx * 8 - 1);

    // tile cells this thread fetches: low bits tile offset, then the halo bit, then the source offset
    unsigned cinfo[CI_SMEM ? 1 : SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        const int i = tid + j * THREADS;
        unsigned ci = 0xffffffffu;
        if (FUSE_IN && i < SLOTS * THREADS) gbtab[i] = make_float2(0.0f, 0.0f);
        if (i < Geo::CELLS) {
            int soff, cz, cy, cx;
            bool halo;
            Geo::cell(i, soff, cz, cy, cx, halo);
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gx = bx * 8 + cx - 1;
            if (FUSE_IN && gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < K) {
                const long long rel = origin + ((long long)cz * p.N + cy) * K + cx;
                gbtab[i] = make_float2(p.gamma[rel], p.beta[rel]);
            }
            if (USE_TMA)  // every cell comes from the staging buffer; the copy zero-fills what lies outside the grid
                ci = (unsigned)soff | (halo ? HALO_BIT : 0u) | ((unsigned)((cz * 10 + cy) * 16 + cx + 3) << SRC_SHIFT);
            else if (gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < K)
                ci = (unsigned)soff | (halo ? HALO_BIT : 0u) | ((unsigned)((cz * p.N + cy) * K + cx) << SRC_SHIFT);
            else {
                tiles[0][soff] = 0.0f;  // outside the grid: zero for the CTA's whole life
                tiles[1][soff] = 0.0f;
            }
        }
        if (CI_SMEM) ctab[i] = ci;
        else cinfo[CI_SMEM ? 0 : j] = ci;
    }
    auto cell_info = [&](int j) { return CI_SMEM ? ctab[tid + j * THREADS] : cinfo[CI_SMEM ? 0 : j]; };
    float dw[27][2][2];
#pragma unroll
    for (int t = 0; t < 27; ++t)
#pragma unroll
        for (int j = 0; j < 2; ++j) dw[t][j][0] = dw[t][j][1] = 0.0f;
    float db[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, ds[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
    __syncthreads();

    const int toff = Geo::window_origin(xp, yp, z);
    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    // Per sample the whole input tile is written once: halo cells into both tiles (they never change),
    // interior cells into tile 0 (iteration 0). Iteration t >= 1 only rewrites the block interior of
    // tile t & 1, every thread its own four cells, from the replayed activations. Loads run one
    // sample (tile cells) resp. one iteration (own activations, deltas) ahead of their use.
    float pf[USE_TMA ? 1 : SLOTS];
    const unsigned bar_base = smem_u32(bars);
    auto fetch_tile = [&](int smp) {
        if (smp < s1) {
            if (USE_TMA) {
                if (tid == 0) {
                    const int par = (smp - s0) & 1;
                    mbar_expect_tx(bar_base + 8 * par, STG * 4);
                    tma_load_4d(smem_u32(staging[par]), &x_map, bar_base + 8 * par, bx * 8 - 4, by * 8 - 1, bz * 8 - 1,
                                smp);
                }
            } else {
                const float *xs = p.x + (size_t)smp * P + origin;
#pragma unroll
                for (int j = 0; j < SLOTS; ++j)
                    if (cell_info(j) != 0xffffffffu) pf[j] = ld_pinned(xs + (cell_info(j) >> SRC_SHIFT));
            }
        }
    };
    if (USE_TMA) {
        if (tid == 0) {
            mbar_init(bar_base, 1);
            mbar_init(bar_base + 8, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            fence_proxy_async();
        }
        __syncthreads();
    }
    float2 xn[2], dn[2];  // own activations and deltas of the step handled next
    float4 tsn = make_float4(0.0f, 1.0f, 1.0f, 1.0f);  // NORM: and its tile statistics
    auto fetch_step = [&](int smp, int it) {
        if (smp < s1) {
            if (NORM) tsn = p.tile_stats[((size_t)it * p.B + smp) * gridDim.x + blk];
            const size_t o = ((size_t)it * p.B + smp) * P + g00;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                dn[j] = ld_pinned2(p.delta + o + (size_t)j * K);
                if (it > 0) xn[j] = ld_pinned2(p.save_x + o - (size_t)p.B * P + (size_t)j * K);
            }
        }
    };
    fetch_tile(s0);
    if (USE_TMA) fetch_tile(s0 + 1);
    fetch_step(s0, 0);
    for (int smp = s0; smp < s1; ++smp) {
        float2 dsv[2];  // consumed after the sample's iterations
#pragma unroll
        for (int j = 0; j < 2; ++j) dsv[j] = ld_pinned2(p.dsb + (size_t)smp * P + g00 + (size_t)j * K);
        const int par = (smp - s0) & 1;
        if (USE_TMA) {
            if (!mbar_wait_bounded(bar_base + 8 * par, ((smp - s0) >> 1) & 1, kSpinLimit) && p.error_flag)
                *p.error_flag = 1;
        }
        __syncthreads();  // the previous sample's tiles are no longer read
        const float2 mr = FUSE_IN ? p.in_stats[smp] : make_float2(0.0f, 1.0f);
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            const unsigned ci = cell_info(j);
            if (ci != 0xffffffffu) {
                float v = USE_TMA ? staging[par][ci >> SRC_SHIFT] : pf[USE_TMA ? 0 : j];
                if (FUSE_IN) {
                    const float2 gb = gbtab[tid + j * THREADS];
                    v = fmaf((v - mr.x) * mr.y, gb.x, gb.y);
                }
                tiles[0][ci & SOFF_MASK] = v;
                if (ci & HALO_BIT) tiles[1][ci & SOFF_MASK] = v;
            }
        }
        if (!USE_TMA) fetch_tile(smp + 1);
        for (int it = 0; it < p.inner; ++it) {
            float dl[2][2] = {{dn[0].x, dn[0].y}, {dn[1].x, dn[1].y}};
            const float tmean = tsn.x, tsd = tsn.w;
            float *tl_w = tiles[it & 1];
            if (it > 0) {
                float *to = tl_w + toff + PS + RS + 1;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    to[j * RS] = xn[j].x;
                    to[j * RS + 1] = xn[j].y;
                }
            }
            if (it + 1 < p.inner) fetch_step(smp, it + 1);
            else fetch_step(smp + 1, 0);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                db[j][0] = NORM ? fmaf(dl[j][0], tsd, db[j][0]) : db[j][0] + dl[j][0];
                db[j][1] = NORM ? fmaf(dl[j][1], tsd, db[j][1]) : db[j][1] + dl[j][1];
            }
            __syncthreads();  // tile complete (the other tile may still be read by slower threads)
            if (USE_TMA && it == 0) fetch_tile(smp + 2);  // everyone has copied this sample's staging buffer
            const float *tl = tl_w + toff;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    float v[4] = {v01.x, v01.y, v23.x, v23.y};
                    if (NORM) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) v[c] -= tmean;
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int bb = r - j;
                        if (bb >= 0 && bb <= 2) {
#pragma unroll
                            for (int c = 0; c < 3; ++c) {
                                dw[a * 9 + bb * 3 + c][j][0] = fmaf(v[c], dl[j][0], dw[a * 9 + bb * 3 + c][j][0]);
                                dw[a * 9 + bb * 3 + c][j][1] = fmaf(v[c + 1], dl[j][1], dw[a * 9 + bb * 3 + c][j][1]);
                            }
                        }
                    }
                }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            ds[j][0] += dsv[j].x;
            ds[j][1] += dsv[j].y;
        }
    }
    if (p.cluster_reduce) {
        // The chunks of one region form a thread-block cluster. In rounds of as many float2 units as
        // the shared-memory pool holds, every CTA parks its partial sums in its own shared memory;
        // CTA r of the cluster then sums the units u = r, r + size, ... of the round over all CTAs
        // in rank order through distributed shared memory and stores them: no atomics, and the
        // result does not depend on scheduling.
        constexpr int UPR = (POOL / 2) / THREADS;  // units per round
        float2 *red = reinterpret_cast<float2 *>(pool);
        cg::cluster_group cl = cg::this_cluster();
        const unsigned rank = cl.block_rank(), size = cl.num_blocks();
#pragma unroll
        for (int base = 0; base < RED_UNITS; base += UPR) {
            __syncthreads();  // the pool is no longer read: by the stencil, or by this CTA's previous round
#pragma unroll
            for (int u = base; u < base + UPR && u < RED_UNITS; ++u) {
                float2 v;
                if (u < 54) v = make_float2(dw[u >> 1][u & 1][0], dw[u >> 1][u & 1][1]);
                else if (u < 56) v = make_float2(db[u & 1][0], db[u & 1][1]);
                else v = make_float2(ds[u & 1][0], ds[u & 1][1]);
                red[(u - base) * THREADS + tid] = v;
            }
            cl.sync();
            const unsigned end = base + UPR < RED_UNITS ? base + UPR : RED_UNITS;
            for (unsigned u = base + rank; u < end; u += size) {
                float2 acc = make_float2(0.0f, 0.0f);
                for (unsigned r = 0; r < size; ++r) {
                    const float2 v = cl.map_shared_rank(red, r)[(u - base) * THREADS + tid];
                    acc.x += v.x;
                    acc.y += v.y;
                }
                const unsigned j = u & 1;
                float *dst = u < 54 ? p.gw + (size_t)(u >> 1) * P : (u < 56 ? p.gb : p.gs);
                *reinterpret_cast<float2 *>(dst + g00 + (size_t)j * K) = acc;
            }
            cl.sync();  // nobody overwrites or leaves while another CTA still reads its shared memory
        }
    } else {
#pragma unroll
        for (int t = 0; t < 27; ++t)
#pragma unroll
            for (int j = 0; j < 2; ++j)
                *reinterpret_cast<float2 *>(p.gw + (size_t)t * P + g00 + (size_t)j * K) = make_float2(dw[t][j][0], dw[t][j][1]);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            *reinterpret_cast<float2 *>(p.gb + g00 + (size_t)j * K) = make_float2(db[j][0], db[j][1]);
            *reinterpret_cast<float2 *>(p.gs + g00 + (size_t)j * K) = make_float2(ds[j][0], ds[j][1]);
        }
    }
}

// ------------------------------------------------------------ gradient across block borders
// First form (bwd_halo8_k; runs block 4, and was the block-8 kernel before the face-split form
// further down, which is 1.25x faster there).
// grad_x of a cell on a block surface also receives w[n][t] * dsum[n] from every neuron n of a
// neighbouring block that reads the cell as a halo cell. One CTA per block and batch chunk, one
// thread per surface cell (296 of the 512 cells). Per sample the CTA stages the one-voxel shell
// of dsum around its block in shared memory (the interior of the tile stays zero), and a thread
// sums all 27 taps from the tile with its weights in registers: taps whose source lies inside the
// block read a zero. A cell of a sample is handled by exactly one thread: no atomics.
// The kernel is bound by the load/store unit: the 488 shell cells and 296 grad_x cells of a
// sample are scattered 4-byte accesses (an x face has one useful float per 32-byte sector).
// Tried and slower: 4-byte asynchronous copies three samples ahead (each costs several
// shared-memory wavefronts), a bulk tensor copy of the whole neighbourhood (its dense rows of
// 16 floats put all cells of an x face on two shared-memory banks), and skipping the taps whose
// weight is zero (the per-lane predicates cost more than the loads they save).
// With block size 4 the CTA still owns an 8 x 8 x 8 region (eight blocks): one thread per cell, 448
// of the 512 lie on a block surface, and the whole 10 x 10 x 10 neighbourhood of dsum is staged
// because neighbouring blocks of the same region feed each other too. There a tap whose source
// lies in the cell's own block reads a real value and multiplies it by a zero weight, so a
// non-finite dsum spreads to the cells around it (the in-block sweep has spread it to them anyway).
template <int SUB>
struct HaloGeo;
template <>
struct HaloGeo<8> {
    static constexpr int THREADS = 320, SLOTS = 4;  // 296 surface cells; ceil(1000 / 320) tile cells fetched per thread
};
template <>
struct HaloGeo<4> {
    static constexpr int THREADS = 512, SLOTS = 2;
};

template <int SUB>
__global__ void __launch_bounds__(HaloGeo<SUB>::THREADS) bwd_halo8_k(const float *__restrict__ w, const float *__restrict__ dsum,
                                                                     float *__restrict__ gx, int B, int M, int N, int K, int spc)
{
    constexpr int THREADS = HaloGeo<SUB>::THREADS, SLOTS = HaloGeo<SUB>::SLOTS, TS = 1000;
    constexpr int SH = SUB == 8 ? 3 : 2;
    __shared__ float tile[2][TS];
    const int tid = threadIdx.x;
    const int nbx = K >> 3, nby = N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)M * N * K;
    const long long origin = ((long long)(bz * 8 - 1) * N + (by * 8 - 1)) * K + (bx * 8 - 1);

    for (int i = tid; i < 2 * TS; i += THREADS) (&tile[0][0])[i] = 0.0f;

    // neighbourhood cells this thread fetches: bits 0..9 tile offset, bits 10.. offset from the origin
    unsigned cinfo[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        const int i = tid + j * THREADS;
        unsigned ci = 0xffffffffu;
        if (i < TS) {
            const int cx = i % 10, cy = (i / 10) % 10, cz = i / 100;
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gxx = bx * 8 + cx - 1;
            // block 8: only the shell is ever read with a non-zero weight, and the interior must stay zero
            const bool wanted = SUB == 4 || cx == 0 || cx == 9 || cy == 0 || cy == 9 || cz == 0 || cz == 9;
            if (wanted && gz >= 0 && gz < M && gy >= 0 && gy < N && gxx >= 0 && gxx < K)
                ci = (unsigned)i | ((unsigned)((cz * N + cy) * K + cx) << 10);
        }
        cinfo[j] = ci;
    }

    // the cell of this thread inside the region
    int lz = 0, ly = 0, lx = 0;
    bool active;
    if (SUB == 8) {  // surface cells only: the two z faces, then the y faces, then the x faces
        active = tid < 296;
        if (tid < 128) {
            lz = (tid >> 6) * 7; ly = (tid >> 3) & 7; lx = tid & 7;
        } else if (tid < 224) {
            const int j = tid - 128;
            ly = (j / 48) * 7; lz = 1 + (j % 48) / 8; lx = j & 7;
        } else if (active) {
            const int j = tid - 224;
            lx = (j / 36) * 7; lz = 1 + (j % 36) / 6; ly = 1 + j % 6;
        }
    } else {
        lz = tid >> 6; ly = (tid >> 3) & 7; lx = tid & 7;
        const int qz = lz & 3, qy = ly & 3, qx = lx & 3;
        active = !(qz > 0 && qz < 3 && qy > 0 && qy < 3 && qx > 0 && qx < 3);  // the 2^3 core of a block has no outside neighbour
    }
    const int z = bz * 8 + lz, y = by * 8 + ly, x = bx * 8 + lx;
    const size_t c = ((size_t)z * N + y) * K + x;
    float wd[27];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        // neuron n = c - offset(t) reaches c through its tap t
        const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
        const int nz = z - dz, ny = y - dy, nx = x - dx;
        const bool other = active && ((nz >> SH) != (z >> SH) || (ny >> SH) != (y >> SH) || (nx >> SH) != (x >> SH)) &&
                           nz >= 0 && nz < M && ny >= 0 && ny < N && nx >= 0 && nx < K;
        wd[t] = other ? w[(size_t)t * P + ((size_t)nz * N + ny) * K + nx] : 0.0f;
    }
    const int tbase = (lz + 1) * 100 + (ly + 1) * 10 + (lx + 1);

    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    float pf[SLOTS];
    auto fetch = [&](int smp) {
        if (smp < s1) {
            const float *src = dsum + (size_t)smp * P + origin;
#pragma unroll
            for (int j = 0; j < SLOTS; ++j)
                if (cinfo[j] != 0xffffffffu) pf[j] = ld_pinned(src + (cinfo[j] >> 10));
        }
    };
    fetch(s0);
    float gnext = 0.0f;
    if (active && s0 < s1) gnext = gx[(size_t)s0 * P + c];
    __syncthreads();  // tiles are zeroed
    for (int smp = s0; smp < s1; ++smp) {
        float *tl = tile[smp & 1];
#pragma unroll
        for (int j = 0; j < SLOTS; ++j)
            if (cinfo[j] != 0xffffffffu) tl[cinfo[j] & 0x3ff] = pf[j];
        fetch(smp + 1);
        float acc = gnext;
        if (active && smp + 1 < s1) gnext = gx[(size_t)(smp + 1) * P + c];
        __syncthreads();  // the other tile may still be read by slower threads; it is rewritten after the next barrier
        if (active) {
#pragma unroll
            for (int t = 0; t < 27; ++t) {
                const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
                acc = fmaf(wd[t], tl[tbase - (dz * 100 + dy * 10 + dx)], acc);
            }
            gx[(size_t)smp * P + c] = acc;
        }
    }
}

// Block 8, second form: the same sums split by the face a tap crosses. Three groups of 128 threads
// work at once, one per axis: a thread of the z group owns one cell of the two z faces (2 x 64)
// and sums the nine taps whose source lies across that face; the y group does the same for the y
// faces with the taps that cross y but not z, the x group for the x faces with the taps that cross
// x only (a tap that crosses several faces at an edge or corner belongs to the first axis in the
// order z, y, x; the other groups carry a zero weight for it). That is 9 shared-memory reads per
// thread instead of 27. The partial sums go to shared memory, and after a barrier one thread per
// surface cell adds the up to three of them to grad_x in the fixed order z, y, x.
// (Also tried: the reverse sweep writing the x faces of the delta sums packed, so that this kernel
// reads them as whole sectors: 3 % here, and it costs the reverse sweep as much. The same face
// split for block 4, with 8 x 6 faces of 16 cells and 768 threads, was 13 % slower than the first
// form there, which therefore still runs block 4.)
namespace border8 {
constexpr int THREADS = 384;
constexpr int TS = 1000;
constexpr int SLOTS = 3;  // ceil(1000 / 384)
}  // namespace border8

// hterm != nullptr (per-block normalisation): every cell of a region's tile, halo included, also owes
// F + x[c] E to that region's statistics (bwd_reverse8 has taken it from the region's own cells); a surface
// cell lies in the tiles of the up to seven neighbouring regions across the faces it touches.
// TWO (the gated update): a second weight set w2 with its own delta sums dsum2 is added in the same pass, so the
// surface cells of grad_x are read and written once for both branches.
template <bool TWO>
__global__ void __launch_bounds__(border8::THREADS) bwd_border8_k(const float *__restrict__ w, const float *__restrict__ dsum,
                                                                  float *__restrict__ gx, int B, int M, int N, int K, int spc,
                                                                  const float2 *__restrict__ hterm,
                                                                  const float *__restrict__ x, size_t tap_stride,
                                                                  const float *__restrict__ w2,
                                                                  const float *__restrict__ dsum2)
{
    using namespace border8;
    __shared__ float tile[2][TS];
    __shared__ float tile2[TWO ? 2 : 1][TWO ? TS : 1];
    __shared__ float part[2][3][128];  // [sample parity][axis][face cell]
    const int tid = threadIdx.x;
    const int nbx = K >> 3, nby = N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)M * N * K;
    const long long origin = ((long long)(bz * 8 - 1) * N + (by * 8 - 1)) * K + (bx * 8 - 1);

    for (int i = tid; i < 2 * TS; i += THREADS) {
        (&tile[0][0])[i] = 0.0f;
        if (TWO) (&tile2[0][0])[i] = 0.0f;
    }

    // shell cells this thread fetches: bits 0..9 tile offset, bits 10.. offset from the origin
    unsigned cinfo[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        const int i = tid + j * THREADS;
        unsigned ci = 0xffffffffu;
        if (i < TS) {
            const int cx = i % 10, cy = (i / 10) % 10, cz = i / 100;
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gxx = bx * 8 + cx - 1;
            const bool shell = cx == 0 || cx == 9 || cy == 0 || cy == 9 || cz == 0 || cz == 9;
            if (shell && gz >= 0 && gz < M && gy >= 0 && gy < N && gxx >= 0 && gxx < K)
                ci = (unsigned)i | ((unsigned)((cz * N + cy) * K + cx) << 10);
        }
        cinfo[j] = ci;
    }

    // ---- role 1: one cell of one face, nine taps across that face
    const int axis = tid >> 7, fc = tid & 127;  // axis 0 = z, 1 = y, 2 = x; fc = face (low / high) * 64 + cell
    const int side = fc >> 6, u = (fc >> 3) & 7, v = fc & 7;
    int l[3];  // local (z, y, x) of the face cell
    l[axis] = side * 7;
    l[axis == 0 ? 1 : 0] = u;
    l[axis == 2 ? 1 : 2] = v;
    const int dcross = side == 0 ? 1 : -1;  // the source n = c - offset lies across the low face when the offset is +1
    float wf[9], wf2[TWO ? 9 : 1];
    int toff[9];
#pragma unroll
    for (int q = 0; q < 9; ++q) {
        int d[3];
        d[axis] = dcross;
        d[axis == 0 ? 1 : 0] = q / 3 - 1;
        d[axis == 2 ? 1 : 2] = q % 3 - 1;
        // an earlier axis (z before y before x) owns the tap if the source also lies across its face
        bool owned = true;
        for (int a = 0; a < axis; ++a) {
            const int s = l[a] - d[a];
            if (s < 0 || s > 7) owned = false;
        }
        const int nz = bz * 8 + l[0] - d[0], ny = by * 8 + l[1] - d[1], nx = bx * 8 + l[2] - d[2];
        const bool ok = owned && nz >= 0 && nz < M && ny >= 0 && ny < N && nx >= 0 && nx < K;
        const int t = (d[0] + 1) * 9 + (d[1] + 1) * 3 + (d[2] + 1);
        wf[q] = ok ? w[(size_t)t * tap_stride + ((size_t)nz * N + ny) * K + nx] : 0.0f;
        if (TWO) wf2[q] = ok ? w2[(size_t)t * tap_stride + ((size_t)nz * N + ny) * K + nx] : 0.0f;
        toff[q] = (l[0] + 1 - d[0]) * 100 + (l[1] + 1 - d[1]) * 10 + (l[2] + 1 - d[2]);
    }

    // ---- role 2: one surface cell (the two z faces, then the y faces, then the x faces), which adds its partial sums to grad_x
    int sz = 0, sy = 0, sx = 0;
    const bool active = tid < 296;
    if (tid < 128) {
        sz = (tid >> 6) * 7; sy = (tid >> 3) & 7; sx = tid & 7;
    } else if (tid < 224) {
        const int j = tid - 128;
        sy = (j / 48) * 7; sz = 1 + (j % 48) / 8; sx = j & 7;
    } else if (active) {
        const int j = tid - 224;
        sx = (j / 36) * 7; sz = 1 + (j % 36) / 6; sy = 1 + j % 6;
    }
    const size_t c = ((size_t)(bz * 8 + sz) * N + by * 8 + sy) * K + bx * 8 + sx;
    // where this cell's partial sums are (-1: the cell is not on a face of that axis)
    const int pz = (sz == 0 || sz == 7) ? (sz / 7) * 64 + sy * 8 + sx : -1;
    const int py = (sy == 0 || sy == 7) ? (sy / 7) * 64 + sz * 8 + sx : -1;
    const int px = (sx == 0 || sx == 7) ? (sx / 7) * 64 + sz * 8 + sy : -1;
    // the neighbouring regions whose tile holds this surface cell, in a fixed order (-1: none)
    int nbr[7];
    {
        const int fz = sz == 0 ? -1 : (sz == 7 ? 1 : 0), fy = sy == 0 ? -1 : (sy == 7 ? 1 : 0), fx = sx == 0 ? -1 : (sx == 7 ? 1 : 0);
        const int nbz = M >> 3;
#pragma unroll
        for (int q = 1; q < 8; ++q) {
            const int dz = (q & 4) ? fz : 0, dy = (q & 2) ? fy : 0, dx = (q & 1) ? fx : 0;
            const bool real = ((q & 4) == 0 || fz != 0) && ((q & 2) == 0 || fy != 0) && ((q & 1) == 0 || fx != 0);
            const int z2 = bz + dz, y2 = by + dy, x2 = bx + dx;
            nbr[q - 1] = (hterm && active && real && z2 >= 0 && z2 < nbz && y2 >= 0 && y2 < nby && x2 >= 0 && x2 < nbx)
                             ? (z2 * nby + y2) * nbx + x2
                             : -1;
        }
    }
    const unsigned nregions = gridDim.x;

    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    float pf[SLOTS], pf2[TWO ? SLOTS : 1];
    auto fetch = [&](int smp) {
        if (smp < s1) {
            const float *src = dsum + (size_t)smp * P + origin;
#pragma unroll
            for (int j = 0; j < SLOTS; ++j)
                if (cinfo[j] != 0xffffffffu) {
                    pf[j] = ld_pinned(src + (cinfo[j] >> 10));
                    if (TWO) pf2[j] = ld_pinned(dsum2 + (size_t)smp * P + origin + (cinfo[j] >> 10));
                }
        }
    };
    fetch(s0);
    float gnext = 0.0f;
    if (active && s0 < s1) gnext = gx[(size_t)s0 * P + c];
    __syncthreads();  // tiles are zeroed
    for (int smp = s0; smp < s1; ++smp) {
        const int par = smp & 1;
        float *tl = tile[par];
        float *tl2 = TWO ? tile2[par] : nullptr;
#pragma unroll
        for (int j = 0; j < SLOTS; ++j)
            if (cinfo[j] != 0xffffffffu) {
                tl[cinfo[j] & 0x3ff] = pf[j];
                if (TWO) tl2[cinfo[j] & 0x3ff] = pf2[j];
            }
        fetch(smp + 1);
        const float gcur = gnext;
        if (active && smp + 1 < s1) gnext = gx[(size_t)(smp + 1) * P + c];
        __syncthreads();  // tile complete
        {
            float acc = 0.0f;
#pragma unroll
            for (int q = 0; q < 9; ++q) acc = fmaf(wf[q], tl[toff[q]], acc);
            if (TWO) {
#pragma unroll
                for (int q = 0; q < 9; ++q) acc = fmaf(wf2[q], tl2[toff[q]], acc);
            }
            part[par][axis][fc] = acc;
        }
        __syncthreads();  // partial sums complete; tile and sums of the other parity are free again
        if (active) {
            float acc = gcur;
            if (pz >= 0) acc += part[par][0][pz];
            if (py >= 0) acc += part[par][1][py];
            if (px >= 0) acc += part[par][2][px];
            if (hterm) {
                float f = 0.0f, e = 0.0f;
#pragma unroll
                for (int q = 0; q < 7; ++q)
                    if (nbr[q] >= 0) {
                        const float2 t = hterm[(size_t)smp * nregions + nbr[q]];
                        f += t.x;
                        e += t.y;
                    }
                acc -= fmaf(x[(size_t)smp * P + c], e, f);
            }
            gx[(size_t)smp * P + c] = acc;
        }
    }
}

// ---------------------------------------------------------------------------------- launcher
size_t bwd_fast8_stash_floats(int B, int M, int N, int K, int inner)
{
    // pre-activations of every iteration and the activations between iterations
    const size_t BP = (size_t)B * M * N * K;
    return (size_t)inner * BP + (size_t)(inner > 1 ? inner - 1 : 0) * BP;
}

// floats that the per-block-normalisation backward needs after the ordinary workspace (whose last 16 bytes hold
// the error flag): the tile statistics [inner][B][regions] float4 and the halo terms [B][regions] float2
size_t bwd_fast8_norm_extra_floats(int B, int M, int N, int K, int inner)
{
    const size_t regions = (size_t)(M / 8) * (N / 8) * (K / 8);
    return (size_t)inner * B * regions * 4 + (size_t)B * regions * 2;
}

size_t bwd_fast8_workspace_floats(int B, int M, int N, int K, int inner, bool with_stash)
{
    // [the stash, unless the forward pass kept it,] deltas, delta sums, scale-gradient terms, and 16 bytes
    // whose first int is the error flag of the bounded waits
    const size_t BP = (size_t)B * M * N * K;
    return (with_stash ? bwd_fast8_stash_floats(B, M, N, K, inner) : 0) + (size_t)inner * BP + 2 * BP + 4;
}

bool bwd_fast8_applicable(const float *w, const float *b, const float *s, const float *x, const float *gy, float *gw,
                          float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner, int block,
                          int normalize)
{
    FastFwdParams f{};
    f.w = w; f.b = b; f.s = s; f.x = x;
    f.B = B; f.M = M; f.N = N; f.K = K; f.inner = inner;
    f.normalize = normalize ? 1 : 0;  // per-block normalisation: block 8 only (fast8_applicable says so)
    if (!fast8_applicable(f, block, f.normalize)) return false;
    auto al8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; };
    return al8(gy) && al8(gw) && al8(gb) && al8(gs) && al8(gx) && al8(x);
}

// wgrad launch for one instantiation: plain when one CTA covers a block's batch, otherwise the
// batch chunks of a block as one thread-block cluster
template <int SUB, bool USE_TMA, bool NORM = false, bool FUSE_IN = false>
static int launch_wgrad(const CUtensorMap &map, const BwdParams &p, long long nb, unsigned chunks, cudaStream_t st)
{
    auto kern = bwd_wgrad8<SUB, USE_TMA, NORM, FUSE_IN>;
    if (chunks <= 1) {
        kern<<<(unsigned)nb, bwd8::THREADS, 0, st>>>(map, p);
        return GN_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nb, chunks, 1);
    cfg.blockDim = dim3(bwd8::THREADS, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = chunks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map, p);
    if (e != cudaSuccess) {
        record_cuda_error(e, "bwd_wgrad8 cluster launch");
        return GN_ERR_CUDA;
    }
    return GN_OK;
}

template <int SUB, int INNER_T>
static void launch_reverse_inner(const BwdParams &p, dim3 grid, int act, cudaStream_t st)
{
    switch (act) {
    case GN_ACT_RELU: bwd_reverse8<SUB, GN_ACT_RELU, INNER_T><<<grid, bwd8::THREADS, 0, st>>>(p); break;
    case GN_ACT_LEAKY_RELU: bwd_reverse8<SUB, GN_ACT_LEAKY_RELU, INNER_T><<<grid, bwd8::THREADS, 0, st>>>(p); break;
    case GN_ACT_SILU: bwd_reverse8<SUB, GN_ACT_SILU, INNER_T><<<grid, bwd8::THREADS, 0, st>>>(p); break;
    default: bwd_reverse8<SUB, GN_ACT_TANH, INNER_T><<<grid, bwd8::THREADS, 0, st>>>(p); break;
    }
}

template <int SUB>
static void launch_reverse(const BwdParams &p, dim3 grid, int act, cudaStream_t st)
{
    // two inner iterations (the large configurations of the reference) get an unrolled instantiation:
    // 5 % faster; unrolling four iterations was 5 % slower than the run-time loop, and the
    // weight-gradient kernel unrolled for two spills registers and is 8 % slower
    if (SUB == 8 && p.inner == 2) launch_reverse_inner<SUB, 2>(p, grid, act, st);
    else launch_reverse_inner<SUB, 0>(p, grid, act, st);
}

int launch_bwd_border8(const float *w, size_t tap_stride, const float *dsum, float *gx, int B, int M, int N, int K,
                       cudaStream_t st, const float *w2, const float *dsum2)
{
    const long long nb = (long long)(M / 8) * (N / 8) * (K / 8);
    const int chunks = pick_batch_chunks_balanced(nb, B, 3, 8.0, 32);
    const int spc = (B + chunks - 1) / chunks;
    dim3 grid((unsigned)nb, (unsigned)((B + spc - 1) / spc));
    if (w2)
        bwd_border8_k<true><<<grid, border8::THREADS, 0, st>>>(w, dsum, gx, B, M, N, K, spc, nullptr, nullptr, tap_stride, w2, dsum2);
    else
        bwd_border8_k<false><<<grid, border8::THREADS, 0, st>>>(w, dsum, gx, B, M, N, K, spc, nullptr, nullptr, tap_stride, nullptr,
                                                                nullptr);
    return check_launch("bwd_border8");
}

int launch_step_bwd_fast8(const float *w, const float *b, const float *s, const float *x, const float *gy, float *gw,
                          float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner, int block, int act,
                          const float *stash, float *ws, cudaStream_t st, int normalize, float eps, const float *in_stats,
                          const float *gamma, const float *beta)
{
    // stash != nullptr: the forward pass kept the pre-activations and intermediate activations
    // (launch_step_fwd_fast8 with save_h / save_x), so the replay is skipped
    const size_t P = (size_t)M * N * K, BP = (size_t)B * P;
    float *save_h = stash ? const_cast<float *>(stash) : ws;
    float *save_x = save_h + (size_t)inner * BP;
    float *delta = stash ? ws : save_x + (size_t)(inner > 1 ? inner - 1 : 0) * BP;
    float *dsum = delta + (size_t)inner * BP;
    float *dsb = dsum + BP;
    int *error_flag = reinterpret_cast<int *>(dsb + BP);
    // per-block normalisation: the replay's tile statistics and the halo terms follow the flag's 16 bytes
    const long long nregions = (long long)(M / 8) * (N / 8) * (K / 8);
    float4 *tile_stats = reinterpret_cast<float4 *>(dsb + BP + 4);
    float2 *hterm = reinterpret_cast<float2 *>(tile_stats + (size_t)inner * B * nregions);
    if (normalize && (stash || block != 8)) return GN_ERR_UNSUPPORTED;
    if (in_stats && (normalize || block != 8 || !gamma || !beta)) return GN_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(error_flag, 0, sizeof(int), st) != cudaSuccess) {
        record_cuda_error(cudaGetLastError(), "cudaMemsetAsync");
        return GN_ERR_CUDA;
    }
    int rc;

    FastFwdParams f{};
    f.w = w; f.b = b; f.s = s; f.x = x; f.y = nullptr;
    f.B = B; f.M = M; f.N = N; f.K = K; f.inner = inner; f.sub = block;
    f.save_h = save_h;
    f.save_x = save_x;
    f.error_flag = error_flag;
    f.normalize = normalize ? 1 : 0;
    f.norm_eps = eps;
    f.tile_stats = normalize ? tile_stats : nullptr;
    f.in_stats = reinterpret_cast<const float2 *>(in_stats);  // x is a raw step output: the replay normalises on load
    f.gamma = gamma;
    f.beta = beta;
    if (!stash) {
        rc = launch_step_fwd_fast8(f, act, st);
        if (rc != GN_OK) return rc;
    }

    const long long nb = (long long)(M / 8) * (N / 8) * (K / 8);  // 8^3 regions, one CTA (per batch chunk) each
    BwdParams p{};
    p.w = w; p.s = s; p.x = x; p.gy = gy; p.save_h = save_h; p.save_x = save_x;
    p.delta = delta; p.dsum = dsum; p.dsb = dsb; p.gw = gw; p.gb = gb; p.gs = gs; p.gx = gx;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner;
    p.error_flag = error_flag;
    p.b = b;
    p.tile_stats = tile_stats;
    p.hterm = hterm;
    p.in_stats = reinterpret_cast<const float2 *>(in_stats);
    p.gamma = gamma;
    p.beta = beta;
    {
        const int chunks = pick_batch_chunks_balanced(nb, B, 3, 1.5, 16);
        p.spc = (B + chunks - 1) / chunks;
        dim3 grid((unsigned)nb, (unsigned)((B + p.spc - 1) / p.spc));
        if (normalize) {
            switch (act) {
            case GN_ACT_RELU: bwd_reverse8<8, GN_ACT_RELU, 0, true><<<grid, bwd8::THREADS, 0, st>>>(p); break;
            case GN_ACT_LEAKY_RELU: bwd_reverse8<8, GN_ACT_LEAKY_RELU, 0, true><<<grid, bwd8::THREADS, 0, st>>>(p); break;
            case GN_ACT_SILU: bwd_reverse8<8, GN_ACT_SILU, 0, true><<<grid, bwd8::THREADS, 0, st>>>(p); break;
            default: bwd_reverse8<8, GN_ACT_TANH, 0, true><<<grid, bwd8::THREADS, 0, st>>>(p); break;
            }
        } else if (block == 4) launch_reverse<4>(p, grid, act, st);
        else launch_reverse<8>(p, grid, act, st);
        rc = check_launch("bwd_reverse8");
        if (rc != GN_OK) return rc;
    }
    {
        // One CTA per region covers the batch when the grid already fills the GPU; otherwise the batch
        // is split into at most 8 chunks that form a cluster and combine their sums on chip.
        const int want = nb >= 4LL * sm_count() * 3 ? 1 : pick_batch_chunks_balanced(nb, B, 3, 2.0, 8);
        p.spc = (B + want - 1) / want;
        const unsigned chunks = (unsigned)((B + p.spc - 1) / p.spc);
        p.cluster_reduce = chunks > 1;
        CUtensorMap map;
        memset(&map, 0, sizeof(map));
        const bool tma = fast8_make_tile_map(&map, x, B, M, N, K);  // tiles by bulk tensor copy whenever x allows it
        if (block == 4) {
            if (!tma) return GN_ERR_UNSUPPORTED;  // excluded by bwd_fast8_applicable
            rc = launch_wgrad<4, true>(map, p, nb, chunks, st);
        } else if (in_stats) {
            if (!tma) return GN_ERR_UNSUPPORTED;
            rc = launch_wgrad<8, true, false, true>(map, p, nb, chunks, st);
        } else if (normalize) {
            rc = tma ? launch_wgrad<8, true, true>(map, p, nb, chunks, st) : launch_wgrad<8, false, true>(map, p, nb, chunks, st);
        } else if (tma) {
            rc = launch_wgrad<8, true>(map, p, nb, chunks, st);
        } else {
            rc = launch_wgrad<8, false>(map, p, nb, chunks, st);
        }
        if (rc != GN_OK) return rc;
        rc = check_launch("bwd_wgrad8");
        if (rc != GN_OK) return rc;
    }
    {
        const int chunks = pick_batch_chunks_balanced(nb, B, 3, 8.0, 32);
        const int spc = (B + chunks - 1) / chunks;
        dim3 grid((unsigned)nb, (unsigned)((B + spc - 1) / spc));
        if (block == 4) bwd_halo8_k<4><<<grid, HaloGeo<4>::THREADS, 0, st>>>(w, dsum, gx, B, M, N, K, spc);
        else bwd_border8_k<false><<<grid, border8::THREADS, 0, st>>>(w, dsum, gx, B, M, N, K, spc, normalize ? hterm : nullptr, x, P,
                                                                     nullptr, nullptr);
    }
    rc = check_launch("bwd_halo8");
    if (rc != GN_OK) return rc;
    // callers of the backward rarely look into the workspace: a set flag also goes to the library's status word
    return launch_propagate_flag(error_flag, st);
}

}  // namespace gn
