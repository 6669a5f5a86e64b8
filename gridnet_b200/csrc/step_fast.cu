// Tuned float forward kernel for the block-local grid update with per-block
// normalisation off (the configuration every reference model trains with,
// gridnet/scripts/train_mnist.py:51) and block size 8.
//
// Mapping. One CTA of 128 threads owns one 8x8x8 block and a range of samples.
// A thread owns a 1x2x2 patch of neurons (z; y = 2*yp, 2*yp+1; x = 2*xp, 2*xp+1)
// and keeps their 4 x 27 weights in registers for the CTA's whole life, so the
// weights cross HBM/L2 once per CTA and are reused over all its samples and all
// inner iterations. The 10x10x10 activation tile of a sample (block + stale
// one-voxel halo) sits in shared memory with a row stride of 12 floats: with that
// stride the 64-bit row loads of a half-warp touch all 32 banks exactly once.
// Per inner iteration a thread reads a 3x4x4 window (48 floats) for its
// 4 x 27 = 108 FMAs, 2.25 FMAs per shared-memory float. Shared-memory wavefronts,
// not HBM and not the FMA pipe, are what this kernel runs out of first, so
// everything around the stencil is arranged to cost as few of them as possible.
//
// Pipeline. Each sample has two tiles; inner iteration i reads one and writes the
// block interior of the other (the halo is stored in both when the tile is
// loaded), so one barrier per iteration is enough and new values never wait in
// registers. Tile cells are fetched global -> registers one stage (one sample)
// ahead, so those loads are in flight while the current stage iterates; they are
// written to shared memory when the stage starts. The last inner iteration goes
// straight to global memory.
//
// Fusion with the whole-grid normalisation (gridnet/scripts/train_mnist.py:62-64):
//   FUSE_IN   the input is the previous step's raw output; (x - mean) * rstd *
//             gamma + beta is applied to each tile cell on its way from the
//             prefetch register into shared memory, so the normalised tensor never
//             exists in HBM.
//   STATS_OUT per-sample sum and sum of squares of what this step writes are
//             reduced over each warp (128 values, in float; at block 8 the shuffle
//             rounds run inside the next sample's first iteration) and stored as
//             double partials for norm_finalize_k (norm.cu), which adds them in double.
//
// Reference semantics: gridnet/backend_torch.py:61-142; the kernel it stands in
// for is gridnet_cuda_forward_kernel, src/gridnet_cuda_kernels.cu:101-200.
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "patch_geo.cuh"
#include "tma.cuh"

namespace gn {

namespace fast8 {
constexpr int THREADS = 128;
#ifndef GN_F8_MIN_CTAS
#define GN_F8_MIN_CTAS 3
#endif
constexpr int MIN_CTAS = GN_F8_MIN_CTAS;     // CTAs per SM the register budget is sized for (168 registers per thread)
constexpr int STG = 10 * 10 * 16;  // floats of one TMA staging buffer
constexpr unsigned kSpinLimit = 1u << 18;
// Per-slot descriptor of a tile cell this thread fetches, one register: low bits tile offset
// (PatchGeo::SOFF_BITS of them), next bit = halo cell (kept in both ping-pong tiles), the rest
// the offset of the source: inside the staging buffer, or in global memory relative to the
// tile's origin cell.
constexpr unsigned kSkip = 0xffffffffu;     // slot beyond the tile cells
constexpr unsigned kOutside = 0xfffffffeu;  // cell outside the grid: reads as zero
constexpr unsigned kFirstSpecial = kOutside;
constexpr long long kMaxRel = 1LL << 20;
}  // namespace fast8

// INNER_T > 0: the inner iteration count is a compile-time constant (loop unrolled, tile parity
// folded into addresses); INNER_T == 0: taken from the parameters.
// SUB: the block size (8: the CTA's region is one block; 4: eight blocks, each with its own tile).
// NORM: per-block normalisation (the reference's normalize=True, gridnet/backend_torch.py:92-97,
// src/gridnet_cuda_kernels.cu:164-170): before every inner iteration the stencil input is
// (tile - mean) / (std + eps) over the 1000 cells of the tile (halo and cells outside the grid included), the
// residual stays un-normalised. The sums come from where the values are produced, and the iteration never waits
// for them: the tile commit reduces the halo and the interior of a fresh tile once per sample (double precision);
// the fresh tile's mean c becomes the sample's pivot; every iteration stores each thread's sums of (v - c) and
// (v - c)^2 over the four values it writes, the barrier that publishes the tile publishes them, and after it
// every warp adds the 128 partial sums (two loads and ten shuffles) WHILE the stencil runs on sum w (v - c),
// which needs neither the mean nor the deviation. They enter at the end: h = (acc - (mean - c) sum w) / (std +
// eps) + bias, with the per-neuron sum of the weights in a register. Shifting by c keeps the float sums and the
// subtraction free of cancellation whatever the tile's offset.
template <int SUB, int ACT, bool FUSE_IN, bool STATS_OUT, bool USE_TMA, int INNER_T, bool NORM = false>
__global__ void __launch_bounds__(fast8::THREADS, fast8::MIN_CTAS)
    step_fwd_fast8(const __grid_constant__ CUtensorMap x_map, const FastFwdParams p)
{
    using namespace fast8;
    using Geo = PatchGeo<SUB>;
    constexpr int RS = Geo::RS, PS = Geo::PS, TS = Geo::TS, SLOTS = Geo::SLOTS;
    constexpr unsigned SOFF_MASK = (1u << Geo::SOFF_BITS) - 1, HALO_BIT = 1u << Geo::SOFF_BITS;
    constexpr int SRC_SHIFT = Geo::SOFF_BITS + 1;
    static_assert(SUB == 8 || USE_TMA, "block 4 tiles are fetched by bulk tensor copy only");
    // tiles[sample parity][ping-pong][TS]: static for block 8; for block 4 (41.5 KB, past the 48 KB
    // static limit together with the rest) in dynamic shared memory
    __shared__ __align__(16) float tiles_static[SUB == 8 ? 4 * TS : 4];
    extern __shared__ __align__(16) float tiles_dynamic[];
    float(*tiles)[2][TS] = reinterpret_cast<float(*)[2][TS]>(SUB == 8 ? tiles_static : tiles_dynamic);
    // USE_TMA: raw 10x10 rows of 16 floats (x from 8*bx - 4, the nearest origin TMA accepts), two samples deep
    __shared__ __align__(128) float staging[USE_TMA ? 2 : 1][USE_TMA ? STG : 4];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ float2 gbtab[FUSE_IN ? SLOTS * THREADS : 1];  // (gamma, beta) per tile cell
    static_assert(!NORM || (SUB == 8 && !FUSE_IN && !STATS_OUT), "per-block normalisation: block 8, plain input and output");
    // NORM: (sum, sum of squares) per warp: of the halo and of the interior of a freshly committed tile
    // [sample parity][halo | interior][warp], and of the interior an iteration wrote [iteration parity][warp]
    __shared__ double2 fresh_sums[NORM ? 2 : 1][2][4];
    __shared__ __align__(16) float2 part_sums[2][NORM ? THREADS : 1];
    // NORM: bias, scale and weight sum of the thread's four neurons (kept out of the registers: used once per
    // iteration), and per warp the sample's (halo sum, halo sum of squares, fresh interior sum, ... of squares)
    // relative to the pivot, then the pivot
    // (block 4 keeps bias and scale there too: its variants run out of registers otherwise, and reading them back
    // once per iteration made its forward pass 9 % faster; at block 8 the registers were there and it cost 1 %)
    constexpr bool CONST_SMEM = NORM || SUB == 4;
    __shared__ float4 tconst[3][CONST_SMEM ? THREADS : 1];
    __shared__ float4 wnorm[2][NORM ? 4 : 1];

    const int tid = threadIdx.x;
    const int xp = tid & 3, yp = (tid >> 2) & 3, z = tid >> 4;
    const int nbx = p.kbn, nby = p.N >> 3;  // blocks along K that this launch updates
    const unsigned blk = blockIdx.x;
    const int bx = p.kb0 + blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g00 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + 2 * yp)) * K + (bx * 8 + 2 * xp);
    // offset of the tile's origin cell (block corner minus one voxel; may lie outside the grid)
    const long long origin = ((long long)(bz * 8 - 1) * p.N + (by * 8 - 1)) * K + (bx * 8 - 1);

    // ---- which tile cells this thread fetches for every sample, and where they go
    unsigned cinfo[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        const int i = tid + j * THREADS;
        unsigned ci = kSkip;
        float2 gb = make_float2(0.0f, 0.0f);
        if (i < Geo::CELLS) {
            int soff, cz, cy, cx;
            bool halo;
            Geo::cell(i, soff, cz, cy, cx, halo);
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gx = bx * 8 + cx - 1;
            const bool inside = gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < K;
            const int rel = (cz * p.N + cy) * K + cx;
            if (inside && FUSE_IN) gb = make_float2(p.gamma[origin + rel], p.beta[origin + rel]);
            if (USE_TMA) {
                // every cell is copied from the staging buffer; TMA has zero-filled what lies outside the
                // grid, and gamma = beta = 0 there keeps it zero through the normalisation
                ci = (unsigned)soff | (halo ? HALO_BIT : 0u) | ((unsigned)((cz * 10 + cy) * 16 + cx + 3) << SRC_SHIFT);
            } else if (inside) {
                ci = (unsigned)soff | (halo ? HALO_BIT : 0u) | ((unsigned)rel << SRC_SHIFT);
            } else {
                ci = kOutside;
                // cells outside the grid stay zero for the CTA's whole life
#pragma unroll
                for (int q = 0; q < 4; ++q) (&tiles[0][0][0])[q * TS + soff] = 0.0f;
            }
        }
        cinfo[j] = ci;
        if (FUSE_IN && i < SLOTS * THREADS) gbtab[i] = gb;
    }

    // ---- this thread's parameters: 4 neurons x (27 weights, bias, scale)
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

    if (CONST_SMEM && !NORM) {
        tconst[0][tid] = make_float4(bias[0][0], bias[0][1], bias[1][0], bias[1][1]);
        tconst[1][tid] = make_float4(scl[0][0], scl[0][1], scl[1][0], scl[1][1]);
    }
    if (NORM) {
        float wsum[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};  // sum of each neuron's 27 weights
#pragma unroll
        for (int t = 0; t < 27; ++t)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                wsum[j][0] += w[t][j][0];
                wsum[j][1] += w[t][j][1];
            }
        tconst[0][tid] = make_float4(bias[0][0], bias[0][1], bias[1][0], bias[1][1]);
        tconst[1][tid] = make_float4(scl[0][0], scl[0][1], scl[1][0], scl[1][1]);
        tconst[2][tid] = make_float4(wsum[0][0], wsum[0][1], wsum[1][0], wsum[1][1]);
    }

    const int s0 = blockIdx.y * p.spc;
    const int s1 = min(p.B, s0 + p.spc);
    const int toff = Geo::window_origin(xp, yp, z);  // window origin of this thread inside a tile

    // Software pipeline over the CTA's samples: while sample i iterates on tile set i & 1, the cells
    // of sample i + 1 (fetched into registers during sample i - 1) are normalised and written into the
    // other tile set, and the loads of sample i + 2 are issued. One barrier ends each sample: it
    // publishes the next sample's tiles and retires the current ones.
    float pf[USE_TMA ? 1 : SLOTS];
    float2 pf_mr = make_float2(0.0f, 1.0f);  // (mean, rstd) of the sample that commit() handles next
    const unsigned bar_base = smem_u32(bars);
    // start the fetch of one sample: a bulk tensor copy into the staging ring (USE_TMA) or loads into
    // registers
    auto prefetch = [&](int smp) {
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
                    if (cinfo[j] < kFirstSpecial) pf[j] = ld_pinned(xs + (cinfo[j] >> SRC_SHIFT));
            }
        }
    };
    // fetched cells -> tile set `set`, normalising on the way when the input is a raw step output
    auto commit = [&](int smp, int set) {
        if (smp < s1) {
            const float2 mr = pf_mr;
            const int par = (smp - s0) & 1;
            if (USE_TMA) {
                if (!mbar_wait_bounded(bar_base + 8 * par, ((smp - s0) >> 1) & 1, kSpinLimit) && p.error_flag)
                    *p.error_flag = 1;
            }
            double hs = 0.0, hq = 0.0, is = 0.0, iq = 0.0;
#pragma unroll
            for (int j = 0; j < SLOTS; ++j) {
                const unsigned ci = cinfo[j];
                if (ci < kFirstSpecial) {
                    float v = USE_TMA ? staging[par][ci >> SRC_SHIFT] : pf[j];
                    if (FUSE_IN) {
                        const float2 gb = gbtab[tid + j * THREADS];
                        v = fmaf((v - mr.x) * mr.y, gb.x, gb.y);
                    }
                    tiles[set][0][ci & SOFF_MASK] = v;
                    if (ci & HALO_BIT) tiles[set][1][ci & SOFF_MASK] = v;
                    if (NORM) {
                        const double d = (double)v;
                        if (ci & HALO_BIT) {
                            hs += d;
                            hq = fma(d, d, hq);
                        } else {
                            is += d;
                            iq = fma(d, d, iq);
                        }
                    }
                }
            }
            if (NORM) {
                hs = warp_sum(hs);
                hq = warp_sum(hq);
                is = warp_sum(is);
                iq = warp_sum(iq);
                if ((tid & 31) == 0) {
                    fresh_sums[set][0][tid >> 5] = make_double2(hs, hq);
                    fresh_sums[set][1][tid >> 5] = make_double2(is, iq);
                }
            }
        }
    };
    auto load_stats = [&](int smp) {
        if (FUSE_IN && smp < s1) pf_mr = p.in_stats[smp];
    };

    if (USE_TMA) {
        if (tid == 0) {
            mbar_init(bar_base, 1);
            mbar_init(bar_base + 8, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            fence_proxy_async();
        }
        __syncthreads();
        prefetch(s0);
        prefetch(s0 + 1);
    } else {
        prefetch(s0);
    }
    load_stats(s0);
    __syncthreads();  // zero fill and gamma/beta table are in place
    commit(s0, 0);
    if (!USE_TMA) prefetch(s0 + 1);
    load_stats(s0 + 1);
    __syncthreads();

    const int inner = INNER_T > 0 ? INNER_T : p.inner;
    // STATS_OUT: the (sum, sum of squares) of the four values this thread wrote for the sample before; its five
    // shuffle rounds over the warp run between the first stencil rows of the NEXT sample's first iteration, where
    // their latency hides (done at the end of the sample they were 13 % of the kernel at two inner iterations)
    // (block 8; the block-4 variants, short of registers, reduce at the end of the sample: deferring cost them 6 %)
    constexpr bool DEFER_STATS = STATS_OUT && SUB == 8;
    float ps_sum = 0.0f, ps_sq = 0.0f;
    for (int smp = s0; smp < s1; ++smp) {
        const int set = (smp - s0) & 1;
        // TMA: the staging buffer of THIS sample was consumed a whole sample ago (a barrier has passed),
        // so the copy for sample smp + 2 can start now; registers: they are free once smp + 1 is committed
        if (USE_TMA) prefetch(smp + 2);
        commit(smp + 1, set ^ 1);
        if (!USE_TMA) prefetch(smp + 2);
        load_stats(smp + 2);
        // NORM: the sample's pivot and, relative to it, the sums of the halo (fixed for the sample) and of the
        // fresh interior; every thread adds the same per-warp sums in the same order
        float pivot = 0.0f;
        if (NORM) {
            if ((tid & 31) == 0) {  // one lane per warp; every warp adds the same sums in the same order
                double hs = 0.0, hq = 0.0, is = 0.0, iq = 0.0;
#pragma unroll
                for (int wq = 0; wq < 4; ++wq) {
                    const double2 h2 = fresh_sums[set][0][wq], i2 = fresh_sums[set][1][wq];
                    hs += h2.x;
                    hq += h2.y;
                    is += i2.x;
                    iq += i2.y;
                }
                const float pv = (float)((hs + is) * (1.0 / Geo::CELLS));
                const double c = (double)pv;
                constexpr double NI = 512.0, NH = Geo::CELLS - 512.0;
                wnorm[0][tid >> 5] = make_float4((float)(hs - NH * c), (float)(hq - 2.0 * c * hs + NH * c * c),
                                                 (float)(is - NI * c), (float)(iq - 2.0 * c * is + NI * c * c));
                wnorm[1][tid >> 5] = make_float4(pv, 0.0f, 0.0f, 0.0f);
            }
            __syncwarp();
            pivot = wnorm[1][tid >> 5].x;
        }
#pragma unroll
        for (int it = 0; it < (INNER_T > 0 ? INNER_T : inner); ++it) {
            const bool last = it + 1 == inner;
            const int cur = it & 1;
            const float *tl = tiles[set][cur] + toff;
            float acc[2][2];
            if (CONST_SMEM) {
                const float4 cb0 = tconst[0][tid];
                acc[0][0] = cb0.x, acc[0][1] = cb0.y, acc[1][0] = cb0.z, acc[1][1] = cb0.w;
            } else {
                acc[0][0] = bias[0][0], acc[0][1] = bias[0][1], acc[1][0] = bias[1][0], acc[1][1] = bias[1][1];
            }
            float old[2][2];
            // NORM: the interior sums of this tile relative to the pivot: this lane's share of the 128 partial
            // sums; the five shuffle rounds that add them over the warp sit between the first stencil rows
            float red_s = 0.0f, red_q = 0.0f;
            if (NORM) {
                if (it > 0) {
                    const float4 a = *reinterpret_cast<const float4 *>(&part_sums[it & 1][(tid & 31) * 4]);
                    const float4 c = *reinterpret_cast<const float4 *>(&part_sums[it & 1][(tid & 31) * 4 + 2]);
                    red_s = (a.x + a.z) + (c.x + c.z);
                    red_q = (a.y + a.w) + (c.y + c.w);
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) acc[j][0] = acc[j][1] = 0.0f;
            }
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    float v[4] = {v01.x, v01.y, v23.x, v23.y};
                    if (a == 1 && (r == 1 || r == 2)) {
                        old[r - 1][0] = v[1];
                        old[r - 1][1] = v[2];
                    }
                    if (DEFER_STATS && it == 0 && a * 4 + r < 5 && smp > s0) {  // uniform over the CTA
                        ps_sum += __shfl_xor_sync(0xffffffffu, ps_sum, 16 >> (a * 4 + r));
                        ps_sq += __shfl_xor_sync(0xffffffffu, ps_sq, 16 >> (a * 4 + r));
                    }
                    if (DEFER_STATS && it == 0 && a * 4 + r == 5 && smp > s0 && (tid & 31) == 0)
                        p.out_partials[(size_t)(smp - 1) * p.nparts + (size_t)blk * 4 + (tid >> 5)] =
                            make_double2((double)ps_sum, (double)ps_sq);
                    if (NORM) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) v[c] -= pivot;
                        if (a * 4 + r < 5) {  // one shuffle round per row (uniform: every lane takes part)
                            red_s += __shfl_xor_sync(0xffffffffu, red_s, 16 >> (a * 4 + r));
                            red_q += __shfl_xor_sync(0xffffffffu, red_q, 16 >> (a * 4 + r));
                        }
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
            if (NORM) {
                const float4 wn = wnorm[0][tid >> 5];
                const float is = it > 0 ? red_s : wn.z, iq = it > 0 ? red_q : wn.w;
                // the tile's mean relative to the pivot and 1 / (std + eps); approximate square root and reciprocal
                // (a few ulp, far inside the tolerance of the comparison with the reference)
                const float tmean = (wn.x + is) * (1.0f / Geo::CELLS);
                const float var = fmaxf(fmaf(-tmean, tmean, (wn.y + iq) * (1.0f / Geo::CELLS)), 0.0f);
                float sd, trs;
                asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(sd) : "f"(var));
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(trs) : "f"(sd + p.norm_eps));
                if (p.tile_stats && tid == 0)  // every thread holds the same values
                    p.tile_stats[((size_t)it * p.B + smp) * gridDim.x + blk] =
                        make_float4(pivot + tmean, trs, sd, sd + p.norm_eps);
                const float4 cb = tconst[0][tid], cs = tconst[1][tid], cw = tconst[2][tid];
                const float bb[2][2] = {{cb.x, cb.y}, {cb.z, cb.w}}, ss[2][2] = {{cs.x, cs.y}, {cs.z, cs.w}};
                const float ww[2][2] = {{cw.x, cw.y}, {cw.z, cw.w}};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        acc[j][i] = fmaf(fmaf(-tmean, ww[j][i], acc[j][i]), trs, bb[j][i]);
                        nv[j][i] = fmaf(Act<ACT, float>::fwd(acc[j][i]), ss[j][i], old[j][i]);
                    }
            } else if (CONST_SMEM) {
                const float4 cs0 = tconst[1][tid];
                const float ss0[2][2] = {{cs0.x, cs0.y}, {cs0.z, cs0.w}};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) nv[j][i] = fmaf(Act<ACT, float>::fwd(acc[j][i]), ss0[j][i], old[j][i]);
            } else {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 2; ++i) nv[j][i] = fmaf(Act<ACT, float>::fwd(acc[j][i]), scl[j][i], old[j][i]);
            }
            if (p.save_h) {  // replay for the backward pass: pre-activations, and activations between iterations
                const size_t o = ((size_t)it * p.B + smp) * P + g00;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    *reinterpret_cast<float2 *>(p.save_h + o + (size_t)j * K) = make_float2(acc[j][0], acc[j][1]);
                    if (!last) *reinterpret_cast<float2 *>(p.save_x + o + (size_t)j * K) = make_float2(nv[j][0], nv[j][1]);
                }
            }
            if (!last) {
                // The two z-planes of a warp would hit the same 16 banks with the same element of
                // the pair; odd planes store the pair in the other order, so each store instruction
                // covers all 32 banks once.
                float *to = tiles[set][cur ^ 1] + toff + PS + RS + 1 + (z & 1);
                const int step = 1 - 2 * (z & 1);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    to[j * RS] = (z & 1) ? nv[j][1] : nv[j][0];
                    to[j * RS + step] = (z & 1) ? nv[j][0] : nv[j][1];
                }
                if (NORM) {
                    const float d0 = nv[0][0] - pivot, d1 = nv[0][1] - pivot, d2 = nv[1][0] - pivot, d3 = nv[1][1] - pivot;
                    part_sums[(it + 1) & 1][tid] =
                        make_float2((d0 + d1) + (d2 + d3), fmaf(d0, d0, d1 * d1) + fmaf(d2, d2, d3 * d3));
                }
                __syncthreads();  // the other tile is complete; this one may be overwritten next
            } else {
                if (p.y) {
                    float *ys = p.y + (size_t)smp * P + g00;
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        *reinterpret_cast<float2 *>(ys + (size_t)j * K) = make_float2(nv[j][0], nv[j][1]);
                }
                // slab mode: the boundary columns go straight to the neighbours' packed face buffers
                if (p.face_left && bx == p.kb0 && xp == 0) {
                    const size_t fi = ((size_t)smp * p.M + bz * 8 + z) * p.N + by * 8 + 2 * yp;
                    if (p.face_stride <= 1) {
                        *reinterpret_cast<float2 *>(p.face_left + fi) = make_float2(nv[0][0], nv[1][0]);
                    } else {
                        p.face_left[fi * p.face_stride] = nv[0][0];
                        p.face_left[(fi + 1) * p.face_stride] = nv[1][0];
                    }
                }
                if (p.face_right && bx == p.kb0 + p.kbn - 1 && xp == 3) {
                    const size_t fi = ((size_t)smp * p.M + bz * 8 + z) * p.N + by * 8 + 2 * yp;
                    if (p.face_stride <= 1) {
                        *reinterpret_cast<float2 *>(p.face_right + fi) = make_float2(nv[0][1], nv[1][1]);
                    } else {
                        p.face_right[fi * p.face_stride] = nv[0][1];
                        p.face_right[(fi + 1) * p.face_stride] = nv[1][1];
                    }
                }
                if (STATS_OUT) {
                    // the 128 values of a warp are added in float (ten shuffles instead of twenty: the shuffles,
                    // not the arithmetic, were 13 % of this kernel at two inner iterations); everything above
                    // the warp - 4 partials per block and sample here, their sum per sample in norm_finalize_k -
                    // is double. A warp's sum of 128 values carries a relative error of a few 1e-7.
                    ps_sum = (nv[0][0] + nv[0][1]) + (nv[1][0] + nv[1][1]);
                    ps_sq = fmaf(nv[0][0], nv[0][0], nv[0][1] * nv[0][1]) + fmaf(nv[1][0], nv[1][0], nv[1][1] * nv[1][1]);
                    if (!DEFER_STATS) {
                        ps_sum = warp_sum(ps_sum);
                        ps_sq = warp_sum(ps_sq);
                        if ((tid & 31) == 0)
                            p.out_partials[(size_t)smp * p.nparts + (size_t)blk * 4 + (tid >> 5)] =
                                make_double2((double)ps_sum, (double)ps_sq);
                    }
                }
            }
        }
        __syncthreads();  // next sample's tiles are complete; this sample's tiles are free
    }
    if (DEFER_STATS && s0 < s1) {  // the last sample's statistics
        ps_sum = warp_sum(ps_sum);
        ps_sq = warp_sum(ps_sq);
        if ((tid & 31) == 0)
            p.out_partials[(size_t)(s1 - 1) * p.nparts + (size_t)blk * 4 + (tid >> 5)] = make_double2((double)ps_sum, (double)ps_sq);
    }
}

// ------------------------------------------------------------------ launcher
bool fast8_applicable(const FastFwdParams &p, int block, int normalize)
{
    if ((block != 8 && block != 4) || p.inner < 1) return false;
    if (normalize != p.normalize) return false;  // the caller says which; the parameters must agree
    if (normalize && (block != 8 || p.in_stats || p.out_partials || p.face_left || p.face_right || p.kbn > 0))
        return false;
    if (p.M % 8 || p.N % 8 || p.K % 8) return false;  // a CTA owns an 8 x 8 x 8 region also with block 4
    if ((long long)p.M * p.N * p.K >= (1LL << 31)) return false;
    auto al = [](const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
    // Without bulk tensor copies the per-cell descriptor holds global offsets relative to the tile origin in 20
    // bits, which limits the size of an (N, K) plane; with them the offsets point into the staging buffer.
    const bool bulk = encode_tiled_fn() && al(p.x, 16) && (p.K & 3) == 0;
    if (!bulk && (9LL * p.N + 9) * p.K + 9 >= fast8::kMaxRel) return false;
    if (!(al(p.w, 8) && al(p.b, 8) && al(p.s, 8) && al(p.x, 4) && al(p.y, 8) && al(p.save_h, 8) && al(p.save_x, 8)))
        return false;
    // block 4 tiles are fetched by bulk tensor copy only
    if (block == 4 && (!encode_tiled_fn() || !al(p.x, 16))) return false;
    return true;
}

int g_fast8_spc_override = 0;

int fast8_default_spc(int B, long long nbricks, int inner)
{
    if (g_fast8_spc_override > 0) return g_fast8_spc_override;
    // evenly filled rounds of 3 CTAs per SM; a CTA's fixed work (weight fetch, pipeline fill) is charged in
    // samples: 1.5 of them, or 3.5 where a sample is cheap (one or two inner iterations; measured on a
    // 256 x 256 x 32 slab with batch 32: one CTA per block, 0.611 ms, beats two, 0.638 ms; with eight inner
    // iterations at block 4 the larger charge picked a split that was 15 % slower). It keeps CTAs long where the
    // batch allows it and still splits a small batch over the whole GPU.
    const double fixed = inner <= 2 ? 3.5 : 1.5;
    const int chunks = pick_batch_chunks_balanced(nbricks, B, fast8::MIN_CTAS, fixed, B < 64 ? B : 64);
    return (B + chunks - 1) / chunks;
}

// Tensor map over a float tensor [B, M, N, K]: dims (fastest first) {K, N, M, B}, box {16, 10, 10, 1}.
bool fast8_make_tile_map(CUtensorMap *map, const float *base, int B, int M, int N, int K)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc || (reinterpret_cast<uintptr_t>(base) & 15) || (K & 3)) return false;
    MapKey key{base, 16, 0, {B, M, N, K}};
    (void)cudaGetDevice(&key.dev);
    if (tensor_map_cache_get(key, map)) return true;
    const cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)B};
    const cuuint64_t strides[3] = {(cuuint64_t)K * 4, (cuuint64_t)N * K * 4, (cuuint64_t)M * N * K * 4};
    const cuuint32_t box[4] = {16, 10, 10, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    tensor_map_cache_put(key, *map);
    return true;
}

int launch_step_fwd_fast8(FastFwdParams p, int act, cudaStream_t st)
{
    const long long nb = (long long)(p.M / 8) * (p.N / 8) * (p.K / 8);
    if (!p.error_flag) p.error_flag = device_status_ptr();  // callers without a flag of their own: the library's status word
    if (p.kbn <= 0) {
        p.kb0 = 0;
        p.kbn = p.K / 8;
    }
    const long long nbl = (long long)(p.M / 8) * (p.N / 8) * p.kbn;
    (void)nb;
    if (p.spc <= 0) p.spc = fast8_default_spc(p.B, nbl, p.inner);
    dim3 grid((unsigned)nbl, (unsigned)((p.B + p.spc - 1) / p.spc));
    const bool fin = p.in_stats != nullptr, sout = p.out_partials != nullptr;
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    const bool tma = fast8_make_tile_map(&map, p.x, p.B, p.M, p.N, p.K);  // tiles by bulk tensor copy whenever x allows it
#define SUB4_(A, FI, SO, IT)                                                                              \
    do {                                                                                                  \
        auto kern = step_fwd_fast8<4, A, FI, SO, true, IT>;                                               \
        const size_t dyn = sizeof(float) * 4 * PatchGeo<4>::TS;                                           \
        static unsigned long long attr_set = 0; /* one mask per instantiation: the macro body is its own scope */ \
        if (first_use_on_device(&attr_set)) {                                                             \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn); \
            if (e != cudaSuccess) {                                                                       \
                record_cuda_error(e, "cudaFuncSetAttribute");                                             \
                return GN_ERR_CUDA;                                                                       \
            }                                                                                             \
        }                                                                                                 \
        kern<<<grid, fast8::THREADS, dyn, st>>>(map, p);                                                  \
    } while (0)
#define ONE_(A, FI, SO)                                                                                   \
    do {                                                                                                  \
        if (p.sub == 4) {                                                                                 \
            if (!tma) return GN_ERR_UNSUPPORTED;                                                          \
            if (p.inner == 8) SUB4_(A, FI, SO, 8);                                                        \
            else SUB4_(A, FI, SO, 0);                                                                     \
        } else if (tma && p.inner == 4) step_fwd_fast8<8, A, FI, SO, true, 4><<<grid, fast8::THREADS, 0, st>>>(map, p);  \
        else if (tma && p.inner == 2) step_fwd_fast8<8, A, FI, SO, true, 2><<<grid, fast8::THREADS, 0, st>>>(map, p); \
        else if (tma) step_fwd_fast8<8, A, FI, SO, true, 0><<<grid, fast8::THREADS, 0, st>>>(map, p);     \
        else step_fwd_fast8<8, A, FI, SO, false, 0><<<grid, fast8::THREADS, 0, st>>>(map, p);             \
    } while (0)
#define LAUNCH_(A)                              \
    do {                                        \
        if (fin && sout) ONE_(A, true, true);   \
        else if (fin) ONE_(A, true, false);     \
        else if (sout) ONE_(A, false, true);    \
        else ONE_(A, false, false);             \
    } while (0)
#define NORM_(A)                                                                                                  \
    do {                                                                                                          \
        if (tma && p.inner == 2) step_fwd_fast8<8, A, false, false, true, 2, true><<<grid, fast8::THREADS, 0, st>>>(map, p); \
        else if (tma && p.inner == 4) step_fwd_fast8<8, A, false, false, true, 4, true><<<grid, fast8::THREADS, 0, st>>>(map, p); \
        else if (tma) step_fwd_fast8<8, A, false, false, true, 0, true><<<grid, fast8::THREADS, 0, st>>>(map, p); \
        else step_fwd_fast8<8, A, false, false, false, 0, true><<<grid, fast8::THREADS, 0, st>>>(map, p);         \
    } while (0)
    if (p.normalize) {
        switch (act) {
        case GN_ACT_RELU: NORM_(GN_ACT_RELU); break;
        case GN_ACT_LEAKY_RELU: NORM_(GN_ACT_LEAKY_RELU); break;
        case GN_ACT_SILU: NORM_(GN_ACT_SILU); break;
        default: NORM_(GN_ACT_TANH); break;
        }
        return check_launch("step_fwd_fast8 (per-block normalisation)");
    }
#undef NORM_
    switch (act) {
    case GN_ACT_RELU: LAUNCH_(GN_ACT_RELU); break;
    case GN_ACT_LEAKY_RELU: LAUNCH_(GN_ACT_LEAKY_RELU); break;
    case GN_ACT_SILU: LAUNCH_(GN_ACT_SILU); break;
    default: LAUNCH_(GN_ACT_TANH); break;
    }
#undef LAUNCH_
#undef ONE_
#undef SUB4_
    return check_launch("step_fwd_fast8");
}

}  // namespace gn
