// Tuned float backward of the gated grid update (block 8):
//   gate = sigmoid(hg), hg = sum_t x[n + o_t] wg[t][n] + bg[n];  a = act(hv), hv = sum_t x[n + o_t] wv[t][n] + bv[n]
//   x_new[n] = gate x[n] + (1 - gate) a
// (gridnet/backend_torch.py:145-267; the kernel this stands in for is the gated backward kernel of
// src/gridnet_cuda_kernels.cu:538-734, which does everything in one kernel with shared-memory atomics).
//
// Same four-kernel decomposition as step_bwd_fast.cu, with the thread map of the gated forward kernel
// (step_gated_fast.cu: 256 threads, a thread owns two neurons along x and keeps 2 x 54 values in registers):
//   replay   gated_fwd_fast8 in replay mode stores hv_t, hg_t of every iteration and the activations between;
//   reverse  gated_bwd_reverse8: iterations backwards. dv = g (1 - gate) act'(hv), dg = g (x_t - a) gate (1 - gate);
//            the gradient carried to the iteration before is g gate plus a 27-tap gather over the two delta tiles
//            with TRANSPOSED weights (cell c receives w[n][26 - t] delta[n] from its neighbour n = c + o_t inside
//            the block): no atomics;
//   wgrad    gated_bwd_wgrad8: dWv[n][t] += x_t[n + o_t] dv_t[n], dWg likewise, plus the two bias gradients,
//            accumulated in registers over samples and iterations; batch chunks of a block form a thread-block
//            cluster and add their partial sums through distributed shared memory in rank order;
//   border   bwd_border8_k (step_bwd_fast.cu) with both branches in one pass: the part of grad_x that crosses block
//            borders needs only the per-neuron sums of dv and dg over the iterations.
// Deterministic: no floating-point atomics. Bounded waits on the bulk tensor copies report through the int at
// the end of the workspace.
#include <cooperative_groups.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace gn {
namespace cg = cooperative_groups;

namespace gbwd8 {
constexpr int RS = 12, PS = 120, TS = 1200;
constexpr int THREADS = 256;
constexpr int SLOTS = 4;           // ceil(1000 / 256) tile cells per thread
constexpr int STG = 10 * 10 * 16;  // floats of one bulk-copied neighbourhood (x from 8 bx - 4)
constexpr unsigned kSpinLimit = 1u << 18;
constexpr int RED_UNITS = 56;  // float2 partial sums per thread: 27 taps x 2 branches, 2 biases
}  // namespace gbwd8

struct GatedBwdParams {
    const float *w, *x, *gy;
    const float *save_hv, *save_hg, *save_x;  // from the replay
    float *dv, *dg;                           // [inner][B][P] each
    float *dsum_v, *dsum_g;                   // [B][P] sums over the iterations
    float *gw, *gb, *gx;
    int B, M, N, K, inner, spc;
    int *error_flag;
    int cluster_reduce;
};

// ---------------------------------------------------------------------------- reverse sweep
template <int ACT>
__global__ void __launch_bounds__(gbwd8::THREADS, 1) gated_bwd_reverse8(const GatedBwdParams p)
{
    using namespace gbwd8;
    __shared__ __align__(16) float Dv[2][TS], Dg[2][TS];
    const int tid = threadIdx.x;
    const int xp = tid & 3, y = 2 * ((tid >> 2) & 3) + ((tid >> 4) & 1), z = tid >> 5;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g0 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + y)) * K + (bx * 8 + 2 * xp);

    // transposed weights of both branches: cell c receives w[26 - t][branch][n] * delta[n] from n = c + offset(t)
    // when n is a neuron of c's block, else 0
    float wtv[27][2], wtg[27][2];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
        const int lz = z + dz, ly = y + dy;
        const float *wp = p.w + (size_t)(2 * (26 - t)) * P + g0 + ((long long)dz * p.N + dy) * K + dx;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int lx = 2 * xp + i + dx;
            const bool same = lz >= 0 && lz < 8 && ly >= 0 && ly < 8 && lx >= 0 && lx < 8;
            wtv[t][i] = same ? __ldg(wp + i) : 0.0f;
            wtg[t][i] = same ? __ldg(wp + P + i) : 0.0f;
        }
    }
    for (int i = tid; i < 2 * TS; i += THREADS) {  // the halo of all four tiles stays zero
        (&Dv[0][0])[i] = 0.0f;
        (&Dg[0][0])[i] = 0.0f;
    }
    __syncthreads();

    const int toff = z * PS + y * RS + 2 * xp;
    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    unsigned step = 0;  // picks the delta tiles: consecutive iterations (also across samples) alternate
    // what the iteration handled next needs is fetched one iteration early
    float2 hvn = make_float2(0.0f, 0.0f), hgn = hvn, xon = hvn, gn = hvn;
    auto fetch = [&](int smp, int it) {
        const size_t o = ((size_t)it * p.B + smp) * P + g0;
        hvn = ld_pinned2(p.save_hv + o);
        hgn = ld_pinned2(p.save_hg + o);
        xon = ld_pinned2(it > 0 ? p.save_x + o - (size_t)p.B * P : p.x + (size_t)smp * P + g0);
    };
    if (s0 < s1) {
        fetch(s0, p.inner - 1);
        gn = ld_pinned2(p.gy + (size_t)s0 * P + g0);
    }
    for (int smp = s0; smp < s1; ++smp) {
        float g[2] = {gn.x, gn.y};
        float sv[2] = {0.0f, 0.0f}, sg[2] = {0.0f, 0.0f};
        for (int it = p.inner - 1; it >= 0; --it, ++step) {
            const size_t o = ((size_t)it * p.B + smp) * P + g0;
            const float hv[2] = {hvn.x, hvn.y}, hg[2] = {hgn.x, hgn.y}, xo[2] = {xon.x, xon.y};
            if (it > 0) fetch(smp, it - 1);
            else if (smp + 1 < s1) {
                fetch(smp + 1, p.inner - 1);
                gn = ld_pinned2(p.gy + (size_t)(smp + 1) * P + g0);
            }
            float dv[2], dg[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float gate = sigmoid_(hg[i]);
                float a, da;
                Act<ACT, float>::both(hv[i], a, da);
                dv[i] = g[i] * (1.0f - gate) * da;
                dg[i] = g[i] * (xo[i] - a) * gate * (1.0f - gate);
                sv[i] += dv[i];
                sg[i] += dg[i];
                g[i] *= gate;  // the part of the gradient that the old value carries
            }
            *reinterpret_cast<float2 *>(p.dv + o) = make_float2(dv[0], dv[1]);
            *reinterpret_cast<float2 *>(p.dg + o) = make_float2(dg[0], dg[1]);
            float *tv = Dv[step & 1], *tg = Dg[step & 1];
            tv[toff + PS + RS + 1] = dv[0];
            tv[toff + PS + RS + 2] = dv[1];
            tg[toff + PS + RS + 1] = dg[0];
            tg[toff + PS + RS + 2] = dg[1];
            __syncthreads();
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tv + toff + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tv + toff + a * PS + r * RS + 2);
                    const float2 u01 = *reinterpret_cast<const float2 *>(tg + toff + a * PS + r * RS);
                    const float2 u23 = *reinterpret_cast<const float2 *>(tg + toff + a * PS + r * RS + 2);
                    const float v[4] = {v01.x, v01.y, v23.x, v23.y}, u[4] = {u01.x, u01.y, u23.x, u23.y};
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + r * 3 + c;
                        g[0] = fmaf(wtv[t][0], v[c], g[0]);
                        g[1] = fmaf(wtv[t][1], v[c + 1], g[1]);
                        g[0] = fmaf(wtg[t][0], u[c], g[0]);
                        g[1] = fmaf(wtg[t][1], u[c + 1], g[1]);
                    }
                }
        }
        const size_t so = (size_t)smp * P + g0;
        *reinterpret_cast<float2 *>(p.gx + so) = make_float2(g[0], g[1]);
        *reinterpret_cast<float2 *>(p.dsum_v + so) = make_float2(sv[0], sv[1]);
        *reinterpret_cast<float2 *>(p.dsum_g + so) = make_float2(sg[0], sg[1]);
    }
}

// ------------------------------------------------------------------------- weight gradients
__global__ void __launch_bounds__(gbwd8::THREADS, 1)
    gated_bwd_wgrad8(const __grid_constant__ CUtensorMap x_map, const GatedBwdParams p)
{
    using namespace gbwd8;
    // one pool: the staging ring (raw 10 x 10 rows of 16 floats of the step input, two samples deep), then the two
    // tiles; the cluster reduction at the end reuses all of it
    constexpr int POOL = 2 * STG + 2 * TS;
    __shared__ __align__(128) float pool[POOL];
    float(*staging)[STG] = reinterpret_cast<float(*)[STG]>(pool);
    float(*tiles)[TS] = reinterpret_cast<float(*)[TS]>(pool + 2 * STG);
    __shared__ __align__(8) unsigned long long bars[2];
    const int tid = threadIdx.x;
    const int xp = tid & 3, y = 2 * ((tid >> 2) & 3) + ((tid >> 4) & 1), z = tid >> 5;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const size_t g0 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + y)) * p.K + (bx * 8 + 2 * xp);

    // tile cells this thread copies out of the staging buffer: bits 0..10 tile offset, bit 11 halo
    // (kept in both tiles), bits 12.. staging offset
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
    float dwv[27][2], dwg[27][2];
#pragma unroll
    for (int t = 0; t < 27; ++t) dwv[t][0] = dwv[t][1] = dwg[t][0] = dwg[t][1] = 0.0f;
    float dbv[2] = {0.0f, 0.0f}, dbg[2] = {0.0f, 0.0f};

    const int toff = z * PS + y * RS + 2 * xp;
    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    const unsigned bar_base = smem_u32(bars);
    auto fetch_tile = [&](int smp) {
        if (smp < s1 && tid == 0) {
            const int par = (smp - s0) & 1;
            mbar_expect_tx(bar_base + 8 * par, STG * 4);
            tma_load_4d(smem_u32(staging[par]), &x_map, bar_base + 8 * par, bx * 8 - 4, by * 8 - 1, bz * 8 - 1, smp);
        }
    };
    if (tid == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    __syncthreads();
    float2 xn = make_float2(0.0f, 0.0f), dvn = xn, dgn = xn;  // own activations and deltas of the step handled next
    auto fetch_step = [&](int smp, int it) {
        if (smp < s1) {
            const size_t o = ((size_t)it * p.B + smp) * P + g0;
            dvn = ld_pinned2(p.dv + o);
            dgn = ld_pinned2(p.dg + o);
            if (it > 0) xn = ld_pinned2(p.save_x + o - (size_t)p.B * P);
        }
    };
    fetch_tile(s0);
    fetch_tile(s0 + 1);
    fetch_step(s0, 0);
    for (int smp = s0; smp < s1; ++smp) {
        const int par = (smp - s0) & 1;
        if (!mbar_wait_bounded(bar_base + 8 * par, ((smp - s0) >> 1) & 1, kSpinLimit) && p.error_flag) *p.error_flag = 1;
        __syncthreads();  // the previous sample's tiles are no longer read
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            const unsigned ci = cinfo[j];
            if (ci != 0xffffffffu) {
                const float v = staging[par][ci >> 12];
                tiles[0][ci & 0x7ff] = v;
                if (ci & 0x800) tiles[1][ci & 0x7ff] = v;
            }
        }
        for (int it = 0; it < p.inner; ++it) {
            const float dv[2] = {dvn.x, dvn.y}, dg[2] = {dgn.x, dgn.y};
            float *tl_w = tiles[it & 1];
            if (it > 0) {
                tl_w[toff + PS + RS + 1] = xn.x;
                tl_w[toff + PS + RS + 2] = xn.y;
            }
            if (it + 1 < p.inner) fetch_step(smp, it + 1);
            else fetch_step(smp + 1, 0);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                dbv[i] += dv[i];
                dbg[i] += dg[i];
            }
            __syncthreads();  // tile complete (the other tile may still be read by slower threads)
            if (it == 0) fetch_tile(smp + 2);  // everyone has copied this sample's staging buffer
            const float *tl = tl_w + toff;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    const float v[4] = {v01.x, v01.y, v23.x, v23.y};
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + r * 3 + c;
                        dwv[t][0] = fmaf(v[c], dv[0], dwv[t][0]);
                        dwv[t][1] = fmaf(v[c + 1], dv[1], dwv[t][1]);
                        dwg[t][0] = fmaf(v[c], dg[0], dwg[t][0]);
                        dwg[t][1] = fmaf(v[c + 1], dg[1], dwg[t][1]);
                    }
                }
        }
    }
    // unit u < 54: tap u / 2, branch u & 1 (the weight tensor's own order [27][2][P]); 54, 55: the two biases
    auto unit = [&](int u) {
        if (u < 54) return (u & 1) ? make_float2(dwg[u >> 1][0], dwg[u >> 1][1]) : make_float2(dwv[u >> 1][0], dwv[u >> 1][1]);
        return u == 54 ? make_float2(dbv[0], dbv[1]) : make_float2(dbg[0], dbg[1]);
    };
    if (p.cluster_reduce) {
        // The chunks of one block form a thread-block cluster: in rounds of as many float2 units as the pool
        // holds, every CTA parks its partial sums in its own shared memory; CTA r then adds the units
        // u = r, r + size, ... of the round over all CTAs in rank order through distributed shared memory.
        constexpr int UPR = (POOL / 2) / THREADS;  // units per round
        float2 *red = reinterpret_cast<float2 *>(pool);
        cg::cluster_group cl = cg::this_cluster();
        const unsigned rank = cl.block_rank(), size = cl.num_blocks();
#pragma unroll
        for (int base = 0; base < RED_UNITS; base += UPR) {
            __syncthreads();  // the pool is no longer read: by the stencil, or by this CTA's previous round
#pragma unroll
            for (int u = base; u < base + UPR && u < RED_UNITS; ++u) red[(u - base) * THREADS + tid] = unit(u);
            cl.sync();
            const unsigned end = base + UPR < RED_UNITS ? base + UPR : RED_UNITS;
            for (unsigned u = base + rank; u < end; u += size) {
                float2 acc = make_float2(0.0f, 0.0f);
                for (unsigned r = 0; r < size; ++r) {
                    const float2 v = cl.map_shared_rank(red, r)[(u - base) * THREADS + tid];
                    acc.x += v.x;
                    acc.y += v.y;
                }
                float *dst = u < 54 ? p.gw + (size_t)u * P : p.gb + (size_t)(u - 54) * P;
                *reinterpret_cast<float2 *>(dst + g0) = acc;
            }
            cl.sync();  // nobody overwrites or leaves while another CTA still reads its shared memory
        }
    } else {
#pragma unroll
        for (int u = 0; u < RED_UNITS; ++u) {
            float *dst = u < 54 ? p.gw + (size_t)u * P : p.gb + (size_t)(u - 54) * P;
            *reinterpret_cast<float2 *>(dst + g0) = unit(u);
        }
    }
}

// ---------------------------------------------------------------------------------- launcher
size_t gated_bwd_fast8_workspace_floats(int B, int M, int N, int K, int inner)
{
    // hv, hg of every iteration; activations between iterations; dv, dg of every iteration; their two sums; and 16
    // bytes whose first int is the error flag of the bounded waits
    const size_t BP = (size_t)B * M * N * K;
    return (size_t)(2 * inner + (inner > 1 ? inner - 1 : 0) + 2 * inner + 2) * BP + 4;
}

bool gated_bwd_fast8_applicable(const float *w, const float *b, const float *x, const float *gy, const float *gw,
                                const float *gb, const float *gx, int M, int N, int K, int inner, int block)
{
    if (!gated_fast8_applicable(w, b, x, gx, M, N, K, block, inner)) return false;
    if ((long long)M * N * K >= (1LL << 31)) return false;
    auto al8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; };
    return al8(gy) && al8(gw) && al8(gb) && al8(gx);
}

int launch_gated_bwd_fast8(const float *w, const float *b, const float *x, const float *gy, float *gw, float *gb, float *gx,
                           int B, int M, int N, int K, int inner, int act, float *ws, cudaStream_t st)
{
    const size_t P = (size_t)M * N * K, BP = (size_t)B * P;
    float *save_hv = ws, *save_hg = save_hv + (size_t)inner * BP, *save_x = save_hg + (size_t)inner * BP;
    float *dv = save_x + (size_t)(inner > 1 ? inner - 1 : 0) * BP, *dg = dv + (size_t)inner * BP;
    float *dsum_v = dg + (size_t)inner * BP, *dsum_g = dsum_v + BP;
    int *error_flag = reinterpret_cast<int *>(dsum_g + BP);
    if (cudaMemsetAsync(error_flag, 0, sizeof(int), st) != cudaSuccess) {
        record_cuda_error(cudaGetLastError(), "cudaMemsetAsync");
        return GN_ERR_CUDA;
    }
    int rc = launch_gated_fwd_fast8(w, b, x, nullptr, B, M, N, K, inner, act, st, save_hv, save_hg, save_x, error_flag);
    if (rc != GN_OK) return rc;

    const long long nb = (long long)(M / 8) * (N / 8) * (K / 8);
    GatedBwdParams p{};
    p.w = w; p.x = x; p.gy = gy; p.save_hv = save_hv; p.save_hg = save_hg; p.save_x = save_x;
    p.dv = dv; p.dg = dg; p.dsum_v = dsum_v; p.dsum_g = dsum_g; p.gw = gw; p.gb = gb; p.gx = gx;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner;
    p.error_flag = error_flag;
    {
        const int chunks = pick_batch_chunks_balanced(nb, B, 1, 1.5, 16);
        p.spc = (B + chunks - 1) / chunks;
        dim3 grid((unsigned)nb, (unsigned)((B + p.spc - 1) / p.spc));
        switch (act) {
        case GN_ACT_RELU: gated_bwd_reverse8<GN_ACT_RELU><<<grid, gbwd8::THREADS, 0, st>>>(p); break;
        case GN_ACT_LEAKY_RELU: gated_bwd_reverse8<GN_ACT_LEAKY_RELU><<<grid, gbwd8::THREADS, 0, st>>>(p); break;
        case GN_ACT_SILU: gated_bwd_reverse8<GN_ACT_SILU><<<grid, gbwd8::THREADS, 0, st>>>(p); break;
        default: gated_bwd_reverse8<GN_ACT_TANH><<<grid, gbwd8::THREADS, 0, st>>>(p); break;
        }
        rc = check_launch("gated_bwd_reverse8");
        if (rc != GN_OK) return rc;
    }
    {
        // one CTA per block covers the batch when the grid already fills the GPU; otherwise the batch is split into
        // at most 8 chunks that form a cluster and combine their sums on chip
        const int want = nb >= 4LL * sm_count() ? 1 : pick_batch_chunks_balanced(nb, B, 1, 2.0, 8);
        p.spc = (B + want - 1) / want;
        const unsigned chunks = (unsigned)((B + p.spc - 1) / p.spc);
        p.cluster_reduce = chunks > 1;
        CUtensorMap map;
        memset(&map, 0, sizeof(map));
        if (!fast8_make_tile_map(&map, x, B, M, N, K)) return GN_ERR_UNSUPPORTED;  // excluded by gated_bwd_fast8_applicable
        if (chunks <= 1) {
            gated_bwd_wgrad8<<<(unsigned)nb, gbwd8::THREADS, 0, st>>>(map, p);
        } else {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)nb, chunks, 1);
            cfg.blockDim = dim3(gbwd8::THREADS, 1, 1);
            cfg.dynamicSmemBytes = 0;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = chunks;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            const cudaError_t e = cudaLaunchKernelEx(&cfg, gated_bwd_wgrad8, map, p);
            if (e != cudaSuccess) {
                record_cuda_error(e, "gated_bwd_wgrad8 cluster launch");
                return GN_ERR_CUDA;
            }
        }
        rc = check_launch("gated_bwd_wgrad8");
        if (rc != GN_OK) return rc;
    }
    // grad_x across block borders, both branches in one pass: the value branch (taps at w + 2 t P) and the gate
    // branch (w + (2 t + 1) P)
    rc = launch_bwd_border8(w, 2 * P, dsum_v, gx, B, M, N, K, st, w + P, dsum_g);
    if (rc != GN_OK) return rc;
    return launch_propagate_flag(error_flag, st);
}

}  // namespace gn
