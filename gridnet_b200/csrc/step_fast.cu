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
//             reduced in double precision per warp and stored as partials for
//             norm_finalize_k (norm.cu).
//
// Reference semantics: gridnet/backend_torch.py:61-142; the kernel it stands in
// for is gridnet_cuda_forward_kernel, src/gridnet_cuda_kernels.cu:101-200.
#include "common.cuh"
#include "kernels.h"

namespace gn {

namespace fast8 {
constexpr int RS = 12;          // row stride (floats)
constexpr int PS = 10 * RS;     // plane stride
constexpr int TS = 10 * PS;     // one tile
constexpr int THREADS = 128;
constexpr int SPS = 1;          // samples per pipeline stage (2 measured slower: the prefetch registers crowd out the stencil)
#ifndef GN_F8_MIN_CTAS
#define GN_F8_MIN_CTAS 3
#endif
constexpr int MIN_CTAS = GN_F8_MIN_CTAS;     // CTAs per SM the register budget is sized for (168 registers per thread)
constexpr int SLOTS = 8;        // tile cells handled per thread when loading (8 * 128 >= 1000)
// Per-slot descriptor, one register: bits 0..10 tile offset, bit 11 = halo cell (kept in both
// ping-pong tiles), bits 12..31 global offset relative to the tile's origin cell.
constexpr unsigned kSkip = 0xffffffffu;     // slot beyond the 1000 tile cells
constexpr unsigned kOutside = 0xfffffffeu;  // cell outside the grid: reads as zero
constexpr unsigned kFirstSpecial = kOutside;
constexpr long long kMaxRel = 1LL << 20;
}  // namespace fast8

// A global load that stays where it is written: the compiler may sink an ordinary read-only
// load past barriers down to its first use, which would put the whole memory latency back on
// the critical path of the next stage.
__device__ __forceinline__ float ld_pinned(const float *ptr)
{
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(ptr) : "memory");
    return v;
}

template <int ACT, bool FUSE_IN, bool STATS_OUT>
__global__ void __launch_bounds__(fast8::THREADS, fast8::MIN_CTAS) step_fwd_fast8(const FastFwdParams p)
{
    using namespace fast8;
    __shared__ __align__(16) float tiles[2][SPS][TS];
    __shared__ float2 gbtab[FUSE_IN ? SLOTS * THREADS : 1];  // (gamma, beta) per tile cell

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
        if (i < 1000) {
            const int cx = i % 10, cy = (i / 10) % 10, cz = i / 100;
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gx = bx * 8 + cx - 1;
            const int soff = cz * PS + cy * RS + cx;
            const bool halo = cx == 0 || cx == 9 || cy == 0 || cy == 9 || cz == 0 || cz == 9;
            if (gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < K) {
                const int rel = (cz * p.N + cy) * K + cx;
                ci = (unsigned)soff | (halo ? 0x800u : 0u) | ((unsigned)rel << 12);
                if (FUSE_IN) gb = make_float2(p.gamma[origin + rel], p.beta[origin + rel]);
            } else {
                ci = kOutside;
                // cells outside the grid stay zero for the CTA's whole life
#pragma unroll
                for (int q = 0; q < 2 * SPS; ++q) (&tiles[0][0][0])[q * TS + soff] = 0.0f;
            }
        }
        cinfo[j] = ci;
        if (FUSE_IN) gbtab[i] = gb;
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

    const int s0 = blockIdx.y * p.spc;
    const int s1 = min(p.B, s0 + p.spc);
    const int nstages = (s1 - s0 + SPS - 1) / SPS;
    const int toff = z * PS + 2 * yp * RS + 2 * xp;  // window origin of this thread inside a tile

    // global -> registers for one stage; consumed by commit() one stage later
    float pf[SPS][SLOTS];
    auto prefetch = [&](int st) {
#pragma unroll
        for (int s = 0; s < SPS; ++s) {
            const int smp = s0 + st * SPS + s;
            if (smp < s1) {
                const float *xs = p.x + (size_t)smp * P + origin;
#pragma unroll
                for (int j = 0; j < SLOTS; ++j)
                    if (cinfo[j] < kFirstSpecial) pf[s][j] = ld_pinned(xs + (cinfo[j] >> 12));
            }
        }
    };
    // registers -> tiles, normalising on the way when the input is a raw step output
    auto commit = [&](int st) {
#pragma unroll
        for (int s = 0; s < SPS; ++s) {
            const int smp = s0 + st * SPS + s;
            if (smp < s1) {
                float2 mr = make_float2(0.0f, 1.0f);
                if (FUSE_IN) mr = p.in_stats[smp];
#pragma unroll
                for (int j = 0; j < SLOTS; ++j) {
                    const unsigned ci = cinfo[j];
                    if (ci < kFirstSpecial) {
                        float v = pf[s][j];
                        if (FUSE_IN) {
                            const float2 gb = gbtab[tid + j * THREADS];
                            v = fmaf((v - mr.x) * mr.y, gb.x, gb.y);
                        }
                        tiles[0][s][ci & 0x7ff] = v;
                        if (ci & 0x800) tiles[1][s][ci & 0x7ff] = v;
                    }
                }
            }
        }
    };

    if (nstages > 0) prefetch(0);

    for (int st = 0; st < nstages; ++st) {
        const int smp0 = s0 + st * SPS;
        __syncthreads();  // the previous stage no longer reads the tiles (and the zero fill is done)
        commit(st);
        __syncthreads();
        if (st + 1 < nstages) prefetch(st + 1);

        const int inner = p.inner;
        for (int it = 0; it < inner; ++it) {
            const bool last = it + 1 == inner;
            const int cur = it & 1;
#pragma unroll
            for (int s = 0; s < SPS; ++s) {
                if (smp0 + s < s1) {
                    const float *tl = tiles[cur][s] + toff;
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
                        for (int i = 0; i < 2; ++i)
                            nv[j][i] = fmaf(Act<ACT, float>::fwd(acc[j][i]), scl[j][i], old[j][i]);
                    if (!last) {
                        // The two z-planes of a warp would hit the same 16 banks with the same
                        // element of the pair; odd planes store the pair in the other order, so
                        // each store instruction covers all 32 banks once.
                        float *to = tiles[cur ^ 1][s] + toff + PS + RS + 1 + (z & 1);
                        const int step = 1 - 2 * (z & 1);
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            to[j * RS] = (z & 1) ? nv[j][1] : nv[j][0];
                            to[j * RS + step] = (z & 1) ? nv[j][0] : nv[j][1];
                        }
                    } else {
                        float *ys = p.y + (size_t)(smp0 + s) * P + g00;
#pragma unroll
                        for (int j = 0; j < 2; ++j)
                            *reinterpret_cast<float2 *>(ys + (size_t)j * K) = make_float2(nv[j][0], nv[j][1]);
                        if (STATS_OUT) {
                            double sm = 0.0, sq = 0.0;
#pragma unroll
                            for (int j = 0; j < 2; ++j)
#pragma unroll
                                for (int i = 0; i < 2; ++i) {
                                    const double v = (double)nv[j][i];
                                    sm += v;
                                    sq = fma(v, v, sq);
                                }
                            sm = warp_sum(sm);
                            sq = warp_sum(sq);
                            if ((tid & 31) == 0)
                                p.out_partials[(size_t)(smp0 + s) * p.nparts + (size_t)blk * 4 + (tid >> 5)] =
                                    make_double2(sm, sq);
                        }
                    }
                }
            }
            if (!last) {
                __syncthreads();  // the other tile is complete; this one may be overwritten next
            }
        }
    }
}

// ------------------------------------------------------------------ launcher
bool fast8_applicable(const FastFwdParams &p, int block, int normalize)
{
    if (block != 8 || normalize || p.inner < 1) return false;
    if ((long long)p.M * p.N * p.K >= (1LL << 31)) return false;
    // the per-cell descriptor holds offsets relative to the tile origin in 20 bits
    if ((9LL * p.N + 9) * p.K + 9 >= fast8::kMaxRel) return false;
    auto al = [](const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
    return al(p.w, 8) && al(p.b, 8) && al(p.s, 8) && al(p.x, 4) && al(p.y, 8);
}

int fast8_default_spc(int B, long long nbricks)
{
    // enough CTAs for several waves of 3 CTAs per SM, but at least 8 samples per
    // CTA (when the batch allows) so that the weight fetch is amortised
    const int chunks = pick_batch_chunks(nbricks, B, 3 * 4, 8);
    return (B + chunks - 1) / chunks;
}

int launch_step_fwd_fast8(FastFwdParams p, int act, cudaStream_t st)
{
    if (p.kbn <= 0) {
        p.kb0 = 0;
        p.kbn = p.K / 8;
    }
    const long long nb = (long long)(p.M / 8) * (p.N / 8) * p.kbn;
    if (p.spc <= 0) p.spc = fast8_default_spc(p.B, nb);
    dim3 grid((unsigned)nb, (unsigned)((p.B + p.spc - 1) / p.spc));
    const bool fin = p.in_stats != nullptr, sout = p.out_partials != nullptr;
#define LAUNCH_(A)                                                                          \
    do {                                                                                    \
        if (fin && sout) step_fwd_fast8<A, true, true><<<grid, fast8::THREADS, 0, st>>>(p);  \
        else if (fin) step_fwd_fast8<A, true, false><<<grid, fast8::THREADS, 0, st>>>(p);    \
        else if (sout) step_fwd_fast8<A, false, true><<<grid, fast8::THREADS, 0, st>>>(p);   \
        else step_fwd_fast8<A, false, false><<<grid, fast8::THREADS, 0, st>>>(p);            \
    } while (0)
    switch (act) {
    case GN_ACT_RELU: LAUNCH_(GN_ACT_RELU); break;
    case GN_ACT_LEAKY_RELU: LAUNCH_(GN_ACT_LEAKY_RELU); break;
    case GN_ACT_SILU: LAUNCH_(GN_ACT_SILU); break;
    default: LAUNCH_(GN_ACT_TANH); break;
    }
#undef LAUNCH_
    return check_launch("step_fwd_fast8");
}

}  // namespace gn
