// Tuned float backward of the block-local grid update (block 8, per-block normalisation off),
// split into four kernels so that every stencil runs with the register-patch mapping of the
// forward kernel (a thread owns a 1x2x2 patch and keeps 4 x 27 values in registers):
//
//   replay   step_fwd_fast8 (step_fast.cu) in replay mode: runs the inner iterations once and
//            stores every iteration's pre-activation h_t and the activations x_t in between —
//            the inner iterations are recomputed here, never kept from the forward pass;
//   reverse  bwd_reverse8: walks the iterations backwards. delta_t = act'(h_t) * g * scale, and
//            the gradient flowing back inside the block is a 27-tap stencil over the delta tile
//            with TRANSPOSED weights (cell c receives w[n][t] * delta[n] from the neuron
//            n = c + o through its tap pointing back at c), so it is a gather, with no atomics;
//   wgrad    bwd_wgrad8: dW[n][t] += x_t[n + offset(t)] * delta_t[n], accumulated in registers
//            over samples and iterations, plus dB and dS;
//   halo     bwd_halo8: the part of dX that crosses block borders. A halo cell never feeds back
//            into its block, so its gradient only needs the per-neuron SUM of deltas:
//            dX[c] += sum over neurons n of other blocks with c = n + offset(t) of w[n][t] * Dsum[n].
//
// Everything is deterministic (no floating-point atomics) as long as one CTA of wgrad covers a
// block's whole batch; when the batch is split for occupancy, weight gradients are combined
// with atomics.
//
// Reference semantics: the gradient of gridnet/backend_torch.py:61-142 with normalize=False;
// the kernel this stands in for is gridnet_cuda_backward_kernel, src/gridnet_cuda_kernels.cu:202-450.
#include "common.cuh"
#include "kernels.h"

namespace gn {

namespace bwd8 {
constexpr int RS = 12, PS = 120, TS = 1200;  // tile strides, as in step_fast.cu
constexpr int THREADS = 128;
constexpr int SLOTS = 8;
}  // namespace bwd8

// wT[t][c] = w[26 - t][c + offset(t)] when that neighbour is a neuron of c's own block, else 0
__global__ void __launch_bounds__(256) bwd_transpose_weights_k(const float *__restrict__ w, float *__restrict__ wT,
                                                               int M, int N, int K)
{
    const size_t P = (size_t)M * N * K;
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= P) return;
    const int x = (int)(c % K), y = (int)((c / K) % N), z = (int)(c / ((size_t)K * N));
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
        const int nz = z + dz, ny = y + dy, nx = x + dx;
        float v = 0.0f;
        if ((nz >> 3) == (z >> 3) && (ny >> 3) == (y >> 3) && (nx >> 3) == (x >> 3) && nz >= 0 && ny >= 0 && nx >= 0)
            v = w[(size_t)(26 - t) * P + ((size_t)nz * N + ny) * K + nx];
        wT[(size_t)t * P + c] = v;
    }
}

struct BwdParams {
    const float *w, *wT, *s, *x, *gy;
    const float *save_h, *save_x;  // from the replay
    float *delta;                  // [inner][B][P]
    float *dsum;                   // [B][P] sum of deltas over the iterations
    float *dsb;                    // [B][P] per-sample gradient of the residual scale
    float *gw, *gb, *gs, *gx;
    int B, M, N, K, inner, spc;
    int atomic_params;
};

// ---------------------------------------------------------------------------- reverse sweep
template <int ACT>
__global__ void __launch_bounds__(bwd8::THREADS, 3) bwd_reverse8(const BwdParams p)
{
    using namespace bwd8;
    __shared__ __align__(16) float D[2][TS];
    const int tid = threadIdx.x;
    const int xp = tid & 3, yp = (tid >> 2) & 3, z = tid >> 4;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g00 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + 2 * yp)) * K + (bx * 8 + 2 * xp);

    float wt[27][2][2];
#pragma unroll
    for (int t = 0; t < 27; ++t)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 v = *reinterpret_cast<const float2 *>(p.wT + (size_t)t * P + g00 + (size_t)j * K);
            wt[t][j][0] = v.x;
            wt[t][j][1] = v.y;
        }
    float scl[2][2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float2 v = *reinterpret_cast<const float2 *>(p.s + g00 + (size_t)j * K);
        scl[j][0] = v.x;
        scl[j][1] = v.y;
    }
    for (int i = tid; i < 2 * TS; i += THREADS) (&D[0][0])[i] = 0.0f;  // the halo of both tiles stays zero
    __syncthreads();

    const int toff = z * PS + 2 * yp * RS + 2 * xp;
    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    unsigned step = 0;  // picks the delta tile: consecutive iterations (also across samples) alternate
    for (int smp = s0; smp < s1; ++smp) {
        const size_t so = (size_t)smp * P + g00;
        float g[2][2], dsum[2][2], dsacc[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 v = *reinterpret_cast<const float2 *>(p.gy + so + (size_t)j * K);
            g[j][0] = v.x;
            g[j][1] = v.y;
            dsum[j][0] = dsum[j][1] = dsacc[j][0] = dsacc[j][1] = 0.0f;
        }
        float2 hn[2];  // pre-activations of the iteration handled next, fetched one iteration early
#pragma unroll
        for (int j = 0; j < 2; ++j)
            hn[j] = *reinterpret_cast<const float2 *>(p.save_h + ((size_t)(p.inner - 1) * p.B + smp) * P + g00 + (size_t)j * K);
        for (int it = p.inner - 1; it >= 0; --it, ++step) {
            const size_t ho = ((size_t)it * p.B + smp) * P + g00;
            float *Dt = D[step & 1];
            float dl[2][2];
            const float2 hc[2] = {hn[0], hn[1]};
            if (it > 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    hn[j] = *reinterpret_cast<const float2 *>(p.save_h + ho - (size_t)p.B * P + (size_t)j * K);
            }
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
            const float *tl = Dt + toff;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    const float v[4] = {v01.x, v01.y, v23.x, v23.y};
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
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            *reinterpret_cast<float2 *>(p.gx + so + (size_t)j * K) = make_float2(g[j][0], g[j][1]);
            *reinterpret_cast<float2 *>(p.dsum + so + (size_t)j * K) = make_float2(dsum[j][0], dsum[j][1]);
            *reinterpret_cast<float2 *>(p.dsb + so + (size_t)j * K) = make_float2(dsacc[j][0], dsacc[j][1]);
        }
    }
}

// ------------------------------------------------------------------------- weight gradients
template <int DUMMY>
__global__ void __launch_bounds__(bwd8::THREADS, 3) bwd_wgrad8(const BwdParams p)
{
    using namespace bwd8;
    __shared__ __align__(16) float tiles[2][TS];
    const int tid = threadIdx.x;
    const int xp = tid & 3, yp = (tid >> 2) & 3, z = tid >> 4;
    const int nbx = p.K >> 3, nby = p.N >> 3;
    const unsigned blk = blockIdx.x;
    const int bx = blk % nbx, by = (blk / nbx) % nby, bz = blk / nbx / nby;
    const size_t P = (size_t)p.M * p.N * p.K;
    const int K = p.K;
    const size_t g00 = ((size_t)(bz * 8 + z) * p.N + (by * 8 + 2 * yp)) * K + (bx * 8 + 2 * xp);
    const long long origin = ((long long)(bz * 8 - 1) * p.N + (by * 8 - 1)) * K + (bx * 8 - 1);

    // tile cells this thread fetches: bits 0..10 tile offset, bit 11 halo, bits 12.. offset from the origin
    unsigned cinfo[SLOTS];
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        const int i = tid + j * THREADS;
        unsigned ci = 0xffffffffu;
        if (i < 1000) {
            const int cx = i % 10, cy = (i / 10) % 10, cz = i / 100;
            const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gx = bx * 8 + cx - 1;
            const int soff = cz * PS + cy * RS + cx;
            const bool halo = cx == 0 || cx == 9 || cy == 0 || cy == 9 || cz == 0 || cz == 9;
            if (gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < K)
                ci = (unsigned)soff | (halo ? 0x800u : 0u) | ((unsigned)((cz * p.N + cy) * K + cx) << 12);
            else {
                tiles[0][soff] = 0.0f;  // outside the grid: zero for the CTA's whole life
                tiles[1][soff] = 0.0f;
            }
        }
        cinfo[j] = ci;
    }
    float dw[27][2][2];
#pragma unroll
    for (int t = 0; t < 27; ++t)
#pragma unroll
        for (int j = 0; j < 2; ++j) dw[t][j][0] = dw[t][j][1] = 0.0f;
    float db[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, ds[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
    __syncthreads();

    const int toff = z * PS + 2 * yp * RS + 2 * xp;
    const int s0 = blockIdx.y * p.spc, s1 = min(p.B, s0 + p.spc);
    // Per sample the whole input tile is written once: halo cells into both tiles (they never change),
    // interior cells into tile 0 (iteration 0). Iteration t >= 1 only rewrites the block interior of
    // tile t & 1, every thread its own four cells, from the replayed activations. Loads run one
    // sample (tile cells) resp. one iteration (own activations, deltas) ahead of their use.
    float pf[SLOTS];
    auto fetch_tile = [&](int smp) {
        if (smp < s1) {
            const float *xs = p.x + (size_t)smp * P + origin;
#pragma unroll
            for (int j = 0; j < SLOTS; ++j)
                if (cinfo[j] != 0xffffffffu) pf[j] = __ldg(xs + (cinfo[j] >> 12));
        }
    };
    float2 xn[2], dn[2];  // own activations and deltas of the step handled next
    auto fetch_step = [&](int smp, int it) {
        if (smp < s1) {
            const size_t o = ((size_t)it * p.B + smp) * P + g00;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                dn[j] = *reinterpret_cast<const float2 *>(p.delta + o + (size_t)j * K);
                if (it > 0) xn[j] = *reinterpret_cast<const float2 *>(p.save_x + o - (size_t)p.B * P + (size_t)j * K);
            }
        }
    };
    fetch_tile(s0);
    fetch_step(s0, 0);
    for (int smp = s0; smp < s1; ++smp) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 v = *reinterpret_cast<const float2 *>(p.dsb + (size_t)smp * P + g00 + (size_t)j * K);
            ds[j][0] += v.x;
            ds[j][1] += v.y;
        }
        __syncthreads();  // the previous sample's tiles are no longer read
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            const unsigned ci = cinfo[j];
            if (ci != 0xffffffffu) {
                tiles[0][ci & 0x7ff] = pf[j];
                if (ci & 0x800) tiles[1][ci & 0x7ff] = pf[j];
            }
        }
        fetch_tile(smp + 1);
        for (int it = 0; it < p.inner; ++it) {
            float dl[2][2] = {{dn[0].x, dn[0].y}, {dn[1].x, dn[1].y}};
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
                db[j][0] += dl[j][0];
                db[j][1] += dl[j][1];
            }
            __syncthreads();  // tile complete (the other tile may still be read by slower threads)
            const float *tl = tl_w + toff;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float2 v01 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS);
                    const float2 v23 = *reinterpret_cast<const float2 *>(tl + a * PS + r * RS + 2);
                    const float v[4] = {v01.x, v01.y, v23.x, v23.y};
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
    }
    if (p.atomic_params) {
#pragma unroll
        for (int t = 0; t < 27; ++t)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                atomicAdd(p.gw + (size_t)t * P + g00 + (size_t)j * K, dw[t][j][0]);
                atomicAdd(p.gw + (size_t)t * P + g00 + (size_t)j * K + 1, dw[t][j][1]);
            }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            atomicAdd(p.gb + g00 + (size_t)j * K, db[j][0]);
            atomicAdd(p.gb + g00 + (size_t)j * K + 1, db[j][1]);
            atomicAdd(p.gs + g00 + (size_t)j * K, ds[j][0]);
            atomicAdd(p.gs + g00 + (size_t)j * K + 1, ds[j][1]);
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
// One thread per grid cell on a block surface and per batch chunk; a cell is handled by exactly
// one thread per sample, so grad_x needs no atomics. grid (ceil(P / 256), chunks).
__global__ void __launch_bounds__(256) bwd_halo8_k(const float *__restrict__ w, const float *__restrict__ dsum,
                                                   float *__restrict__ gx, int B, int M, int N, int K, int spc)
{
    const size_t P = (size_t)M * N * K;
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= P) return;
    const int x = (int)(c % K), y = (int)((c / K) % N), z = (int)(c / ((size_t)K * N));
    const int lx = x & 7, ly = y & 7, lz = z & 7;
    if (lx > 0 && lx < 7 && ly > 0 && ly < 7 && lz > 0 && lz < 7) return;  // no neighbour in another block
    float wd[27];
    unsigned valid = 0;
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        // neuron n = c - offset(t) reaches c through its tap t
        const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
        const int nz = z - dz, ny = y - dy, nx = x - dx;
        const bool other = ((nz >> 3) != (z >> 3) || (ny >> 3) != (y >> 3) || (nx >> 3) != (x >> 3)) && nz >= 0 &&
                           nz < M && ny >= 0 && ny < N && nx >= 0 && nx < K;
        wd[t] = other ? w[(size_t)t * P + (c - ((long long)dz * N + dy) * K - dx)] : 0.0f;
        valid |= (other ? 1u : 0u) << t;
    }
    const int b0 = blockIdx.y * spc, b1 = min(B, b0 + spc);
    for (int b = b0; b < b1; ++b) {
        const float *ds = dsum + (size_t)b * P + c;
        float acc = 0.0f;
#pragma unroll
        for (int t = 0; t < 27; ++t) {
            const int dz = t / 9 - 1, dy = (t / 3) % 3 - 1, dx = t % 3 - 1;
            if (valid & (1u << t)) acc = fmaf(wd[t], ds[-(((long long)dz * N + dy) * K + dx)], acc);
        }
        gx[(size_t)b * P + c] += acc;
    }
}

// ---------------------------------------------------------------------------------- launcher
size_t bwd_fast8_workspace_floats(int B, int M, int N, int K, int inner)
{
    const size_t P = (size_t)M * N * K, BP = (size_t)B * P;
    return 27 * P + (size_t)inner * BP + (size_t)(inner > 1 ? inner - 1 : 0) * BP + (size_t)inner * BP + 2 * BP;
}

bool bwd_fast8_applicable(const float *w, const float *b, const float *s, const float *x, const float *gy, float *gw,
                          float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner, int block,
                          int normalize)
{
    FastFwdParams f{};
    f.w = w; f.b = b; f.s = s; f.x = x;
    f.B = B; f.M = M; f.N = N; f.K = K; f.inner = inner;
    if (!fast8_applicable(f, block, normalize)) return false;
    auto al8 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 7) == 0; };
    return al8(gy) && al8(gw) && al8(gb) && al8(gs) && al8(gx) && al8(x);
}

int launch_step_bwd_fast8(const float *w, const float *b, const float *s, const float *x, const float *gy, float *gw,
                          float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner, int act,
                          float *ws, cudaStream_t st)
{
    const size_t P = (size_t)M * N * K, BP = (size_t)B * P;
    float *wT = ws;
    float *save_h = wT + 27 * P;
    float *save_x = save_h + (size_t)inner * BP;
    float *delta = save_x + (size_t)(inner > 1 ? inner - 1 : 0) * BP;
    float *dsum = delta + (size_t)inner * BP;
    float *dsb = dsum + BP;

    bwd_transpose_weights_k<<<(unsigned)((P + 255) / 256), 256, 0, st>>>(w, wT, M, N, K);
    int rc = check_launch("bwd_transpose_weights");
    if (rc != GN_OK) return rc;

    FastFwdParams f{};
    f.w = w; f.b = b; f.s = s; f.x = x; f.y = nullptr;
    f.B = B; f.M = M; f.N = N; f.K = K; f.inner = inner;
    f.save_h = save_h;
    f.save_x = save_x;
    rc = launch_step_fwd_fast8(f, act, st);
    if (rc != GN_OK) return rc;

    const long long nb = (long long)(M / 8) * (N / 8) * (K / 8);
    BwdParams p{};
    p.w = w; p.wT = wT; p.s = s; p.x = x; p.gy = gy; p.save_h = save_h; p.save_x = save_x;
    p.delta = delta; p.dsum = dsum; p.dsb = dsb; p.gw = gw; p.gb = gb; p.gs = gs; p.gx = gx;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner;
    {
        const int chunks = pick_batch_chunks(nb, B, 3 * 4, 8);
        p.spc = (B + chunks - 1) / chunks;
        dim3 grid((unsigned)nb, (unsigned)((B + p.spc - 1) / p.spc));
        switch (act) {
        case GN_ACT_RELU: bwd_reverse8<GN_ACT_RELU><<<grid, bwd8::THREADS, 0, st>>>(p); break;
        case GN_ACT_LEAKY_RELU: bwd_reverse8<GN_ACT_LEAKY_RELU><<<grid, bwd8::THREADS, 0, st>>>(p); break;
        case GN_ACT_SILU: bwd_reverse8<GN_ACT_SILU><<<grid, bwd8::THREADS, 0, st>>>(p); break;
        default: bwd_reverse8<GN_ACT_TANH><<<grid, bwd8::THREADS, 0, st>>>(p); break;
        }
        rc = check_launch("bwd_reverse8");
        if (rc != GN_OK) return rc;
    }
    {
        // one CTA per block covers the batch when the grid already fills the GPU (deterministic plain
        // stores); otherwise the batch is split and the parameter gradients are combined with atomics
        const int chunks = nb >= 4LL * kNumSMs * 3 ? 1 : pick_batch_chunks(nb, B, 3 * 2, 8);
        p.spc = (B + chunks - 1) / chunks;
        dim3 grid((unsigned)nb, (unsigned)((B + p.spc - 1) / p.spc));
        p.atomic_params = grid.y > 1;
        if (p.atomic_params) {
            cudaError_t e = cudaMemsetAsync(gw, 0, sizeof(float) * 27 * P, st);
            if (e == cudaSuccess) e = cudaMemsetAsync(gb, 0, sizeof(float) * P, st);
            if (e == cudaSuccess) e = cudaMemsetAsync(gs, 0, sizeof(float) * P, st);
            if (e != cudaSuccess) {
                record_cuda_error(e, "cudaMemsetAsync");
                return GN_ERR_CUDA;
            }
        }
        bwd_wgrad8<0><<<grid, bwd8::THREADS, 0, st>>>(p);
        rc = check_launch("bwd_wgrad8");
        if (rc != GN_OK) return rc;
    }
    {
        const int chunks = B >= 8 ? 8 : 1;
        const int spc = (B + chunks - 1) / chunks;
        dim3 grid((unsigned)((P + 255) / 256), (unsigned)((B + spc - 1) / spc));
        bwd_halo8_k<<<grid, 256, 0, st>>>(w, dsum, gx, B, M, N, K, spc);
    }
    return check_launch("bwd_halo8");
}

}  // namespace gn
