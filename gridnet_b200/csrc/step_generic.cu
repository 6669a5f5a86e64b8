// General kernels for the block-local grid update: every activation, per-block
// normalisation on or off, block 4 or 8, float or double, plain and gated,
// forward and backward. One CTA owns one bs^3 block of the grid and walks over a
// range of samples; one thread owns one neuron and keeps that neuron's 27 (or 54)
// weights in registers for the CTA's whole life, so weights are read from HBM
// once per CTA instead of once per sample.
//
// Semantics follow gridnet/backend_torch.py:61-142 (plain) and :241-265 (gated);
// the launch surface they replace is src/gridnet_cuda_kernels.cu:736-930.
//
// The tuned float path for normalize = 0 lives in step_fast.cu; this file is the
// reference-complete fallback and the double-precision implementation.
#include "common.cuh"

namespace gn {

// Tile geometry. The tile is stored with padded strides so that a warp's 32 window reads fall
// into 32 different banks: block 8 -> rows of 10, planes of 104 (= 8 mod 32) with a warp spanning
// 8 x-positions x 4 z-planes; block 4 -> rows of 8, planes of 68 (= 4 mod 32) with a warp spanning
// 4 x-positions x 4 rows x 2 planes.
template <int BS>
struct Geo {
    static constexpr int E = BS + 2;
    static constexpr int T = E * E * E;          // logical cells
    static constexpr int NT = BS * BS * BS;
    static constexpr int RS = BS == 8 ? 10 : 8;  // row stride
    static constexpr int PS = BS == 8 ? 104 : 68;  // plane stride
    static constexpr int TP = E * PS;            // padded tile size
    // logical cell number (z-major) -> offset in the padded tile
    static __device__ __forceinline__ int pad(int i) { return (i / (E * E)) * PS + ((i / E) % E) * RS + i % E; }
};

struct BlockPos {
    int bx, by, bz;
    int tx, ty, tz;
    size_t g;  // offset of this thread's neuron inside one [M,N,K] grid
    int own;   // this thread's cell inside the padded tile
};

template <int BS>
__device__ __forceinline__ BlockPos block_pos(int N, int K)
{
    BlockPos p;
    const int tid = threadIdx.x;
    if (BS == 8) {  // a warp = 8 x-positions x 4 z-planes of one row
        p.tx = tid & 7;
        p.tz = (tid >> 3) & 7;
        p.ty = tid >> 6;
    } else {
        p.tx = tid & 3;
        p.ty = (tid >> 2) & 3;
        p.tz = tid >> 4;
    }
    const int nbx = K / BS, nby = N / BS;
    const unsigned blk = blockIdx.x;
    p.bx = blk % nbx;
    p.by = (blk / nbx) % nby;
    p.bz = blk / nbx / nby;
    p.g = ((size_t)(p.bz * BS + p.tz) * N + (p.by * BS + p.ty)) * K + (p.bx * BS + p.tx);
    p.own = (p.tz + 1) * Geo<BS>::PS + (p.ty + 1) * Geo<BS>::RS + p.tx + 1;
    return p;
}

// Gather the (bs+2)^3 tile of one sample; cells outside the grid read as zero.
template <typename R, int BS>
__device__ __forceinline__ void load_tile(R *tile, const R *xs, const BlockPos &p, int M, int N, int K)
{
    constexpr int E = Geo<BS>::E, T = Geo<BS>::T, NT = Geo<BS>::NT;
    for (int i = threadIdx.x; i < T; i += NT) {
        const int px = i % E, py = (i / E) % E, pz = i / (E * E);
        const int gz = p.bz * BS + pz - 1, gy = p.by * BS + py - 1, gx = p.bx * BS + px - 1;
        R v = R(0);
        if (gz >= 0 && gz < M && gy >= 0 && gy < N && gx >= 0 && gx < K)
            v = xs[((size_t)gz * N + gy) * K + gx];
        tile[Geo<BS>::pad(i)] = v;
    }
}

// mean and 1/(std + eps) over all tile cells, zero padding included
// (gridnet/backend_torch.py:126-129); two passes, like torch's std.
template <typename R, int BS>
__device__ __forceinline__ void tile_stats(const R *tile, R *red, R eps, R &mu, R &sd)
{
    constexpr int T = Geo<BS>::T, NT = Geo<BS>::NT;
    R s = R(0);
    for (int i = threadIdx.x; i < T; i += NT) s += tile[Geo<BS>::pad(i)];
    mu = block_sum(s, red) / R(T);
    R q = R(0);
    for (int i = threadIdx.x; i < T; i += NT) {
        const R d = tile[Geo<BS>::pad(i)] - mu;
        q += d * d;
    }
    sd = sqrt_<R>(block_sum(q, red) / R(T));
    (void)eps;
}

// ============================================================== plain forward
template <typename R, int BS, int ACT, bool NORM>
__global__ void __launch_bounds__(BS *BS *BS)
    step_fwd_generic(const R *__restrict__ w, const R *__restrict__ b, const R *__restrict__ s,
                     const R *__restrict__ x, R *__restrict__ y, int B, int M, int N, int K,
                     int inner, R eps, int spc)
{
    constexpr int T = Geo<BS>::T, RS = Geo<BS>::RS, PS = Geo<BS>::PS, TP = Geo<BS>::TP;
    __shared__ R tile[TP];
    __shared__ R red[33];
    const BlockPos p = block_pos<BS>(N, K);
    const size_t P = (size_t)M * N * K;
    R wr[27];
#pragma unroll
    for (int t = 0; t < 27; ++t) wr[t] = w[(size_t)t * P + p.g];
    const R br = b[p.g], sr = s[p.g];
    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    for (int smp = s0; smp < s1; ++smp) {
        __syncthreads();
        load_tile<R, BS>(tile, x + (size_t)smp * P, p, M, N, K);
        __syncthreads();
        for (int it = 0; it < inner; ++it) {
            R mu = R(0), inv = R(1);
            if (NORM) {
                R sd;
                tile_stats<R, BS>(tile, red, eps, mu, sd);
                inv = R(1) / (sd + eps);
            }
            R acc = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        if (NORM) v = (v - mu) * inv;
                        acc = fma(v, wr[a * 9 + bb * 3 + c], acc);
                    }
            const R nv = fma(Act<ACT, R>::fwd(acc + br), sr, tile[p.own]);
            __syncthreads();
            tile[p.own] = nv;
            __syncthreads();
        }
        y[(size_t)smp * P + p.g] = tile[p.own];
    }
}

// ============================================================= plain backward
// Dynamic shared memory: tile[TP] | G[TP] | Gin[TP] | red[40] | stash[inner][NT] (TP = padded tile)
// Recomputes the inner iterations (stashing each neuron's own activation per
// iteration), then walks them in reverse. The 27 contributions of a neuron to the
// gradient tile are scattered with shared-memory atomics, so the float summation
// order (and the last bits of the result) can vary from run to run.
template <typename R, int BS, int ACT, bool NORM>
__global__ void __launch_bounds__(BS *BS *BS)
    step_bwd_generic(const R *__restrict__ w, const R *__restrict__ b, const R *__restrict__ s,
                     const R *__restrict__ x, const R *__restrict__ gy, R *__restrict__ gw,
                     R *__restrict__ gb, R *__restrict__ gs, R *__restrict__ gx, int B, int M,
                     int N, int K, int inner, R eps, int spc, int atomic_params)
{
    constexpr int E = Geo<BS>::E, T = Geo<BS>::T, NT = Geo<BS>::NT, RS = Geo<BS>::RS, PS = Geo<BS>::PS, TP = Geo<BS>::TP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    R *tile = reinterpret_cast<R *>(smem_raw);
    R *G = tile + TP;
    R *Gin = G + TP;
    R *red = Gin + TP;
    R *stash = red + 40;
    const BlockPos p = block_pos<BS>(N, K);
    const size_t P = (size_t)M * N * K;
    const int tid = threadIdx.x;
    R wr[27], dw[27];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        wr[t] = w[(size_t)t * P + p.g];
        dw[t] = R(0);
    }
    const R br = b[p.g], sr = s[p.g];
    R db = R(0), ds = R(0);
    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    for (int smp = s0; smp < s1; ++smp) {
        __syncthreads();
        load_tile<R, BS>(tile, x + (size_t)smp * P, p, M, N, K);
        for (int i = tid; i < T; i += NT) {
            G[Geo<BS>::pad(i)] = R(0);
            Gin[Geo<BS>::pad(i)] = R(0);
        }
        __syncthreads();
        // forward replay
        for (int it = 0; it < inner; ++it) {
            stash[it * NT + tid] = tile[p.own];
            R mu = R(0), inv = R(1);
            if (NORM) {
                R sd;
                tile_stats<R, BS>(tile, red, eps, mu, sd);
                inv = R(1) / (sd + eps);
            }
            R acc = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        if (NORM) v = (v - mu) * inv;
                        acc = fma(v, wr[a * 9 + bb * 3 + c], acc);
                    }
            const R nv = fma(Act<ACT, R>::fwd(acc + br), sr, tile[p.own]);
            __syncthreads();
            tile[p.own] = nv;
            __syncthreads();
        }
        G[p.own] = gy[(size_t)smp * P + p.g];
        // reverse sweep
        for (int it = inner - 1; it >= 0; --it) {
            tile[p.own] = stash[it * NT + tid];
            const R go = G[p.own];  // dL/d(output of this iteration) for this neuron
            __syncthreads();
            R mu = R(0), inv = R(1), sd = R(1);
            if (NORM) {
                tile_stats<R, BS>(tile, red, eps, mu, sd);
                inv = R(1) / (sd + eps);
            }
            R xv[27];
            R acc = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        if (NORM) v = (v - mu) * inv;
                        xv[a * 9 + bb * 3 + c] = v;
                        acc = fma(v, wr[a * 9 + bb * 3 + c], acc);
                    }
            R f, d;
            Act<ACT, R>::both(acc + br, f, d);
            ds = fma(f, go, ds);
            const R dl = d * go * sr;
            db += dl;
            R *dst = NORM ? Gin : G;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + bb * 3 + c;
                        dw[t] = fma(xv[t], dl, dw[t]);
                        atomicAdd(&dst[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c], wr[t] * dl);
                    }
            __syncthreads();
            if (NORM) {
                // inputs were (cur - mu) * inv with inv = 1/(sd + eps): chain rule through mu, sd
                R sg = R(0), sgc = R(0);
                for (int i = tid; i < T; i += NT) {
                    const int pi = Geo<BS>::pad(i);
                    sg += Gin[pi];
                    sgc += Gin[pi] * (tile[pi] - mu);
                }
                sg = block_sum(sg, red);
                sgc = block_sum(sgc, red);
                const R dsd = -sgc * inv * inv;
                for (int i = tid; i < T; i += NT) {
                    const int pi = Geo<BS>::pad(i);
                    R v = Gin[pi] * inv - sg * inv / R(T);
                    v += dsd * (tile[pi] - mu) / (R(T) * sd);
                    G[pi] += v;
                    Gin[pi] = R(0);
                }
                __syncthreads();
            }
        }
        __syncthreads();
        // the tile gradient lands on the input grid; halo cells belong to neighbour blocks
        R *gxs = gx + (size_t)smp * P;
        for (int i = tid; i < T; i += NT) {
            const int px = i % E, py = (i / E) % E, pz = i / (E * E);
            const int gz = p.bz * BS + pz - 1, gyy = p.by * BS + py - 1, gxx = p.bx * BS + px - 1;
            if (gz >= 0 && gz < M && gyy >= 0 && gyy < N && gxx >= 0 && gxx < K)
                atomicAdd(&gxs[((size_t)gz * N + gyy) * K + gxx], G[Geo<BS>::pad(i)]);
        }
    }
    if (atomic_params) {
#pragma unroll
        for (int t = 0; t < 27; ++t) atomicAdd(&gw[(size_t)t * P + p.g], dw[t]);
        atomicAdd(&gb[p.g], db);
        atomicAdd(&gs[p.g], ds);
    } else {
#pragma unroll
        for (int t = 0; t < 27; ++t) gw[(size_t)t * P + p.g] = dw[t];
        gb[p.g] = db;
        gs[p.g] = ds;
    }
}

// ================================================= plain backward, normalize off
// Dynamic shared memory: tile[TP] | D[TP] | wsm[27][NT] | stash[inner][NT]
// Same replay-and-reverse structure, but without shared-memory atomics: the gradient that flows
// back to a block cell is GATHERED by the thread that owns the cell, from the per-iteration delta
// tile D and a shared-memory copy of the block's weights (cell c receives w[n][t] * delta[n] from
// every neuron n with c = n + offset(t)). The running gradient of an owned cell is a register.
// Halo cells never feed back into the block, so their gradient is built once per sample from the
// per-neuron sum of deltas. Everything inside the CTA is deterministic; only the final
// accumulation into grad_x, where tiles of neighbouring blocks overlap, uses global atomics.
template <typename R, int BS, int ACT>
__global__ void __launch_bounds__(BS *BS *BS)
    step_bwd_gather(const R *__restrict__ w, const R *__restrict__ b, const R *__restrict__ s,
                    const R *__restrict__ x, const R *__restrict__ gy, R *__restrict__ gw, R *__restrict__ gb,
                    R *__restrict__ gs, R *__restrict__ gx, int B, int M, int N, int K, int inner, int spc,
                    int atomic_params)
{
    constexpr int E = Geo<BS>::E, T = Geo<BS>::T, NT = Geo<BS>::NT, RS = Geo<BS>::RS, PS = Geo<BS>::PS, TP = Geo<BS>::TP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    R *tile = reinterpret_cast<R *>(smem_raw);
    R *D = tile + TP;
    R *wsm = D + TP;
    R *stash = wsm + 27 * NT;
    const BlockPos p = block_pos<BS>(N, K);
    const size_t P = (size_t)M * N * K;
    const int tid = threadIdx.x;
    // thread-index distance to the neighbour one step along x, y, z (see block_pos)
    constexpr int DX = 1, DY = BS == 8 ? 64 : 4, DZ = BS == 8 ? 8 : 16;
    R wr[27], dw[27];
    unsigned inside = 0;  // bit t: the neighbour at offset(t) is a neuron of this block
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        wr[t] = w[(size_t)t * P + p.g];
        wsm[t * NT + tid] = wr[t];
        dw[t] = R(0);
        const int a = t / 9, bb = (t / 3) % 3, c = t % 3;
        const bool in = (unsigned)(p.tz + a - 1) < (unsigned)BS && (unsigned)(p.ty + bb - 1) < (unsigned)BS &&
                        (unsigned)(p.tx + c - 1) < (unsigned)BS;
        inside |= (in ? 1u : 0u) << t;
    }
    const R br = b[p.g], sr = s[p.g];
    R db = R(0), ds = R(0);
    for (int i = tid; i < T; i += NT) D[Geo<BS>::pad(i)] = R(0);  // the halo of D stays zero
    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    for (int smp = s0; smp < s1; ++smp) {
        __syncthreads();
        load_tile<R, BS>(tile, x + (size_t)smp * P, p, M, N, K);
        __syncthreads();
        for (int it = 0; it < inner; ++it) {  // forward replay
            stash[it * NT + tid] = tile[p.own];
            R acc = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                        acc = fma(tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c], wr[a * 9 + bb * 3 + c], acc);
            const R nv = fma(Act<ACT, R>::fwd(acc + br), sr, tile[p.own]);
            __syncthreads();
            tile[p.own] = nv;
            __syncthreads();
        }
        R g = gy[(size_t)smp * P + p.g];  // gradient w.r.t. this neuron's current activation
        R dsum = R(0);                    // sum of this neuron's deltas over the iterations
        for (int it = inner - 1; it >= 0; --it) {
            tile[p.own] = stash[it * NT + tid];
            __syncthreads();
            R xv[27];
            R acc = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + bb * 3 + c;
                        xv[t] = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        acc = fma(xv[t], wr[t], acc);
                    }
            R f, d;
            Act<ACT, R>::both(acc + br, f, d);
            ds = fma(f, g, ds);
            const R dl = d * g * sr;
            db += dl;
            dsum += dl;
#pragma unroll
            for (int t = 0; t < 27; ++t) dw[t] = fma(xv[t], dl, dw[t]);
            D[p.own] = dl;
            __syncthreads();
            // gather: the neighbour at offset o = offset(t) reaches this cell through its tap 26 - t
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + bb * 3 + c;
                        if (inside & (1u << t)) {
                            const int nb_tid = tid + (c - 1) * DX + (bb - 1) * DY + (a - 1) * DZ;
                            g = fma(wsm[(26 - t) * NT + nb_tid], D[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c], g);
                        }
                    }
            __syncthreads();  // D and the tile may be overwritten by the next iteration
        }
        // ---- gradient of the input tile: owned cells from registers, halo cells from the delta sums
        R *gxs = gx + (size_t)smp * P;
        atomicAdd(&gxs[p.g], g);
        D[p.own] = dsum;
        __syncthreads();
        for (int i = tid; i < T; i += NT) {
            const int px = i % E, py = (i / E) % E, pz = i / (E * E);
            const bool halo = px == 0 || px == E - 1 || py == 0 || py == E - 1 || pz == 0 || pz == E - 1;
            const int gz = p.bz * BS + pz - 1, gyy = p.by * BS + py - 1, gxx = p.bx * BS + px - 1;
            if (halo && gz >= 0 && gz < M && gyy >= 0 && gyy < N && gxx >= 0 && gxx < K) {
                R acc = R(0);
                // (fixed 27-trip loop with a validity test: measured faster than clipped loop bounds)
                for (int a = 0; a < 3; ++a)
                    for (int bb = 0; bb < 3; ++bb)
                        for (int c = 0; c < 3; ++c) {
                            // neuron n = cell - offset(t) in padded coordinates; it must be a block neuron
                            const int nz = pz - (a - 1), ny = py - (bb - 1), nx = px - (c - 1);
                            if (nz >= 1 && nz <= BS && ny >= 1 && ny <= BS && nx >= 1 && nx <= BS) {
                                const int ntid = BS == 8 ? (nx - 1) + 8 * (nz - 1) + 64 * (ny - 1)
                                                         : (nx - 1) + 4 * (ny - 1) + 16 * (nz - 1);
                                acc = fma(wsm[(a * 9 + bb * 3 + c) * NT + ntid], D[nz * PS + ny * RS + nx], acc);
                            }
                        }
                atomicAdd(&gxs[((size_t)gz * N + gyy) * K + gxx], acc);
            }
        }
        __syncthreads();
        D[p.own] = R(0);  // (halo of D is still zero)
    }
    if (atomic_params) {
#pragma unroll
        for (int t = 0; t < 27; ++t) atomicAdd(&gw[(size_t)t * P + p.g], dw[t]);
        atomicAdd(&gb[p.g], db);
        atomicAdd(&gs[p.g], ds);
    } else {
#pragma unroll
        for (int t = 0; t < 27; ++t) gw[(size_t)t * P + p.g] = dw[t];
        gb[p.g] = db;
        gs[p.g] = ds;
    }
}

// ============================================================== gated forward
template <typename R, int BS, int ACT>
__global__ void __launch_bounds__(BS *BS *BS)
    gated_fwd_generic(const R *__restrict__ w, const R *__restrict__ b, const R *__restrict__ x,
                      R *__restrict__ y, int B, int M, int N, int K, int inner, int spc)
{
    constexpr int T = Geo<BS>::T, RS = Geo<BS>::RS, PS = Geo<BS>::PS, TP = Geo<BS>::TP;
    __shared__ R tile[TP];
    const BlockPos p = block_pos<BS>(N, K);
    const size_t P = (size_t)M * N * K;
    R wv[27], wg[27];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        wv[t] = w[(size_t)(2 * t) * P + p.g];
        wg[t] = w[(size_t)(2 * t + 1) * P + p.g];
    }
    const R bv = b[p.g], bg = b[P + p.g];
    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    for (int smp = s0; smp < s1; ++smp) {
        __syncthreads();
        load_tile<R, BS>(tile, x + (size_t)smp * P, p, M, N, K);
        __syncthreads();
        for (int it = 0; it < inner; ++it) {
            R av = R(0), ag = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        av = fma(v, wv[a * 9 + bb * 3 + c], av);
                        ag = fma(v, wg[a * 9 + bb * 3 + c], ag);
                    }
            const R gate = sigmoid_(ag + bg);
            const R nv = gate * tile[p.own] + (R(1) - gate) * Act<ACT, R>::fwd(av + bv);
            __syncthreads();
            tile[p.own] = nv;
            __syncthreads();
        }
        y[(size_t)smp * P + p.g] = tile[p.own];
    }
}

// ============================================== gated backward without shared-memory atomics
// Dynamic shared memory: tile[TP] | Dv[TP] | Dg[TP] | wsm[54][NT] | stash[inner][NT]
// The gated counterpart of step_bwd_gather: the gradient flowing back to a block cell is gathered by
// the thread that owns the cell from the two per-iteration delta tiles (value path and gate path)
// and a shared-memory copy of the block's weights; the running gradient of an owned cell is a
// register that is scaled by the gate before the gathered terms are added (the remembered part of
// the state passes its gradient straight through). Halo cells are handled once per sample from the
// per-neuron sums of the two deltas. Deterministic inside the CTA; the final accumulation into
// grad_x uses global atomics where tiles of neighbouring blocks overlap.
template <typename R, int BS, int ACT>
__global__ void __launch_bounds__(BS *BS *BS)
    gated_bwd_gather(const R *__restrict__ w, const R *__restrict__ b, const R *__restrict__ x,
                     const R *__restrict__ gy, R *__restrict__ gw, R *__restrict__ gb, R *__restrict__ gx, int B,
                     int M, int N, int K, int inner, int spc, int atomic_params)
{
    constexpr int E = Geo<BS>::E, T = Geo<BS>::T, NT = Geo<BS>::NT, RS = Geo<BS>::RS, PS = Geo<BS>::PS, TP = Geo<BS>::TP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    R *tile = reinterpret_cast<R *>(smem_raw);
    R *Dv = tile + TP;
    R *Dg = Dv + TP;
    R *wsm = Dg + TP;  // [0..26] value weights, [27..53] gate weights, each [NT]
    R *stash = wsm + 54 * NT;
    const BlockPos p = block_pos<BS>(N, K);
    const size_t P = (size_t)M * N * K;
    const int tid = threadIdx.x;
    constexpr int DX = 1, DY = BS == 8 ? 64 : 4, DZ = BS == 8 ? 8 : 16;  // thread-index distance to the x, y, z neighbour
    R wv[27], wg[27], dwv[27], dwg[27];
    unsigned inside = 0;  // bit t: the neighbour at offset(t) is a neuron of this block
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        wv[t] = w[(size_t)(2 * t) * P + p.g];
        wg[t] = w[(size_t)(2 * t + 1) * P + p.g];
        wsm[t * NT + tid] = wv[t];
        wsm[(27 + t) * NT + tid] = wg[t];
        dwv[t] = R(0);
        dwg[t] = R(0);
        const int a = t / 9, bb = (t / 3) % 3, c = t % 3;
        const bool in = (unsigned)(p.tz + a - 1) < (unsigned)BS && (unsigned)(p.ty + bb - 1) < (unsigned)BS &&
                        (unsigned)(p.tx + c - 1) < (unsigned)BS;
        inside |= (in ? 1u : 0u) << t;
    }
    const R bv = b[p.g], bg = b[P + p.g];
    R dbv = R(0), dbg = R(0);
    for (int i = tid; i < T; i += NT) {  // the halo of both delta tiles stays zero
        Dv[Geo<BS>::pad(i)] = R(0);
        Dg[Geo<BS>::pad(i)] = R(0);
    }
    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    for (int smp = s0; smp < s1; ++smp) {
        __syncthreads();
        load_tile<R, BS>(tile, x + (size_t)smp * P, p, M, N, K);
        __syncthreads();
        for (int it = 0; it < inner; ++it) {  // forward replay
            stash[it * NT + tid] = tile[p.own];
            R av = R(0), ag = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        av = fma(v, wv[a * 9 + bb * 3 + c], av);
                        ag = fma(v, wg[a * 9 + bb * 3 + c], ag);
                    }
            const R gate = sigmoid_(ag + bg);
            const R nv = gate * tile[p.own] + (R(1) - gate) * Act<ACT, R>::fwd(av + bv);
            __syncthreads();
            tile[p.own] = nv;
            __syncthreads();
        }
        R g = gy[(size_t)smp * P + p.g];  // gradient w.r.t. this neuron's current activation
        R dvsum = R(0), dgsum = R(0);     // sums of this neuron's two deltas over the iterations
        for (int it = inner - 1; it >= 0; --it) {
            const R xo = stash[it * NT + tid];
            tile[p.own] = xo;
            __syncthreads();
            R av = R(0), ag = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        av = fma(v, wv[a * 9 + bb * 3 + c], av);
                        ag = fma(v, wg[a * 9 + bb * 3 + c], ag);
                    }
            const R gate = sigmoid_(ag + bg);
            R f, d;
            Act<ACT, R>::both(av + bv, f, d);
            const R dv = g * (R(1) - gate) * d;
            const R dg = g * gate * (R(1) - gate) * (xo - f);
            dbv += dv;
            dbg += dg;
            dvsum += dv;
            dgsum += dg;
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + bb * 3 + c;
                        const R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        dwv[t] = fma(v, dv, dwv[t]);
                        dwg[t] = fma(v, dg, dwg[t]);
                    }
            Dv[p.own] = dv;
            Dg[p.own] = dg;
            g *= gate;  // the remembered part of the state
            __syncthreads();
            // gather: the neighbour at offset o = offset(t) reaches this cell through its tap 26 - t
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + bb * 3 + c;
                        if (inside & (1u << t)) {
                            const int nb_tid = tid + (c - 1) * DX + (bb - 1) * DY + (a - 1) * DZ;
                            const int ci = (p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c;
                            g = fma(wsm[(26 - t) * NT + nb_tid], Dv[ci], g);
                            g = fma(wsm[(27 + 26 - t) * NT + nb_tid], Dg[ci], g);
                        }
                    }
            __syncthreads();  // the delta tiles and the tile may be overwritten by the next iteration
        }
        // ---- gradient of the input tile: owned cells from registers, halo cells from the delta sums
        R *gxs = gx + (size_t)smp * P;
        atomicAdd(&gxs[p.g], g);
        Dv[p.own] = dvsum;
        Dg[p.own] = dgsum;
        __syncthreads();
        for (int i = tid; i < T; i += NT) {
            const int px = i % E, py = (i / E) % E, pz = i / (E * E);
            const bool halo = px == 0 || px == E - 1 || py == 0 || py == E - 1 || pz == 0 || pz == E - 1;
            const int gz = p.bz * BS + pz - 1, gyy = p.by * BS + py - 1, gxx = p.bx * BS + px - 1;
            if (halo && gz >= 0 && gz < M && gyy >= 0 && gyy < N && gxx >= 0 && gxx < K) {
                R acc = R(0);
                for (int a = 0; a < 3; ++a)
                    for (int bb = 0; bb < 3; ++bb)
                        for (int c = 0; c < 3; ++c) {
                            // neuron n = cell - offset(t) in padded coordinates; it must be a block neuron
                            const int nz = pz - (a - 1), ny = py - (bb - 1), nx = px - (c - 1);
                            if (nz >= 1 && nz <= BS && ny >= 1 && ny <= BS && nx >= 1 && nx <= BS) {
                                const int ntid = BS == 8 ? (nx - 1) + 8 * (nz - 1) + 64 * (ny - 1)
                                                         : (nx - 1) + 4 * (ny - 1) + 16 * (nz - 1);
                                const int t = a * 9 + bb * 3 + c, ci = nz * PS + ny * RS + nx;
                                acc = fma(wsm[t * NT + ntid], Dv[ci], acc);
                                acc = fma(wsm[(27 + t) * NT + ntid], Dg[ci], acc);
                            }
                        }
                atomicAdd(&gxs[((size_t)gz * N + gyy) * K + gxx], acc);
            }
        }
        __syncthreads();
        Dv[p.own] = R(0);  // (the halo of the delta tiles is still zero)
        Dg[p.own] = R(0);
    }
    if (atomic_params) {
#pragma unroll
        for (int t = 0; t < 27; ++t) {
            atomicAdd(&gw[(size_t)(2 * t) * P + p.g], dwv[t]);
            atomicAdd(&gw[(size_t)(2 * t + 1) * P + p.g], dwg[t]);
        }
        atomicAdd(&gb[p.g], dbv);
        atomicAdd(&gb[P + p.g], dbg);
    } else {
#pragma unroll
        for (int t = 0; t < 27; ++t) {
            gw[(size_t)(2 * t) * P + p.g] = dwv[t];
            gw[(size_t)(2 * t + 1) * P + p.g] = dwg[t];
        }
        gb[p.g] = dbv;
        gb[P + p.g] = dbg;
    }
}

// ============================================================= gated backward
// Dynamic shared memory: tile[TP] | G[TP] | stash[inner][NT]
template <typename R, int BS, int ACT>
__global__ void __launch_bounds__(BS *BS *BS)
    gated_bwd_generic(const R *__restrict__ w, const R *__restrict__ b, const R *__restrict__ x,
                      const R *__restrict__ gy, R *__restrict__ gw, R *__restrict__ gb,
                      R *__restrict__ gx, int B, int M, int N, int K, int inner, int spc,
                      int atomic_params)
{
    constexpr int E = Geo<BS>::E, T = Geo<BS>::T, NT = Geo<BS>::NT, RS = Geo<BS>::RS, PS = Geo<BS>::PS, TP = Geo<BS>::TP;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    R *tile = reinterpret_cast<R *>(smem_raw);
    R *G = tile + TP;
    R *stash = G + TP;
    const BlockPos p = block_pos<BS>(N, K);
    const size_t P = (size_t)M * N * K;
    const int tid = threadIdx.x;
    R wv[27], wg[27], dwv[27], dwg[27];
#pragma unroll
    for (int t = 0; t < 27; ++t) {
        wv[t] = w[(size_t)(2 * t) * P + p.g];
        wg[t] = w[(size_t)(2 * t + 1) * P + p.g];
        dwv[t] = R(0);
        dwg[t] = R(0);
    }
    const R bv = b[p.g], bg = b[P + p.g];
    R dbv = R(0), dbg = R(0);
    const int s0 = blockIdx.y * spc, s1 = min(B, s0 + spc);
    for (int smp = s0; smp < s1; ++smp) {
        __syncthreads();
        load_tile<R, BS>(tile, x + (size_t)smp * P, p, M, N, K);
        for (int i = tid; i < T; i += NT) G[Geo<BS>::pad(i)] = R(0);
        __syncthreads();
        for (int it = 0; it < inner; ++it) {
            stash[it * NT + tid] = tile[p.own];
            R av = R(0), ag = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        av = fma(v, wv[a * 9 + bb * 3 + c], av);
                        ag = fma(v, wg[a * 9 + bb * 3 + c], ag);
                    }
            const R gate = sigmoid_(ag + bg);
            const R nv = gate * tile[p.own] + (R(1) - gate) * Act<ACT, R>::fwd(av + bv);
            __syncthreads();
            tile[p.own] = nv;
            __syncthreads();
        }
        G[p.own] = gy[(size_t)smp * P + p.g];
        for (int it = inner - 1; it >= 0; --it) {
            const R xo = stash[it * NT + tid];
            tile[p.own] = xo;
            const R go = G[p.own];
            __syncthreads();
            R av = R(0), ag = R(0);
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const R v = tile[(p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c];
                        av = fma(v, wv[a * 9 + bb * 3 + c], av);
                        ag = fma(v, wg[a * 9 + bb * 3 + c], ag);
                    }
            const R gate = sigmoid_(ag + bg);
            R f, d;
            Act<ACT, R>::both(av + bv, f, d);
            const R dv = go * (R(1) - gate) * d;
            const R dg = go * gate * (R(1) - gate) * (xo - f);
            dbv += dv;
            dbg += dg;
            // the interior gradient is rebuilt from the gate path; the halo keeps accumulating
            G[p.own] = gate * go;
            __syncthreads();
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int bb = 0; bb < 3; ++bb)
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int t = a * 9 + bb * 3 + c;
                        const int ci = (p.tz + a) * PS + (p.ty + bb) * RS + p.tx + c;
                        const R v = tile[ci];
                        dwv[t] = fma(v, dv, dwv[t]);
                        dwg[t] = fma(v, dg, dwg[t]);
                        atomicAdd(&G[ci], fma(wv[t], dv, wg[t] * dg));
                    }
            __syncthreads();
        }
        if (inner == 0) __syncthreads();  // no iteration ran: the G cells written above are read by other threads below
        R *gxs = gx + (size_t)smp * P;
        for (int i = tid; i < T; i += NT) {
            const int px = i % E, py = (i / E) % E, pz = i / (E * E);
            const int gz = p.bz * BS + pz - 1, gyy = p.by * BS + py - 1, gxx = p.bx * BS + px - 1;
            if (gz >= 0 && gz < M && gyy >= 0 && gyy < N && gxx >= 0 && gxx < K)
                atomicAdd(&gxs[((size_t)gz * N + gyy) * K + gxx], G[Geo<BS>::pad(i)]);
        }
    }
    if (atomic_params) {
#pragma unroll
        for (int t = 0; t < 27; ++t) {
            atomicAdd(&gw[(size_t)(2 * t) * P + p.g], dwv[t]);
            atomicAdd(&gw[(size_t)(2 * t + 1) * P + p.g], dwg[t]);
        }
        atomicAdd(&gb[p.g], dbv);
        atomicAdd(&gb[P + p.g], dbg);
    } else {
#pragma unroll
        for (int t = 0; t < 27; ++t) {
            gw[(size_t)(2 * t) * P + p.g] = dwv[t];
            gw[(size_t)(2 * t + 1) * P + p.g] = dwg[t];
        }
        gb[p.g] = dbv;
        gb[P + p.g] = dbg;
    }
}

// ================================================================== launchers
static constexpr size_t kMaxDynSmem = 227 * 1024;

template <typename R>
static size_t bwd_smem_bytes(int bs, int inner, bool gated)
{
    const size_t T = (size_t)(bs + 2) * (bs == 8 ? 104 : 68), NT = (size_t)bs * bs * bs;  // padded tile
    const size_t fixed = gated ? 2 * T : 3 * T + 40;
    return (fixed + (size_t)inner * NT) * sizeof(R);
}

int step_backward_max_inner(int block, int elem_size)
{
    if ((block != 4 && block != 8) || (elem_size != 4 && elem_size != 8)) return -1;
    const size_t T = (size_t)(block + 2) * (block == 8 ? 104 : 68), NT = (size_t)block * block * block;
    const size_t fixed = (3 * T + 40) * elem_size;
    return (int)((kMaxDynSmem - fixed) / (NT * elem_size));
}

#define GN_ACT_SWITCH(act, MACRO)                    \
    switch (act) {                                   \
    case GN_ACT_RELU: MACRO(GN_ACT_RELU); break;     \
    case GN_ACT_LEAKY_RELU: MACRO(GN_ACT_LEAKY_RELU); break; \
    case GN_ACT_SILU: MACRO(GN_ACT_SILU); break;     \
    default: MACRO(GN_ACT_TANH); break;              \
    }

template <typename R>
int launch_step_fwd_generic(const R *w, const R *b, const R *s, const R *x, R *y, int B, int M, int N,
                            int K, int inner, int bs, R eps, int normalize, int act, cudaStream_t st)
{
    const long long nb = (long long)(M / bs) * (N / bs) * (K / bs);
    const int chunks = pick_batch_chunks(nb, B, bs == 8 ? 2 : 16);
    const int spc = (B + chunks - 1) / chunks;
    dim3 grid((unsigned)nb, (unsigned)((B + spc - 1) / spc));
#define LAUNCH_(A)                                                                                      \
    do {                                                                                                \
        if (bs == 8) {                                                                                  \
            if (normalize) step_fwd_generic<R, 8, A, true><<<grid, 512, 0, st>>>(w, b, s, x, y, B, M, N, K, inner, eps, spc); \
            else step_fwd_generic<R, 8, A, false><<<grid, 512, 0, st>>>(w, b, s, x, y, B, M, N, K, inner, eps, spc);          \
        } else {                                                                                        \
            if (normalize) step_fwd_generic<R, 4, A, true><<<grid, 64, 0, st>>>(w, b, s, x, y, B, M, N, K, inner, eps, spc);  \
            else step_fwd_generic<R, 4, A, false><<<grid, 64, 0, st>>>(w, b, s, x, y, B, M, N, K, inner, eps, spc);           \
        }                                                                                               \
    } while (0)
    GN_ACT_SWITCH(act, LAUNCH_)
#undef LAUNCH_
    return check_launch("step_fwd_generic");
}

template <typename K_>
static int opt_in_smem(K_ kernel, size_t bytes)
{
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaFuncSetAttribute");
            return GN_ERR_CUDA;
        }
    }
    return GN_OK;
}

template <typename R>
int launch_step_bwd_generic(const R *w, const R *b, const R *s, const R *x, const R *gy, R *gw, R *gb,
                            R *gs, R *gx, int B, int M, int N, int K, int inner, int bs, R eps,
                            int normalize, int act, cudaStream_t st)
{
    const size_t P = (size_t)M * N * K;
    const long long nb = (long long)(M / bs) * (N / bs) * (K / bs);
    // one CTA per block covers the whole batch whenever the grid already fills the GPU: parameter
    // gradients are then plain stores (splitting the batch further was measured slower: the atomics
    // on 27 weight gradients per neuron cost more than the last partial wave)
    const int chunks = pick_batch_chunks(nb, B, bs == 8 ? 1 : 8);
    const int spc = (B + chunks - 1) / chunks;
    dim3 grid((unsigned)nb, (unsigned)((B + spc - 1) / spc));
    const int atomic_params = grid.y > 1;
    const size_t tp = (size_t)(bs + 2) * (bs == 8 ? 104 : 68), nt = (size_t)bs * bs * bs;
    const size_t smem_gather = (2 * tp + 27 * nt + (size_t)inner * nt) * sizeof(R);
    const bool gather = !normalize && smem_gather <= kMaxDynSmem;
    const size_t smem = gather ? smem_gather : bwd_smem_bytes<R>(bs, inner, false);
    if (smem > kMaxDynSmem) return GN_ERR_BAD_INNER;
    cudaError_t e = cudaMemsetAsync(gx, 0, sizeof(R) * B * P, st);
    if (e == cudaSuccess && atomic_params) {
        e = cudaMemsetAsync(gw, 0, sizeof(R) * 27 * P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gb, 0, sizeof(R) * P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gs, 0, sizeof(R) * P, st);
    }
    if (e != cudaSuccess) {
        record_cuda_error(e, "cudaMemsetAsync");
        return GN_ERR_CUDA;
    }
#define ONE_(BSV, A, NRM)                                                                      \
    do {                                                                                       \
        auto kern = step_bwd_generic<R, BSV, A, NRM>;                                          \
        int rc = opt_in_smem(kern, smem);                                                      \
        if (rc != GN_OK) return rc;                                                            \
        kern<<<grid, BSV * BSV * BSV, smem, st>>>(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, \
                                                  inner, eps, spc, atomic_params);             \
    } while (0)
#define GATHER_(BSV, A)                                                                              \
    do {                                                                                             \
        auto kern = step_bwd_gather<R, BSV, A>;                                                      \
        int rc = opt_in_smem(kern, smem);                                                            \
        if (rc != GN_OK) return rc;                                                                  \
        kern<<<grid, BSV * BSV * BSV, smem, st>>>(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, \
                                                  spc, atomic_params);                               \
    } while (0)
#define LAUNCH_(A)                           \
    do {                                     \
        if (bs == 8) {                       \
            if (normalize) ONE_(8, A, true); \
            else if (gather) GATHER_(8, A);  \
            else ONE_(8, A, false);          \
        } else {                             \
            if (normalize) ONE_(4, A, true); \
            else if (gather) GATHER_(4, A);  \
            else ONE_(4, A, false);          \
        }                                    \
    } while (0)
    GN_ACT_SWITCH(act, LAUNCH_)
#undef LAUNCH_
#undef GATHER_
#undef ONE_
    return check_launch("step_bwd");
}

template <typename R>
int launch_gated_fwd_generic(const R *w, const R *b, const R *x, R *y, int B, int M, int N, int K,
                             int inner, int bs, int act, cudaStream_t st)
{
    const long long nb = (long long)(M / bs) * (N / bs) * (K / bs);
    const int chunks = pick_batch_chunks(nb, B, bs == 8 ? 1 : 8);
    const int spc = (B + chunks - 1) / chunks;
    dim3 grid((unsigned)nb, (unsigned)((B + spc - 1) / spc));
#define LAUNCH_(A)                                                                                  \
    do {                                                                                            \
        if (bs == 8) gated_fwd_generic<R, 8, A><<<grid, 512, 0, st>>>(w, b, x, y, B, M, N, K, inner, spc); \
        else gated_fwd_generic<R, 4, A><<<grid, 64, 0, st>>>(w, b, x, y, B, M, N, K, inner, spc);   \
    } while (0)
    GN_ACT_SWITCH(act, LAUNCH_)
#undef LAUNCH_
    return check_launch("gated_fwd_generic");
}

template <typename R>
int launch_gated_bwd_generic(const R *w, const R *b, const R *x, const R *gy, R *gw, R *gb, R *gx, int B,
                             int M, int N, int K, int inner, int bs, int act, cudaStream_t st)
{
    const size_t P = (size_t)M * N * K;
    const long long nb = (long long)(M / bs) * (N / bs) * (K / bs);
    const int chunks = pick_batch_chunks(nb, B, bs == 8 ? 1 : 8);
    const int spc = (B + chunks - 1) / chunks;
    dim3 grid((unsigned)nb, (unsigned)((B + spc - 1) / spc));
    const int atomic_params = grid.y > 1;
    const size_t tp = (size_t)(bs + 2) * (bs == 8 ? 104 : 68), nt = (size_t)bs * bs * bs;
    const size_t smem_gather = (3 * tp + 54 * nt + (size_t)inner * nt) * sizeof(R);
    // block 4 only: at block 8 the 110 KB weight copy leaves one CTA per SM and the kernel spills
    // registers (measured 3.96 ms against 2.27 ms for the atomic kernel on 64^3 x 64 samples, 2 inner;
    // block 4, 8 inner: 4.73 ms against 6.25 ms)
    const bool gather = bs == 4 && smem_gather <= kMaxDynSmem;
    const size_t smem = gather ? smem_gather : bwd_smem_bytes<R>(bs, inner, true);
    if (smem > kMaxDynSmem) return GN_ERR_BAD_INNER;
    cudaError_t e = cudaMemsetAsync(gx, 0, sizeof(R) * B * P, st);
    if (e == cudaSuccess && atomic_params) {
        e = cudaMemsetAsync(gw, 0, sizeof(R) * 54 * P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gb, 0, sizeof(R) * 2 * P, st);
    }
    if (e != cudaSuccess) {
        record_cuda_error(e, "cudaMemsetAsync");
        return GN_ERR_CUDA;
    }
#define ONE_(BSV, A)                                                                          \
    do {                                                                                      \
        auto kern = gated_bwd_generic<R, BSV, A>;                                             \
        int rc = opt_in_smem(kern, smem);                                                     \
        if (rc != GN_OK) return rc;                                                           \
        kern<<<grid, BSV * BSV * BSV, smem, st>>>(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, \
                                                  spc, atomic_params);                        \
    } while (0)
#define GATHER_(BSV, A)                                                                       \
    do {                                                                                      \
        auto kern = gated_bwd_gather<R, BSV, A>;                                              \
        int rc = opt_in_smem(kern, smem);                                                     \
        if (rc != GN_OK) return rc;                                                           \
        kern<<<grid, BSV * BSV * BSV, smem, st>>>(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, \
                                                  spc, atomic_params);                        \
    } while (0)
#define LAUNCH_(A)                          \
    do {                                    \
        if (bs == 8) {                      \
            ONE_(8, A);                     \
        } else {                            \
            if (gather) GATHER_(4, A);      \
            else ONE_(4, A);                \
        }                                   \
    } while (0)
    GN_ACT_SWITCH(act, LAUNCH_)
#undef LAUNCH_
#undef GATHER_
#undef ONE_
    return check_launch("gated_bwd");
}

// explicit instantiations used by api.cu
template int launch_step_fwd_generic<float>(const float *, const float *, const float *, const float *, float *, int, int, int, int, int, int, float, int, int, cudaStream_t);
template int launch_step_fwd_generic<double>(const double *, const double *, const double *, const double *, double *, int, int, int, int, int, int, double, int, int, cudaStream_t);
template int launch_step_bwd_generic<float>(const float *, const float *, const float *, const float *, const float *, float *, float *, float *, float *, int, int, int, int, int, int, float, int, int, cudaStream_t);
template int launch_step_bwd_generic<double>(const double *, const double *, const double *, const double *, const double *, double *, double *, double *, double *, int, int, int, int, int, int, double, int, int, cudaStream_t);
template int launch_gated_fwd_generic<float>(const float *, const float *, const float *, float *, int, int, int, int, int, int, int, cudaStream_t);
template int launch_gated_fwd_generic<double>(const double *, const double *, const double *, double *, int, int, int, int, int, int, int, cudaStream_t);
template int launch_gated_bwd_generic<float>(const float *, const float *, const float *, const float *, float *, float *, float *, int, int, int, int, int, int, int, cudaStream_t);
template int launch_gated_bwd_generic<double>(const double *, const double *, const double *, const double *, double *, double *, double *, int, int, int, int, int, int, int, cudaStream_t);

}  // namespace gn
