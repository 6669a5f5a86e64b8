// "Lanes = samples" forward kernel for the fused model loop (float, block 8, per-block
// normalisation off). It exists because the register-patch kernel in step_fast.cu runs out of
// shared-memory wavefronts: there a shared-memory float feeds 2.25 FMAs. Here
//
//   * the activations of 16 samples are interleaved ("IL16": [group][z][y][x][16 samples]), in
//     HBM between the steps of the fused loop and in shared memory inside the kernel, so a
//     thread works on a PAIR of samples and the 8 pairs of a group sit in 8 neighbouring lanes;
//   * a thread sweeps four z-planes of a 1x4 strip of neurons (fixed y, x = 4*xh .. 4*xh+3) and
//     keeps a 3x3x6 window of sample pairs in registers: each step loads one new plane slice
//     (18 LDS.64) for 4 x 27 x 2 = 216 FMAs, 6 FMAs per shared-memory float;
//   * the block's 512 x 27 weights live in shared memory and reach the lanes as broadcast
//     LDS.128 (4 taps of one neuron per load, used for both samples of the pair).
//
// The 10x10x10 tile of a group (block + stale halo) arrives by TMA: in the IL16 layout the
// tile's x origin is (8*bx - 1) * 64 bytes, which satisfies TMA's 16-byte rule that the plain
// [B,M,N,K] layout cannot (origin 8*bx - 1 floats). Rows are fetched 11 cells wide so that the
// row stride is odd and the four strips of a warp spread over all 32 banks. Cells outside the
// grid are zero-filled by the TMA unit. Tiles are double buffered: the next group's tile is in
// flight while the current one iterates. New activations wait in registers until every thread
// has read the old ones (two barriers per inner iteration).
//
// Work is a list of (block, group) items, block-major, cut into one contiguous range per CTA
// (persistent CTAs, one per SM); weights are re-staged only when the range moves to a new block.
//
// Reference semantics: gridnet/backend_torch.py:61-142 (step), gridnet/scripts/train_mnist.py:62-64
// (LayerNorm between steps: applied here to the tile right after it lands, FUSE_IN).
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace gn {

namespace lanes {
constexpr int THREADS = 256;
constexpr int ROWC = 11;                       // cells per tile row as fetched (10 used)
constexpr int CELLF = 16;                      // floats per cell (16 samples)
constexpr int ROWF = ROWC * CELLF;             // 176 floats
constexpr int PLANEF = 10 * ROWF;              // 1760
constexpr int TILEF = 10 * PLANEF;             // 17600 floats = 70400 bytes
constexpr int TILE_BYTES = TILEF * 4;
constexpr int WSTRIDE = 28;                    // floats per neuron in shared memory: 27 taps + bias
constexpr int W_FLOATS = 512 * WSTRIDE;
constexpr int GB_CELLS = 10 * 10 * ROWC;       // gamma/beta table entries (pad cell included)
constexpr unsigned kSpinLimit = 1u << 18;      // bounded wait on the TMA barrier

// dynamic shared memory carve-up (bytes)
constexpr int OFF_TILE0 = 0;
constexpr int OFF_TILE1 = OFF_TILE0 + TILE_BYTES;
constexpr int OFF_W = OFF_TILE1 + TILE_BYTES;
constexpr int OFF_SCALE = OFF_W + W_FLOATS * 4;
constexpr int OFF_GB = OFF_SCALE + 512 * 4;
constexpr int OFF_RED = OFF_GB + GB_CELLS * 8;
constexpr int OFF_BAR = OFF_RED + 8 * 16 * 2 * 8;  // 8 warps x 16 samples x (sum, sq) doubles
constexpr int SMEM_BYTES = OFF_BAR + 64;
}  // namespace lanes

struct LanesParams {
    const float *w, *b, *s;        // [27,M,N,K], [M,N,K], [M,N,K]
    const float *gamma, *beta;     // [M,N,K] (FUSE_IN)
    const float2 *in_stats;        // [G*16] (mean, rstd) of the input, or nullptr
    double2 *out_partials;         // [G*16][nblocks] (sum, sum of squares) of the output, or nullptr
    float *y;                      // IL16 output
    int *error_flag;               // set to 1 if a bounded wait gave up
    int M, N, K, G, inner;
    int nblocks, nitems;
};

// ---- the kernel ----------------------------------------------------------------------------
template <int ACT, bool FUSE_IN, bool STATS_OUT>
__global__ void __launch_bounds__(lanes::THREADS, 1)
    step_fwd_lanes16(const __grid_constant__ CUtensorMap in_map, const LanesParams p)
{
    using namespace lanes;
    extern __shared__ __align__(1024) unsigned char smem[];
    float *const tile0 = reinterpret_cast<float *>(smem + OFF_TILE0);
    float *const tile1 = reinterpret_cast<float *>(smem + OFF_TILE1);
    float *const wsm = reinterpret_cast<float *>(smem + OFF_W);
    float *const ssm = reinterpret_cast<float *>(smem + OFF_SCALE);
    float2 *const gbt = reinterpret_cast<float2 *>(smem + OFF_GB);
    double *const red = reinterpret_cast<double *>(smem + OFF_RED);
    const unsigned bar_base = smem_u32(smem + OFF_BAR);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int pr = tid & 7;  // sample pair inside the group
    const int q = tid >> 3;  // strip: 32 per CTA
    const int xh = q & 1, ylo = (q >> 1) & 1, yhi = (q >> 2) & 3, zh = q >> 4;
    const int yy = yhi * 2 + ylo;

    const int it0 = (int)((long long)p.nitems * blockIdx.x / gridDim.x);
    const int it1 = (int)((long long)p.nitems * (blockIdx.x + 1) / gridDim.x);
    if (it0 >= it1) return;

    if (tid == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    __syncthreads();

    const int nbx = p.K >> 3, nby = p.N >> 3;
    const size_t P = (size_t)p.M * p.N * p.K;

    auto issue = [&](int item, int buf) {
        if (tid == 0) {
            const int brick = item / p.G, g = item - brick * p.G;
            const int bx = brick % nbx, by = (brick / nbx) % nby, bz = brick / nbx / nby;
            fence_proxy_async();  // earlier generic-proxy writes to this buffer precede the bulk write
            const unsigned bar = bar_base + 8 * buf;
            mbar_expect_tx(bar, TILE_BYTES);
            tma_load_4d(smem_u32(buf ? tile1 : tile0), &in_map, bar, (bx * 8 - 1) * CELLF, by * 8 - 1, bz * 8 - 1, g);
        }
    };

    unsigned phase0 = 0, phase1 = 0;
    int cur_brick = -1;
    int bx = 0, by = 0, bz = 0;
    issue(it0, 0);

    for (int item = it0; item < it1; ++item) {
        const int buf = (item - it0) & 1;
        const int brick = item / p.G, g = item - brick * p.G;
        if (brick != cur_brick) {
            // ---- stage this block's parameters (the previous item ended with a barrier)
            cur_brick = brick;
            bx = brick % nbx;
            by = (brick / nbx) % nby;
            bz = brick / nbx / nby;
            for (int idx = tid; idx < 28 * 512; idx += THREADS) {
                const int t = idx >> 9, n = idx & 511;
                const int z = n >> 6, y = (n >> 3) & 7, x = n & 7;
                const size_t gi = ((size_t)(bz * 8 + z) * p.N + (by * 8 + y)) * p.K + (bx * 8 + x);
                // neurons that the four strips of a warp touch together are neighbours in shared memory
                const int pn = (((z * 4 + (y >> 1)) * 4 + (x & 3)) * 4) + ((y & 1) * 2 + (x >> 2));
                if (t < 27) wsm[pn * WSTRIDE + t] = p.w[(size_t)t * P + gi];
                else {
                    wsm[pn * WSTRIDE + 27] = p.b[gi];
                    ssm[pn] = p.s[gi];
                }
            }
            if (FUSE_IN) {
                for (int cidx = tid; cidx < GB_CELLS; cidx += THREADS) {
                    const int cx = cidx % ROWC, cy = (cidx / ROWC) % 10, cz = cidx / (ROWC * 10);
                    const int gz = bz * 8 + cz - 1, gy = by * 8 + cy - 1, gx = bx * 8 + cx - 1;
                    float2 gb = make_float2(0.0f, 0.0f);  // outside the grid: the zero fill stays zero
                    if (cx < 10 && gz >= 0 && gz < p.M && gy >= 0 && gy < p.N && gx >= 0 && gx < p.K) {
                        const size_t gi = ((size_t)gz * p.N + gy) * p.K + gx;
                        gb = make_float2(p.gamma[gi], p.beta[gi]);
                    }
                    gbt[cidx] = gb;
                }
            }
            __syncthreads();
        }
        if (item + 1 < it1) issue(item + 1, buf ^ 1);

        // ---- wait for this item's tile (bounded)
        {
            const unsigned bar = bar_base + 8 * buf;
            const unsigned ph = buf ? phase1 : phase0;
            unsigned spins = 0;
            while (!mbar_try_wait(bar, ph)) {
                if (++spins > kSpinLimit) {
                    if (p.error_flag) *p.error_flag = 1;
                    break;
                }
            }
            if (buf) phase1 ^= 1;
            else phase0 ^= 1;
        }
        float *const T = buf ? tile1 : tile0;

        if (FUSE_IN) {
            // the tile holds the previous step's raw output: normalise it in place
            const float2 m0 = p.in_stats[g * 16 + 2 * pr], m1 = p.in_stats[g * 16 + 2 * pr + 1];
            for (int cidx = q; cidx < GB_CELLS; cidx += 32) {
                const float2 gb = gbt[cidx];
                float2 *ptr = reinterpret_cast<float2 *>(T + cidx * CELLF + 2 * pr);
                float2 v = *ptr;
                v.x = fmaf((v.x - m0.x) * m0.y, gb.x, gb.y);
                v.y = fmaf((v.y - m1.x) * m1.y, gb.x, gb.y);
                *ptr = v;
            }
            __syncthreads();
        }

        // this thread's window origin: planes 4*zh.., rows yy.., cells 4*xh.. (all in padded coordinates)
        float *const wbase = T + ((4 * zh * 10 + yy) * ROWC + 4 * xh) * CELLF + 2 * pr;

        for (int it = 0; it < p.inner; ++it) {
            const bool last = it + 1 == p.inner;
            float2 win[3][3][6];
            float2 out[4][4];
            auto load_plane = [&](int prel, int slot) {
#pragma unroll
                for (int r = 0; r < 3; ++r)
#pragma unroll
                    for (int c = 0; c < 6; ++c)
                        win[slot][r][c] = *reinterpret_cast<const float2 *>(wbase + ((prel * 10 + r) * ROWC + c) * CELLF);
            };
            load_plane(0, 0);
            load_plane(1, 1);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                load_plane(k + 2, (k + 2) % 3);
                const int z = 4 * zh + k;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int pn = (((z * 4 + yhi) * 4 + i) * 4) + (ylo * 2 + xh);
                    const float4 *wp = reinterpret_cast<const float4 *>(wsm + pn * WSTRIDE);
                    float wv[28];
#pragma unroll
                    for (int v4 = 0; v4 < 7; ++v4) {
                        const float4 t4 = wp[v4];
                        wv[4 * v4] = t4.x;
                        wv[4 * v4 + 1] = t4.y;
                        wv[4 * v4 + 2] = t4.z;
                        wv[4 * v4 + 3] = t4.w;
                    }
                    float ax = wv[27], ay = wv[27];  // bias
#pragma unroll
                    for (int a = 0; a < 3; ++a)
#pragma unroll
                        for (int b = 0; b < 3; ++b)
#pragma unroll
                            for (int c = 0; c < 3; ++c) {
                                const float wt = wv[a * 9 + b * 3 + c];
                                const float2 v = win[(k + a) % 3][b][i + c];
                                ax = fmaf(wt, v.x, ax);
                                ay = fmaf(wt, v.y, ay);
                            }
                    const float2 old = win[(k + 1) % 3][1][i + 1];
                    const float sc = ssm[pn];
                    out[k][i] = make_float2(fmaf(Act<ACT, float>::fwd(ax), sc, old.x),
                                            fmaf(Act<ACT, float>::fwd(ay), sc, old.y));
                }
            }
            if (!last) {
                __syncthreads();  // every thread has read the old activations
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<float2 *>(wbase + (((k + 1) * 10 + 1) * ROWC + i + 1) * CELLF) = out[k][i];
                __syncthreads();
            } else {
                float *yb = p.y + ((((size_t)g * p.M + (bz * 8 + 4 * zh)) * p.N + (by * 8 + yy)) * p.K + (bx * 8 + 4 * xh)) * CELLF + 2 * pr;
                double s0 = 0.0, q0 = 0.0, s1 = 0.0, q1 = 0.0;
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        *reinterpret_cast<float2 *>(yb + ((size_t)k * p.N * p.K + i) * CELLF) = out[k][i];
                        if (STATS_OUT) {
                            const double vx = (double)out[k][i].x, vy = (double)out[k][i].y;
                            s0 += vx;
                            q0 = fma(vx, vx, q0);
                            s1 += vy;
                            q1 = fma(vy, vy, q1);
                        }
                    }
                if (STATS_OUT) {
                    // lanes of one warp that share a pair differ in bits 3 and 4
#pragma unroll
                    for (int o = 8; o <= 16; o <<= 1) {
                        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                        q0 += __shfl_xor_sync(0xffffffffu, q0, o);
                        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                        q1 += __shfl_xor_sync(0xffffffffu, q1, o);
                    }
                    if ((tid & 31) < 8) {
                        double *r = red + (warp * 16 + 2 * pr) * 2;
                        r[0] = s0;
                        r[1] = q0;
                        r[2] = s1;
                        r[3] = q1;
                    }
                    __syncthreads();
                    if (tid < 16) {
                        double s = 0.0, qq = 0.0;
#pragma unroll
                        for (int wi = 0; wi < 8; ++wi) {
                            s += red[(wi * 16 + tid) * 2];
                            qq += red[(wi * 16 + tid) * 2 + 1];
                        }
                        p.out_partials[(size_t)(g * 16 + tid) * p.nblocks + brick] = make_double2(s, qq);
                    }
                }
            }
        }
        fence_proxy_async();
        __syncthreads();  // the tile, the weights and the reduction scratch are free again
    }
}


// ---- layout conversion at the two ends of the fused loop --------------------------------------
// [B, P] -> IL16 [G][P][16]; samples beyond B are written as zeros. grid (P / 32, G), 256 threads.
__global__ void __launch_bounds__(256) to_il16_k(const float *__restrict__ x, float *__restrict__ il, int B, size_t P)
{
    __shared__ float t[16][33];
    const int g = blockIdx.y;
    const size_t p0 = (size_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int sidx = ty + 8 * h, b = g * 16 + sidx;
        t[sidx][tx] = b < B ? x[(size_t)b * P + p0 + tx] : 0.0f;
    }
    __syncthreads();
    float *o = il + ((size_t)g * P + p0) * 16;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int idx = threadIdx.x + 256 * h;
        o[idx] = t[idx & 15][idx >> 4];
    }
}

// IL16 raw step output -> y [B, P] = (v - mean) * rstd * gamma + beta. grid (P / 32, G), 256 threads.
__global__ void __launch_bounds__(256) norm_apply_from_il16_k(const float *__restrict__ il,
                                                              const float2 *__restrict__ stats,
                                                              const float *__restrict__ gamma,
                                                              const float *__restrict__ beta, float *__restrict__ y,
                                                              int B, size_t P)
{
    __shared__ float t[16][33];
    const int g = blockIdx.y;
    const size_t p0 = (size_t)blockIdx.x * 32;
    const float *in = il + ((size_t)g * P + p0) * 16;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int idx = threadIdx.x + 256 * h;
        t[idx & 15][idx >> 4] = in[idx];
    }
    __syncthreads();
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const float gm = gamma[p0 + tx], bt = beta[p0 + tx];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int sidx = ty + 8 * h, b = g * 16 + sidx;
        if (b < B) {
            const float2 mr = stats[b];
            y[(size_t)b * P + p0 + tx] = fmaf((t[sidx][tx] - mr.x) * mr.y, gm, bt);
        }
    }
}

// ---- host side --------------------------------------------------------------------------------
EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

bool lanes16_applicable(int M, int N, int K, int block, int inner, const void *w, const void *b, const void *s)
{
    if (block != 8 || inner < 1) return false;
    if ((long long)M * N * K >= (1LL << 31) / 16) return false;  // IL16 element offsets inside one group stay below 2^31
    if ((long long)K * 16 >= (1LL << 32)) return false;
    auto al = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 3) == 0; };
    if (!al(w) || !al(b) || !al(s)) return false;
    return encode_tiled_fn() != nullptr;
}

// Tensor map over an IL16 buffer: dims (fastest first) {K*16, N, M, G}, box {11 cells, 10, 10, 1}.
static int make_il16_map(CUtensorMap *map, const float *il, int M, int N, int K, int G)
{
    const cuuint64_t dims[4] = {(cuuint64_t)K * 16, (cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)G};
    const cuuint64_t strides[3] = {(cuuint64_t)K * 64, (cuuint64_t)N * K * 64, (cuuint64_t)M * N * K * 64};
    const cuuint32_t box[4] = {lanes::ROWF, 10, 10, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(il), dims, strides,
                                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
        return GN_ERR_CUDA;
    }
    return GN_OK;
}

int launch_to_il16(const float *x, float *il, int B, int G, long long P, cudaStream_t st)
{
    dim3 grid((unsigned)(P / 32), (unsigned)G);
    to_il16_k<<<grid, 256, 0, st>>>(x, il, B, (size_t)P);
    return check_launch("to_il16");
}

int launch_norm_apply_from_il16(const float *il, const float2 *stats, const float *gamma, const float *beta, float *y,
                                int B, int G, long long P, cudaStream_t st)
{
    dim3 grid((unsigned)(P / 32), (unsigned)G);
    norm_apply_from_il16_k<<<grid, 256, 0, st>>>(il, stats, gamma, beta, y, B, (size_t)P);
    return check_launch("norm_apply_from_il16");
}

int launch_step_fwd_lanes16(const LanesStep &a, int act, cudaStream_t st)
{
    CUtensorMap map;
    int rc = make_il16_map(&map, a.in_il16, a.M, a.N, a.K, a.G);
    if (rc != GN_OK) return rc;
    LanesParams p{};
    p.w = a.w; p.b = a.b; p.s = a.s; p.gamma = a.gamma; p.beta = a.beta;
    p.in_stats = a.in_stats; p.out_partials = a.out_partials; p.y = a.out_il16; p.error_flag = a.error_flag;
    p.M = a.M; p.N = a.N; p.K = a.K; p.G = a.G; p.inner = a.inner;
    p.nblocks = (a.M / 8) * (a.N / 8) * (a.K / 8);
    p.nitems = p.nblocks * a.G;
    int dev = 0, sms = kNumSMs;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = p.nitems < sms ? p.nitems : sms;
    const bool fin = a.in_stats != nullptr, sout = a.out_partials != nullptr;
#define ONE_(A, FI, SO)                                                                                    \
    do {                                                                                                   \
        auto kern = step_fwd_lanes16<A, FI, SO>;                                                           \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lanes::SMEM_BYTES); \
        if (e != cudaSuccess) {                                                                            \
            record_cuda_error(e, "cudaFuncSetAttribute(step_fwd_lanes16)");                               \
            return GN_ERR_CUDA;                                                                            \
        }                                                                                                  \
        kern<<<grid, lanes::THREADS, lanes::SMEM_BYTES, st>>>(map, p);                                     \
    } while (0)
#define LAUNCH_(A)                          \
    do {                                    \
        if (fin && sout) ONE_(A, true, true);   \
        else if (fin) ONE_(A, true, false);     \
        else if (sout) ONE_(A, false, true);    \
        else ONE_(A, false, false);             \
    } while (0)
    switch (act) {
    case GN_ACT_RELU: LAUNCH_(GN_ACT_RELU); break;
    case GN_ACT_LEAKY_RELU: LAUNCH_(GN_ACT_LEAKY_RELU); break;
    case GN_ACT_SILU: LAUNCH_(GN_ACT_SILU); break;
    default: LAUNCH_(GN_ACT_TANH); break;
    }
#undef LAUNCH_
#undef ONE_
    return check_launch("step_fwd_lanes16");
}

}  // namespace gn
