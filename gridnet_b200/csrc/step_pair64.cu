// "Lanes = samples" forward kernel for large batches (float, block 8, per-block normalisation off).
//
// The register-patch kernel of step_fast.cu keeps a neuron's weights in registers and therefore
// reads 48 shared-memory floats for 108 FMAs; it runs out of shared-memory wavefronts at about a
// quarter of the FP32 peak. Here the roles are swapped: a lane owns SAMPLES, and the weights are what
// is fetched from shared memory, once per warp for all the samples of its lanes.
//
//   * Activations are interleaved by groups of 64 samples ("IL64": [group][z][y][x][64 samples]), in
//     HBM between the steps of the fused loop and in shared memory inside the kernel. A cell is 256
//     bytes; 16 lanes x one 128-bit load fetch it for all 64 samples.
//   * A half-warp (16 lanes x 4 samples) works on a 2x2 (z, y) patch of neurons and sweeps along x,
//     one tile column per step. A column is 4x4 cells; it feeds the three x-taps of three
//     neighbouring output columns at once, so the 16 cell loads of a step serve 4 x 27 FMAs per
//     sample. The two half-warps of a warp take the two halves of the x range and sweep towards the
//     middle (columns 0..5 and 9..4), which doubles the number of independent work units.
//   * The weights of a step (36 floats per x-tap: 4 neurons x 9 (z, y) taps) are read as 128-bit
//     loads whose address is uniform per half-warp: two wavefronts per load, amortised over four
//     samples per lane. FMAs are issued as packed fma.rn.f32x2 over sample pairs.
//   * The 64-sample tile of a whole block does not fit one SM (256 KB), so a block is split along z
//     over the two CTAs of a thread-block cluster (6 x 10 x 10 cells x 64 samples = 150 KB each).
//     After every inner iteration the plane next to the cut is handed to the partner through
//     distributed shared memory (plain st.shared::cluster stores into a buffer that alternates with
//     the iteration's parity) followed by a cluster barrier whose wait sits one step later.
//   * New activations go back into the tile in place. A column may be overwritten once every warp
//     has read it; four mbarriers carry that order: a warp arrives after the reads of a step and
//     waits one step later, so nobody stalls as long as the warps stay within a step of each other.
//   * The tile is stored column by column (x outermost), and every column arrives by its own 5-d
//     bulk tensor copy (TMA; zero fill outside the grid). In the last inner iteration of a work
//     item a column is dead as soon as every warp has read it, so the same column of the NEXT item
//     is fetched right then: the tile is re-filled in place underneath the running iteration and
//     no second buffer is needed. The block's pre-packed weights (pair64_pack_k) arrive by one
//     bulk copy. All of these complete on mbarriers with bounded waits.
//
// Fusion with the whole-grid normalisation (gridnet/scripts/train_mnist.py:62-64): FUSE_IN
// normalises the freshly loaded tile in place, STATS_OUT reduces per-sample sum / sum of squares of
// the step's output to one partial per (sample, block half).
//
// Reference semantics: gridnet/backend_torch.py:61-142; the kernel it stands in for is
// gridnet_cuda_forward_kernel, src/gridnet_cuda_kernels.cu:101-200.
#include <string.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace gn {

namespace pair64 {
constexpr int THREADS = 256;
constexpr int NS = 64;                       // samples per group = floats per cell
// tile[x column 0..9][z plane 0..5][y row 0..9][64 samples]: a column is contiguous, so it can be
// fetched (and re-filled for the next work item) by one bulk tensor copy of its own
constexpr int YS = NS, ZS = 10 * NS, XS = 60 * NS;
constexpr int COL_BYTES = XS * 4;            // 15360
constexpr int TILE_F = 10 * XS;              // 38400 floats
constexpr int TILE_BYTES = TILE_F * 4;       // 153600
// alternate buffer of the exchange plane: alt[x column][y row][64 samples]
constexpr int AXS = 10 * NS;
constexpr int PLANE_BYTES = 100 * NS * 4;    // 25600
// packed parameters of half a block: 8 chunks (x half h, output column xo), each 3 x-taps x 8 units x 36
// weights, then 8 units x 4 biases, then 8 units x 4 scales; a chunk is fetched by one bulk copy
constexpr int WCH_W = 864, WCH_F = WCH_W + 64, WCH_BYTES = WCH_F * 4;  // 3712 bytes
constexpr int WPK_F = 8 * WCH_F;             // 7424
constexpr int WPK_BYTES = WPK_F * 4;         // 29696
constexpr int GB_CELLS = 600;
// after the chunks: (gamma, beta) of the 600 tile cells of the block half, zero outside the grid
constexpr int GB_BYTES = GB_CELLS * 8;       // 4800
constexpr int PK_F = WPK_F + 2 * GB_CELLS;   // floats per block half in the packed buffer: 8624
constexpr unsigned kSpinLimit = 1u << 20;    // bounded waits on mbarriers

constexpr int OFF_TILE = 0;
constexpr int OFF_ALT = OFF_TILE + TILE_BYTES;
constexpr int OFF_W = OFF_ALT + PLANE_BYTES;
constexpr int OFF_GB = OFF_W + WPK_BYTES;
constexpr int OFF_RED = OFF_GB + GB_CELLS * 8;
constexpr int OFF_BAR = OFF_RED + 16 * NS * 16;  // 16 contributors x 64 samples x double2
constexpr int SMEM_BYTES = OFF_BAR + 256;
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one SM");
}  // namespace pair64

struct Pair64Params {
    const float *wpk;            // [blocks][2][PK_F] from pair64_pack_k
        const float2 *in_stats;      // [G*64] (mean, rstd) of the input (FUSE_IN)
    double2 *out_partials;       // [G*64][nparts]; this kernel fills slots 0 .. 2*blocks-1 of every row (STATS_OUT)
    int nparts;
    float *y;                    // IL64 output
    int *error_flag;             // set to 1 if a bounded wait gave up
    int M, N, K, G, inner;
    int nblocks, nitems;
};

typedef unsigned long long u64;
struct Quad {
    u64 lo, hi;  // samples (0,1) and (2,3) of the lane
};

__device__ __forceinline__ u64 pack2(float a, float b)
{
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float &a, float &b)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ void ffma2(u64 &acc, u64 a, u64 w)
{
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(w));
}
__device__ __forceinline__ u64 fmul2(u64 a, u64 b)
{
    u64 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 fadd2(u64 a, u64 b)
{
    u64 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 ffma2r(u64 a, u64 b, u64 c)
{
    u64 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// cen + sc * act(h) for a pair of samples. silu is done on the pair: the multiplies and adds are packed, only the
// two MUFU operations per value are scalar. 2^t overflows to +inf for very negative h; the reciprocal is then 0
// and h * 0 = -0, the right limit, so no clamp is needed.
template <int ACT>
__device__ __forceinline__ u64 act_residual2(u64 h, float sc, u64 cen)
{
    const u64 sc2 = pack2(sc, sc);
    if (ACT == GN_ACT_SILU) {
        const u64 t = fmul2(h, pack2(-1.4426950408889634f, -1.4426950408889634f));
        float t0, t1, e0, e1, r0, r1;
        unpack2(t, t0, t1);
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(t0));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(t1));
        const u64 d = fadd2(pack2(e0, e1), pack2(1.0f, 1.0f));
        float d0, d1;
        unpack2(d, d0, d1);
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d0));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d1));
        return ffma2r(fmul2(h, pack2(r0, r1)), sc2, cen);
    }
    float h0, h1;
    unpack2(h, h0, h1);
    return ffma2r(pack2(Act<ACT, float>::fwd(h0), Act<ACT, float>::fwd(h1)), sc2, cen);
}
__device__ __forceinline__ Quad lds_quad(const float *p)
{
    const ulonglong2 t = *reinterpret_cast<const ulonglong2 *>(p);
    Quad q;
    q.lo = t.x;
    q.hi = t.y;
    return q;
}
__device__ __forceinline__ unsigned cluster_rank()
{
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
// Arrival without a fence: enough where the arrival only says "I have finished READING" (the loads have
// returned before the instruction issues); a release arrival would also wait for every global store in flight.
__device__ __forceinline__ void cluster_arrive_relaxed()
{
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned map_to_rank(unsigned local_addr, unsigned rank)
{
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f4(unsigned addr, float4 v)
{
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_5d(unsigned dst, const CUtensorMap *map, unsigned bar, int c0, int c1, int c2, int c3,
                                            int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void bulk_load_1d(unsigned dst, const void *src, unsigned bytes, unsigned bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- the kernel ----------------------------------------------------------------------------
// Barriers in shared memory (8 bytes each, from OFF_BAR): C[0..4] column pair (j, 9-j) of the tile has
// landed; W[0..3] the parameter chunks of output column xo (both x halves) have landed; R1, R2, R3, R5
// every warp has finished step 1 / 2 / 3 / 5 (and every tile write it does before that point); D[0..4] in
// a work item's last iteration every warp has read column pair j for the last time (pairs 0..3 in step j,
// pair 4 = columns 4 and 5 in step 5), so the columns can be re-filled for the next item; E[0..3] likewise
// for the parameter chunks of output column xo, last used in step xo + 2; G the (gamma, beta) table has landed.
template <int ACT, bool FUSE_IN, bool STATS_OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pair64::THREADS, 1)
    step_fwd_pair64(const __grid_constant__ CUtensorMap in_map, const Pair64Params p)
{
    using namespace pair64;
    extern __shared__ __align__(1024) unsigned char smem[];
    float *const tile = reinterpret_cast<float *>(smem + OFF_TILE);
    float *const alt = reinterpret_cast<float *>(smem + OFF_ALT);
    float *const wsm = reinterpret_cast<float *>(smem + OFF_W);
    float2 *const gbt = reinterpret_cast<float2 *>(smem + OFF_GB);
    double2 *const red = reinterpret_cast<double2 *>(smem + OFF_RED);
    const unsigned bar0 = smem_u32(smem + OFF_BAR);
    const unsigned bar_c = bar0, bar_w = bar0 + 40, bar_r = bar0 + 72, bar_d = bar0 + 104, bar_e = bar0 + 144,
                   bar_g = bar0 + 176;

    const int tid = threadIdx.x, lane = tid & 31, u = tid >> 5;
    const int h = lane >> 4, li = lane & 15;  // x half (0: columns 0..5 upwards, 1: columns 9..4 downwards), sample quad
    const int zp = u >> 2, yp = u & 3;
    const unsigned rank = cluster_rank();
    const int cl = blockIdx.x >> 1, ncl = gridDim.x >> 1;
    const int it0 = (int)((long long)p.nitems * cl / ncl);
    const int it1 = (int)((long long)p.nitems * (cl + 1) / ncl);

    if (tid == 0) {
        for (int i = 0; i < 5; ++i) mbar_init(bar_c + 8 * i, 1);
        for (int i = 0; i < 4; ++i) mbar_init(bar_w + 8 * i, 1);
        for (int i = 0; i < 4; ++i) mbar_init(bar_e + 8 * i, 8);
        mbar_init(bar_g, 1);
        for (int i = 0; i < 4; ++i) mbar_init(bar_r + 8 * i, 8);
        for (int i = 0; i < 5; ++i) mbar_init(bar_d + 8 * i, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_proxy_async();
    }
    cluster_arrive_relaxed();  // pairs with the wait before the first item's first exchange

    const int nbx = p.K >> 3, nby = p.N >> 3;
    const int xs = h ? -XS : XS, axs = h ? -AXS : AXS;
    // exchange plane: the tile plane that belongs to the partner CTA (rank 0: plane 5, rank 1: plane 0)
    const int ez = rank ? 0 : 5;
    const int exrow = ez - 2 * zp;                                 // this unit's window row on that plane, if in 0..3
    const bool exporter = rank ? (zp == 0) : (zp == 1);            // this unit owns the plane the partner needs
    const int edz = rank ? 0 : 1;                                  // ... its neurons with this dz
    // the partner's two buffers for my plane (its exchange plane): parity 0 = inside its tile, 1 = its alt plane
    const unsigned partner = rank ^ 1u;
    const int pez = partner ? 0 : 5;
    const unsigned rem_tile = map_to_rank(smem_u32(tile + pez * ZS), partner), rem_alt = map_to_rank(smem_u32(alt), partner);
    const int col0 = h ? 9 : 0;
    const float *const wp = wsm + h * 4 * WCH_F + u * 36;          // + xo * WCH_F + c * 288 + 4 * tap
    const float *const bp = wsm + h * 4 * WCH_F + WCH_W + u * 4;   // + xo * WCH_F: biases; 32 floats further: scales

    unsigned ph_w = 0, ph_g = 0, ph1 = 0, ph2 = 0, ph3 = 0, ph5 = 0;
    bool failed = false;
    auto wait_bar = [&](unsigned bar, unsigned &ph) {
#ifdef GN_PAIR64_NOSYNC  // timing experiment only (racy): skip the waits on the R barriers
        if (bar >= bar_r && bar < bar_d) {
            ph ^= 1;
            return;
        }
#endif
        if (!mbar_wait_bounded(bar, ph, kSpinLimit)) failed = true;
        ph ^= 1;
    };
    auto arrive = [&](unsigned bar) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar);
    };
    // thread 0: fetch column pair j of the tile whose origin cell is (tx0, ty0, tz0) in sample group tg
    struct TileOrigin {
        int x, y, z, g;
    };
    auto tile_origin = [&](int item) {
        const int brick = item / p.G, g = item - brick * p.G;
        TileOrigin o;
        o.x = (brick % nbx) * 8 - 1;
        o.y = ((brick / nbx) % nby) * 8 - 1;
        o.z = (brick / nbx / nby) * 8 + 4 * (int)rank - 1;
        o.g = g;
        return o;
    };
    auto issue_cols = [&](const TileOrigin &o, int j) {
        fence_proxy_async();  // earlier generic-proxy accesses to these columns precede the bulk writes
        mbar_expect_tx(bar_c + 8 * j, 2 * COL_BYTES);
        tma_load_5d(smem_u32(tile + j * XS), &in_map, bar_c + 8 * j, 0, o.x + j, o.y, o.z, o.g);
        tma_load_5d(smem_u32(tile + (9 - j) * XS), &in_map, bar_c + 8 * j, 0, o.x + 9 - j, o.y, o.z, o.g);
    };
    // thread 0: fetch the parameter chunks of output column xo (one per x half) of a block
    auto issue_weights = [&](int brick, int xo) {
        const float *src = p.wpk + ((size_t)brick * 2 + rank) * PK_F;
        fence_proxy_async();
        mbar_expect_tx(bar_w + 8 * xo, 2 * WCH_BYTES);
        bulk_load_1d(smem_u32(wsm + xo * WCH_F), src + xo * WCH_F, WCH_BYTES, bar_w + 8 * xo);
        bulk_load_1d(smem_u32(wsm + (4 + xo) * WCH_F), src + (4 + xo) * WCH_F, WCH_BYTES, bar_w + 8 * xo);
    };

    // thread 0: fetch the (gamma, beta) table of a block half
    auto issue_gb_table = [&](int brick) {
        fence_proxy_async();
        mbar_expect_tx(bar_g, GB_BYTES);
        bulk_load_1d(smem_u32(gbt), p.wpk + ((size_t)brick * 2 + rank) * PK_F + WPK_F, GB_BYTES, bar_g);
    };
    __syncthreads();  // barriers initialised

    if (tid == 0 && it0 < it1) {
        const TileOrigin o = tile_origin(it0);
        for (int j = 0; j < 5; ++j) issue_cols(o, j);
        for (int xo = 0; xo < 4; ++xo) issue_weights(it0 / p.G, xo);
        if (FUSE_IN) issue_gb_table(it0 / p.G);
    }

#ifdef GN_PAIR64_TRACE
    long long *trace = reinterpret_cast<long long *>(p.error_flag);
    int tr = 0;
#define TRACE_() do { if (blockIdx.x == 0 && tid == 0 && tr < 120) trace[tr++] = clock64(); } while (0)
#else
#define TRACE_() do { } while (0)
#endif
    int cur_brick = -1;
    for (int item = it0; item < it1; ++item) {
        TRACE_();
        const int brick = item / p.G, g = item - brick * p.G;
        const int bx = brick % nbx, by = (brick / nbx) % nby, bz = brick / nbx / nby;
        const bool new_brick = brick != cur_brick;
        cur_brick = brick;
        const bool has_next = item + 1 < it1;
        unsigned ph_item = (unsigned)(item - it0) & 1u;  // C and D barriers complete once per item
        const int next_brick = has_next ? (item + 1) / p.G : brick;
        const bool next_is_new_brick = next_brick != brick;
        float na[4], nb[4];  // normalise: v * na + nb, then * gamma + beta
        if (FUSE_IN) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 mr = p.in_stats[g * NS + 4 * li + q];
                na[q] = mr.y;
                nb[q] = -mr.x * mr.y;
            }
        }
        if (FUSE_IN && new_brick) wait_bar(bar_g, ph_g);
        // normalise the columns in place as they land: 16 lanes per cell, 16 cells at a time, four rounds per column
        for (int j = 0; j < 5; ++j) {
            unsigned phc = ph_item;
            wait_bar(bar_c + 8 * j, phc);
            if (FUSE_IN) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int cx = half ? 9 - j : j;
                    float4 *cp = reinterpret_cast<float4 *>(tile + cx * XS + 4 * li) + (tid >> 4) * (NS / 4);
                    const float2 *gp = gbt + cx * 60 + (tid >> 4);
                    const bool tail = (tid >> 4) < 12;  // rows 48 .. 59 of the column
                    float4 v[4];
                    float2 gb[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (k < 3 || tail) {
                            v[k] = cp[k * 16 * (NS / 4)];
                            gb[k] = gp[k * 16];
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (k < 3 || tail) {
                            v[k].x = fmaf(fmaf(v[k].x, na[0], nb[0]), gb[k].x, gb[k].y);
                            v[k].y = fmaf(fmaf(v[k].y, na[1], nb[1]), gb[k].x, gb[k].y);
                            v[k].z = fmaf(fmaf(v[k].z, na[2], nb[2]), gb[k].x, gb[k].y);
                            v[k].w = fmaf(fmaf(v[k].w, na[3], nb[3]), gb[k].x, gb[k].y);
                            cp[k * 16 * (NS / 4)] = v[k];
                        }
                    }
                }
            }
        }
        if (new_brick) {
            for (int xo = 0; xo < 4; ++xo) {
                unsigned phw = ph_w;
                wait_bar(bar_w + 8 * xo, phw);
            }
            ph_w ^= 1;
        }
        TRACE_();
        __syncthreads();
        TRACE_();
        if (FUSE_IN && tid == 0 && next_is_new_brick) issue_gb_table(next_brick);  // the table is not read again in this item
        cluster_wait();  // the partner has finished the previous item: its exchange buffers may be written
        TRACE_();
        // The rim of the exchange plane (stale halo cells) also goes to the plane's alternate buffer, which is first
        // read in iteration 1: the arrive / wait chain of iteration 0 orders these stores before those loads.
        for (int k = tid >> 4; k < 36; k += THREADS / 16) {
            // rim cells in order: row 0 (10), row 9 (10), then columns 0 and 9 of rows 1..8
            const int cy = k < 10 ? 0 : (k < 20 ? 9 : 1 + ((k - 20) >> 1));
            const int cx = k < 20 ? (k < 10 ? k : k - 10) : ((k & 1) ? 9 : 0);
            *reinterpret_cast<float4 *>(alt + cx * AXS + cy * NS + 4 * li) =
                *reinterpret_cast<const float4 *>(tile + cx * XS + ez * ZS + cy * YS + 4 * li);
        }

        // output position of (dz = 0, dy = 0, first column of this half) in the IL64 output
        float *const yb = p.y +
                          ((((size_t)g * p.M + (bz * 8 + 4 * (int)rank + 2 * zp)) * p.N + (by * 8 + 2 * yp)) * p.K +
                           (bx * 8 + (h ? 7 : 0))) * NS + 4 * li;
        const size_t ydz = (size_t)p.N * p.K * NS, ydy = (size_t)p.K * NS;
        const int ysx = h ? -NS : NS;
        float ssum[4] = {0.f, 0.f, 0.f, 0.f}, ssq[4] = {0.f, 0.f, 0.f, 0.f};
        float4 carry[4];  // output column 3 of the previous iteration: written after every warp has finished step 5

        TileOrigin nxt{};
        if (has_next) nxt = tile_origin(item + 1);

        // One inner iteration. LAST: the results go to global memory instead of the tile, and the tile's
        // columns are handed over to the next item's bulk copies as they die.
        auto iteration = [&](auto last_tag, const int t) {
            constexpr bool LAST = decltype(last_tag)::value;
            const int par = t & 1;
            // window rows: planes 2*zp .. 2*zp+3, rows 2*yp .. 2*yp+3 of column col0; the exchange plane alternates
            // between its place in the tile and the alternate buffer
            const float *rowp[4];
            int rxs[4];
#pragma unroll
            for (int rz = 0; rz < 4; ++rz) {
                const bool ex = rz == exrow && par;
                rowp[rz] = (ex ? alt + col0 * AXS : tile + col0 * XS + (2 * zp + rz) * ZS) + (2 * yp) * YS + 4 * li;
                rxs[rz] = ex ? axs : xs;
            }
            float *const wrow = tile + col0 * XS + (2 * zp + 1) * ZS + (2 * yp + 1) * YS + 4 * li;  // own cell (dz 0, dy 0)
            // where the partner reads my plane next iteration: the buffer of the other parity
            const unsigned rem = par ? rem_tile + 4u * (unsigned)(col0 * XS + (2 * yp + 1) * YS + 4 * li)
                                     : rem_alt + 4u * (unsigned)(col0 * AXS + (2 * yp + 1) * YS + 4 * li);
            const int rstep = par ? xs : axs;

            Quad acc[4][4], cen[4][4];
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                if (j == 1 && t > 0) cluster_wait();  // the partner's plane of the previous iteration has landed
                Quad col[4][4];
#pragma unroll
                for (int rz = 0; rz < 4; ++rz)
#pragma unroll
                    for (int ry = 0; ry < 4; ++ry) col[rz][ry] = lds_quad(rowp[rz] + j * rxs[rz] + ry * YS);
                if (LAST) {
                    // this warp is done with column pair j of the item's tile (columns 4 and 5: after step 5)
                    if (j <= 3) arrive(bar_d + 8 * j);
                    if (j == 5) arrive(bar_d + 32);
                    // ... and with the parameters of output column j - 3 (last used in step j - 1)
                    if (j >= 3) arrive(bar_e + 8 * (j - 3));
                    if (tid == 0 && j >= 1 && j <= 4 && has_next) {
                        unsigned phd = ph_item;
                        wait_bar(bar_d + 8 * (j - 1), phd);
                        issue_cols(nxt, j - 1);
                    }
                    if (tid == 0 && j >= 4 && next_is_new_brick) {
                        unsigned phe = ph_item;
                        wait_bar(bar_e + 8 * (j - 4), phe);
                        issue_weights(next_brick, j - 4);
                    }
                }
                if (j >= 1 && j <= 4) {
#pragma unroll
                    for (int jn = 0; jn < 4; ++jn) cen[j - 1][jn] = col[1 + (jn >> 1)][1 + (jn & 1)];
                }
                if (j <= 3) {
                    const float4 b4 = *reinterpret_cast<const float4 *>(bp + j * WCH_F);
                    acc[j][0].lo = acc[j][0].hi = pack2(b4.x, b4.x);
                    acc[j][1].lo = acc[j][1].hi = pack2(b4.y, b4.y);
                    acc[j][2].lo = acc[j][2].hi = pack2(b4.z, b4.z);
                    acc[j][3].lo = acc[j][3].hi = pack2(b4.w, b4.w);
                }
                // taps outermost: the 8 to 24 FMAs of one (z, y) tap go to different accumulators
#pragma unroll
                for (int ab = 0; ab < 9; ++ab) {
                    const int a = ab / 3, b = ab % 3;
#pragma unroll
                    for (int c = 0; c < 3; ++c) {
                        const int xo = j - c;
                        if (xo < 0 || xo > 3) continue;
                        const float4 w4 = *reinterpret_cast<const float4 *>(wp + xo * WCH_F + c * 288 + 4 * ab);
                        const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for (int jn = 0; jn < 4; ++jn) {
                            const Quad v = col[(jn >> 1) + a][(jn & 1) + b];
                            const u64 ww = pack2(wv[jn], wv[jn]);
                            ffma2(acc[xo][jn].lo, v.lo, ww);
                            ffma2(acc[xo][jn].hi, v.hi, ww);
                        }
                    }
                }
                float4 o[4];
                if (j >= 2) {
                    const int xo = j - 2;
                    const float4 s4 = *reinterpret_cast<const float4 *>(bp + 32 + xo * WCH_F);
                    const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                    for (int jn = 0; jn < 4; ++jn) {
                        const u64 lo = act_residual2<ACT>(acc[xo][jn].lo, sv[jn], cen[xo][jn].lo);
                        const u64 hi = act_residual2<ACT>(acc[xo][jn].hi, sv[jn], cen[xo][jn].hi);
                        unpack2(lo, o[jn].x, o[jn].y);
                        unpack2(hi, o[jn].z, o[jn].w);
                    }
                    if (LAST) {
#pragma unroll
                        for (int jn = 0; jn < 4; ++jn) {
                            *reinterpret_cast<float4 *>(yb + (jn >> 1) * ydz + (jn & 1) * ydy + xo * ysx) = o[jn];
                            if (STATS_OUT) {
                                ssum[0] += o[jn].x; ssq[0] = fmaf(o[jn].x, o[jn].x, ssq[0]);
                                ssum[1] += o[jn].y; ssq[1] = fmaf(o[jn].y, o[jn].y, ssq[1]);
                                ssum[2] += o[jn].z; ssq[2] = fmaf(o[jn].z, o[jn].z, ssq[2]);
                                ssum[3] += o[jn].w; ssq[3] = fmaf(o[jn].w, o[jn].w, ssq[3]);
                            }
                        }
                    } else if (exporter) {
#pragma unroll
                        for (int dy = 0; dy < 2; ++dy)
                            st_cluster_f4(rem + 4u * (unsigned)(dy * YS + (xo + 1) * rstep), edz ? o[2 + dy] : o[dy]);
                    }
                }
                // Tile writes. Output column xo overwrites tile column xo+1 (counted from this half's outer end), which
                // this half read one step earlier and the other half never reads - except xo = 3, whose column the other
                // half reads in step 5: that one waits for the next iteration's step 0.
                if (j == 0 && t > 0) {
                    wait_bar(bar_r + 24, ph5);
#pragma unroll
                    for (int jn = 0; jn < 4; ++jn)
                        *reinterpret_cast<float4 *>(wrow + (jn >> 1) * ZS + (jn & 1) * YS + 4 * xs) = carry[jn];
                }
                if (j == 1 && (!LAST || t > 0)) arrive(bar_r);
                if (j == 2 && (!LAST || t > 0)) wait_bar(bar_r, ph1);
                if (!LAST) {
                    if (j == 3) wait_bar(bar_r + 8, ph2);
                    if (j == 4) wait_bar(bar_r + 16, ph3);
                    if (j >= 2 && j <= 4) {
#pragma unroll
                        for (int jn = 0; jn < 4; ++jn)
                            *reinterpret_cast<float4 *>(wrow + (jn >> 1) * ZS + (jn & 1) * YS + (j - 1) * xs) = o[jn];
                    }
                    if (j == 2) arrive(bar_r + 8);
                    if (j == 3) arrive(bar_r + 16);
                    if (j == 5) {
#pragma unroll
                        for (int jn = 0; jn < 4; ++jn) carry[jn] = o[jn];
                        arrive(bar_r + 24);
                        cluster_arrive();  // all exports of this iteration are stored
                    }
                }
            }
        };
        for (int t = 0; t + 1 < p.inner; ++t) {
            iteration(std::false_type{}, t);
            TRACE_();
        }
        iteration(std::true_type{}, p.inner - 1);
        TRACE_();
        if (tid == 0 && has_next) {
            unsigned phd = ph_item;
            wait_bar(bar_d + 32, phd);
            issue_cols(nxt, 4);
        }
        // the parameters of output columns 2 and 3 are last used in steps 4 and 5
        arrive(bar_e + 24);
        if (tid == 0 && next_is_new_brick) {
            for (int xo = 2; xo < 4; ++xo) {
                unsigned phe = ph_item;
                wait_bar(bar_e + 8 * xo, phe);
                issue_weights(next_brick, xo);
            }
        }

        if (STATS_OUT) {
            // 16 contributors per sample: 8 units x 2 halves
#pragma unroll
            for (int q = 0; q < 4; ++q) red[(u * 2 + h) * NS + 4 * li + q] = make_double2((double)ssum[q], (double)ssq[q]);
        }
        cluster_arrive_relaxed();  // this CTA no longer reads its exchange buffers of this item
        TRACE_();
        __syncthreads();  // the partials are in place
        TRACE_();
        if (STATS_OUT && tid < NS) {
            double s = 0.0, q = 0.0;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const double2 v = red[k * NS + tid];
                s += v.x;
                q += v.y;
            }
            p.out_partials[(size_t)(g * NS + tid) * p.nparts + (size_t)brick * 2 + rank] = make_double2(s, q);
        }
    }
    cluster_wait();  // no CTA leaves while its partner may still store into its shared memory
#ifndef GN_PAIR64_TRACE
    if (failed && p.error_flag) *p.error_flag = 1;
#endif
}

// ---- weight packing ---------------------------------------------------------------------------
// One CTA per block: the block's 27 x 512 weights, biases and scales are staged in shared memory with
// coalesced reads and written out in the order the step kernel reads them:
//   [block][rank][chunk (h, xo)][ (c, unit) x 36 floats ((a * 3 + b) * 4 + jn) | bias (unit, jn) | scale (unit, jn) ]
// rank = z half of the block, h = x half, xo = output column counted from the half's outer end,
// c = x tap in sweep order (h = 1 sweeps downwards, so its taps are mirrored), unit = (zp, yp) patch,
// jn = (dz, dy) inside the patch, (a, b) = (z, y) tap. Tap numbering a * 9 + b * 3 + c follows
// gridnet/backend_torch.py:283-298.
__global__ void __launch_bounds__(256) pair64_pack_k(const float *__restrict__ w, const float *__restrict__ b,
                                                     const float *__restrict__ s, const float *__restrict__ gamma,
                                                     const float *__restrict__ beta, float *__restrict__ out, int M, int N,
                                                     int K)
{
    extern __shared__ __align__(16) float stage[];  // [29][512]: 27 taps, bias, scale
    const int nbx = K >> 3, nby = N >> 3;
    const int brick = blockIdx.x;
    const int bx = brick % nbx, by = (brick / nbx) % nby, bz = brick / nbx / nby;
    const size_t P = (size_t)M * N * K;
    const bool vec = ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(s)) & 15) == 0;
    if (vec) {  // K is a multiple of 8, so half a block row is an aligned float4
        for (int idx = threadIdx.x; idx < 29 * 128; idx += 256) {
            const int t = idx >> 7, n = (idx & 127) * 4;
            const int z = n >> 6, y = (n >> 3) & 7, x = n & 7;
            const size_t gi = ((size_t)(bz * 8 + z) * N + (by * 8 + y)) * K + (bx * 8 + x);
            const float *src = t < 27 ? w + (size_t)t * P + gi : (t == 27 ? b + gi : s + gi);
            *reinterpret_cast<float4 *>(stage + t * 512 + n) = *reinterpret_cast<const float4 *>(src);
        }
    } else {
        for (int idx = threadIdx.x; idx < 29 * 512; idx += 256) {
            const int t = idx >> 9, n = idx & 511;
            const int z = n >> 6, y = (n >> 3) & 7, x = n & 7;
            const size_t gi = ((size_t)(bz * 8 + z) * N + (by * 8 + y)) * K + (bx * 8 + x);
            stage[idx] = t < 27 ? w[(size_t)t * P + gi] : (t == 27 ? b[gi] : s[gi]);
        }
    }
    __syncthreads();
    float *o = out + (size_t)brick * 2 * pair64::PK_F;
    // (gamma, beta) of the 6 x 10 x 10 tile cells of each block half, in the tile's order [x][z][y]; cells outside
    // the grid get (0, 0), which keeps the zero fill of the bulk copies at zero through the normalisation
    for (int idx = threadIdx.x; idx < 2 * pair64::GB_CELLS; idx += 256) {
        const int rank = idx / pair64::GB_CELLS, c = idx - rank * pair64::GB_CELLS;
        const int cy = c % 10, cz = (c / 10) % 6, cx = c / 60;
        const int gz = bz * 8 + 4 * rank - 1 + cz, gy = by * 8 - 1 + cy, gx = bx * 8 - 1 + cx;
        float2 gb = make_float2(0.0f, 0.0f);
        if (gamma && gz >= 0 && gz < M && gy >= 0 && gy < N && gx >= 0 && gx < K) {
            const size_t gi = ((size_t)gz * N + gy) * K + gx;
            gb = make_float2(gamma[gi], beta[gi]);
        }
        reinterpret_cast<float2 *>(o + rank * pair64::PK_F + pair64::WPK_F)[c] = gb;
    }
    for (int idx = threadIdx.x; idx < 2 * pair64::WPK_F; idx += 256) {
        const int rank = idx / pair64::WPK_F, e = idx - rank * pair64::WPK_F;
        const int chunk = e / pair64::WCH_F, k = e - chunk * pair64::WCH_F;  // chunk = h * 4 + xo
        const int h = chunk >> 2, xo = chunk & 3;
        int un, jn, src_t;
        if (k < pair64::WCH_W) {
            const int c = k / 288, r = k - c * 288;  // x tap in sweep order, then [unit][tap (a, b)][jn]
            un = r / 36;
            const int ab = (r - un * 36) >> 2;
            jn = r & 3;
            src_t = (ab / 3) * 9 + (ab % 3) * 3 + (h ? 2 - c : c);
        } else {
            const int r = (k - pair64::WCH_W) & 31;
            src_t = k - pair64::WCH_W < 32 ? 27 : 28;
            un = r >> 2;
            jn = r & 3;
        }
        const int z = 4 * rank + 2 * (un >> 2) + (jn >> 1), y = 2 * (un & 3) + (jn & 1), x = h ? 7 - xo : xo;
        o[rank * pair64::PK_F + e] = stage[src_t * 512 + (z * 8 + y) * 8 + x];
    }
}

// ---- layout conversion at the two ends of the fused loop --------------------------------------
// [B, P] -> IL64 [G][P][64]; samples beyond B are written as zeros. grid (P / 32, G), 256 threads.
__global__ void __launch_bounds__(256) to_il64_k(const float *__restrict__ x, float *__restrict__ il, int B, size_t P)
{
    __shared__ float t[64][33];
    const int g = blockIdx.y;
    const size_t p0 = (size_t)blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int sidx = ty + 8 * k, bb = g * 64 + sidx;
        t[sidx][tx] = bb < B ? x[(size_t)bb * P + p0 + tx] : 0.0f;
    }
    __syncthreads();
    float *o = il + ((size_t)g * P + p0) * 64;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int idx = threadIdx.x + 256 * k;
        o[idx] = t[idx & 63][idx >> 6];
    }
}

// IL64 raw step output -> y [B, P] = (v - mean) * rstd * gamma + beta (stats == nullptr: plain copy).
__global__ void __launch_bounds__(256) from_il64_k(const float *__restrict__ il, const float2 *__restrict__ stats,
                                                   const float *__restrict__ gamma, const float *__restrict__ beta,
                                                   float *__restrict__ y, int B, size_t P)
{
    __shared__ float t[64][33];
    const int g = blockIdx.y;
    const size_t p0 = (size_t)blockIdx.x * 32;
    const float *in = il + ((size_t)g * P + p0) * 64;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int idx = threadIdx.x + 256 * k;
        t[idx & 63][idx >> 6] = in[idx];
    }
    __syncthreads();
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    float gm = 1.0f, bt = 0.0f;
    if (stats) {
        gm = gamma[p0 + tx];
        bt = beta[p0 + tx];
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int sidx = ty + 8 * k, bb = g * 64 + sidx;
        if (bb < B) {
            float v = t[sidx][tx];
            if (stats) {
                const float2 mr = stats[bb];
                v = fmaf((v - mr.x) * mr.y, gm, bt);
            }
            y[(size_t)bb * P + p0 + tx] = v;
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

size_t pair64_packed_floats(int M, int N, int K)
{
    return (size_t)(M / 8) * (N / 8) * (K / 8) * 2 * pair64::PK_F;
}

bool pair64_applicable(int M, int N, int K, int block, int inner)
{
    if (block != 8 || inner < 1) return false;
    if (M % 8 || N % 8 || K % 8) return false;
    if ((long long)M * N * K >= (1LL << 31) / 64) return false;  // element offsets inside one group stay below 2^31
    return encode_tiled_fn() != nullptr;
}

// Tensor map over an IL64 buffer: dims (fastest first) {64, K, N, M, G}, box {64, 1, 10, 6, 1}: one tile column.
static int make_il64_map(CUtensorMap *map, const float *il, int M, int N, int K, int G)
{
    MapKey key{il, 64, 0, {M, N, K, G}};
    (void)cudaGetDevice(&key.dev);
    if (tensor_map_cache_get(key, map)) return GN_OK;
    const cuuint64_t dims[5] = {64, (cuuint64_t)K, (cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)G};
    const cuuint64_t strides[4] = {256, (cuuint64_t)K * 256, (cuuint64_t)N * K * 256, (cuuint64_t)M * N * K * 256};
    const cuuint32_t box[5] = {64, 1, 10, 6, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(il), dims, strides,
                                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
        return GN_ERR_CUDA;
    }
    tensor_map_cache_put(key, *map);
    return GN_OK;
}

int launch_pair64_pack(const float *w, const float *b, const float *s, const float *gamma, const float *beta, float *packed,
                       int M, int N, int K, cudaStream_t st)
{
    static unsigned long long attr_set = 0;
    const int smem = 29 * 512 * 4;
    if (first_use_on_device(&attr_set)) {
        cudaError_t e = cudaFuncSetAttribute(pair64_pack_k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaFuncSetAttribute(pair64_pack_k)");
            return GN_ERR_CUDA;
        }
    }
    const int nblocks = (M / 8) * (N / 8) * (K / 8);
    pair64_pack_k<<<nblocks, 256, smem, st>>>(w, b, s, gamma, beta, packed, M, N, K);
    return check_launch("pair64_pack");
}

int launch_to_il64(const float *x, float *il, int B, int G, long long P, cudaStream_t st)
{
    dim3 grid((unsigned)(P / 32), (unsigned)G);
    to_il64_k<<<grid, 256, 0, st>>>(x, il, B, (size_t)P);
    return check_launch("to_il64");
}

int launch_from_il64(const float *il, const float2 *stats, const float *gamma, const float *beta, float *y, int B, int G,
                     long long P, cudaStream_t st)
{
    dim3 grid((unsigned)(P / 32), (unsigned)G);
    from_il64_k<<<grid, 256, 0, st>>>(il, stats, gamma, beta, y, B, (size_t)P);
    return check_launch("from_il64");
}

int launch_step_fwd_pair64(const Pair64Step &a, int act, cudaStream_t st)
{
    CUtensorMap map;
    int rc = make_il64_map(&map, a.in_il64, a.M, a.N, a.K, a.G);
    if (rc != GN_OK) return rc;
    Pair64Params p{};
    p.wpk = a.packed;
    p.in_stats = a.in_stats; p.out_partials = a.out_partials; p.nparts = a.nparts;
    p.y = a.out_il64;
    p.error_flag = a.error_flag ? a.error_flag : device_status_ptr();
    p.M = a.M; p.N = a.N; p.K = a.K; p.G = a.G; p.inner = a.inner;
    p.nblocks = (a.M / 8) * (a.N / 8) * (a.K / 8);
    p.nitems = p.nblocks * a.G;
    int ncl = sm_count() / 2;
    if (ncl > p.nitems) ncl = p.nitems;
    // evenly filled rounds: with r = ceil(items / clusters) rounds, use just as many clusters as r rounds need
    const int rounds = (p.nitems + ncl - 1) / ncl;
    ncl = (p.nitems + rounds - 1) / rounds;
    const bool fin = a.in_stats != nullptr, sout = a.out_partials != nullptr;
    static unsigned long long attr_done[4][2][2] = {};
#define ONE_(A, FI, SO)                                                                                    \
    do {                                                                                                   \
        auto kern = step_fwd_pair64<A, FI, SO>;                                                            \
        if (first_use_on_device(&attr_done[A][FI][SO])) {                                                  \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pair64::SMEM_BYTES); \
            if (e != cudaSuccess) {                                                                        \
                record_cuda_error(e, "cudaFuncSetAttribute(step_fwd_pair64)");                            \
                return GN_ERR_CUDA;                                                                        \
            }                                                                                              \
        }                                                                                                  \
        kern<<<2 * ncl, pair64::THREADS, pair64::SMEM_BYTES, st>>>(map, p);                                \
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
    return check_launch("step_fwd_pair64");
}

}  // namespace gn
