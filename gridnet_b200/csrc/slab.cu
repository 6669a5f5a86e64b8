// Helpers of the slab mode (a grid split along K across GPUs; gridnet_b200/slab.py).
#include "common.cuh"
#include "kernels.h"

namespace gn {

// x[b][m][n][col_left] = from_left[b][m][n] and x[b][m][n][col_right] = from_right[b][m][n]: the
// neighbours' boundary faces, delivered packed, go into the ghost columns the step kernel reads
// as halo cells. Either source may be null (end of the grid).
__global__ void __launch_bounds__(256) slab_unpack_faces_k(const float *__restrict__ from_left,
                                                           const float *__restrict__ from_right, float *__restrict__ x,
                                                           size_t cells, int K, int col_left, int col_right)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= cells) return;
    if (from_left) x[i * K + col_left] = from_left[i];
    if (from_right) x[i * K + col_right] = from_right[i];
}

int launch_slab_unpack_faces(const float *from_left, const float *from_right, float *x, int B, int M, int N, int K,
                             int col_left, int col_right, cudaStream_t st)
{
    const size_t cells = (size_t)B * M * N;
    if (cells == 0 || (!from_left && !from_right)) return GN_OK;
    slab_unpack_faces_k<<<(unsigned)((cells + 255) / 256), 256, 0, st>>>(from_left, from_right, x, cells, K, col_left,
                                                                        col_right);
    return check_launch("slab_unpack_faces");
}

// ---- the statistics exchange without a collective call ------------------------------------------------------
// Every rank owns a "mailbox" (normally in memory that all ranks have mapped): for each of two step parities and
// each source rank, [B] (sum, sum of squares) in double and a 64-bit flag. After its step kernel a rank adds up
// its own partials per sample and stores the sums into slot [parity][its rank] of EVERY rank's mailbox (plain
// peer stores), fences, and then stores the step number into the matching flags. The receiving side waits, with
// an iteration limit, until the flags of all ranks show the step number, adds the sums in rank order (so every
// rank gets the same bits), finishes the statistics and unpacks the two faces that the neighbours' step kernels
// stored before they published. A flag only ever grows, so nothing has to be cleared between steps; two parities
// suffice because a rank cannot be more than one step ahead of a neighbour it needs sums from.

constexpr int kMaxSlabWorld = 16;
constexpr unsigned kMailboxSpinLimit = 1u << 22;  // x ~100 ns of sleep between polls: well under a second

struct SlabMailboxes {
    unsigned char *base[kMaxSlabWorld];  // every rank's mailbox (own rank included)
};

// layout of one mailbox, in bytes
__host__ __device__ inline size_t mailbox_sums_offset(int parity, int src, int world, int B)
{
    return ((size_t)(parity * world + src) * B) * sizeof(double2);
}
__host__ __device__ inline size_t mailbox_flags_offset(int world, int B)
{
    return (size_t)2 * world * B * sizeof(double2);
}
constexpr int kPublishSlices = 8;  // CTAs that share the partials of one sample

// after the flags: the CTA counter of the whole launch, per-sample counters, per-sample slice sums (own use only)
__host__ __device__ inline size_t mailbox_scratch_offset(int world, int B)
{
    return mailbox_flags_offset(world, B) + (size_t)2 * world * sizeof(unsigned long long);
}
size_t slab_mailbox_bytes(int world, int B)
{
    size_t n = mailbox_scratch_offset(world, B) + 16 + (size_t)B * sizeof(unsigned);
    n = (n + 15) / 16 * 16;
    return n + (size_t)B * kPublishSlices * sizeof(double2);
}

// grid B * kPublishSlices: a CTA adds up one slice of a sample's partials (fixed order); the CTA of a sample that
// finishes last adds the slice sums in slice order and stores the pair into every mailbox; the CTA that finishes
// last of all publishes the flags
// FINALIZE: the CTA that publishes the flags then also waits (with the iteration limit of slab_finalize_unpack_k)
// for the other ranks' flags and finishes the statistics of all samples, which saves the separate kernel where
// nothing has to be unpacked. Every other CTA has left by then, so the wait cannot hold anything up.
template <bool FINALIZE>
__global__ void __launch_bounds__(256) slab_publish_sums_k(const double2 *__restrict__ partials, int nparts, int B,
                                                           int rank, int world, SlabMailboxes boxes, int parity,
                                                           unsigned long long step, long long count, float eps,
                                                           float2 *__restrict__ stats, int *error_flag)
{
    __shared__ double red[33];
    __shared__ bool last_of_sample, last_of_all;
    const int b = blockIdx.x / kPublishSlices, slice = blockIdx.x - b * kPublishSlices;
    unsigned char *own = boxes.base[rank] + mailbox_scratch_offset(world, B);
    unsigned *all_counter = reinterpret_cast<unsigned *>(own);
    unsigned *sample_counter = reinterpret_cast<unsigned *>(own + 16) + b;
    double2 *slice_sums = reinterpret_cast<double2 *>(own + (16 + (size_t)B * sizeof(unsigned) + 15) / 16 * 16) + (size_t)b * kPublishSlices;
    const int per = (nparts + kPublishSlices - 1) / kPublishSlices;
    const int lo = slice * per, hi = min(nparts, lo + per);
    const double2 *ps = partials + (size_t)b * nparts;
    double s = 0.0, q = 0.0;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const double2 v = ps[i];
        s += v.x;
        q += v.y;
    }
    s = block_sum(s, red);
    q = block_sum(q, red);
    if (threadIdx.x == 0) {
        __stcg(&slice_sums[slice], make_double2(s, q));
        __threadfence();
        last_of_sample = atomicAdd(sample_counter, 1u) == (unsigned)kPublishSlices - 1;
        last_of_all = false;
        if (last_of_sample) {
            *sample_counter = 0;
            __threadfence();
        }
    }
    __syncthreads();
    if (!last_of_sample) return;
    if (threadIdx.x < world) {
        double ts = 0.0, tq = 0.0;
        for (int k = 0; k < kPublishSlices; ++k) {
            const double2 v = __ldcg(&slice_sums[k]);
            ts += v.x;
            tq += v.y;
        }
        double2 *dst = reinterpret_cast<double2 *>(boxes.base[threadIdx.x] + mailbox_sums_offset(parity, rank, world, B));
        dst[b] = make_double2(ts, tq);
    }
    __threadfence_system();  // the sums are out before this sample counts as done
    __syncthreads();
    if (threadIdx.x == 0) {
        last_of_all = atomicAdd(all_counter, 1u) == (unsigned)B - 1;
        if (last_of_all) *all_counter = 0;  // ready for the next step (launches on a stream do not overlap)
    }
    __syncthreads();
    if (last_of_all && threadIdx.x < world) {
        __threadfence_system();  // order the other CTAs' stores, seen through the counter, before the flags
        unsigned long long *flag = reinterpret_cast<unsigned long long *>(boxes.base[threadIdx.x] + mailbox_flags_offset(world, B)) +
                                   parity * world + rank;
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(step) : "memory");
    }
    if (FINALIZE && last_of_all) {
        const unsigned char *box = boxes.base[rank];
        if (threadIdx.x < world) {  // one thread per rank polls that rank's flag in this rank's own mailbox
            const unsigned long long *flag =
                reinterpret_cast<const unsigned long long *>(box + mailbox_flags_offset(world, B)) + parity * world + threadIdx.x;
            unsigned spins = 0;
            unsigned long long v;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
                if (v >= step) break;
                if (++spins > kMailboxSpinLimit) {
                    if (error_flag) *error_flag = 1;
                    break;
                }
                __nanosleep(100);
            }
        }
        __syncthreads();
        for (int b2 = threadIdx.x; b2 < B; b2 += blockDim.x) {
            double ts = 0.0, tq = 0.0;
            for (int r = 0; r < world; ++r) {  // rank order: the same bits on every rank
                const double2 v = __ldcg(reinterpret_cast<const double2 *>(box + mailbox_sums_offset(parity, r, world, B)) + b2);
                ts += v.x;
                tq += v.y;
            }
            const double mean = ts / (double)count;
            double var = tq / (double)count - mean * mean;
            if (var < 0.0) var = 0.0;
            stats[b2] = make_float2((float)mean, (float)(1.0 / sqrt(var + (double)eps)));
        }
    }
}

// Waits for the step's flags of all ranks in this rank's mailbox, then: CTAs 0 .. B-1 finish the statistics of one
// sample each; all CTAs unpack the two faces (as slab_unpack_faces_k). A wait that runs out sets *error_flag and
// carries on.
__global__ void __launch_bounds__(256) slab_finalize_unpack_k(const unsigned char *__restrict__ box, int world, int B,
                                                              int parity, unsigned long long step, long long count, float eps,
                                                              float2 *__restrict__ stats, const float *__restrict__ from_left,
                                                              const float *__restrict__ from_right, float *__restrict__ x,
                                                              size_t cells, int K, int col_left, int col_right,
                                                              int *error_flag)
{
    if (threadIdx.x == 0) {
        const unsigned long long *flags =
            reinterpret_cast<const unsigned long long *>(box + mailbox_flags_offset(world, B)) + parity * world;
        bool all = true;
        for (int r = 0; r < world; ++r) {
            unsigned spins = 0;
            unsigned long long v;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + r) : "memory");
                if (v >= step) break;
                if (++spins > kMailboxSpinLimit) {
                    all = false;
                    break;
                }
                __nanosleep(100);
            }
        }
        if (!all && error_flag) *error_flag = 1;
    }
    __syncthreads();
    if ((int)blockIdx.x < B && threadIdx.x == 0) {
        const int b = blockIdx.x;
        double s = 0.0, q = 0.0;
        for (int r = 0; r < world; ++r) {
            const double2 v = reinterpret_cast<const double2 *>(box + mailbox_sums_offset(parity, r, world, B))[b];
            s += v.x;
            q += v.y;
        }
        const double mean = s / (double)count;
        double var = q / (double)count - mean * mean;
        if (var < 0.0) var = 0.0;
        stats[b] = make_float2((float)mean, (float)(1.0 / sqrt(var + (double)eps)));
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < cells; i += (size_t)gridDim.x * blockDim.x) {
        if (from_left) x[i * K + col_left] = from_left[i];
        if (from_right) x[i * K + col_right] = from_right[i];
    }
}

int launch_slab_publish_sums(const double2 *partials, int nparts, int B, int rank, int world, void *const *mailboxes,
                             int parity, unsigned long long step, cudaStream_t st)
{
    if (world < 1 || world > kMaxSlabWorld || rank < 0 || rank >= world) return GN_ERR_BAD_SHAPE;
    SlabMailboxes boxes{};
    for (int r = 0; r < world; ++r) {
        if (!mailboxes[r]) return GN_ERR_NULL_POINTER;
        boxes.base[r] = static_cast<unsigned char *>(mailboxes[r]);
    }
    slab_publish_sums_k<false><<<B * kPublishSlices, 256, 0, st>>>(partials, nparts, B, rank, world, boxes, parity, step, 1, 0.0f,
                                                                   nullptr, nullptr);
    return check_launch("slab_publish_sums");
}

int launch_slab_publish_finalize(const double2 *partials, int nparts, int B, int rank, int world, void *const *mailboxes,
                                 int parity, unsigned long long step, long long count, float eps, float2 *stats,
                                 int *error_flag, cudaStream_t st)
{
    if (world < 1 || world > kMaxSlabWorld || rank < 0 || rank >= world) return GN_ERR_BAD_SHAPE;
    SlabMailboxes boxes;
    for (int r = 0; r < world; ++r) {
        if (!mailboxes[r]) return GN_ERR_NULL_POINTER;
        boxes.base[r] = static_cast<unsigned char *>(mailboxes[r]);
    }
    if (!error_flag) error_flag = device_status_ptr();
    slab_publish_sums_k<true><<<B * kPublishSlices, 256, 0, st>>>(partials, nparts, B, rank, world, boxes, parity, step, count,
                                                                  eps, stats, error_flag);
    return check_launch("slab_publish_finalize");
}

int launch_slab_finalize_unpack(const void *mailbox, int world, int B, int parity, unsigned long long step, long long count,
                                float eps, float2 *stats, const float *from_left, const float *from_right, float *x, int M,
                                int N, int K, int col_left, int col_right, int *error_flag, cudaStream_t st)
{
    if (world < 1 || world > kMaxSlabWorld) return GN_ERR_BAD_SHAPE;
    const size_t cells = (from_left || from_right) ? (size_t)B * M * N : 0;
    size_t ctas = (cells + 255) / 256;
    if (ctas < (size_t)B) ctas = B;
    const size_t cap = (size_t)sm_count() * 8;
    if (ctas > cap) ctas = cap > (size_t)B ? cap : (size_t)B;
    slab_finalize_unpack_k<<<(unsigned)ctas, 256, 0, st>>>(static_cast<const unsigned char *>(mailbox), world, B, parity, step,
                                                           count, eps, stats, from_left, from_right, x, cells, K, col_left,
                                                           col_right, error_flag);
    return check_launch("slab_finalize_unpack");
}

}  // namespace gn
