// Internal launcher declarations shared by the .cu files and api.cu.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace gn {

// ---- step_generic.cu
template <typename R>
int launch_step_fwd_generic(const R *w, const R *b, const R *s, const R *x, R *y, int B, int M, int N,
                            int K, int inner, int bs, R eps, int normalize, int act, cudaStream_t st);
template <typename R>
int launch_step_bwd_generic(const R *w, const R *b, const R *s, const R *x, const R *gy, R *gw, R *gb,
                            R *gs, R *gx, int B, int M, int N, int K, int inner, int bs, R eps,
                            int normalize, int act, cudaStream_t st);
template <typename R>
int launch_gated_fwd_generic(const R *w, const R *b, const R *x, R *y, int B, int M, int N, int K,
                             int inner, int bs, int act, cudaStream_t st);
template <typename R>
int launch_gated_bwd_generic(const R *w, const R *b, const R *x, const R *gy, R *gw, R *gb, R *gx, int B,
                             int M, int N, int K, int inner, int bs, int act, cudaStream_t st);
int step_backward_max_inner(int block, int elem_size);

// ---- step_fast.cu
struct FastFwdParams {
    const float *w, *b, *s, *x;
    float *y;
    const float *gamma, *beta;  // used when in_stats != nullptr
    const float2 *in_stats;     // [B] (mean, rstd) of x: normalise while loading; nullptr = x is used as is
    double2 *out_partials;      // [B][nparts] (sum, sum of squares) of y per warp; nullptr = not wanted
    int nparts;                 // partial slots per sample (= blocks * 4)
    int B, M, N, K, inner;
    int sub;                    // block size: 8 (also when 0) or 4; a CTA owns an 8 x 8 x 8 region either way
    int spc;                    // samples per CTA; <= 0 picks a default
    // Slab mode: only blocks kb0 .. kb0 + kbn - 1 along K are updated (kbn == 0: all of them). Tile
    // cells in the columns outside that range are read like any other cell, so they can carry a
    // neighbour slab's boundary face.
    int kb0, kbn;
    int *error_flag;            // optional device int, set to 1 if a bounded wait on a bulk copy gave up
    // Replay mode of the backward pass: keep what the reverse sweep needs. save_h [inner][B][M,N,K]
    // receives every iteration's pre-activation, save_x [inner-1][B][M,N,K] the activations after
    // iterations 1 .. inner-1 (y may then be nullptr: the final output is not wanted).
    float *save_h, *save_x;
    // Slab mode with direct face delivery: the CTAs of the first / last updated K-block also store their
    // first / last column, packed as [B][M][N], to these addresses (normally a buffer in the neighbouring
    // GPU's memory, written over NVLink); nullptr = no neighbour on that side.
    float *face_left, *face_right;
    // Distance, in floats, between consecutive entries of those face arrays: 0 or 1 = packed; K of the neighbour's
    // padded slab = the entries are that slab's ghost column itself (the face lands where the neighbour's next step
    // reads it, nothing is unpacked).
    long long face_stride;
    // Per-block normalisation (the reference's normalize=True): block 8 only, and none of the fusions, the
    // replay mode or the slab mode above. norm_eps is added to the tile's standard deviation.
    int normalize;
    float norm_eps;
    // Replay mode with per-block normalisation: [inner][B][regions] (mean, 1 / (std + eps), std, std + eps) of the
    // tile every iteration normalised, for the backward kernels; nullptr = not wanted.
    float4 *tile_stats;
};
bool fast8_applicable(const FastFwdParams &p, int block, int normalize);
extern int g_fast8_spc_override;  // tuning knob: samples per CTA of the tuned forward kernel, 0 = automatic
int launch_step_fwd_fast8(FastFwdParams p, int act, cudaStream_t st);
// Tensor map for 16 x 10 x 10 tile boxes of a float tensor [B, M, N, K]; false when bulk tensor copies cannot
// be used (base not 16-byte aligned, K not a multiple of 4, driver entry point missing).
bool fast8_make_tile_map(CUtensorMap *map, const float *base, int B, int M, int N, int K);

// ---- step_gated_fast.cu (tuned float forward of the gated update, block 8; tiles by bulk tensor copy only)
bool gated_fast8_applicable(const float *w, const float *b, const float *x, const float *y, int M, int N, int K, int block,
                            int inner);
int launch_gated_fwd_fast8(const float *w, const float *b, const float *x, float *y, int B, int M, int N, int K, int inner,
                           int act, cudaStream_t st, float *save_hv = nullptr, float *save_hg = nullptr,
                           float *save_x = nullptr, int *error_flag = nullptr);

// ---- step_gated_bwd_fast.cu (tuned float backward of the gated update, block 8: replay, reverse sweep, weight
// gradients, and the cross-block kernel of step_bwd_fast.cu once per branch)
size_t gated_bwd_fast8_workspace_floats(int B, int M, int N, int K, int inner);
bool gated_bwd_fast8_applicable(const float *w, const float *b, const float *x, const float *gy, const float *gw,
                                const float *gb, const float *gx, int M, int N, int K, int inner, int block);
int launch_gated_bwd_fast8(const float *w, const float *b, const float *x, const float *gy, float *gw, float *gb, float *gx,
                           int B, int M, int N, int K, int inner, int act, float *ws, cudaStream_t st);
// the cross-block part of grad_x for one weight set: w + tap * tap_stride + cell (step_bwd_fast.cu)
// (w2, dsum2: a second weight set with its own delta sums, added in the same pass)
int launch_bwd_border8(const float *w, size_t tap_stride, const float *dsum, float *gx, int B, int M, int N, int K,
                       cudaStream_t st, const float *w2 = nullptr, const float *dsum2 = nullptr);

// ---- slab.cu
int launch_slab_unpack_faces(const float *from_left, const float *from_right, float *x, int B, int M, int N, int K,
                             int col_left, int col_right, cudaStream_t st);

// statistics exchange of the slab mode through mailboxes in peer-mapped memory (no collective call)
size_t slab_mailbox_bytes(int world, int B);
int launch_slab_publish_sums(const double2 *partials, int nparts, int B, int rank, int world, void *const *mailboxes,
                             int parity, unsigned long long step, cudaStream_t st);
int launch_slab_publish_finalize(const double2 *partials, int nparts, int B, int rank, int world, void *const *mailboxes,
                                 int parity, unsigned long long step, long long count, float eps, float2 *stats,
                                 int *error_flag, cudaStream_t st);
int launch_slab_finalize_unpack(const void *mailbox, int world, int B, int parity, unsigned long long step, long long count,
                                float eps, float2 *stats, const float *from_left, const float *from_right, float *x, int M,
                                int N, int K, int col_left, int col_right, int *error_flag, cudaStream_t st);

// ---- step_bwd_fast.cu (tuned float backward, block 8, normalize off; needs a workspace)
size_t bwd_fast8_stash_floats(int B, int M, int N, int K, int inner);
size_t bwd_fast8_workspace_floats(int B, int M, int N, int K, int inner, bool with_stash);
bool bwd_fast8_applicable(const float *w, const float *b, const float *s, const float *x, const float *gy, float *gw,
                          float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner, int block,
                          int normalize);
int launch_step_bwd_fast8(const float *w, const float *b, const float *s, const float *x, const float *gy, float *gw,
                          float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner, int block, int act,
                          const float *stash, float *ws, cudaStream_t st, int normalize = 0, float eps = 0.0f,
                          const float *in_stats = nullptr, const float *gamma = nullptr, const float *beta = nullptr);
size_t bwd_fast8_norm_extra_floats(int B, int M, int N, int K, int inner);

// ---- step_pair64.cu ("lanes = samples" kernel for large batches; activations in the IL64 layout
// [group][z][y][x][64 samples], weights pre-packed per block half)
struct Pair64Step {
    const float *packed;      // pair64_packed_floats(M, N, K) floats from launch_pair64_pack (holds gamma, beta too)
    const float *in_il64;
    float *out_il64;
    const float2 *in_stats;   // [G*64] or nullptr
    double2 *out_partials;    // [G*64][nparts] or nullptr; slots 0 .. 2*blocks-1 of every row are written
    int nparts;
    int *error_flag;          // device int, set when a bounded wait gave up
    int M, N, K, G, inner;
};
bool pair64_applicable(int M, int N, int K, int block, int inner);
size_t pair64_packed_floats(int M, int N, int K);
int launch_pair64_pack(const float *w, const float *b, const float *s, const float *gamma, const float *beta, float *packed,
                       int M, int N, int K, cudaStream_t st);
int launch_step_fwd_pair64(const Pair64Step &a, int act, cudaStream_t st);
int launch_to_il64(const float *x, float *il, int B, int G, long long P, cudaStream_t st);
// stats == nullptr: plain layout conversion; otherwise y = (v - mean) * rstd * gamma + beta
int launch_from_il64(const float *il, const float2 *stats, const float *gamma, const float *beta, float *y, int B, int G,
                     long long P, cudaStream_t st);

// ---- status.cu: device address of the per-device status word that kernels set when a bounded wait gives up
// and the caller passed no flag of its own (nullptr if it cannot be resolved)
int *device_status_ptr();
// multiprocessor count of the current device, cached
int sm_count();
// For once-per-device set-up of a kernel (cudaFuncSetAttribute is per device): true the first time it is called
// with this mask while a given device is current, false afterwards. One mask per kernel instantiation.
bool first_use_on_device(unsigned long long *mask);
// cache of tensor maps keyed on (kind of map, device, base pointer, four extents)
struct MapKey {
    const void *ptr;
    int kind, dev;
    int d[4];
};
bool tensor_map_cache_get(const MapKey &key, CUtensorMap *out);
void tensor_map_cache_put(const MapKey &key, const CUtensorMap &map);
int launch_propagate_flag(const int *flag, cudaStream_t st);

// ---- probe.cu (FFMA-only kernel for the measured FP32 peak)
int launch_ffma_probe(float *sink, int iters, long long *fma_count, cudaStream_t st);

// ---- outer_small.cu (the whole fused loop as one persistent cooperative kernel, for launch-bound problems)
int outer_small_spc(int B, int M, int N, int K, int block, int inner, int outer, const void *w, const void *b, const void *s,
                    const void *gamma, const void *beta, const void *x, const void *y);
int launch_outer_small(const float *w, const float *b, const float *s, const float *gamma, const float *beta, const float *x,
                       float *y, float *buf0, float *buf1, double2 *partials, unsigned *barrier, int *error_flag, int B, int M,
                       int N, int K, int inner, int outer, int spc, float eps, int act, cudaStream_t st);

// ---- norm.cu
constexpr int kNormMaxParts = 64;
// per-sample (sum, sum of squares) of x in double, `parts` slices per sample
int launch_norm_partial_stats(const float *x, double2 *partials, int B, long long P, int parts, cudaStream_t st);
// partials [B][nparts] -> stats [B] = (mean, 1/sqrt(var + eps))
int launch_norm_finalize(const double2 *partials, int nparts, float2 *stats, int B, long long P, float eps,
                         cudaStream_t st);
int launch_norm_apply(const float *x, const float *gamma, const float *beta, const float2 *stats, float *y,
                      int B, long long P, cudaStream_t st);
int launch_norm_backward(const float *x, const float *gamma, const float *gy, const float2 *stats,
                         double2 *partials, float2 *ac, float *gx, float *ggamma, float *gbeta, int B,
                         long long P, int parts, cudaStream_t st);
int norm_pick_parts(long long P);
// The same normalisation in pieces, for a grid that is sharded over several ranks: per-sample sums over the local
// part (the caller adds them up over the ranks), then the element-wise passes with the global figures.
int launch_norm_residual_combine(const float *h, const float *y, const float *gamma, const float *beta,
                                 const float2 *stats, float *out, double2 *partials, int B, long long P, int parts,
                                 cudaStream_t st);
int launch_norm_local_sums(const float *x, double2 *partials, double2 *sums, int B, long long P, int parts,
                           cudaStream_t st);
int launch_norm_backward_local_sums(const float *x, const float *gamma, const float *gy, const float2 *stats,
                                    double2 *partials, double2 *sums, int B, long long P, int parts, cudaStream_t st);
int launch_norm_backward_apply(const float *x, const float *gamma, const float *gy, const float2 *stats,
                               const double2 *sums, long long P_total, float2 *ac, float *gx, float *ggamma, float *gbeta,
                               int B, long long P, cudaStream_t st);

}  // namespace gn
