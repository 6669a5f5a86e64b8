/*
 * gridnet_b200 — C ABI of the B200 (sm_100a) kernels for gridnet's block-local
 * recurrent grid update and the whole-grid normalisation between outer steps.
 *
 * This header is the drop-in boundary: it carries what the reference's native
 * extension `gridnet_cuda` exposes through pybind11 (src/gridnet_cuda.cpp:188-194),
 * as plain `extern "C"` entry points with raw device pointers, sizes and a CUDA
 * stream handle. No torch types appear in any signature.
 *
 * Conventions (same as the reference, src/gridnet_cuda.cpp:6-10,
 * gridnet/backend_cuda.py:19-50):
 *   - every pointer is a DEVICE pointer to a dense row-major array;
 *   - activations are [B, M, N, K]; K is the fastest dimension;
 *   - weight is [27, M, N, K] with tap = a*9 + b*3 + c reading the neighbour at
 *     offset (a-1, b-1, c-1) along (M, N, K); gated weight is [27, 2, M, N, K]
 *     (0 = value, 1 = gate), gated bias [2, M, N, K];
 *   - block must be 4 or 8 and divide M, N and K;
 *   - the caller owns every buffer; the library never allocates or frees device
 *     memory, never synchronises, and launches only on the stream it is given;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - every function returns GN_OK (0) or a negative gn_status; gn_status_string()
 *     turns it into text. A launch error is reported as GN_ERR_CUDA and the CUDA
 *     error text is available from gn_last_cuda_error().
 *
 * Gradient outputs are OVERWRITTEN (the reference accumulates into tensors the
 * caller zeroed, gridnet/backend_cuda.py:78-81; with zeroed tensors the two are
 * the same thing).
 */
#ifndef GRIDNET_B200_H
#define GRIDNET_B200_H

#include <stddef.h>

#if defined(__GNUC__)
#define GN_API __attribute__((visibility("default")))
#else
#define GN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum gn_status {
    GN_OK = 0,
    GN_ERR_NULL_POINTER = -1,
    GN_ERR_BAD_BLOCK = -2,      /* block not in {4, 8} or not dividing M, N, K */
    GN_ERR_BAD_SHAPE = -3,      /* non-positive or too large dimension */
    GN_ERR_BAD_ACTIVATION = -4, /* activation id outside gn_activation */
    GN_ERR_BAD_INNER = -5,      /* negative, or too many inner iterations for the backward stash */
    GN_ERR_WORKSPACE = -6,      /* workspace missing, misaligned or too small */
    GN_ERR_CUDA = -7,           /* CUDA reported an error; see gn_last_cuda_error() */
    GN_ERR_UNSUPPORTED = -8,    /* combination not available in this entry point */
    GN_ERR_TOO_LARGE = -9       /* size beyond a fixed built-in limit */
} gn_status;

/* The strings the reference accepts (src/activations.h:6-17) map to these ids. */
typedef enum gn_activation {
    GN_ACT_RELU = 0,
    GN_ACT_LEAKY_RELU = 1, /* slope 0.01 */
    GN_ACT_SILU = 2,
    GN_ACT_TANH = 3
} gn_activation;

GN_API const char *gn_status_string(int status);
GN_API const char *gn_last_cuda_error(void);
/* -1 for an unknown name */
GN_API int gn_activation_from_name(const char *name);
GN_API int gn_version(void);
/* Process-wide tuning switches (not needed for normal use). Keys:
 *   "outer_kernel": which kernel gn_outer_forward_f32 uses: 0 = automatic (default: the whole
 *                   loop as one persistent kernel when the problem is so small that launches are
 *                   what it costs; the large-batch kernel when at most a quarter of the last group
 *                   of 64 samples would be padding; else the register-patch kernel), 1 = the
 *                   register-patch kernel, 2 = the large-batch kernel, 3 = the persistent kernel
 *                   (GN_ERR_UNSUPPORTED from gn_outer_forward_f32 when the forced one does not apply).
 *   "forward_samples_per_cta": samples one CTA of the tuned float forward kernel walks through;
 *                   0 = chosen from the grid and batch size (default). */
GN_API int gn_config_set(const char *key, int value);

/* Kernels that fetch tiles by bulk copy wait for them with an iteration limit, so that a failed copy
 * can never hang the GPU; a wait that gives up makes the call's results invalid. Entry points with a
 * workspace record that in a flag inside the workspace (gn_*_error_flag_offset); entry points without
 * one (gn_step_forward_f32, gn_step_forward_fused_f32, the slab forms, gn_gated_forward_f32,
 * gn_step_forward_pair64_f32 with error_flag == NULL) and the workspace backward set one int per device
 * inside the library instead. gn_device_status(clear) returns 1 if it is set on the current device, 0 if
 * not, a negative status on a CUDA error; clear != 0 resets it. It copies the word back with a blocking
 * copy: synchronise the streams you care about first. gn_device_status_set(v) writes the word (tests).
 * No counterpart in the reference, whose kernels never wait. */
GN_API int gn_device_status(int clear);
GN_API int gn_device_status_set(int value);

/* Measurement helper, on no product path and without a counterpart in the reference: launches a
 * kernel of nothing but dependent-chain-free FP32 FMAs on every SM (sink: one device float that is
 * practically never written) and returns in *fma_count (host, may be NULL) how many FMAs it executes.
 * Timed with events around it, it gives the FP32 pipe rate the roofline fractions are quoted against. */
GN_API int gn_probe_fp32_fma(float *sink, int iters_per_chain, long long *fma_count, void *stream);

/* ------------------------------------------------------------------ plain step
 * Replaces gridnet_cuda.forward (src/gridnet_cuda.cpp:61-89 ->
 * src/gridnet_cuda_kernels.cu:736-784): y = one outer-loop step of x.
 * inner == 0 copies x to y. */
GN_API int gn_step_forward_f32(const float *weight, const float *bias, const float *scale,
                        const float *x, float *y, int B, int M, int N, int K, int inner,
                        int block, float eps, int normalize, int activation, void *stream);
GN_API int gn_step_forward_f64(const double *weight, const double *bias, const double *scale,
                        const double *x, double *y, int B, int M, int N, int K, int inner,
                        int block, double eps, int normalize, int activation, void *stream);

/* Replaces gridnet_cuda.backward (src/gridnet_cuda.cpp:91-131 ->
 * src/gridnet_cuda_kernels.cu:786-851). Writes grad_weight [27,M,N,K],
 * grad_bias, grad_scale [M,N,K] and grad_x [B,M,N,K]. */
GN_API int gn_step_backward_f32(const float *weight, const float *bias, const float *scale,
                         const float *x, const float *grad_y, float *grad_weight,
                         float *grad_bias, float *grad_scale, float *grad_x, int B, int M,
                         int N, int K, int inner, int block, float eps, int normalize,
                         int activation, void *stream);
GN_API int gn_step_backward_f64(const double *weight, const double *bias, const double *scale,
                         const double *x, const double *grad_y, double *grad_weight,
                         double *grad_bias, double *grad_scale, double *grad_x, int B, int M,
                         int N, int K, int inner, int block, double eps, int normalize,
                         int activation, void *stream);
/* gn_step_backward_f32 with a scratch buffer. With normalize = 0, block 8 (or block 4 on a grid
 * whose sides are multiples of 8 and a 16-byte-aligned x) and
 * gn_step_backward_workspace_bytes(...) bytes of 16-byte-aligned workspace the gradient is
 * computed by the tuned four-kernel path (replay of the inner iterations, reverse sweep with
 * transposed weights, weight gradients, cross-block halo terms), which is about twice as fast as
 * the one-kernel path and free of floating-point atomics: two calls on the same inputs return
 * the same bits. In every other case (workspace NULL, misaligned or too small, other block size,
 * normalize = 1) it behaves exactly like gn_step_backward_f32. gn_step_backward_workspace_bytes
 * returns 0 when the tuned path does not apply. The workspace holds
 * (3 * inner + 1) * B * M*N*K floats and, at byte offset
 * gn_step_backward_error_flag_offset(...), an int that the call clears and that a kernel sets to
 * 1 if a bounded wait on a bulk copy gave up (the gradients are then not valid). The inner
 * iteration count is not limited on this path. */
GN_API size_t gn_step_backward_workspace_bytes(int B, int M, int N, int K, int inner, int block,
                                        int normalize, int elem_size);
GN_API size_t gn_step_backward_error_flag_offset(int B, int M, int N, int K, int inner);
GN_API int gn_step_backward_ws_f32(const float *weight, const float *bias, const float *scale,
                            const float *x, const float *grad_y, float *grad_weight,
                            float *grad_bias, float *grad_scale, float *grad_x, int B, int M,
                            int N, int K, int inner, int block, float eps, int normalize,
                            int activation, void *workspace, size_t workspace_bytes,
                            void *stream);
/* The tuned pair with the intermediate results kept from the forward pass ("stash"), for callers
 * that can afford the memory: gn_step_forward_stash_f32 is gn_step_forward_f32 (normalize = 0) that
 * also stores every inner iteration's pre-activation and the activations between iterations into
 * `stash` ((2 * inner - 1) * B * M*N*K floats, 16-byte aligned, gn_step_stash_bytes); the stash must
 * stay untouched until gn_step_backward_stash_f32 has consumed it. That call then skips the
 * recomputation of the inner iterations (about a quarter of the tuned backward) and needs only
 * gn_step_backward_stash_workspace_bytes of scratch ((inner + 2) * B * M*N*K floats; error flag at
 * gn_step_backward_stash_error_flag_offset). Same results, bit for bit, as gn_step_backward_ws_f32.
 * GN_ERR_UNSUPPORTED where the tuned path does not apply (the size queries return 0 there): grid
 * sides not multiples of 8, misaligned pointers, no bulk-tensor-copy support for block 4.
 * The reference always recomputes (src/gridnet_cuda_kernels.cu:246-300); no counterpart. */
GN_API size_t gn_step_stash_bytes(int B, int M, int N, int K, int inner, int block);
GN_API size_t gn_step_backward_stash_workspace_bytes(int B, int M, int N, int K, int inner, int block);
GN_API size_t gn_step_backward_stash_error_flag_offset(int B, int M, int N, int K, int inner);
GN_API int gn_step_forward_stash_f32(const float *weight, const float *bias, const float *scale,
                              const float *x, float *y, int B, int M, int N, int K, int inner,
                              int block, int activation, void *stash, size_t stash_bytes,
                              void *stream);
GN_API int gn_step_backward_stash_f32(const float *weight, const float *bias, const float *scale,
                               const float *x, const float *grad_y, float *grad_weight,
                               float *grad_bias, float *grad_scale, float *grad_x, int B, int M,
                               int N, int K, int inner, int block, int activation,
                               const void *stash, size_t stash_bytes, void *workspace,
                               size_t workspace_bytes, void *stream);
/* gn_step_backward_ws_f32 / gn_step_backward_stash_f32 for a step inside the model loop
 * (gridnet/scripts/train_mnist.py:62-64), whose input is the LayerNorm of the step before: x_raw is that step's RAW
 * output, in_mean_rstd [B][2] its statistics, norm_weight / norm_bias the LayerNorm parameters; the kernels
 * normalise x_raw while loading it, so the caller does not rebuild the normalised tensor. grad_x is the gradient
 * with respect to the NORMALISED input, as in the other entry points. stash: what gn_step_forward_train_f32 kept
 * (then workspace >= gn_step_backward_stash_workspace_bytes), or NULL (the inner iterations are replayed; workspace
 * >= gn_step_backward_workspace_bytes(..., normalize 0, elem 4)). Float, block 8, x_raw 16-byte aligned;
 * GN_ERR_UNSUPPORTED otherwise (normalise with gn_norm_apply_f32 and call the entry points above). */
GN_API int gn_step_backward_fused_in_f32(const float *weight, const float *bias, const float *scale, const float *x_raw,
                                  const float *in_mean_rstd, const float *norm_weight, const float *norm_bias,
                                  const float *grad_y, float *grad_weight, float *grad_bias, float *grad_scale,
                                  float *grad_x, int B, int M, int N, int K, int inner, int block, int activation,
                                  const void *stash, size_t stash_bytes, void *workspace, size_t workspace_bytes,
                                  void *stream);
/* Largest `inner` the backward entry points accept for this block size and
 * element size (the per-iteration stash lives in shared memory). */
GN_API int gn_step_backward_max_inner(int block, int elem_size);

/* ------------------------------------------------------------------ gated step
 * Replace gridnet_cuda.forward_gated / backward_gated
 * (src/gridnet_cuda.cpp:133-186 -> src/gridnet_cuda_kernels.cu:853-930). */
GN_API int gn_gated_forward_f32(const float *weight, const float *bias, const float *x, float *y,
                         int B, int M, int N, int K, int inner, int block, int activation,
                         void *stream);
GN_API int gn_gated_forward_f64(const double *weight, const double *bias, const double *x, double *y,
                         int B, int M, int N, int K, int inner, int block, int activation,
                         void *stream);
GN_API int gn_gated_backward_f32(const float *weight, const float *bias, const float *x,
                          const float *grad_y, float *grad_weight, float *grad_bias,
                          float *grad_x, int B, int M, int N, int K, int inner, int block,
                          int activation, void *stream);
GN_API int gn_gated_backward_f64(const double *weight, const double *bias, const double *x,
                          const double *grad_y, double *grad_weight, double *grad_bias,
                          double *grad_x, int B, int M, int N, int K, int inner, int block,
                          int activation, void *stream);
/* gn_gated_backward_f32 with a caller-supplied scratch buffer (16-byte aligned, at least
 * gn_gated_backward_workspace_bytes(...) bytes; 0 = no tuned path for these arguments: call gn_gated_backward_f32).
 * With it the float backward at block 8 runs as four kernels with the forward kernel's register-patch mapping
 * (replay, reverse sweep, weight gradients, cross-block part of grad_x), without floating-point atomics, so two calls
 * return the same bits, and with no limit on `inner`; otherwise it behaves exactly like gn_gated_backward_f32. The
 * int at gn_gated_backward_error_flag_offset(...) inside the workspace is 1 afterwards if a bounded wait on a bulk
 * tile copy gave up (the results are then invalid). Same reference entry point as gn_gated_backward_f32
 * (src/gridnet_cuda.cpp:159-186 -> src/gridnet_cuda_kernels.cu:538-734). */
GN_API size_t gn_gated_backward_workspace_bytes(int B, int M, int N, int K, int inner, int block, int elem_size);
GN_API size_t gn_gated_backward_error_flag_offset(int B, int M, int N, int K, int inner);
GN_API int gn_gated_backward_ws_f32(const float *weight, const float *bias, const float *x, const float *grad_y,
                             float *grad_weight, float *grad_bias, float *grad_x, int B, int M, int N, int K,
                             int inner, int block, int activation, void *workspace, size_t workspace_bytes,
                             void *stream);

/* ------------------------------------------------- whole-grid normalisation
 * The reference's models apply torch.nn.LayerNorm over the full [M,N,K] grid
 * after every step (gridnet/scripts/train_mnist.py:54,62-64;
 * gridnet/scripts/train_imagenet.py:67,85-86). Per sample over P = M*N*K values:
 * y = (x - mean) / sqrt(var + eps) * gamma + beta with the biased variance.
 * `workspace` holds the per-sample partial sums between the two kernels.
 * mean_rstd (optional, may be NULL) receives [B][2] floats (mean, 1/std). */
GN_API size_t gn_norm_workspace_bytes(int B, long long P);
GN_API int gn_norm_forward_f32(const float *x, const float *gamma, const float *beta, float *y,
                        float *mean_rstd, int B, long long P, float eps, void *workspace,
                        size_t workspace_bytes, void *stream);
/* grad_x [B,P], grad_gamma [P], grad_beta [P] are overwritten. */
GN_API int gn_norm_backward_f32(const float *x, const float *gamma, const float *grad_y, float *grad_x,
                         float *grad_gamma, float *grad_beta, int B, long long P, float eps,
                         void *workspace, size_t workspace_bytes, void *stream);

/* The residual form of the model loop, gridnet/scripts/train_imagenet.py:81-83: n = LayerNorm(h); h' = h + (net(n) - n).
 * Given h [B,P], y = net(n) [B,P] and the (mean, rstd) of h, writes out = h + (y - LayerNorm(h)) (out may alias h or
 * y) and the (mean, rstd) of out for the next step, so the normalised tensor itself is never stored: the step
 * kernel normalises h while loading it (gn_step_forward_train_f32 with in_mean_rstd). workspace:
 * gn_norm_workspace_bytes(B, P). */
GN_API int gn_norm_residual_combine_f32(const float *h, const float *y, const float *gamma, const float *beta,
                                        const float *mean_rstd_h, float *out, float *mean_rstd_out, int B, long long P,
                                        float eps, void *workspace, size_t workspace_bytes, void *stream);

/* The same normalisation in pieces, for a grid whose positions are spread over several ranks (slab sharding:
 * each rank holds P of the P_total positions of every sample). The caller adds the [B][2] double sums of the
 * ranks (an all-reduce) between the calls; no counterpart in the reference, which is single-device.
 *   forward:  gn_norm_local_sums_f32 -> (sum x, sum x^2) per sample over the local part; all-reduce;
 *             gn_norm_finalize_f32(sums, 1, mean_rstd, B, P_total, eps); gn_norm_apply_f32 on the local part.
 *   backward: gn_norm_backward_local_sums_f32 -> (sum gy gamma, sum gy gamma xhat) per sample, local; all-reduce;
 *             gn_norm_backward_apply_f32 with the global sums and P_total: grad_x, grad_gamma, grad_beta of the
 *             local part (overwritten).
 * workspace: gn_norm_workspace_bytes(B, P). */
GN_API int gn_norm_local_sums_f32(const float *x, double *sums, int B, long long P, void *workspace,
                           size_t workspace_bytes, void *stream);
GN_API int gn_norm_backward_local_sums_f32(const float *x, const float *gamma, const float *grad_y,
                                    const float *mean_rstd, double *sums, int B, long long P, void *workspace,
                                    size_t workspace_bytes, void *stream);
GN_API int gn_norm_backward_apply_f32(const float *x, const float *gamma, const float *grad_y, const float *mean_rstd,
                               const double *sums, long long P_total, float *grad_x, float *grad_gamma,
                               float *grad_beta, int B, long long P, void *workspace, size_t workspace_bytes,
                               void *stream);

/* gn_norm_forward_static_f32: gn_norm_forward_f32 without a workspace argument and without
 * any allocation, for callers that are not allowed to allocate device memory (a host
 * application that has frozen its memory plan, a plug-in running inside another program's
 * execution loop, a process under a hard memory cap). It has no counterpart in the
 * reference. The partial sums live in a fixed array inside the library image (about
 * 0.26 MB on every GPU that loads the library, held until the process exits), so:
 *   - at most gn_norm_static_max_batch() (256) samples per call; a larger B returns
 *     GN_ERR_TOO_LARGE and nothing is launched;
 *   - the first call on each device looks up the array's device address (with that device
 *     current) and keeps it for the life of the process; make that first call before any stream
 *     capture begins. The kept address belongs to the device's primary context: a process that
 *     calls cudaDeviceReset, or makes another context current on the same device, must not use
 *     this entry point afterwards;
 *   - all calls on a device share the array: two calls whose kernels can overlap on the
 *     GPU (different streams, no ordering between them) race on it. Calls on one stream,
 *     or otherwise ordered, are safe; nothing needs clearing between calls.
 * It calls no cudaMalloc / cudaFree or any allocating routine. Results are identical to
 * gn_norm_forward_f32. */
GN_API int gn_norm_static_max_batch(void);
GN_API int gn_norm_forward_static_f32(const float *x, const float *gamma, const float *beta, float *y,
                               int B, long long P, float eps, void *stream);

/* Building blocks of the fused loop below, for callers that drive the outer loop
 * themselves (a slab-sharded grid exchanges halos and statistics between steps).
 *
 * gn_step_forward_fused_f32: one plain step with normalize = 0 whose input may be
 * the RAW output of the previous step: with in_mean_rstd != NULL every tile cell is
 * turned into (x - mean) * rstd * gamma + beta while it is loaded (in_mean_rstd is
 * [B][2] floats; gamma, beta [M,N,K]); with out_partials != NULL the per-sample
 * sum and sum of squares of y are written as gn_step_stats_partials() pairs of
 * doubles per sample ([B][nparts][2]) for gn_norm_finalize_f32. Block size 8 and
 * inner >= 1 only (GN_ERR_UNSUPPORTED otherwise). No counterpart in the
 * reference, whose LayerNorm is a separate torch module.
 * gn_norm_finalize_f32: partials -> [B][2] (mean, 1/sqrt(var + eps)).
 * gn_norm_apply_f32: y = (x - mean) * rstd * gamma + beta. */
GN_API int gn_step_stats_partials(int M, int N, int K, int block);
GN_API int gn_step_forward_fused_f32(const float *weight, const float *bias, const float *scale,
                              const float *x, float *y, const float *gamma, const float *beta,
                              const float *in_mean_rstd, double *out_partials, int B, int M,
                              int N, int K, int inner, int block, int activation, void *stream);
/* gn_step_forward_fused_f32 for the forward pass of TRAINING (block 8 or 4): the same fusion with the
 * normalisation, and with stash != NULL (gn_step_stash_bytes bytes, 16-byte aligned) it also keeps what
 * gn_step_backward_stash_f32 needs, like gn_step_forward_stash_f32. The x that the matching backward wants is the
 * NORMALISED input: gn_norm_apply_f32(x, gamma, beta, in_mean_rstd). No counterpart in the reference. */
GN_API int gn_step_forward_train_f32(const float *weight, const float *bias, const float *scale, const float *x,
                              float *y, const float *gamma, const float *beta, const float *in_mean_rstd,
                              double *out_partials, int B, int M, int N, int K, int inner, int block,
                              int activation, void *stash, size_t stash_bytes, void *stream);
/* Large-batch form of gn_step_forward_fused_f32 (block 8, normalize = 0, inner >= 1, M, N, K
 * multiples of 8): same arithmetic as src/gridnet_cuda_kernels.cu:101-200, but a thread owns
 * samples instead of neurons, which needs the activations interleaved by groups of 64 samples
 * ("IL64": [ceil(B/64)][M][N][K][64] floats, samples beyond B zero) and the parameters re-ordered
 * per block half. No counterpart in the reference.
 *   gn_pair64_supported            1 if this device and shape can run it
 *   gn_pair64_stats_partials       (sum, sum of squares) pairs per sample that a step writes: 2 per block
 *   gn_pair64_packed_weight_bytes  size of the re-ordered parameters (weights, bias, scale, gamma, beta)
 *   gn_pair64_pack_weights_f32     weight [27,M,N,K], bias, scale [M,N,K] and the whole-grid norm's gamma, beta
 *                                  [M,N,K] (both NULL if no step will normalise its input) -> packed
 *                                  (16-byte aligned)
 *   gn_pair64_interleave_f32       x [B,M,N,K] -> x_il64
 *   gn_step_forward_pair64_f32     one step, IL64 in, IL64 out; in_mean_rstd ([64*ceil(B/64)][2]; the gamma
 *                                  and beta it goes with are the packed ones) and out_partials
 *                                  ([64*ceil(B/64)][partials_per_sample][2] doubles; the first
 *                                  gn_pair64_stats_partials(M,N,K) pairs of every row are written) as in
 *                                  gn_step_forward_fused_f32;
 *                                  error_flag (device int, may be NULL) is set to 1 if a bounded wait on a
 *                                  bulk copy gave up
 *   gn_pair64_deinterleave_f32     y_il64 -> y [B,M,N,K]; with mean_rstd != NULL y = (v - mean) * rstd *
 *                                  gamma + beta */
GN_API int gn_pair64_supported(int M, int N, int K, int block, int inner);
GN_API int gn_pair64_stats_partials(int M, int N, int K);
GN_API size_t gn_pair64_packed_weight_bytes(int M, int N, int K);
GN_API int gn_pair64_pack_weights_f32(const float *weight, const float *bias, const float *scale, const float *gamma,
                               const float *beta, float *packed, int M, int N, int K, void *stream);
GN_API int gn_pair64_interleave_f32(const float *x, float *x_il64, int B, int M, int N, int K, void *stream);
GN_API int gn_pair64_deinterleave_f32(const float *y_il64, const float *mean_rstd, const float *gamma,
                               const float *beta, float *y, int B, int M, int N, int K, void *stream);
GN_API int gn_step_forward_pair64_f32(const float *packed, const float *x_il64, float *y_il64,
                               const float *in_mean_rstd, double *out_partials,
                               int partials_per_sample, int B, int M, int N, int K, int inner, int activation,
                               int *error_flag, void *stream);
/* Slab form of gn_step_forward_fused_f32 for a grid that is split along K across GPUs. The
 * arrays have the usual layout with K = the local width INCLUDING one ghost block of 8 columns
 * on each side that is not updated; only blocks k_block_first .. k_block_first + k_block_count - 1
 * (in units of 8 columns) are computed and written. The last column of the left ghost block and the
 * first column of the right ghost block carry the neighbours' boundary faces (zeros at the ends of
 * the grid) and are read as ordinary halo cells. out_partials receives
 * 4 * (M/8) * (N/8) * k_block_count pairs per sample, laid out [B][partials_per_sample][2];
 * partials_per_sample = 0 means exactly that count, a larger value lets several launches (for
 * example boundary blocks first, interior blocks later) fill disjoint parts of one buffer, each
 * launch being handed out_partials advanced to its first pair. No counterpart in the reference
 * (it is single-GPU). */
GN_API int gn_step_forward_slab_f32(const float *weight, const float *bias, const float *scale,
                             const float *x, float *y, const float *gamma, const float *beta,
                             const float *in_mean_rstd, double *out_partials, int partials_per_sample,
                             int B, int M, int N, int K, int k_block_first, int k_block_count,
                             int inner, int activation, void *stream);
/* gn_step_forward_slab_f32 that also delivers the boundary faces: the first updated K-block stores
 * its first column, the last one its last column, packed as [B][M][N] floats, to face_to_left /
 * face_to_right (8-byte aligned; NULL = no neighbour on that side). The addresses are normally
 * buffers in the neighbouring GPUs' memory mapped into this process, so the faces cross NVLink
 * from inside the step kernel and no pack kernel or send/recv call is needed; the receiver moves
 * them into its ghost columns with gn_slab_unpack_faces_f32 once it knows the sender's kernel
 * has finished (for instance after the all-reduce of the statistics of the same step). The raw
 * step output is sent: the receiver normalises it on load like every other cell.
 * No counterpart in the reference (it is single-GPU). */
GN_API int gn_step_forward_slab_faces_f32(const float *weight, const float *bias, const float *scale,
                                   const float *x, float *y, const float *norm_weight,
                                   const float *norm_bias, const float *in_mean_rstd,
                                   double *out_partials, int partials_per_sample, int B, int M,
                                   int N, int K, int k_block_first, int k_block_count, int inner,
                                   int activation, float *face_to_left, float *face_to_right,
                                   void *stream);
/* gn_step_forward_slab_faces_f32 whose face entries are face_stride floats apart (4-byte aligned addresses;
 * face_stride <= 1: packed, as above). With face_stride = K of the neighbour's padded slab and face_to_left /
 * face_to_right = the address of the ghost column [0][0][0][col] of the buffer the neighbour reads in its next
 * step, the faces land where they are read and gn_slab_unpack_faces_f32 is not needed: that pass writes four
 * useful bytes per 32-byte sector, here the same scattered stores leave the step kernel one by one while it
 * computes. The neighbour must not be reading or writing that column meanwhile (it does not: its own step
 * writes only the real columns of that buffer, and it starts its next step after this rank's kernel has
 * finished). No counterpart in the reference (it is single-GPU). */
GN_API int gn_step_forward_slab_faces_strided_f32(const float *weight, const float *bias, const float *scale,
                                           const float *x, float *y, const float *norm_weight,
                                           const float *norm_bias, const float *in_mean_rstd,
                                           double *out_partials, int partials_per_sample, int B, int M,
                                           int N, int K, int k_block_first, int k_block_count, int inner,
                                           int activation, float *face_to_left, float *face_to_right,
                                           long long face_stride, void *stream);
/* x[b][m][n][col_left] = from_left[b][m][n], x[b][m][n][col_right] = from_right[b][m][n] for a
 * float array x [B, M, N, K]; either source may be NULL. */
GN_API int gn_slab_unpack_faces_f32(const float *from_left, const float *from_right, float *x, int B,
                             int M, int N, int K, int col_left, int col_right, void *stream);
/* The statistics exchange of the slab mode without a collective call. Every rank owns a mailbox of
 * gn_slab_mailbox_bytes(world, B) bytes, zero-filled once, in memory that all ranks have mapped (world <= 16).
 * After the step kernel of outer step number `step` (1, 2, 3, ...; parity = step & 1):
 *   gn_slab_publish_sums_f32     adds this rank's partials per sample and stores the [B][2] double sums into
 *                                every rank's mailbox (mailboxes[r] = rank r's mailbox as mapped here), then
 *                                publishes them by storing `step` into the mailboxes' flags (release, system scope);
 *   gn_slab_finalize_unpack_f32  waits, with an iteration limit, until this rank's mailbox shows `step` from all
 *                                ranks, adds the sums in rank order, writes mean_rstd [B][2] over `count` values
 *                                per sample, and moves the two faces (as gn_slab_unpack_faces_f32; either may be
 *                                NULL). If the wait runs out it sets *error_flag (NULL: the library's status word,
 *                                gn_device_status) and returns garbage statistics rather than hang.
 * The waiting kernel and the publishing kernels of the other ranks must be able to run at the same time: one rank
 * per GPU (or, with all ranks on one GPU, every rank's publish launched before any finalize). No counterpart in
 * the reference (it is single-GPU). */
GN_API size_t gn_slab_mailbox_bytes(int world, int B);
GN_API int gn_slab_publish_sums_f32(const double *partials, int partials_per_sample, int B, int rank, int world,
                             void *const *mailboxes, int parity, unsigned long long step, void *stream);
/* gn_slab_publish_sums_f32 and the statistics half of gn_slab_finalize_unpack_f32 in one launch, for exchanges
 * that have nothing to unpack (faces stored in place): the CTA that publishes this rank's flags then waits, with the
 * same iteration limit, for the other ranks' flags and writes mean_rstd [B][2]. Same requirement: the other ranks'
 * kernels must be able to run at the same time (one rank per GPU). */
GN_API int gn_slab_publish_finalize_f32(const double *partials, int partials_per_sample, int B, int rank, int world,
                                 void *const *mailboxes, int parity, unsigned long long step, long long count,
                                 float eps, float *mean_rstd, int *error_flag, void *stream);
GN_API int gn_slab_finalize_unpack_f32(const void *mailbox, int world, int B, int parity, unsigned long long step,
                                long long count, float eps, float *mean_rstd, const float *from_left,
                                const float *from_right, float *x, int M, int N, int K, int col_left,
                                int col_right, int *error_flag, void *stream);
GN_API int gn_norm_finalize_f32(const double *partials, int nparts, float *mean_rstd, int B,
                         long long P, float eps, void *stream);
GN_API int gn_norm_apply_f32(const float *x, const float *gamma, const float *beta,
                      const float *mean_rstd, float *y, int B, long long P, void *stream);

/* ------------------------------------------------------ fused model loop
 * `outer` repetitions of (plain step with normalize = 0, whole-grid LayerNorm):
 * the loop of gridnet/scripts/train_mnist.py:62-64 as one call. The
 * normalisation is never a pass of its own: each step kernel reduces the
 * per-sample statistics of what it writes, and the next step applies
 * (x - mean) * rstd * gamma + beta while it loads its tiles; only the last
 * step's output is normalised by a separate kernel into y.
 * workspace: two [B rounded up to 64, M,N,K] float buffers, the statistics partials and, for
 * block 8, the weights re-ordered for the large-batch kernel (29/27 of the weight tensor).
 * With the large-batch kernel (see gn_step_forward_pair64_f32 below) the activations stay
 * interleaved by groups of 64 samples between steps, [group][M][N][K][64], and are read by TMA. */
/* Which kernel gn_outer_forward_f32 would take for this problem with suitably aligned buffers: 3 = the whole loop
 * as one persistent kernel (1 launch), 2 = the large-batch kernel (2 launches per outer step + 3), 1 = the
 * register-patch kernel (2 per outer step + 1), 4 = the step-by-step composition of the generic kernels,
 * 0 = bad arguments or the kernel forced with gn_config_set does not apply. */
GN_API int gn_outer_forward_plan(int B, int M, int N, int K, int inner, int outer, int block);
GN_API size_t gn_outer_forward_workspace_bytes(int B, int M, int N, int K, int block);
/* Byte offset, inside the workspace, of an int that gn_outer_forward_f32 sets to 1 when a bounded
 * wait on a bulk tile copy gave up (the results of that call are then invalid). It is cleared at
 * the start of every call; read it after synchronising the stream. */
GN_API size_t gn_outer_forward_error_flag_offset(int B, int M, int N, int K, int block);
GN_API int gn_outer_forward_f32(const float *weight, const float *bias, const float *scale,
                         const float *gamma, const float *beta, const float *x, float *y,
                         int B, int M, int N, int K, int inner, int outer, int block,
                         float ln_eps, int activation, void *workspace,
                         size_t workspace_bytes, void *stream);
/* gn_outer_forward_f32 with flags. GN_OUTER_PARAMS_UNCHANGED: the previous call with this workspace had the same
 * weight, bias, scale, gamma and beta (same values, same shape) and nothing else has written to the workspace
 * since, so the re-ordered copy of the parameters that the large-batch kernel keeps there is still good and is
 * not rebuilt (an inference server calls the loop many times between weight updates). */
#define GN_OUTER_PARAMS_UNCHANGED 1
GN_API int gn_outer_forward_flags_f32(const float *weight, const float *bias, const float *scale,
                               const float *norm_weight, const float *norm_bias, const float *x, float *y,
                               int B, int M, int N, int K, int inner, int outer, int block, float ln_eps,
                               int activation, void *workspace, size_t workspace_bytes, int flags,
                               void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GRIDNET_B200_H */
