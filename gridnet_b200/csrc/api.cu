// extern "C" entry points declared in include/gridnet_b200.h: argument checks,
// kernel selection, and the fused model loop.
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace gn {

static thread_local char g_cuda_error[256] = "";

void record_cuda_error(cudaError_t e, const char *where)
{
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(e));
}

int check_launch(const char *where)
{
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        record_cuda_error(e, where);
        (void)cudaGetLastError();  // clear a non-sticky launch error
        return GN_ERR_CUDA;
    }
    return GN_OK;
}

static int check_geometry(int B, int M, int N, int K, int inner, int block, int act)
{
    if (B < 0 || M <= 0 || N <= 0 || K <= 0) return GN_ERR_BAD_SHAPE;
    if (B > 65535 * 64) return GN_ERR_BAD_SHAPE;
    if (block != 4 && block != 8) return GN_ERR_BAD_BLOCK;
    if (M % block || N % block || K % block) return GN_ERR_BAD_BLOCK;
    if (inner < 0) return GN_ERR_BAD_INNER;
    if (act < GN_ACT_RELU || act > GN_ACT_TANH) return GN_ERR_BAD_ACTIVATION;
    const long long nb = (long long)(M / block) * (N / block) * (K / block);
    if (nb > 0x7fffffffLL) return GN_ERR_BAD_SHAPE;
    return GN_OK;
}

template <typename R>
static int copy_through(const R *x, R *y, int B, int M, int N, int K, cudaStream_t st)
{
    if (x == y) return GN_OK;
    const cudaError_t e =
        cudaMemcpyAsync(y, x, sizeof(R) * (size_t)B * M * N * K, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) {
        record_cuda_error(e, "cudaMemcpyAsync");
        return GN_ERR_CUDA;
    }
    return GN_OK;
}

template <typename R>
static int step_forward(const R *w, const R *b, const R *s, const R *x, R *y, int B, int M, int N, int K,
                        int inner, int block, R eps, int normalize, int act, cudaStream_t st);

template <>
int step_forward<double>(const double *w, const double *b, const double *s, const double *x, double *y, int B,
                         int M, int N, int K, int inner, int block, double eps, int normalize, int act,
                         cudaStream_t st)
{
    return launch_step_fwd_generic<double>(w, b, s, x, y, B, M, N, K, inner, block, eps, normalize, act, st);
}

template <>
int step_forward<float>(const float *w, const float *b, const float *s, const float *x, float *y, int B, int M,
                        int N, int K, int inner, int block, float eps, int normalize, int act, cudaStream_t st)
{
    FastFwdParams p{};
    p.w = w; p.b = b; p.s = s; p.x = x; p.y = y;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.sub = block;
    p.normalize = normalize ? 1 : 0;
    p.norm_eps = eps;
    if (fast8_applicable(p, block, p.normalize)) return launch_step_fwd_fast8(p, act, st);
    return launch_step_fwd_generic<float>(w, b, s, x, y, B, M, N, K, inner, block, eps, normalize, act, st);
}

template <typename R>
static int api_step_forward(const R *w, const R *b, const R *s, const R *x, R *y, int B, int M, int N, int K,
                            int inner, int block, R eps, int normalize, int act, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (B == 0) return GN_OK;
    if (!w || !b || !s || !x || !y) return GN_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (inner == 0) return copy_through(x, y, B, M, N, K, st);
    return step_forward<R>(w, b, s, x, y, B, M, N, K, inner, block, eps, normalize, act, st);
}

template <typename R>
static int api_step_backward(const R *w, const R *b, const R *s, const R *x, const R *gy, R *gw, R *gb, R *gs,
                             R *gx, int B, int M, int N, int K, int inner, int block, R eps, int normalize,
                             int act, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (!w || !b || !s || !gw || !gb || !gs) return GN_ERR_NULL_POINTER;
    if (B > 0 && (!x || !gy || !gx)) return GN_ERR_NULL_POINTER;
    if (inner > step_backward_max_inner(block, (int)sizeof(R))) return GN_ERR_BAD_INNER;
    cudaStream_t st = (cudaStream_t)stream;
    if (B == 0) {
        const size_t P = (size_t)M * N * K;
        cudaError_t e = cudaMemsetAsync(gw, 0, sizeof(R) * 27 * P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gb, 0, sizeof(R) * P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gs, 0, sizeof(R) * P, st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemsetAsync");
            return GN_ERR_CUDA;
        }
        return GN_OK;
    }
    return launch_step_bwd_generic<R>(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, eps, normalize,
                                      act, st);
}

template <typename R>
static int api_gated_forward(const R *w, const R *b, const R *x, R *y, int B, int M, int N, int K, int inner,
                             int block, int act, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (B == 0) return GN_OK;
    if (!w || !b || !x || !y) return GN_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (inner == 0) return copy_through(x, y, B, M, N, K, st);
    if (sizeof(R) == sizeof(float)) {  // tuned float kernel where it applies
        const float *fw = reinterpret_cast<const float *>(w), *fb = reinterpret_cast<const float *>(b);
        const float *fx = reinterpret_cast<const float *>(x);
        float *fy = reinterpret_cast<float *>(y);
        if (gated_fast8_applicable(fw, fb, fx, fy, M, N, K, block, inner))
            return launch_gated_fwd_fast8(fw, fb, fx, fy, B, M, N, K, inner, act, st);
    }
    return launch_gated_fwd_generic<R>(w, b, x, y, B, M, N, K, inner, block, act, st);
}

template <typename R>
static int api_gated_backward(const R *w, const R *b, const R *x, const R *gy, R *gw, R *gb, R *gx, int B, int M,
                              int N, int K, int inner, int block, int act, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (!w || !b || !gw || !gb) return GN_ERR_NULL_POINTER;
    if (B > 0 && (!x || !gy || !gx)) return GN_ERR_NULL_POINTER;
    if (inner > step_backward_max_inner(block, (int)sizeof(R))) return GN_ERR_BAD_INNER;
    cudaStream_t st = (cudaStream_t)stream;
    if (B == 0) {
        const size_t P = (size_t)M * N * K;
        cudaError_t e = cudaMemsetAsync(gw, 0, sizeof(R) * 54 * P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gb, 0, sizeof(R) * 2 * P, st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemsetAsync");
            return GN_ERR_CUDA;
        }
        return GN_OK;
    }
    return launch_gated_bwd_generic<R>(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, block, act, st);
}

// ---- workspace carving ------------------------------------------------------
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct NormWs {
    double2 *partials;  // [B][kNormMaxParts]
    float2 *stats;      // [B]
    float2 *ac;         // [B]
    size_t bytes;
};

static NormWs carve_norm(void *base, int B)
{
    NormWs w;
    size_t off = 0;
    unsigned char *p = (unsigned char *)base;
    w.partials = (double2 *)(p + off);
    off = align_up(off + sizeof(double2) * (size_t)B * kNormMaxParts, 256);
    w.stats = (float2 *)(p + off);
    off = align_up(off + sizeof(float2) * (size_t)B, 256);
    w.ac = (float2 *)(p + off);
    off = align_up(off + sizeof(float2) * (size_t)B, 256);
    w.bytes = off;
    return w;
}

struct OuterWs {
    float *buf[2];      // [Bpad,M,N,K] each (Bpad = batch rounded up to 64: the IL64 layout works in groups of 64)
    double2 *partials;  // [Bpad][blocks * 4]
    float2 *stats;      // [Bpad]
    float *packed;      // block 8 only: pair64_packed_floats(M, N, K) floats (weights in the large-batch kernel's order)
    int *error_flag;
    size_t bytes;
};

static int round_up64(int B) { return (B + 63) / 64 * 64; }

static OuterWs carve_outer(void *base, int B, int M, int N, int K, int block)
{
    OuterWs w;
    const size_t P = (size_t)M * N * K;
    const size_t nb = (size_t)(M / block) * (N / block) * (K / block);
    const bool pair = block == 8 && M % 8 == 0 && N % 8 == 0 && K % 8 == 0;
    const size_t Bp = pair ? (size_t)round_up64(B) : (size_t)B;
    size_t off = 0;
    unsigned char *p = (unsigned char *)base;
    for (int i = 0; i < 2; ++i) {
        w.buf[i] = (float *)(p + off);
        off = align_up(off + sizeof(float) * Bp * P, 256);
    }
    w.partials = (double2 *)(p + off);
    off = align_up(off + sizeof(double2) * Bp * nb * 4, 256);
    w.stats = (float2 *)(p + off);
    off = align_up(off + sizeof(float2) * Bp, 256);
    w.packed = (float *)(p + off);
    if (pair) off = align_up(off + sizeof(float) * pair64_packed_floats(M, N, K), 256);
    w.error_flag = (int *)(p + off);
    off = align_up(off + sizeof(int), 256);
    w.bytes = off;
    return w;
}

// 0 = choose automatically (the one persistent kernel of outer_small.cu for problems so small that launches are
// what they cost; the large-batch kernel of step_pair64.cu when the batch fills its groups of 64 samples well; else
// the register-patch kernel of step_fast.cu, one launch per outer step), 1 = always the register-patch kernel,
// 2 = always the large-batch kernel, 3 = always the persistent kernel
static int g_outer_kernel = 0;

// The large-batch kernel computes whole groups of 64 samples: worth it when at most a quarter of the
// last group is padding.
static bool pair64_fills_groups(int B) { return round_up64(B) * 3 <= B * 4; }

static int check_ws(const void *ws, size_t have, size_t need)
{
    if (!ws) return GN_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(ws) % 16) return GN_ERR_WORKSPACE;
    if (have < need) return GN_ERR_WORKSPACE;
    return GN_OK;
}

}  // namespace gn

using namespace gn;

extern "C" {

GN_API const char *gn_status_string(int status)
{
    switch (status) {
    case GN_OK: return "ok";
    case GN_ERR_NULL_POINTER: return "a required pointer is NULL";
    case GN_ERR_BAD_BLOCK: return "block size must be 4 or 8 and divide M, N and K";
    case GN_ERR_BAD_SHAPE: return "invalid or unsupported tensor shape";
    case GN_ERR_BAD_ACTIVATION: return "unknown activation function";
    case GN_ERR_BAD_INNER: return "invalid inner iteration count (negative, or too many for the backward stash)";
    case GN_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case GN_ERR_CUDA: return "CUDA error (see gn_last_cuda_error)";
    case GN_ERR_UNSUPPORTED: return "combination not supported by this entry point";
    case GN_ERR_TOO_LARGE: return "size exceeds a fixed built-in limit";
    default: return "unknown status";
    }
}

GN_API const char *gn_last_cuda_error(void) { return g_cuda_error; }

GN_API int gn_activation_from_name(const char *name)
{
    if (!name) return -1;
    if (!strcmp(name, "relu")) return GN_ACT_RELU;
    if (!strcmp(name, "leaky_relu")) return GN_ACT_LEAKY_RELU;
    if (!strcmp(name, "silu")) return GN_ACT_SILU;
    if (!strcmp(name, "tanh")) return GN_ACT_TANH;
    return -1;
}

GN_API int gn_config_set(const char *key, int value)
{
    if (!key) return GN_ERR_NULL_POINTER;
    if (!strcmp(key, "outer_kernel")) {
        if (value < 0 || value > 3) return GN_ERR_UNSUPPORTED;
        g_outer_kernel = value;
        return GN_OK;
    }
    if (!strcmp(key, "forward_samples_per_cta")) {  // 0: chosen from the grid and batch size
        if (value < 0) return GN_ERR_UNSUPPORTED;
        g_fast8_spc_override = value;
        return GN_OK;
    }
    return GN_ERR_UNSUPPORTED;
}

GN_API int gn_version(void) { return 1; }

GN_API int gn_step_forward_f32(const float *w, const float *b, const float *s, const float *x, float *y, int B, int M,
                        int N, int K, int inner, int block, float eps, int normalize, int act, void *stream)
{
    return api_step_forward<float>(w, b, s, x, y, B, M, N, K, inner, block, eps, normalize, act, stream);
}
GN_API int gn_step_forward_f64(const double *w, const double *b, const double *s, const double *x, double *y, int B,
                        int M, int N, int K, int inner, int block, double eps, int normalize, int act,
                        void *stream)
{
    return api_step_forward<double>(w, b, s, x, y, B, M, N, K, inner, block, eps, normalize, act, stream);
}
GN_API int gn_step_backward_f32(const float *w, const float *b, const float *s, const float *x, const float *gy,
                         float *gw, float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner,
                         int block, float eps, int normalize, int act, void *stream)
{
    return api_step_backward<float>(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, eps, normalize, act,
                                    stream);
}
GN_API int gn_step_backward_f64(const double *w, const double *b, const double *s, const double *x, const double *gy,
                         double *gw, double *gb, double *gs, double *gx, int B, int M, int N, int K, int inner,
                         int block, double eps, int normalize, int act, void *stream)
{
    return api_step_backward<double>(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, eps, normalize,
                                     act, stream);
}
GN_API size_t gn_step_backward_workspace_bytes(int B, int M, int N, int K, int inner, int block, int normalize,
                                               int elem_size)
{
    if (elem_size != 4 || (block != 8 && block != 4) || inner < 1 || B <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
    if (normalize && block != 8) return 0;  // per-block normalisation: the tuned path covers block 8
    if (M % 8 || N % 8 || K % 8) return 0;
    // with per-block normalisation the tile statistics and halo terms follow the ordinary workspace
    const size_t extra = normalize ? bwd_fast8_norm_extra_floats(B, M, N, K, inner) : 0;
    return align_up(sizeof(float) * (bwd_fast8_workspace_floats(B, M, N, K, inner, true) + extra), 256);
}

GN_API size_t gn_step_backward_error_flag_offset(int B, int M, int N, int K, int inner)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0 || inner < 1) return 0;
    return sizeof(float) * (bwd_fast8_workspace_floats(B, M, N, K, inner, true) - 4);
}

GN_API int gn_step_backward_ws_f32(const float *w, const float *b, const float *s, const float *x, const float *gy,
                                   float *gw, float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner,
                                   int block, float eps, int normalize, int act, void *workspace,
                                   size_t workspace_bytes, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    const size_t need = gn_step_backward_workspace_bytes(B, M, N, K, inner, block, normalize, 4);
    if (B > 0 && need > 0 && workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) % 16) == 0 &&
        w && b && s && x && gy && gw && gb && gs && gx &&
        bwd_fast8_applicable(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, normalize))
        return launch_step_bwd_fast8(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, act, nullptr,
                                     (float *)workspace, (cudaStream_t)stream, normalize ? 1 : 0, eps);
    return api_step_backward<float>(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, eps, normalize, act,
                                    stream);
}

// ---- the same pair with the replay's results kept from the forward pass (a "stash")
static bool stash_geometry_ok(int B, int M, int N, int K, int inner, int block)
{
    return (block == 8 || block == 4) && inner >= 1 && B > 0 && M > 0 && N > 0 && K > 0 && !(M % 8 || N % 8 || K % 8);
}

GN_API size_t gn_step_stash_bytes(int B, int M, int N, int K, int inner, int block)
{
    if (!stash_geometry_ok(B, M, N, K, inner, block)) return 0;
    return align_up(sizeof(float) * bwd_fast8_stash_floats(B, M, N, K, inner), 256);
}

GN_API size_t gn_step_backward_stash_workspace_bytes(int B, int M, int N, int K, int inner, int block)
{
    if (!stash_geometry_ok(B, M, N, K, inner, block)) return 0;
    return align_up(sizeof(float) * bwd_fast8_workspace_floats(B, M, N, K, inner, false), 256);
}

GN_API size_t gn_step_backward_stash_error_flag_offset(int B, int M, int N, int K, int inner)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0 || inner < 1) return 0;
    return sizeof(float) * (bwd_fast8_workspace_floats(B, M, N, K, inner, false) - 4);
}

GN_API int gn_step_forward_stash_f32(const float *w, const float *b, const float *s, const float *x, float *y, int B,
                                     int M, int N, int K, int inner, int block, int act, void *stash, size_t stash_bytes,
                                     void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (B == 0) return GN_OK;
    if (!w || !b || !s || !x || !y || !stash) return GN_ERR_NULL_POINTER;
    const size_t need = gn_step_stash_bytes(B, M, N, K, inner, block);
    if (need == 0) return GN_ERR_UNSUPPORTED;
    if (stash_bytes < need || reinterpret_cast<uintptr_t>(stash) % 16) return GN_ERR_WORKSPACE;
    FastFwdParams p{};
    p.w = w; p.b = b; p.s = s; p.x = x; p.y = y;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.sub = block;
    p.save_h = static_cast<float *>(stash);
    p.save_x = p.save_h + (size_t)inner * B * M * N * K;
    if (!fast8_applicable(p, block, 0)) return GN_ERR_UNSUPPORTED;
    return launch_step_fwd_fast8(p, act, (cudaStream_t)stream);
}

GN_API int gn_step_backward_stash_f32(const float *w, const float *b, const float *s, const float *x, const float *gy,
                                      float *gw, float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner,
                                      int block, int act, const void *stash, size_t stash_bytes, void *workspace,
                                      size_t workspace_bytes, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (!w || !b || !s || !gw || !gb || !gs) return GN_ERR_NULL_POINTER;
    if (B == 0) return GN_ERR_UNSUPPORTED;  // nothing was stashed: use gn_step_backward_f32
    if (!x || !gy || !gx || !stash || !workspace) return GN_ERR_NULL_POINTER;
    const size_t need_stash = gn_step_stash_bytes(B, M, N, K, inner, block);
    const size_t need_ws = gn_step_backward_stash_workspace_bytes(B, M, N, K, inner, block);
    if (need_stash == 0) return GN_ERR_UNSUPPORTED;
    if (stash_bytes < need_stash || workspace_bytes < need_ws || reinterpret_cast<uintptr_t>(stash) % 16 ||
        reinterpret_cast<uintptr_t>(workspace) % 16)
        return GN_ERR_WORKSPACE;
    if (!bwd_fast8_applicable(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, 0)) return GN_ERR_UNSUPPORTED;
    return launch_step_bwd_fast8(w, b, s, x, gy, gw, gb, gs, gx, B, M, N, K, inner, block, act,
                                 static_cast<const float *>(stash), static_cast<float *>(workspace), (cudaStream_t)stream);
}

GN_API size_t gn_gated_backward_workspace_bytes(int B, int M, int N, int K, int inner, int block, int elem_size)
{
    if (elem_size != 4 || block != 8 || inner < 1 || B <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
    if (M % 8 || N % 8 || K % 8) return 0;
    return align_up(sizeof(float) * gated_bwd_fast8_workspace_floats(B, M, N, K, inner), 256);
}

GN_API size_t gn_gated_backward_error_flag_offset(int B, int M, int N, int K, int inner)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0 || inner < 1) return 0;
    return sizeof(float) * (gated_bwd_fast8_workspace_floats(B, M, N, K, inner) - 4);
}

GN_API int gn_gated_backward_ws_f32(const float *w, const float *b, const float *x, const float *gy, float *gw, float *gb,
                                    float *gx, int B, int M, int N, int K, int inner, int block, int act, void *workspace,
                                    size_t workspace_bytes, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    const size_t need = gn_gated_backward_workspace_bytes(B, M, N, K, inner, block, 4);
    if (B > 0 && need > 0 && workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) % 16) == 0 &&
        w && b && x && gy && gw && gb && gx && gated_bwd_fast8_applicable(w, b, x, gy, gw, gb, gx, M, N, K, inner, block))
        return launch_gated_bwd_fast8(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, act, (float *)workspace,
                                      (cudaStream_t)stream);
    return api_gated_backward<float>(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, block, act, stream);
}

GN_API int gn_step_backward_fused_in_f32(const float *w, const float *b, const float *s, const float *x_raw,
                                         const float *in_mean_rstd, const float *gamma, const float *beta, const float *gy,
                                         float *gw, float *gb, float *gs, float *gx, int B, int M, int N, int K, int inner,
                                         int block, int act, const void *stash, size_t stash_bytes, void *workspace,
                                         size_t workspace_bytes, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (!w || !b || !s || !gw || !gb || !gs) return GN_ERR_NULL_POINTER;
    if (B == 0 || block != 8 || inner < 1) return GN_ERR_UNSUPPORTED;
    if (!x_raw || !in_mean_rstd || !gamma || !beta || !gy || !gx || !workspace) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(in_mean_rstd) % 8 || reinterpret_cast<uintptr_t>(workspace) % 16) return GN_ERR_WORKSPACE;
    const size_t need_ws = stash ? gn_step_backward_stash_workspace_bytes(B, M, N, K, inner, block)
                                 : gn_step_backward_workspace_bytes(B, M, N, K, inner, block, 0, 4);
    if (need_ws == 0) return GN_ERR_UNSUPPORTED;
    if (workspace_bytes < need_ws) return GN_ERR_WORKSPACE;
    if (stash) {
        const size_t need_stash = gn_step_stash_bytes(B, M, N, K, inner, block);
        if (need_stash == 0) return GN_ERR_UNSUPPORTED;
        if (stash_bytes < need_stash || reinterpret_cast<uintptr_t>(stash) % 16) return GN_ERR_WORKSPACE;
    }
    // bulk tensor copies are what the normalise-on-load path of the weight-gradient kernel is built on
    CUtensorMap probe_map;
    if (!bwd_fast8_applicable(w, b, s, x_raw, gy, gw, gb, gs, gx, B, M, N, K, inner, block, 0) ||
        !fast8_make_tile_map(&probe_map, x_raw, B, M, N, K))
        return GN_ERR_UNSUPPORTED;
    return launch_step_bwd_fast8(w, b, s, x_raw, gy, gw, gb, gs, gx, B, M, N, K, inner, block, act,
                                 static_cast<const float *>(stash), static_cast<float *>(workspace), (cudaStream_t)stream, 0,
                                 0.0f, in_mean_rstd, gamma, beta);
}

GN_API int gn_step_backward_max_inner(int block, int elem_size) { return step_backward_max_inner(block, elem_size); }

GN_API int gn_gated_forward_f32(const float *w, const float *b, const float *x, float *y, int B, int M, int N, int K,
                         int inner, int block, int act, void *stream)
{
    return api_gated_forward<float>(w, b, x, y, B, M, N, K, inner, block, act, stream);
}
GN_API int gn_gated_forward_f64(const double *w, const double *b, const double *x, double *y, int B, int M, int N,
                         int K, int inner, int block, int act, void *stream)
{
    return api_gated_forward<double>(w, b, x, y, B, M, N, K, inner, block, act, stream);
}
GN_API int gn_gated_backward_f32(const float *w, const float *b, const float *x, const float *gy, float *gw, float *gb,
                          float *gx, int B, int M, int N, int K, int inner, int block, int act, void *stream)
{
    return api_gated_backward<float>(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, block, act, stream);
}
GN_API int gn_gated_backward_f64(const double *w, const double *b, const double *x, const double *gy, double *gw,
                          double *gb, double *gx, int B, int M, int N, int K, int inner, int block, int act,
                          void *stream)
{
    return api_gated_backward<double>(w, b, x, gy, gw, gb, gx, B, M, N, K, inner, block, act, stream);
}

GN_API size_t gn_norm_workspace_bytes(int B, long long P)
{
    (void)P;
    if (B <= 0) return 256;
    return carve_norm(nullptr, B).bytes;
}

GN_API int gn_norm_forward_f32(const float *x, const float *gamma, const float *beta, float *y, float *mean_rstd, int B,
                        long long P, float eps, void *workspace, size_t workspace_bytes, void *stream)
{
    if (B < 0 || P <= 0 || (long long)B * ((P + 1023) / 1024) > 0x7fffffffLL) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!x || !gamma || !beta || !y) return GN_ERR_NULL_POINTER;
    int rc = check_ws(workspace, workspace_bytes, gn_norm_workspace_bytes(B, P));
    if (rc != GN_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const NormWs ws = carve_norm(workspace, B);
    const int parts = norm_pick_parts(P);
    rc = launch_norm_partial_stats(x, ws.partials, B, P, parts, st);
    if (rc != GN_OK) return rc;
    rc = launch_norm_finalize(ws.partials, parts, ws.stats, B, P, eps, st);
    if (rc != GN_OK) return rc;
    rc = launch_norm_apply(x, gamma, beta, ws.stats, y, B, P, st);
    if (rc != GN_OK) return rc;
    if (mean_rstd) {
        const cudaError_t e =
            cudaMemcpyAsync(mean_rstd, ws.stats, sizeof(float2) * (size_t)B, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemcpyAsync");
            return GN_ERR_CUDA;
        }
    }
    return GN_OK;
}

GN_API int gn_norm_backward_f32(const float *x, const float *gamma, const float *gy, float *gx, float *ggamma,
                         float *gbeta, int B, long long P, float eps, void *workspace, size_t workspace_bytes,
                         void *stream)
{
    if (B < 0 || P <= 0 || (long long)B * ((P + 1023) / 1024) > 0x7fffffffLL) return GN_ERR_BAD_SHAPE;
    if (!gamma || !ggamma || !gbeta) return GN_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (B == 0) {
        cudaError_t e = cudaMemsetAsync(ggamma, 0, sizeof(float) * (size_t)P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gbeta, 0, sizeof(float) * (size_t)P, st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemsetAsync");
            return GN_ERR_CUDA;
        }
        return GN_OK;
    }
    if (!x || !gy || !gx) return GN_ERR_NULL_POINTER;
    int rc = check_ws(workspace, workspace_bytes, gn_norm_workspace_bytes(B, P));
    if (rc != GN_OK) return rc;
    const NormWs ws = carve_norm(workspace, B);
    const int parts = norm_pick_parts(P);
    rc = launch_norm_partial_stats(x, ws.partials, B, P, parts, st);
    if (rc != GN_OK) return rc;
    rc = launch_norm_finalize(ws.partials, parts, ws.stats, B, P, eps, st);
    if (rc != GN_OK) return rc;
    return launch_norm_backward(x, gamma, gy, ws.stats, ws.partials, ws.ac, gx, ggamma, gbeta, B, P, parts, st);
}

GN_API int gn_norm_residual_combine_f32(const float *h, const float *y, const float *gamma, const float *beta,
                                        const float *mean_rstd_h, float *out, float *mean_rstd_out, int B, long long P,
                                        float eps, void *workspace, size_t workspace_bytes, void *stream)
{
    if (B < 0 || P <= 0) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!h || !y || !gamma || !beta || !mean_rstd_h || !out || !mean_rstd_out) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(mean_rstd_h) % 8 || reinterpret_cast<uintptr_t>(mean_rstd_out) % 8)
        return GN_ERR_UNSUPPORTED;
    int rc = check_ws(workspace, workspace_bytes, gn_norm_workspace_bytes(B, P));
    if (rc != GN_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const NormWs ws = carve_norm(workspace, B);
    const int parts = norm_pick_parts(P);
    rc = launch_norm_residual_combine(h, y, gamma, beta, reinterpret_cast<const float2 *>(mean_rstd_h), out, ws.partials,
                                      B, P, parts, st);
    if (rc != GN_OK) return rc;
    return launch_norm_finalize(ws.partials, parts, reinterpret_cast<float2 *>(mean_rstd_out), B, P, eps, st);
}

GN_API int gn_norm_local_sums_f32(const float *x, double *sums, int B, long long P, void *workspace,
                                  size_t workspace_bytes, void *stream)
{
    if (B < 0 || P <= 0) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!x || !sums) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(sums) % 16) return GN_ERR_UNSUPPORTED;
    int rc = check_ws(workspace, workspace_bytes, gn_norm_workspace_bytes(B, P));
    if (rc != GN_OK) return rc;
    const NormWs ws = carve_norm(workspace, B);
    return launch_norm_local_sums(x, ws.partials, reinterpret_cast<double2 *>(sums), B, P, norm_pick_parts(P),
                                  (cudaStream_t)stream);
}

GN_API int gn_norm_backward_local_sums_f32(const float *x, const float *gamma, const float *gy, const float *mean_rstd,
                                           double *sums, int B, long long P, void *workspace, size_t workspace_bytes,
                                           void *stream)
{
    if (B < 0 || P <= 0) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!x || !gamma || !gy || !mean_rstd || !sums) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(sums) % 16 || reinterpret_cast<uintptr_t>(mean_rstd) % 8) return GN_ERR_UNSUPPORTED;
    int rc = check_ws(workspace, workspace_bytes, gn_norm_workspace_bytes(B, P));
    if (rc != GN_OK) return rc;
    const NormWs ws = carve_norm(workspace, B);
    return launch_norm_backward_local_sums(x, gamma, gy, reinterpret_cast<const float2 *>(mean_rstd), ws.partials,
                                           reinterpret_cast<double2 *>(sums), B, P, norm_pick_parts(P),
                                           (cudaStream_t)stream);
}

GN_API int gn_norm_backward_apply_f32(const float *x, const float *gamma, const float *gy, const float *mean_rstd,
                                      const double *sums, long long P_total, float *gx, float *ggamma, float *gbeta,
                                      int B, long long P, void *workspace, size_t workspace_bytes, void *stream)
{
    if (B < 0 || P <= 0 || P_total <= 0) return GN_ERR_BAD_SHAPE;  // P may count padding cells whose grad_y is zero
    if (!gamma || !ggamma || !gbeta) return GN_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (B == 0) {
        cudaError_t e = cudaMemsetAsync(ggamma, 0, sizeof(float) * (size_t)P, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gbeta, 0, sizeof(float) * (size_t)P, st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemsetAsync");
            return GN_ERR_CUDA;
        }
        return GN_OK;
    }
    if (!x || !gy || !mean_rstd || !sums || !gx) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(sums) % 16 || reinterpret_cast<uintptr_t>(mean_rstd) % 8) return GN_ERR_UNSUPPORTED;
    int rc = check_ws(workspace, workspace_bytes, gn_norm_workspace_bytes(B, P));
    if (rc != GN_OK) return rc;
    const NormWs ws = carve_norm(workspace, B);
    return launch_norm_backward_apply(x, gamma, gy, reinterpret_cast<const float2 *>(mean_rstd),
                                      reinterpret_cast<const double2 *>(sums), P_total, ws.ac, gx, ggamma, gbeta, B, P, st);
}

GN_API int gn_step_stats_partials(int M, int N, int K, int block)
{
    if (M <= 0 || N <= 0 || K <= 0 || (block != 8 && block != 4) || M % 8 || N % 8 || K % 8) return 0;
    const long long n = (long long)(M / 8) * (N / 8) * (K / 8) * 4;
    return n > 0x7fffffffLL ? 0 : (int)n;
}

GN_API int gn_step_forward_fused_f32(const float *w, const float *b, const float *s, const float *x, float *y,
                              const float *gamma, const float *beta, const float *in_mean_rstd,
                              double *out_partials, int B, int M, int N, int K, int inner, int block, int act,
                              void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (B == 0) return GN_OK;
    if (!w || !b || !s || !x || !y) return GN_ERR_NULL_POINTER;
    if (in_mean_rstd && (!gamma || !beta)) return GN_ERR_NULL_POINTER;
    FastFwdParams p{};
    p.w = w; p.b = b; p.s = s; p.x = x; p.y = y; p.gamma = gamma; p.beta = beta;
    p.in_stats = reinterpret_cast<const float2 *>(in_mean_rstd);
    p.out_partials = reinterpret_cast<double2 *>(out_partials);
    p.nparts = gn_step_stats_partials(M, N, K, block);
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.sub = block;
    if (!fast8_applicable(p, block, 0)) return GN_ERR_UNSUPPORTED;
    if ((in_mean_rstd && reinterpret_cast<uintptr_t>(in_mean_rstd) % 8) ||
        (out_partials && reinterpret_cast<uintptr_t>(out_partials) % 16))
        return GN_ERR_UNSUPPORTED;
    return launch_step_fwd_fast8(p, act, (cudaStream_t)stream);
}

GN_API int gn_step_forward_train_f32(const float *w, const float *b, const float *s, const float *x, float *y,
                                     const float *gamma, const float *beta, const float *in_mean_rstd,
                                     double *out_partials, int B, int M, int N, int K, int inner, int block, int act,
                                     void *stash, size_t stash_bytes, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (B == 0) return GN_OK;
    if (!w || !b || !s || !x || !y) return GN_ERR_NULL_POINTER;
    if (in_mean_rstd && (!gamma || !beta)) return GN_ERR_NULL_POINTER;
    FastFwdParams p{};
    p.w = w; p.b = b; p.s = s; p.x = x; p.y = y; p.gamma = gamma; p.beta = beta;
    p.in_stats = reinterpret_cast<const float2 *>(in_mean_rstd);
    p.out_partials = reinterpret_cast<double2 *>(out_partials);
    p.nparts = gn_step_stats_partials(M, N, K, block);
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.sub = block;
    if (stash) {
        const size_t need = gn_step_stash_bytes(B, M, N, K, inner, block);
        if (need == 0) return GN_ERR_UNSUPPORTED;
        if (stash_bytes < need || reinterpret_cast<uintptr_t>(stash) % 16) return GN_ERR_WORKSPACE;
        p.save_h = static_cast<float *>(stash);
        p.save_x = p.save_h + (size_t)inner * B * M * N * K;
    }
    if (!fast8_applicable(p, block, 0)) return GN_ERR_UNSUPPORTED;
    if ((in_mean_rstd && reinterpret_cast<uintptr_t>(in_mean_rstd) % 8) ||
        (out_partials && reinterpret_cast<uintptr_t>(out_partials) % 16))
        return GN_ERR_UNSUPPORTED;
    return launch_step_fwd_fast8(p, act, (cudaStream_t)stream);
}

static int slab_forward(const float *w, const float *b, const float *s, const float *x, float *y,
                             const float *gamma, const float *beta, const float *in_mean_rstd,
                             double *out_partials, int partials_per_sample, int B, int M, int N, int K,
                             int k_block_first, int k_block_count, int inner, int act, float *face_to_left,
                             float *face_to_right, void *stream, long long face_stride = 1)
{
    const int rc = check_geometry(B, M, N, K, inner, 8, act);
    if (rc != GN_OK) return rc;
    if (k_block_first < 0 || k_block_count <= 0 || k_block_first + k_block_count > K / 8) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!w || !b || !s || !x || !y) return GN_ERR_NULL_POINTER;
    if (in_mean_rstd && (!gamma || !beta)) return GN_ERR_NULL_POINTER;
    FastFwdParams p{};
    p.w = w; p.b = b; p.s = s; p.x = x; p.y = y; p.gamma = gamma; p.beta = beta;
    p.in_stats = reinterpret_cast<const float2 *>(in_mean_rstd);
    p.out_partials = reinterpret_cast<double2 *>(out_partials);
    p.nparts = (M / 8) * (N / 8) * k_block_count * 4;
    if (partials_per_sample > 0) {  // several launches share one partial buffer
        if (partials_per_sample < p.nparts) return GN_ERR_BAD_SHAPE;
        p.nparts = partials_per_sample;
    }
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner;
    p.kb0 = k_block_first; p.kbn = k_block_count;
    p.face_left = face_to_left; p.face_right = face_to_right;
    p.face_stride = face_stride;
    if (face_stride < 0) return GN_ERR_BAD_SHAPE;
    // packed faces are stored two floats at a time; strided ones float by float
    if ((reinterpret_cast<uintptr_t>(face_to_left) | reinterpret_cast<uintptr_t>(face_to_right)) & (face_stride <= 1 ? 7 : 3))
        return GN_ERR_UNSUPPORTED;
    if (!fast8_applicable(p, 8, 0)) return GN_ERR_UNSUPPORTED;
    if ((in_mean_rstd && reinterpret_cast<uintptr_t>(in_mean_rstd) % 8) ||
        (out_partials && reinterpret_cast<uintptr_t>(out_partials) % 16))
        return GN_ERR_UNSUPPORTED;
    return launch_step_fwd_fast8(p, act, (cudaStream_t)stream);
}

GN_API int gn_step_forward_slab_f32(const float *w, const float *b, const float *s, const float *x, float *y,
                             const float *gamma, const float *beta, const float *in_mean_rstd,
                             double *out_partials, int partials_per_sample, int B, int M, int N, int K,
                             int k_block_first, int k_block_count, int inner, int act, void *stream)
{
    return slab_forward(w, b, s, x, y, gamma, beta, in_mean_rstd, out_partials, partials_per_sample, B, M, N, K,
                        k_block_first, k_block_count, inner, act, nullptr, nullptr, stream);
}

GN_API int gn_step_forward_slab_faces_f32(const float *w, const float *b, const float *s, const float *x, float *y,
                                   const float *gamma, const float *beta, const float *in_mean_rstd,
                                   double *out_partials, int partials_per_sample, int B, int M, int N, int K,
                                   int k_block_first, int k_block_count, int inner, int act, float *face_to_left,
                                   float *face_to_right, void *stream)
{
    return slab_forward(w, b, s, x, y, gamma, beta, in_mean_rstd, out_partials, partials_per_sample, B, M, N, K,
                        k_block_first, k_block_count, inner, act, face_to_left, face_to_right, stream);
}

GN_API int gn_step_forward_slab_faces_strided_f32(const float *w, const float *b, const float *s, const float *x, float *y,
                                                  const float *gamma, const float *beta, const float *in_mean_rstd,
                                                  double *out_partials, int partials_per_sample, int B, int M, int N,
                                                  int K, int k_block_first, int k_block_count, int inner, int act,
                                                  float *face_to_left, float *face_to_right, long long face_stride,
                                                  void *stream)
{
    return slab_forward(w, b, s, x, y, gamma, beta, in_mean_rstd, out_partials, partials_per_sample, B, M, N, K,
                        k_block_first, k_block_count, inner, act, face_to_left, face_to_right, stream, face_stride);
}

GN_API int gn_slab_unpack_faces_f32(const float *from_left, const float *from_right, float *x, int B, int M, int N, int K,
                             int col_left, int col_right, void *stream)
{
    if (B < 0 || M <= 0 || N <= 0 || K <= 0 || col_left < 0 || col_left >= K || col_right < 0 || col_right >= K)
        return GN_ERR_BAD_SHAPE;
    if (!x) return GN_ERR_NULL_POINTER;
    return launch_slab_unpack_faces(from_left, from_right, x, B, M, N, K, col_left, col_right, (cudaStream_t)stream);
}

GN_API size_t gn_slab_mailbox_bytes(int world, int B)
{
    if (world < 1 || world > 16 || B <= 0) return 0;
    return slab_mailbox_bytes(world, B);
}

GN_API int gn_slab_publish_sums_f32(const double *partials, int partials_per_sample, int B, int rank, int world,
                                    void *const *mailboxes, int parity, unsigned long long step, void *stream)
{
    if (B <= 0 || partials_per_sample <= 0 || (parity != 0 && parity != 1) || step == 0) return GN_ERR_BAD_SHAPE;
    if (!partials || !mailboxes) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(partials) % 16) return GN_ERR_UNSUPPORTED;
    return launch_slab_publish_sums(reinterpret_cast<const double2 *>(partials), partials_per_sample, B, rank, world, mailboxes,
                                    parity, step, (cudaStream_t)stream);
}

GN_API int gn_slab_publish_finalize_f32(const double *partials, int partials_per_sample, int B, int rank, int world,
                                        void *const *mailboxes, int parity, unsigned long long step, long long count,
                                        float eps, float *mean_rstd, int *error_flag, void *stream)
{
    if (B <= 0 || partials_per_sample <= 0 || count <= 0 || (parity != 0 && parity != 1) || step == 0) return GN_ERR_BAD_SHAPE;
    if (!partials || !mailboxes || !mean_rstd) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(partials) % 16 || reinterpret_cast<uintptr_t>(mean_rstd) % 8) return GN_ERR_UNSUPPORTED;
    return launch_slab_publish_finalize(reinterpret_cast<const double2 *>(partials), partials_per_sample, B, rank, world,
                                        mailboxes, parity, step, count, eps, reinterpret_cast<float2 *>(mean_rstd), error_flag,
                                        (cudaStream_t)stream);
}

GN_API int gn_slab_finalize_unpack_f32(const void *mailbox, int world, int B, int parity, unsigned long long step,
                                       long long count, float eps, float *mean_rstd, const float *from_left,
                                       const float *from_right, float *x, int M, int N, int K, int col_left, int col_right,
                                       int *error_flag, void *stream)
{
    if (B <= 0 || count <= 0 || (parity != 0 && parity != 1) || step == 0) return GN_ERR_BAD_SHAPE;
    if ((from_left || from_right) && (M <= 0 || N <= 0 || K <= 0 || col_left < 0 || col_left >= K || col_right < 0 || col_right >= K))
        return GN_ERR_BAD_SHAPE;
    if (!mailbox || !mean_rstd) return GN_ERR_NULL_POINTER;
    if ((from_left || from_right) && !x) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(mailbox) % 16 || reinterpret_cast<uintptr_t>(mean_rstd) % 8) return GN_ERR_UNSUPPORTED;
    return launch_slab_finalize_unpack(mailbox, world, B, parity, step, count, eps, reinterpret_cast<float2 *>(mean_rstd),
                                       from_left, from_right, x, M, N, K, col_left, col_right,
                                       error_flag ? error_flag : device_status_ptr(), (cudaStream_t)stream);
}

GN_API int gn_norm_finalize_f32(const double *partials, int nparts, float *mean_rstd, int B, long long P, float eps,
                         void *stream)
{
    if (B < 0 || P <= 0 || nparts <= 0) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!partials || !mean_rstd) return GN_ERR_NULL_POINTER;
    return launch_norm_finalize(reinterpret_cast<const double2 *>(partials), nparts,
                                reinterpret_cast<float2 *>(mean_rstd), B, P, eps, (cudaStream_t)stream);
}

GN_API int gn_norm_apply_f32(const float *x, const float *gamma, const float *beta, const float *mean_rstd, float *y,
                      int B, long long P, void *stream)
{
    if (B < 0 || P <= 0 || (long long)B * ((P + 1023) / 1024) > 0x7fffffffLL) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!x || !gamma || !beta || !mean_rstd || !y) return GN_ERR_NULL_POINTER;
    return launch_norm_apply(x, gamma, beta, reinterpret_cast<const float2 *>(mean_rstd), y, B, P,
                             (cudaStream_t)stream);
}

GN_API int gn_probe_fp32_fma(float *sink, int iters_per_chain, long long *fma_count, void *stream)
{
    if (!sink) return GN_ERR_NULL_POINTER;
    if (iters_per_chain <= 0) return GN_ERR_BAD_SHAPE;
    return launch_ffma_probe(sink, iters_per_chain, fma_count, (cudaStream_t)stream);
}

GN_API int gn_pair64_supported(int M, int N, int K, int block, int inner)
{
    return pair64_applicable(M, N, K, block, inner) ? 1 : 0;
}

GN_API int gn_pair64_stats_partials(int M, int N, int K)
{
    if (M <= 0 || N <= 0 || K <= 0 || M % 8 || N % 8 || K % 8) return 0;
    return 2 * (M / 8) * (N / 8) * (K / 8);
}

GN_API size_t gn_pair64_packed_weight_bytes(int M, int N, int K)
{
    if (M <= 0 || N <= 0 || K <= 0 || M % 8 || N % 8 || K % 8) return 0;
    return sizeof(float) * pair64_packed_floats(M, N, K);
}

GN_API int gn_pair64_pack_weights_f32(const float *w, const float *b, const float *s, const float *gamma,
                                      const float *beta, float *packed, int M, int N, int K, void *stream)
{
    if (M <= 0 || N <= 0 || K <= 0) return GN_ERR_BAD_SHAPE;
    if (M % 8 || N % 8 || K % 8) return GN_ERR_BAD_BLOCK;
    if (!w || !b || !s || !packed) return GN_ERR_NULL_POINTER;
    if ((gamma == nullptr) != (beta == nullptr)) return GN_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(packed) % 16) return GN_ERR_UNSUPPORTED;
    return launch_pair64_pack(w, b, s, gamma, beta, packed, M, N, K, (cudaStream_t)stream);
}

GN_API int gn_pair64_interleave_f32(const float *x, float *x_il64, int B, int M, int N, int K, void *stream)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0) return GN_ERR_BAD_SHAPE;
    if (((long long)M * N * K) % 32) return GN_ERR_BAD_SHAPE;
    if (!x || !x_il64) return GN_ERR_NULL_POINTER;
    return launch_to_il64(x, x_il64, B, round_up64(B) / 64, (long long)M * N * K, (cudaStream_t)stream);
}

GN_API int gn_pair64_deinterleave_f32(const float *y_il64, const float *mean_rstd, const float *gamma, const float *beta,
                                      float *y, int B, int M, int N, int K, void *stream)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0) return GN_ERR_BAD_SHAPE;
    if (((long long)M * N * K) % 32) return GN_ERR_BAD_SHAPE;
    if (!y_il64 || !y) return GN_ERR_NULL_POINTER;
    if (mean_rstd && (!gamma || !beta)) return GN_ERR_NULL_POINTER;
    return launch_from_il64(y_il64, reinterpret_cast<const float2 *>(mean_rstd), gamma, beta, y, B, round_up64(B) / 64,
                            (long long)M * N * K, (cudaStream_t)stream);
}

GN_API int gn_step_forward_pair64_f32(const float *packed, const float *x_il64, float *y_il64,
                                      const float *in_mean_rstd, double *out_partials,
                                      int partials_per_sample, int B, int M, int N, int K, int inner, int act,
                                      int *error_flag, void *stream)
{
    const int rc = check_geometry(B, M, N, K, inner, 8, act);
    if (rc != GN_OK) return rc;
    if (B == 0) return GN_OK;
    if (!packed || !x_il64 || !y_il64) return GN_ERR_NULL_POINTER;
    if (!pair64_applicable(M, N, K, 8, inner)) return GN_ERR_UNSUPPORTED;
    const int nblocks = (M / 8) * (N / 8) * (K / 8);
    if (out_partials && partials_per_sample < nblocks * 2) return GN_ERR_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(x_il64) | reinterpret_cast<uintptr_t>(y_il64)) % 16)
        return GN_ERR_UNSUPPORTED;
    if ((in_mean_rstd && reinterpret_cast<uintptr_t>(in_mean_rstd) % 8) ||
        (out_partials && reinterpret_cast<uintptr_t>(out_partials) % 16))
        return GN_ERR_UNSUPPORTED;
    Pair64Step a{};
    a.packed = packed;
    a.in_il64 = x_il64; a.out_il64 = y_il64;
    a.in_stats = reinterpret_cast<const float2 *>(in_mean_rstd);
    a.out_partials = reinterpret_cast<double2 *>(out_partials);
    a.nparts = partials_per_sample;
    a.error_flag = error_flag;
    a.M = M; a.N = N; a.K = K; a.G = round_up64(B) / 64; a.inner = inner;
    return launch_step_fwd_pair64(a, act, (cudaStream_t)stream);
}

GN_API int gn_outer_forward_plan(int B, int M, int N, int K, int inner, int outer, int block)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0 || inner < 1 || outer < 1 || (block != 4 && block != 8)) return 0;
    alignas(16) static const double aligned[2] = {0.0, 0.0};  // any 16-byte aligned address: only alignment is looked at
    const void *a = aligned;
    if ((g_outer_kernel == 0 || g_outer_kernel == 3) && outer_small_spc(B, M, N, K, block, inner, outer, a, a, a, a, a, a, a) > 0)
        return 3;
    if (g_outer_kernel == 3) return 0;
    if (pair64_applicable(M, N, K, block, inner) && (g_outer_kernel == 2 || (g_outer_kernel == 0 && pair64_fills_groups(B))))
        return 2;
    if (g_outer_kernel == 2) return 0;
    FastFwdParams p{};
    p.w = p.b = p.s = p.x = reinterpret_cast<const float *>(a);
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.sub = block;
    return fast8_applicable(p, block, 0) ? 1 : 4;
}

GN_API size_t gn_outer_forward_workspace_bytes(int B, int M, int N, int K, int block)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0 || (block != 4 && block != 8)) return 256;
    return carve_outer(nullptr, B, M, N, K, block).bytes;
}

GN_API size_t gn_outer_forward_error_flag_offset(int B, int M, int N, int K, int block)
{
    if (B <= 0 || M <= 0 || N <= 0 || K <= 0 || (block != 4 && block != 8)) return 0;
    const OuterWs w = carve_outer(nullptr, B, M, N, K, block);
    return (size_t)((unsigned char *)w.error_flag - (unsigned char *)nullptr);
}

static int outer_forward_impl(const float *w, const float *b, const float *s, const float *gamma, const float *beta,
                              const float *x, float *y, int B, int M, int N, int K, int inner, int outer, int block,
                              float ln_eps, int act, void *workspace, size_t workspace_bytes, int flags, void *stream);

GN_API int gn_outer_forward_f32(const float *w, const float *b, const float *s, const float *gamma, const float *beta,
                         const float *x, float *y, int B, int M, int N, int K, int inner, int outer, int block,
                         float ln_eps, int act, void *workspace, size_t workspace_bytes, void *stream)
{
    return outer_forward_impl(w, b, s, gamma, beta, x, y, B, M, N, K, inner, outer, block, ln_eps, act, workspace,
                              workspace_bytes, 0, stream);
}

GN_API int gn_outer_forward_flags_f32(const float *w, const float *b, const float *s, const float *gamma, const float *beta,
                                      const float *x, float *y, int B, int M, int N, int K, int inner, int outer, int block,
                                      float ln_eps, int act, void *workspace, size_t workspace_bytes, int flags, void *stream)
{
    if (flags & ~GN_OUTER_PARAMS_UNCHANGED) return GN_ERR_UNSUPPORTED;
    return outer_forward_impl(w, b, s, gamma, beta, x, y, B, M, N, K, inner, outer, block, ln_eps, act, workspace,
                              workspace_bytes, flags, stream);
}

}  // extern "C"

static int outer_forward_impl(const float *w, const float *b, const float *s, const float *gamma, const float *beta,
                              const float *x, float *y, int B, int M, int N, int K, int inner, int outer, int block,
                              float ln_eps, int act, void *workspace, size_t workspace_bytes, int flags, void *stream)
{
    int rc = check_geometry(B, M, N, K, inner, block, act);
    if (rc != GN_OK) return rc;
    if (outer < 0) return GN_ERR_BAD_SHAPE;
    if ((long long)B * (((long long)M * N * K + 1023) / 1024) > 0x7fffffffLL) return GN_ERR_BAD_SHAPE;
    if (B == 0) return GN_OK;
    if (!w || !b || !s || !gamma || !beta || !x || !y) return GN_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (outer == 0) return copy_through(x, y, B, M, N, K, st);
    rc = check_ws(workspace, workspace_bytes, gn_outer_forward_workspace_bytes(B, M, N, K, block));
    if (rc != GN_OK) return rc;
    const OuterWs ws = carve_outer(workspace, B, M, N, K, block);
    const long long P = (long long)M * N * K;

    FastFwdParams p{};
    p.w = w; p.b = b; p.s = s; p.gamma = gamma; p.beta = beta;
    p.B = B; p.M = M; p.N = N; p.K = K; p.inner = inner; p.sub = block;
    p.x = x; p.y = ws.buf[0];
    const bool fused = fast8_applicable(p, block, 0);
    const int nparts_fused = (int)((long long)(M / 8) * (N / 8) * (K / 8) * 4);

    if (g_outer_kernel == 0 || g_outer_kernel == 3) {
        const int spc = outer_small_spc(B, M, N, K, block, inner, outer, w, b, s, gamma, beta, x, y);
        if (spc > 0) {
            // the int after the error flag is the counter of the kernel's grid-wide barrier
            const cudaError_t e = cudaMemsetAsync(ws.error_flag, 0, 2 * sizeof(int), st);
            if (e != cudaSuccess) {
                record_cuda_error(e, "cudaMemsetAsync");
                return GN_ERR_CUDA;
            }
            return launch_outer_small(w, b, s, gamma, beta, x, y, ws.buf[0], ws.buf[1], ws.partials,
                                      reinterpret_cast<unsigned *>(ws.error_flag + 1), ws.error_flag, B, M, N, K, inner, outer,
                                      spc, ln_eps, act, st);
        }
        if (g_outer_kernel == 3) return GN_ERR_UNSUPPORTED;
    }
    const bool pair_ok = pair64_applicable(M, N, K, block, inner);
    if (pair_ok && (g_outer_kernel == 2 || (g_outer_kernel == 0 && pair64_fills_groups(B)))) {
        const int Bp = round_up64(B), G = Bp / 64;
        const int nblocks = (M / 8) * (N / 8) * (K / 8);
        cudaError_t e = cudaMemsetAsync(ws.error_flag, 0, sizeof(int), st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "cudaMemsetAsync");
            return GN_ERR_CUDA;
        }
        if (!(flags & GN_OUTER_PARAMS_UNCHANGED)) {  // else the workspace still holds them from the previous call
            rc = launch_pair64_pack(w, b, s, gamma, beta, ws.packed, M, N, K, st);
            if (rc != GN_OK) return rc;
        }
        rc = launch_to_il64(x, ws.buf[0], B, G, P, st);
        if (rc != GN_OK) return rc;
        for (int o = 0; o < outer; ++o) {
            Pair64Step a{};
            a.packed = ws.packed;
            a.in_il64 = ws.buf[o & 1];
            a.out_il64 = ws.buf[(o + 1) & 1];
            a.in_stats = o > 0 ? ws.stats : nullptr;
            a.out_partials = ws.partials;
            a.nparts = nblocks * 2;
            a.error_flag = ws.error_flag;
            a.M = M; a.N = N; a.K = K; a.G = G; a.inner = inner;
            rc = launch_step_fwd_pair64(a, act, st);
            if (rc != GN_OK) return rc;
            rc = launch_norm_finalize(ws.partials, nblocks * 2, ws.stats, Bp, P, ln_eps, st);
            if (rc != GN_OK) return rc;
        }
        return launch_from_il64(ws.buf[outer & 1], ws.stats, gamma, beta, y, B, G, P, st);
    }
    if (g_outer_kernel == 2) return GN_ERR_UNSUPPORTED;

    if (cudaMemsetAsync(ws.error_flag, 0, sizeof(int), st) != cudaSuccess) {
        record_cuda_error(cudaGetLastError(), "cudaMemsetAsync");
        return GN_ERR_CUDA;
    }
    const float *src = x;
    for (int o = 0; o < outer; ++o) {
        float *dst = ws.buf[o & 1];
        if (fused) {
            p.x = src;
            p.y = dst;
            p.error_flag = ws.error_flag;
            p.in_stats = o > 0 ? ws.stats : nullptr;  // raw output of the previous step: normalise on load
            p.out_partials = ws.partials;
            p.nparts = nparts_fused;
            rc = launch_step_fwd_fast8(p, act, st);
            if (rc != GN_OK) return rc;
            rc = launch_norm_finalize(ws.partials, nparts_fused, ws.stats, B, P, ln_eps, st);
            if (rc != GN_OK) return rc;
            src = dst;
        } else {
            // unfused composition: step, statistics, normalise in place
            if (inner == 0) rc = copy_through(src, dst, B, M, N, K, st);
            else rc = launch_step_fwd_generic<float>(w, b, s, src, dst, B, M, N, K, inner, block, 0.0f, 0, act, st);
            if (rc != GN_OK) return rc;
            const int parts = norm_pick_parts(P);
            rc = launch_norm_partial_stats(dst, ws.partials, B, P, parts, st);
            if (rc != GN_OK) return rc;
            rc = launch_norm_finalize(ws.partials, parts, ws.stats, B, P, ln_eps, st);
            if (rc != GN_OK) return rc;
            float *out = (o + 1 == outer) ? y : dst;
            rc = launch_norm_apply(dst, gamma, beta, ws.stats, out, B, P, st);
            if (rc != GN_OK) return rc;
            src = out;
        }
    }
    if (fused) return launch_norm_apply(src, gamma, beta, ws.stats, y, B, P, st);
    return GN_OK;
}
