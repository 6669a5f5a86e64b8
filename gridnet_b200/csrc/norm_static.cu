// gn_norm_forward_static_f32: the whole-grid normalisation for callers that must not
// allocate device memory and have no workspace to hand over.
//
// Who that is: code that runs after a host application has frozen its memory plan — an
// inference server whose framework has already reserved the whole device pool, a plug-in
// called from somebody else's execution loop where cudaMalloc is forbidden (it would
// synchronise the device and could fail mid-service), or a process under a hard memory
// cap that is only allowed the memory the loaded modules bring with them.
//
// The per-sample partial sums that gn_norm_forward_f32 keeps in a caller-provided
// workspace live here in a fixed array inside the library image instead. Every GPU that
// loads the library carries that array (about 0.26 MB) until the process exits.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace gn {

// Limit of this entry point: at most this many samples per call.
constexpr int kStaticNormMaxBatch = 256;
constexpr size_t kStaticPartialBytes = sizeof(double2) * (size_t)kStaticNormMaxBatch * kNormMaxParts;
constexpr size_t kStaticStatsBytes = sizeof(float2) * (size_t)kStaticNormMaxBatch;
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticStatsBytes;

// The scratch itself. In host code this name is only a handle for the runtime (it is not a
// device address and must never be passed to a kernel); the address comes from
// cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_norm_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void *g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the CURRENT device; resolved on first use.
static int static_scratch(void **out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        record_cuda_error(e, "cudaGetDevice");
        return GN_ERR_CUDA;
    }
    if (dev < 0 || dev >= kMaxDevices) return GN_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_norm_static_scratch);
        if (e != cudaSuccess || !p) {
            record_cuda_error(e, "cudaGetSymbolAddress(g_norm_static_scratch)");
            return GN_ERR_CUDA;
        }
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return GN_OK;
}

}  // namespace gn

using namespace gn;

extern "C" {

GN_API int gn_norm_static_max_batch(void) { return kStaticNormMaxBatch; }

GN_API int gn_norm_forward_static_f32(const float *x, const float *gamma, const float *beta, float *y, int B,
                                      long long P, float eps, void *stream)
{
    if (B < 0 || P <= 0) return GN_ERR_BAD_SHAPE;
    if (B > kStaticNormMaxBatch) return GN_ERR_TOO_LARGE;  // more samples than the built-in scratch holds
    if (B == 0) return GN_OK;
    if (!x || !gamma || !beta || !y) return GN_ERR_NULL_POINTER;
    void *base = nullptr;
    int rc = static_scratch(&base);
    if (rc != GN_OK) return rc;
    double2 *partials = reinterpret_cast<double2 *>(base);
    float2 *stats = reinterpret_cast<float2 *>(static_cast<unsigned char *>(base) + kStaticPartialBytes);
    cudaStream_t st = (cudaStream_t)stream;
    // Nothing in the scratch has to start at zero: every slot that is read below is written
    // first by this call (partials by the first kernel, stats by the second), so whatever
    // an earlier call left behind is simply overwritten.
    const int parts = norm_pick_parts(P);
    rc = launch_norm_partial_stats(x, partials, B, P, parts, st);
    if (rc != GN_OK) return rc;
    rc = launch_norm_finalize(partials, parts, stats, B, P, eps, st);
    if (rc != GN_OK) return rc;
    return launch_norm_apply(x, gamma, beta, stats, y, B, P, st);
}

}  // extern "C"
