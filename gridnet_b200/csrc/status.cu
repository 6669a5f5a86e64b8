// A status word on the device for the bounded waits of the tile pipelines.
//
// Every kernel that fetches tiles by bulk copy waits for them with an iteration limit; when a wait
// gives up the kernel carries on (it must never hang the GPU) and its results are garbage. Entry
// points that take a workspace record that in a flag inside the workspace. Entry points without
// one (gn_step_forward_f32, gn_gated_forward_f32, ...) record it here, in one int per device inside
// the library image, which gn_device_status() reads back.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace gn {

static __device__ int g_wait_status;  // 0 = no bounded wait has given up since the last clear

constexpr int kMaxDevices = 64;
static std::mutex g_status_mutex;
static int *g_status_ptr[kMaxDevices] = {nullptr};

// Device address of the status word on the CURRENT device (resolved once per device; the name of a
// __device__ variable is not an address in host code). nullptr if it cannot be resolved: the kernels
// then simply have nowhere to report to.
int *device_status_ptr()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!g_status_ptr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_wait_status) != cudaSuccess || !p) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_status_ptr[dev] = static_cast<int *>(p);
    }
    return g_status_ptr[dev];
}

// Multiprocessor count of the CURRENT device (148 on B200), looked up once per device.
int sm_count()
{
    static int cached[kMaxDevices] = {0};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return kNumSMs;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = kNumSMs;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

bool first_use_on_device(unsigned long long *mask)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    std::lock_guard<std::mutex> lock(g_status_mutex);
    const unsigned long long bit = 1ULL << dev;
    if (*mask & bit) return false;
    *mask |= bit;
    return true;
}

// A few recently built tensor maps, so that a loop of launches on the same buffers does not encode the same
// descriptor again and again (the encoding is a driver call of a microsecond or two).
struct MapSlot {
    MapKey key;
    CUtensorMap map;
    bool used;
};
static MapSlot g_maps[16];
static int g_map_next = 0;

bool tensor_map_cache_get(const MapKey &key, CUtensorMap *out)
{
    std::lock_guard<std::mutex> lock(g_status_mutex);
    for (const MapSlot &s : g_maps)
        if (s.used && s.key.ptr == key.ptr && s.key.kind == key.kind && s.key.dev == key.dev && s.key.d[0] == key.d[0] &&
            s.key.d[1] == key.d[1] && s.key.d[2] == key.d[2] && s.key.d[3] == key.d[3]) {
            *out = s.map;
            return true;
        }
    return false;
}

void tensor_map_cache_put(const MapKey &key, const CUtensorMap &map)
{
    std::lock_guard<std::mutex> lock(g_status_mutex);
    MapSlot &s = g_maps[g_map_next];
    g_map_next = (g_map_next + 1) % 16;
    s.key = key;
    s.map = map;
    s.used = true;
}

__global__ void propagate_flag_k(const int *flag, int *status)
{
    if (*flag) *status = 1;
}

// Copies a set workspace flag into the status word (one thread), for entry points whose callers
// normally never look into the workspace.
int launch_propagate_flag(const int *flag, cudaStream_t st)
{
    int *status = device_status_ptr();
    if (!status || !flag) return GN_OK;
    propagate_flag_k<<<1, 1, 0, st>>>(flag, status);
    return check_launch("propagate_flag");
}

}  // namespace gn

using namespace gn;

extern "C" {

GN_API int gn_device_status(int clear)
{
    int *p = device_status_ptr();
    if (!p) return GN_ERR_CUDA;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && clear && v != 0) e = cudaMemset(p, 0, sizeof(int));
    if (e != cudaSuccess) {
        record_cuda_error(e, "gn_device_status");
        return GN_ERR_CUDA;
    }
    return v != 0 ? 1 : 0;
}

GN_API int gn_device_status_set(int value)
{
    int *p = device_status_ptr();
    if (!p) return GN_ERR_CUDA;
    const int v = value ? 1 : 0;
    const cudaError_t e = cudaMemcpy(p, &v, sizeof(int), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        record_cuda_error(e, "gn_device_status_set");
        return GN_ERR_CUDA;
    }
    return GN_OK;
}

}  // extern "C"
