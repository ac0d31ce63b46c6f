// Status plumbing, device discovery, fill and scale.
#include "common.cuh"
#include "tma.cuh"

#include <atomic>
#include <dlfcn.h>
#include <mutex>
#include <string>
#include <vector>

namespace acro_b200_detail
{

static thread_local std::string g_last_error;

void set_last_error(const std::string &text) { g_last_error = text; }

int fail_invalid(const std::string &text)
{
    set_last_error(text);
    return ACRO_B200_EINVAL;
}

int fail_unsupported(const std::string &text)
{
    set_last_error(text);
    return ACRO_B200_EUNSUPPORTED;
}

int fail_cuda(cudaError_t status, const char *where)
{
    set_last_error(std::string("CUDA error in ") + where + ": " + cudaGetErrorString(status));
    return ACRO_B200_ECUDA;
}

int sm_count()
{
    static std::mutex lock;
    static std::vector<int> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    std::lock_guard<std::mutex> guard(lock);
    if (static_cast<int>(cache.size()) <= dev) cache.resize(dev + 1, 0);
    if (cache[dev] == 0)
    {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 0;
        cache[dev] = n;
    }
    return cache[dev];
}

}

static __device__ int g_wait_timed_out = 0;

namespace
{
// Address of g_wait_timed_out on each device.  A device symbol has one address per CUDA context, so
// acro_b200_set_context clears the table.
constexpr int kMaxDevices = 64;
std::mutex g_wait_flag_lock;
int *g_wait_flag_of_device[kMaxDevices] = {nullptr};
std::atomic<unsigned long long> g_context_epoch{0};
}

namespace acro_b200_detail
{
unsigned long long context_epoch() { return g_context_epoch.load(); }

int *wait_flag_device_ptr()
{
    std::mutex &lock = g_wait_flag_lock;
    int **ptr_of_device = g_wait_flag_of_device;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> guard(lock);
    if (ptr_of_device[dev] == nullptr)
    {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_wait_timed_out) != cudaSuccess) return nullptr;
        ptr_of_device[dev] = static_cast<int *>(p);
    }
    return ptr_of_device[dev];
}
}

using namespace acro_b200_detail;

namespace
{

__global__ void fill_kernel(double *__restrict__ data, int64_t n, double val)
{
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) data[i] = val;
}

__global__ void scale_kernel(double *__restrict__ data, int64_t n, double c)
{
    int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) data[i] *= c;
}

int elementwise_grid(int64_t n)
{
    int64_t blocks = (n + 255) / 256;
    int64_t cap = static_cast<int64_t>(sm_count() > 0 ? sm_count() : 1) * 16;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}

extern "C" {

const char *acro_b200_last_error(void) { return g_last_error.c_str(); }

int acro_b200_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess)
    {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int acro_b200_set_context(void *cuda_context)
{
    // The driver library is looked up at run time so that this library still loads on a
    // machine without a driver (where only the host-side planner can be used).
    typedef int (*set_current_fn)(void *);
    static set_current_fn set_current = nullptr;
    if (set_current == nullptr)
    {
        void *driver = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (driver == nullptr) return fail_cuda(cudaErrorNoDevice, "acro_b200_set_context (the CUDA driver library is not available)");
        set_current = reinterpret_cast<set_current_fn>(dlsym(driver, "cuCtxSetCurrent"));
        if (set_current == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_set_context (cuCtxSetCurrent not found in the driver library)");
    }
    const int status = set_current(cuda_context);
    if (status != 0)
    {
        set_last_error("acro_b200_set_context: cuCtxSetCurrent failed with driver status " + std::to_string(status));
        return ACRO_B200_ECUDA;
    }
    std::lock_guard<std::mutex> guard(g_wait_flag_lock);
    for (int d = 0; d < kMaxDevices; ++d) g_wait_flag_of_device[d] = nullptr;
    ++g_context_epoch;      // every other cached device-symbol address is stale too
    return ACRO_B200_OK;
}

int acro_b200_device_status(void)
{
    // Blocks until the device is idle, then reads (and clears) the bounded-wait flag.
    cudaError_t status = cudaDeviceSynchronize();
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_device_status");
    int flag = 0;
    status = cudaMemcpyFromSymbol(&flag, g_wait_timed_out, sizeof flag);
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_device_status");
    if (flag != 0)
    {
        const int zero = 0;
        cudaMemcpyToSymbol(g_wait_timed_out, &zero, sizeof zero);
        set_last_error("a bounded device-side wait on an asynchronous copy gave up; results of that launch are invalid");
        return ACRO_B200_ETIMEOUT;
    }
    return ACRO_B200_OK;
}

int acro_b200_fill(double *data, int64_t n, double val, void *stream)
{
    if (n < 0 || (n > 0 && data == nullptr)) return fail_invalid("acro_b200_fill: bad arguments");
    if (n == 0) return ACRO_B200_OK;
    fill_kernel<<<elementwise_grid(n), 256, 0, as_stream(stream)>>>(data, n, val);
    return launch_status("acro_b200_fill");
}

int acro_b200_scale(double *data, int64_t n, double c, void *stream)
{
    if (n < 0 || (n > 0 && data == nullptr)) return fail_invalid("acro_b200_scale: bad arguments");
    if (n == 0) return ACRO_B200_OK;
    scale_kernel<<<elementwise_grid(n), 256, 0, as_stream(stream)>>>(data, n, c);
    return launch_status("acro_b200_scale");
}

}
