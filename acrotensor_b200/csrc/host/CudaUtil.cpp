// Device discovery, context/stream selection and the CUDA error convention.
#include "CudaUtil.hpp"

#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <iostream>

namespace acro
{

namespace
{
// Per host thread, so that one thread can copy results back on its own stream while
// another uploads the next inputs.
thread_local void *g_stream = nullptr;
}

bool isCudaReady()
{
    int count = 0;
    cudaError_t status = cudaGetDeviceCount(&count);
    if (status != cudaSuccess)
    {
        cudaGetLastError();   // a missing driver is an answer, not a sticky error
        return false;
    }
    return count > 0;
}

void setCudaContext(void *cuda_context)
{
    // The driver library is looked up at run time so that this library still loads on a
    // machine without a driver (where only the host-side planner can be used).
    typedef int (*set_current_fn)(void *);
    static set_current_fn set_current = nullptr;
    if (set_current == nullptr)
    {
        void *driver = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        ACROBATIC_ASSERT(driver != nullptr, "setCudaContext: the CUDA driver library is not available.");
        set_current = reinterpret_cast<set_current_fn>(dlsym(driver, "cuCtxSetCurrent"));
        ACROBATIC_ASSERT(set_current != nullptr, "setCudaContext: cuCtxSetCurrent not found in the CUDA driver library.");
    }
    int status = set_current(cuda_context);
    ACROBATIC_ASSERT(status == 0, "setCudaContext failed with driver status " + std::to_string(status));
}

void setCudaStream(void *cuda_stream) { g_stream = cuda_stream; }
void *getCudaStream() { return g_stream; }

namespace detail
{
void cudaCheck(int status, const char *file, int line)
{
    if (status == static_cast<int>(cudaSuccess)) return;
    std::string msg = std::string("CUDA error: ") + cudaGetErrorString(static_cast<cudaError_t>(status));
    std::cerr << file << ":" << line << "  " << msg << std::endl;
    throw_error(located(file, line, msg));
}
}

}
