// Device discovery, context/stream selection and the CUDA error convention.
#include "CudaUtil.hpp"
#include "acro_b200.h"

#include <cuda_runtime_api.h>
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
    if (acro_b200_set_context(cuda_context) != ACRO_B200_OK) throw_error(std::string("setCudaContext: ") + acro_b200_last_error());
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
