// Device/runtime helpers of the acro:: API that survive from util/CudaUtil.hpp
// of LLNL/acrotensor: isCudaReady() (:175-184), setCudaContext() (:93-98) and
// the error-check convention (:59-89).  The NVRTC machinery (CudaKernel) has
// no counterpart here: kernels are compiled ahead of time for sm_100a.
#ifndef ACRO_B200_CUDA_UTIL_HPP
#define ACRO_B200_CUDA_UTIL_HPP

#include <string>
#include "Error.hpp"

// User code built with -DACRO_HAVE_CUDA gets the driver and runtime declarations through this
// header, as it does from util/CudaUtil.hpp:17-21 (it may call cudaMalloc or cuCtxCreate itself).
// Without the macro no CUDA header is needed to use the library.
#ifdef ACRO_HAVE_CUDA
#include <cuda.h>
#include <cuda_runtime.h>
#endif

namespace acro
{

// True when a CUDA device can be used by this process.
bool isCudaReady();

// Adopt an externally created driver context (a CUcontext passed as void*)
// for the calling thread; later library calls run in it.
void setCudaContext(void *cuda_context);

// The stream the calling host thread's launches and copies are issued on (a
// cudaStream_t passed as void*; nullptr = the legacy default stream).  The setting is
// per thread: a second thread with its own stream can, for example, copy results
// back while the first one uploads the next inputs.
void setCudaStream(void *cuda_stream);
void *getCudaStream();

namespace detail
{
// Translates a CUDA runtime status (an int to keep CUDA headers out of user
// code) into the library's exception.
void cudaCheck(int status, const char *file, int line);
}

#define acroCudaErrorCheck(call) ::acro::detail::cudaCheck(static_cast<int>(call), __FILE__, __LINE__)

}

#endif
