// Shared plumbing of the kernel layer: status reporting and launch checks.
#ifndef ACRO_B200_KERNELS_COMMON_CUH
#define ACRO_B200_KERNELS_COMMON_CUH

#include <cuda_runtime.h>
#include <cstdint>
#include <string>

#include "acro_b200.h"

namespace acro_b200_detail
{

void set_last_error(const std::string &text);

int fail_invalid(const std::string &text);
int fail_unsupported(const std::string &text);
int fail_cuda(cudaError_t status, const char *where);

// Number of SMs of the current device (cached per device).
int sm_count();

// Device address of the per-device flag a kernel raises when one of its bounded waits gave
// up (nullptr on failure); acro_b200_device_status() reads and clears it.
int *wait_flag_device_ptr();

// Number of acro_b200_set_context calls so far.  The address of a __device__ symbol belongs to one CUDA
// context, so code that caches such an address stores this value with it and looks the address up
// again when the value has moved on.
unsigned long long context_epoch();

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

// To be called right after a kernel launch.
inline int launch_status(const char *where)
{
    cudaError_t status = cudaGetLastError();
    return status == cudaSuccess ? ACRO_B200_OK : fail_cuda(status, where);
}

// Streaming variant of batched_gemm for matrices up to 16 x 16 x 16 (batched_gemm_small.cu).
bool batched_gemm_small_supported(int m, int n, int k);
int batched_gemm_small_launch(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k, int trans_a, int trans_b, int op,
                              cudaStream_t stream);

// Element matrix times element vector (batched_matvec.cu): form 0  Y_i = sum_k M_ik X_k, form 1  Y_j = sum_k X_k M_kj.
bool batched_matvec_supported(int rows, int cols);
int batched_matvec_launch(const double *M, const double *X, double *Y, int64_t batch, int rows, int cols, int form, int op, cudaStream_t stream);

// Streaming variant of the Gram form for a, b <= 16 (gram_stream.cu): one a x b tile of partial sums per CTA at
// partials, *parts = number of tiles written (at most max_parts).
bool gram_stream_supported(int a, int b);
int gram_stream_launch(const double *X, const double *Y, double *partials, int64_t rows, int a, int b, int max_parts, int *parts, cudaStream_t stream);

// Pairs of elements by bulk copy for matrices of 17 .. 32 with rows of an odd length (batched_gemm_pairs.cu); the Gram form
// over pairs of row slabs writes 2 * grid partial tiles (*parts) at partials.
bool batched_gemm_pairs_supported(int m, int n, int k, int trans_a, int trans_b);
int batched_gemm_pairs_launch(const double *A, const double *B, double *C, int64_t pairs, int m, int n, int k, int trans_a, int trans_b, int op,
                              cudaStream_t stream);
int gram_pairs_launch(const double *X, const double *Y, double *partials, int64_t pairs, int slab_rows, int a, int b, int max_parts, int *parts,
                      cudaStream_t stream);

__host__ __device__ inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}

#endif
