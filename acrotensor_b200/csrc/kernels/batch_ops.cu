// Non-contraction batched operations that sit either side of the contraction path:
//   batch_inv_det  inverse and/or determinant of a batch of 1x1, 2x2 or 3x3 matrices
//   flat_scatter   Aout[i] = Ain[M[i]]
//   flat_sum_gather  Aout[d] = sum of Ain[k] over the positions k with M[k] = d
//
// The arithmetic repeats the reference's CPU formulas operation by operation, without
// fused multiply-add (ops/NativeCPUOps.hpp:38-86, ops/NativeCPUOps.cpp:11-144 of
// LLNL/acrotensor), so results are bit-identical to its CPU path.  Note that the
// reference's 3x3 "inverse" stores entry (r,c) of the true inverse at position (c,r);
// this library keeps that layout because user kernels are written against it.
//
// batch_inv_det streams 8*d*d bytes in and 8*d*d (+8) bytes out per matrix: tiles of 256
// matrices travel as contiguous spans through a ring of asynchronous bulk copies, one
// thread inverts one matrix in place in shared memory, and the tile leaves as one bulk
// store; determinants go straight to global memory (one coalesced 8-byte store per thread).
#include "common.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kTile = 256;

template <int DIM>
__device__ __forceinline__ double det_of(const double *a)
{
    if (DIM == 1) return a[0];
    if (DIM == 2) return __dsub_rn(__dmul_rn(a[0], a[3]), __dmul_rn(a[1], a[2]));
    // a0*a4*a8 + a1*a5*a6 + a2*a3*a7 - a6*a4*a2 - a7*a5*a0 - a8*a3*a1, evaluated left to right
    double d = __dmul_rn(__dmul_rn(a[0], a[4]), a[8]);
    d = __dadd_rn(d, __dmul_rn(__dmul_rn(a[1], a[5]), a[6]));
    d = __dadd_rn(d, __dmul_rn(__dmul_rn(a[2], a[3]), a[7]));
    d = __dsub_rn(d, __dmul_rn(__dmul_rn(a[6], a[4]), a[2]));
    d = __dsub_rn(d, __dmul_rn(__dmul_rn(a[7], a[5]), a[0]));
    d = __dsub_rn(d, __dmul_rn(__dmul_rn(a[8], a[3]), a[1]));
    return d;
}

__device__ __forceinline__ double cof(double invdet, double p, double q, double r, double s)
{
    return __dmul_rn(invdet, __dsub_rn(__dmul_rn(p, q), __dmul_rn(r, s)));
}

template <int DIM>
__device__ __forceinline__ void inverse_of(const double *a, double det, double *inv)
{
    const double invdet = __ddiv_rn(1.0, det);
    if (DIM == 1) inv[0] = invdet;
    else if (DIM == 2)
    {
        inv[0] = __dmul_rn(invdet, a[3]);
        inv[1] = __dmul_rn(-invdet, a[1]);
        inv[2] = __dmul_rn(-invdet, a[2]);
        inv[3] = __dmul_rn(invdet, a[0]);
    }
    else
    {
        inv[0] = cof(invdet, a[4], a[8], a[5], a[7]);
        inv[1] = cof(invdet, a[5], a[6], a[3], a[8]);
        inv[2] = cof(invdet, a[3], a[7], a[4], a[6]);
        inv[3] = cof(invdet, a[2], a[7], a[1], a[8]);
        inv[4] = cof(invdet, a[0], a[8], a[2], a[6]);
        inv[5] = cof(invdet, a[1], a[6], a[0], a[7]);
        inv[6] = cof(invdet, a[1], a[5], a[2], a[4]);
        inv[7] = cof(invdet, a[2], a[3], a[0], a[5]);
        inv[8] = cof(invdet, a[0], a[4], a[1], a[3]);
    }
}

struct InvDetArgs
{
    const double *A;
    double *Ainv;   // may be null (determinant only); may alias A
    double *Adet;   // may be null (inverse only)
    int64_t count;
    int *wait_flag;
};

// Plain kernel: any alignment, any count; also serves the ragged tail of the pipelined one.
template <int DIM>
__global__ void __launch_bounds__(kTile)
inv_det_kernel(const InvDetArgs a, int64_t first)
{
    constexpr int BLK = DIM * DIM;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kTile;
    for (int64_t m = first + static_cast<int64_t>(blockIdx.x) * kTile + threadIdx.x; m < a.count; m += stride)
    {
        double x[BLK], inv[BLK];
#pragma unroll
        for (int i = 0; i < BLK; ++i) x[i] = a.A[m * BLK + i];
        const double det = det_of<DIM>(x);
        if (a.Adet != nullptr) a.Adet[m] = det;
        if (a.Ainv != nullptr)
        {
            inverse_of<DIM>(x, det, inv);
#pragma unroll
            for (int i = 0; i < BLK; ++i) a.Ainv[m * BLK + i] = inv[i];
        }
    }
}

// Pipelined kernel for whole tiles of 16-byte aligned operands.
template <int DIM, int STAGES>
__global__ void __launch_bounds__(kTile)
inv_det_pipe_kernel(const InvDetArgs a)
{
    constexpr int BLK = DIM * DIM;
    constexpr int TILE = kTile * BLK;
    constexpr uint32_t TILE_BYTES = TILE * 8;
    extern __shared__ __align__(128) double smem[];
    __shared__ uint64_t full[STAGES];
    const int tid = threadIdx.x;
    const int64_t n_full = a.count / kTile;
    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1);
        fence_mbar_init();
    }
    __syncthreads();
    auto load_tile = [&](int64_t tile, int st) {
        mbar_arrive_expect_tx(&full[st], TILE_BYTES);
        bulk_load(smem + st * TILE, a.A + tile * TILE, TILE_BYTES, &full[st]);
    };
    if (tid == 0)
    {
        for (int j = 0; j < STAGES - 1; ++j)
        {
            const int64_t tile = blockIdx.x + static_cast<int64_t>(j) * gridDim.x;
            if (tile < n_full) load_tile(tile, j);
        }
    }
    int64_t i = 0;
    for (int64_t tile = blockIdx.x; tile < n_full; tile += gridDim.x, ++i)
    {
        const int st = static_cast<int>(i % STAGES);
        if (!mbar_wait(&full[st], static_cast<uint32_t>((i / STAGES) & 1))) atomicExch(a.wait_flag, 1);
        double *p = smem + st * TILE + tid * BLK;
        double x[BLK], inv[BLK];
#pragma unroll
        for (int k = 0; k < BLK; ++k) x[k] = p[k];
        const double det = det_of<DIM>(x);
        if (a.Adet != nullptr) __stcs(a.Adet + tile * kTile + tid, det);
        if (a.Ainv != nullptr)
        {
            inverse_of<DIM>(x, det, inv);
#pragma unroll
            for (int k = 0; k < BLK; ++k) p[k] = inv[k];
            fence_proxy_async();
        }
        __syncthreads();
        if (tid == 0)
        {
            if (a.Ainv != nullptr)
            {
                bulk_store(a.Ainv + tile * TILE, smem + st * TILE, TILE_BYTES);
                bulk_commit();
            }
            const int64_t next = tile + static_cast<int64_t>(STAGES - 1) * gridDim.x;
            if (next < n_full)
            {
                if (a.Ainv != nullptr) bulk_wait_read<1>();
                load_tile(next, static_cast<int>((i + STAGES - 1) % STAGES));
            }
        }
    }
    if (tid == 0) bulk_wait_all<0>();
}

template <int DIM>
int launch_inv_det(const InvDetArgs &args, cudaStream_t s)
{
    constexpr int BLK = DIM * DIM;
    constexpr int STAGES = 4;
    int64_t done = 0;
    const bool in_place = args.Ainv == args.A;
    // In place, a tile's store could still be draining while the same span is loaded again
    // only if tiles overlapped, which they do not; aliasing is therefore safe in the ring.
    (void)in_place;
    if (args.count >= kTile && aligned16(args.A) && (args.Ainv == nullptr || aligned16(args.Ainv)))
    {
        const size_t smem = static_cast<size_t>(STAGES) * kTile * BLK * sizeof(double);
        auto kernel = inv_det_pipe_kernel<DIM, STAGES>;
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batch_inv_det (shared memory opt-in)");
        const int64_t n_full = args.count / kTile;
        int64_t grid = static_cast<int64_t>(sm_count()) * 3;
        if (grid > n_full) grid = n_full;
        kernel<<<static_cast<int>(grid), kTile, smem, s>>>(args);
        const int rc = launch_status("acro_b200_batch_inv_det (pipelined)");
        if (rc != ACRO_B200_OK) return rc;
        done = n_full * kTile;
    }
    if (done < args.count)
    {
        const int64_t left = args.count - done;
        int64_t grid = (left + kTile - 1) / kTile;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
        if (grid > cap) grid = cap;
        inv_det_kernel<DIM><<<static_cast<int>(grid), kTile, 0, s>>>(args, done);
        return launch_status("acro_b200_batch_inv_det");
    }
    return ACRO_B200_OK;
}

__global__ void flat_scatter_kernel(double *__restrict__ out, const double *__restrict__ in, const int *__restrict__ map, int64_t n)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = in[map[i]];
}

__global__ void flat_sum_gather_kernel(double *__restrict__ out, const double *__restrict__ in, const int *__restrict__ inv_map,
                                       const int *__restrict__ offsets, int64_t domain)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t d = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; d < domain; d += stride)
    {
        // ascending position: the reference's order.  Four positions at a time: their indices, then their values, are
        // fetched together (the kernel is bound by the latency of these dependent loads), the additions stay in order.
        double sum = 0.0;
        int k = offsets[d];
        const int end = offsets[d + 1];
        for (; k + 4 <= end; k += 4)
        {
            const int i0 = inv_map[k], i1 = inv_map[k + 1], i2 = inv_map[k + 2], i3 = inv_map[k + 3];
            const double v0 = in[i0], v1 = in[i1], v2 = in[i2], v3 = in[i3];
            sum = __dadd_rn(__dadd_rn(__dadd_rn(__dadd_rn(sum, v0), v1), v2), v3);
        }
        for (; k < end; ++k) sum = __dadd_rn(sum, in[inv_map[k]]);
        out[d] = sum;
    }
}

int grid_for(int64_t n)
{
    int64_t blocks = (n + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count() > 0 ? sm_count() : 1) * 16;
    if (blocks > cap) blocks = cap;
    return static_cast<int>(blocks > 0 ? blocks : 1);
}

}

extern "C" {

int acro_b200_batch_inv_det(const double *A, double *Ainv, double *Adet, int64_t count, int dim, void *stream)
{
    if (A == nullptr || (Ainv == nullptr && Adet == nullptr)) return fail_invalid("acro_b200_batch_inv_det: null argument");
    if (count < 1) return fail_invalid("acro_b200_batch_inv_det: matrix count must be positive");
    if (dim < 1 || dim > 3) return fail_unsupported("acro_b200_batch_inv_det: matrix dimension must be 1, 2 or 3");
    if (sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_batch_inv_det");
    InvDetArgs args;
    args.A = A;
    args.Ainv = Ainv;
    args.Adet = Adet;
    args.count = count;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_batch_inv_det (status flag)");
    cudaStream_t s = as_stream(stream);
    switch (dim)
    {
        case 1: return launch_inv_det<1>(args, s);
        case 2: return launch_inv_det<2>(args, s);
        default: return launch_inv_det<3>(args, s);
    }
}

int acro_b200_flat_scatter(double *Aout, const double *Ain, const int *map, int64_t range_size, void *stream)
{
    if (Aout == nullptr || Ain == nullptr || map == nullptr || range_size < 1) return fail_invalid("acro_b200_flat_scatter: bad arguments");
    if (sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_flat_scatter");
    flat_scatter_kernel<<<grid_for(range_size), 256, 0, as_stream(stream)>>>(Aout, Ain, map, range_size);
    return launch_status("acro_b200_flat_scatter");
}

int acro_b200_flat_sum_gather(double *Aout, const double *Ain, const int *inv_map, const int *inv_offsets, int64_t domain_size, void *stream)
{
    if (Aout == nullptr || Ain == nullptr || inv_map == nullptr || inv_offsets == nullptr || domain_size < 1)
        return fail_invalid("acro_b200_flat_sum_gather: bad arguments");
    if (sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_flat_sum_gather");
    flat_sum_gather_kernel<<<grid_for(domain_size), 256, 0, as_stream(stream)>>>(Aout, Ain, inv_map, inv_offsets, domain_size);
    return launch_status("acro_b200_flat_sum_gather");
}

}
