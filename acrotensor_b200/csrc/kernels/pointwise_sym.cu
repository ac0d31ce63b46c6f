// pointwise_sym: D[p,m,n] (op)= s[p] * sum_l X[p,m,l] * Y[p,n,l], s[p] = product of point-wise factors.
//
// A CTA owns tiles of kTile consecutive points.  The X (and Y) blocks of a tile are one
// contiguous span of kTile*DIM*DIM doubles: it is copied to shared memory with coalesced
// 16-byte loads, each thread then computes the DIM x DIM block of its own point out of
// shared memory (odd strides: no bank conflicts), writes it back into the same shared
// slots, and the tile leaves as one contiguous coalesced store.  Arithmetic follows the
// reference's order term by term — ((s*X)*Y), added one by one, no fused multiply-add —
// so "=" results are bit-identical to its CPU executor.
//
// Algorithmic HBM traffic per point: 8*DIM*DIM (X) [+ 8*DIM*DIM (Y != X)] + 8*DIM*DIM (D)
// + 8 bytes per point-wise factor that varies with every point.
#include "common.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kTile = 256;   // points per tile = threads per CTA

struct PointwiseArgs
{
    acro_b200_pointwise_desc d;
    const double *scalar[ACRO_B200_MAX_SCALARS];
    const double *X;
    const double *Y;
    double *D;
    int64_t points;        // points this launch covers
    int64_t first_point;   // global number of its first point (X, Y, D already point at it)
    int *wait_flag;
};

__device__ inline void copy_in(double *dst, const double *src, int count, bool vec)
{
    if (vec)
    {
        const double2 *s2 = reinterpret_cast<const double2 *>(src);
        double2 *d2 = reinterpret_cast<double2 *>(dst);
        for (int i = threadIdx.x; i < count / 2; i += kTile) d2[i] = __ldcs(s2 + i);
        if ((count & 1) && threadIdx.x == 0) dst[count - 1] = src[count - 1];
    }
    else
    {
        for (int i = threadIdx.x; i < count; i += kTile) dst[i] = __ldcs(src + i);
    }
}

template <int DIM, bool SAME_XY>
__global__ void __launch_bounds__(kTile)
pointwise_sym_kernel(const __grid_constant__ PointwiseArgs a)
{
    constexpr int BLK = DIM * DIM;
    extern __shared__ __align__(128) double smem[];
    double *sx = smem;
    double *sy = SAME_XY ? smem : smem + kTile * BLK;

    const int64_t tiles = (a.points + kTile - 1) / kTile;
    const bool vec_x = aligned16(a.X), vec_y = aligned16(a.Y), vec_d = aligned16(a.D);

    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x)
    {
        const int64_t p0 = tile * kTile;
        const int64_t left = a.points - p0;
        const int n_pts = left < kTile ? static_cast<int>(left) : kTile;
        const int count = n_pts * BLK;
        // kTile*BLK is even, so every tile starts on a 16-byte boundary when the base does.
        copy_in(sx, a.X + p0 * BLK, count, vec_x);
        if (!SAME_XY) copy_in(sy, a.Y + p0 * BLK, count, vec_y);
        __syncthreads();

        if (threadIdx.x < n_pts)
        {
            const int64_t p = p0 + threadIdx.x;
            // Point-wise factors, multiplied left to right.
            double s = 1.0;
            if (a.d.n_scalars > 0)
            {
                int64_t idx[ACRO_B200_MAX_POINT_LOOPS];
                int64_t rest = a.first_point + p;
#pragma unroll
                for (int j = ACRO_B200_MAX_POINT_LOOPS - 1; j >= 0; --j)
                {
                    if (j < a.d.n_point_loops)
                    {
                        idx[j] = rest % a.d.point_extent[j];
                        rest /= a.d.point_extent[j];
                    }
                    else idx[j] = 0;
                }
#pragma unroll
                for (int i = 0; i < ACRO_B200_MAX_SCALARS; ++i)
                {
                    if (i < a.d.n_scalars)
                    {
                        int64_t off = 0;
#pragma unroll
                        for (int j = 0; j < ACRO_B200_MAX_POINT_LOOPS; ++j) off += idx[j] * a.d.scalar_step[i][j];
                        const double f = __ldg(a.scalar[i] + off);
                        s = (i == 0) ? f : __dmul_rn(s, f);
                    }
                }
            }
            double x[BLK], y[BLK];
#pragma unroll
            for (int i = 0; i < BLK; ++i)
            {
                x[i] = sx[threadIdx.x * BLK + i];
                y[i] = SAME_XY ? x[i] : sy[threadIdx.x * BLK + i];
            }
#pragma unroll
            for (int m = 0; m < DIM; ++m)
            {
                // With at least one factor the reference's product starts (s*X); without, it is X*Y.
                double sxm[DIM];
#pragma unroll
                for (int l = 0; l < DIM; ++l) sxm[l] = (a.d.n_scalars > 0) ? __dmul_rn(s, x[m * DIM + l]) : x[m * DIM + l];
#pragma unroll
                for (int n = 0; n < DIM; ++n)
                {
                    double acc = (a.d.op == ACRO_B200_OP_ADD) ? a.D[p * BLK + m * DIM + n] : 0.0;
#pragma unroll
                    for (int l = 0; l < DIM; ++l) acc = __dadd_rn(acc, __dmul_rn(sxm[l], y[n * DIM + l]));
                    if (a.d.op == ACRO_B200_OP_SUB) acc = __dsub_rn(a.D[p * BLK + m * DIM + n], acc);
                    sx[threadIdx.x * BLK + m * DIM + n] = acc;   // own slots only: no hazard with other threads
                }
            }
        }
        __syncthreads();

        double *dst = a.D + p0 * BLK;
        if (vec_d)
        {
            const double2 *s2 = reinterpret_cast<const double2 *>(sx);
            double2 *d2 = reinterpret_cast<double2 *>(dst);
            for (int i = threadIdx.x; i < count / 2; i += kTile) __stcs(d2 + i, s2[i]);
            if ((count & 1) && threadIdx.x == 0) dst[count - 1] = sx[count - 1];
        }
        else
        {
            for (int i = threadIdx.x; i < count; i += kTile) __stcs(dst + i, sx[i]);
        }
        __syncthreads();
    }
}


// Point-wise factor product s[p] for global point number gp (left to right, as the reference).
__device__ __forceinline__ double scalar_product(const PointwiseArgs &a, int64_t gp)
{
    double s = 1.0;
    int64_t idx[ACRO_B200_MAX_POINT_LOOPS];
    int64_t rest = gp;
#pragma unroll
    for (int j = ACRO_B200_MAX_POINT_LOOPS - 1; j >= 0; --j)
    {
        if (j < a.d.n_point_loops)
        {
            idx[j] = rest % a.d.point_extent[j];
            rest /= a.d.point_extent[j];
        }
        else idx[j] = 0;
    }
#pragma unroll
    for (int i = 0; i < ACRO_B200_MAX_SCALARS; ++i)
    {
        if (i < a.d.n_scalars)
        {
            int64_t off = 0;
#pragma unroll
            for (int j = 0; j < ACRO_B200_MAX_POINT_LOOPS; ++j) off += idx[j] * a.d.scalar_step[i][j];
            const double f = __ldg(a.scalar[i] + off);
            s = (i == 0) ? f : __dmul_rn(s, f);
        }
    }
    return s;
}

// Pipelined variant for "=": whole tiles travel by asynchronous bulk copies through a ring of
// shared-memory buffers.  While the threads compute tile i in place, the loads of the next
// tiles are in flight and the store of tile i-1 drains; one CTA barrier per tile.
template <int DIM, bool SAME_XY, int STAGES>
__global__ void __launch_bounds__(kTile)
pointwise_sym_pipe_kernel(const __grid_constant__ PointwiseArgs a)
{
    constexpr int BLK = DIM * DIM;
    constexpr int TILE = kTile * BLK;                 // doubles per tile buffer
    constexpr uint32_t TILE_BYTES = TILE * 8;
    extern __shared__ __align__(128) double smem[];
    double *bx = smem;                                 // [STAGES][TILE]
    double *by = smem + (SAME_XY ? 0 : STAGES * TILE);
    __shared__ uint64_t full[STAGES];

    const int64_t n_full = a.points / kTile;           // the ragged tail is a separate launch
    const int tid = threadIdx.x;
    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1);
        fence_mbar_init();
    }
    __syncthreads();

    auto load_tile = [&](int64_t tile, int st) {
        mbar_arrive_expect_tx(&full[st], SAME_XY ? TILE_BYTES : 2 * TILE_BYTES);
        bulk_load(bx + st * TILE, a.X + tile * TILE, TILE_BYTES, &full[st]);
        if (!SAME_XY) bulk_load(by + st * TILE, a.Y + tile * TILE, TILE_BYTES, &full[st]);
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
        // the point-wise factors come straight from global memory: fetch them before waiting
        const double s = a.d.n_scalars > 0 ? scalar_product(a, a.first_point + tile * kTile + tid) : 1.0;
        if (!mbar_wait(&full[st], static_cast<uint32_t>((i / STAGES) & 1))) atomicExch(a.wait_flag, 1);

        double *px = bx + st * TILE + tid * BLK;
        const double *py = by + st * TILE + tid * BLK;
        double x[BLK], y[BLK];
#pragma unroll
        for (int k = 0; k < BLK; ++k)
        {
            x[k] = px[k];
            y[k] = SAME_XY ? x[k] : py[k];
        }
#pragma unroll
        for (int m = 0; m < DIM; ++m)
        {
            double sxm[DIM];
#pragma unroll
            for (int l = 0; l < DIM; ++l) sxm[l] = (a.d.n_scalars > 0) ? __dmul_rn(s, x[m * DIM + l]) : x[m * DIM + l];
#pragma unroll
            for (int n = 0; n < DIM; ++n)
            {
                double acc = 0.0;
#pragma unroll
                for (int l = 0; l < DIM; ++l) acc = __dadd_rn(acc, __dmul_rn(sxm[l], y[n * DIM + l]));
                px[m * DIM + n] = acc;
            }
        }
        fence_proxy_async();     // the results must be visible to the bulk store
        __syncthreads();
        if (tid == 0)
        {
            bulk_store(a.D + tile * TILE, bx + st * TILE, TILE_BYTES);
            bulk_commit();
            // Refill the buffer tile i-1 used: its store is the second youngest group.
            const int64_t next = tile + static_cast<int64_t>(STAGES - 1) * gridDim.x;
            if (next < n_full)
            {
                bulk_wait_read<1>();
                load_tile(next, static_cast<int>((i + STAGES - 1) % STAGES));
            }
        }
    }
    if (tid == 0) bulk_wait_all<0>();   // shared memory must outlive the stores that read it
}

template <int DIM, bool SAME_XY, int STAGES>
int launch_pipe(const PointwiseArgs &args, cudaStream_t s, int ctas_per_sm)
{
    constexpr int BLK = DIM * DIM;
    const size_t smem = static_cast<size_t>(STAGES) * kTile * BLK * sizeof(double) * (SAME_XY ? 1 : 2);
    auto kernel = pointwise_sym_pipe_kernel<DIM, SAME_XY, STAGES>;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_pointwise_sym (shared memory opt-in)");
    const int64_t n_full = args.points / kTile;
    int64_t grid = static_cast<int64_t>(sm_count()) * ctas_per_sm;
    if (grid > n_full) grid = n_full;
    kernel<<<static_cast<int>(grid), kTile, smem, s>>>(args);
    return launch_status("acro_b200_pointwise_sym (pipelined)");
}

template <int DIM>
int launch(const PointwiseArgs &args_in, cudaStream_t s)
{
    PointwiseArgs args = args_in;
    // "=" on 16-byte aligned operands: whole tiles through the bulk-copy pipeline, then the
    // ragged tail (if any) through the plain kernel below.
    if (args.d.op == ACRO_B200_OP_ASSIGN && args.points >= kTile && aligned16(args.X) && aligned16(args.Y) && aligned16(args.D))
    {
        const bool same_xy = args.X == args.Y;
        int rc;
        if (DIM == 3) rc = same_xy ? launch_pipe<DIM, true, 4>(args, s, 3) : launch_pipe<DIM, false, 3>(args, s, 2);
        else rc = same_xy ? launch_pipe<DIM, true, 4>(args, s, 4) : launch_pipe<DIM, false, 4>(args, s, 4);
        if (rc != ACRO_B200_OK) return rc;
        const int64_t done = (args.points / kTile) * kTile;
        if (done == args.points) return ACRO_B200_OK;
        constexpr int BLK2 = DIM * DIM;
        args.X += done * BLK2;
        args.Y += done * BLK2;
        args.D += done * BLK2;
        args.first_point += done;
        args.points -= done;
    }
    constexpr int BLK = DIM * DIM;
    const bool same = args.X == args.Y;
    const size_t smem = static_cast<size_t>(kTile) * BLK * sizeof(double) * (same ? 1 : 2);
    const int64_t tiles = (args.points + kTile - 1) / kTile;
    int64_t grid = static_cast<int64_t>(sm_count()) * 8;
    if (grid > tiles) grid = tiles;
    if (same) pointwise_sym_kernel<DIM, true><<<static_cast<int>(grid), kTile, smem, s>>>(args);
    else pointwise_sym_kernel<DIM, false><<<static_cast<int>(grid), kTile, smem, s>>>(args);
    return launch_status("acro_b200_pointwise_sym");
}

}

extern "C" {

int acro_b200_pointwise_sym_supported(const acro_b200_pointwise_desc *d)
{
    if (d == nullptr) return 0;
    if (d->dim < 1 || d->dim > 3) return 0;
    if (d->n_point_loops < 1 || d->n_point_loops > ACRO_B200_MAX_POINT_LOOPS) return 0;
    if (d->n_scalars < 0 || d->n_scalars > ACRO_B200_MAX_SCALARS) return 0;
    if (d->op < 0 || d->op > 2) return 0;
    for (int j = 0; j < d->n_point_loops; ++j)
    {
        if (d->point_extent[j] < 1) return 0;
    }
    return 1;
}

int acro_b200_pointwise_sym(const acro_b200_pointwise_desc *desc, const double *const *scalars, const double *X,
                            const double *Y, double *D, void *stream)
{
    if (desc == nullptr || X == nullptr || Y == nullptr || D == nullptr) return fail_invalid("acro_b200_pointwise_sym: null argument");
    if (!acro_b200_pointwise_sym_supported(desc)) return fail_unsupported("acro_b200_pointwise_sym: unsupported descriptor");
    if (sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_pointwise_sym");
    PointwiseArgs args;
    args.d = *desc;
    args.X = X;
    args.Y = Y;
    args.D = D;
    args.points = 1;
    for (int j = 0; j < desc->n_point_loops; ++j) args.points *= desc->point_extent[j];
    args.first_point = 0;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_pointwise_sym (status flag)");
    for (int i = 0; i < ACRO_B200_MAX_SCALARS; ++i)
    {
        args.scalar[i] = nullptr;
        if (i < desc->n_scalars)
        {
            if (scalars == nullptr || scalars[i] == nullptr) return fail_invalid("acro_b200_pointwise_sym: null scalar factor");
            args.scalar[i] = scalars[i];
        }
    }
    cudaStream_t s = as_stream(stream);
    switch (desc->dim)
    {
        case 1: return launch<1>(args, s);
        case 2: return launch<2>(args, s);
        default: return launch<3>(args, s);
    }
}

}
