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


// ------------------------------------------------------------------ cell-major output
// D[cell][m][n][k]: the K points of a cell come after the block indices.  Block (a,b) of a
// point, blk[a][b] = sum_l (s X[a][l]) Y[b][l], lands at (m,n) = (a,b), or (b,a) when the
// string lists the n-operand first.

// blk holds the starting values on entry (0, or the old output for "+=", whose terms the
// reference adds one by one onto the existing value) and the sums on return.
template <int DIM>
__device__ __forceinline__ void point_block(const PointwiseArgs &a, double s, const double *x, const double *y, double *blk)
{
#pragma unroll
    for (int p = 0; p < DIM; ++p)
    {
        double sx[DIM];
#pragma unroll
        for (int l = 0; l < DIM; ++l) sx[l] = (a.d.n_scalars > 0) ? __dmul_rn(s, x[p * DIM + l]) : x[p * DIM + l];
#pragma unroll
        for (int q = 0; q < DIM; ++q)
        {
            double acc = blk[p * DIM + q];
#pragma unroll
            for (int l = 0; l < DIM; ++l) acc = __dadd_rn(acc, __dmul_rn(sx[l], y[q * DIM + l]));
            blk[p * DIM + q] = acc;
        }
    }
}

// Direct kernel: one thread per point, operands straight from global memory.  Consecutive
// threads are consecutive points of a cell, so each of the dim*dim stores is coalesced.
// Serves "+=" / "-=", unaligned operands and the ragged tail of the pipelined kernel.
template <int DIM>
__global__ void __launch_bounds__(kTile)
pointwise_cell_direct_kernel(const __grid_constant__ PointwiseArgs a)
{
    constexpr int BLK = DIM * DIM;
    const int64_t K = a.d.cell_points;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kTile;
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * kTile + threadIdx.x; p < a.points; p += stride)
    {
        const int64_t gp = a.first_point + p;
        const double s = a.d.n_scalars > 0 ? scalar_product(a, gp) : 1.0;
        double x[BLK], y[BLK], blk[BLK];
#pragma unroll
        for (int i = 0; i < BLK; ++i)
        {
            x[i] = a.X[p * BLK + i];
            y[i] = a.Y[p * BLK + i];
        }
        double *cell = a.D + (p / K) * BLK * K + (p % K);
#pragma unroll
        for (int i = 0; i < BLK; ++i)
        {
            const int pos = a.d.swapped ? (i % DIM) * DIM + i / DIM : i;
            blk[i] = (a.d.op == ACRO_B200_OP_ADD) ? cell[pos * K] : 0.0;
        }
        point_block<DIM>(a, s, x, y, blk);
#pragma unroll
        for (int i = 0; i < BLK; ++i)
        {
            const int pos = a.d.swapped ? (i % DIM) * DIM + i / DIM : i;
            double *dst = cell + pos * K;
            if (a.d.op == ACRO_B200_OP_SUB) *dst = __dsub_rn(*dst, blk[i]);
            else *dst = blk[i];
        }
    }
}

// Pipelined kernel for "=": tiles of whole cells (tile_pts points, a multiple of K, at most
// kTile) through the same ring of bulk copies as the point-major kernel.  The result is
// written back into the tile buffer in cell-major order, which is not the thread's own slots,
// hence one more CTA barrier between reading the operands and writing the results.
template <int DIM, bool SAME_XY, int STAGES>
__global__ void __launch_bounds__(kTile)
pointwise_cell_pipe_kernel(const __grid_constant__ PointwiseArgs a, int tile_pts)
{
    constexpr int BLK = DIM * DIM;
    constexpr int SLOT = kTile * BLK;                    // doubles reserved per ring slot
    extern __shared__ __align__(128) double smem[];
    double *bx = smem;
    double *by = smem + (SAME_XY ? 0 : STAGES * SLOT);
    __shared__ uint64_t full[STAGES];

    const int tid = threadIdx.x;
    const int K = static_cast<int>(a.d.cell_points);
    const int tile_doubles = tile_pts * BLK;
    const uint32_t tile_bytes = static_cast<uint32_t>(tile_doubles) * 8u;
    const int64_t n_full = a.points / tile_pts;
    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1);
        fence_mbar_init();
    }
    __syncthreads();

    auto load_tile = [&](int64_t tile, int st) {
        mbar_arrive_expect_tx(&full[st], SAME_XY ? tile_bytes : 2 * tile_bytes);
        bulk_load(bx + st * SLOT, a.X + tile * tile_doubles, tile_bytes, &full[st]);
        if (!SAME_XY) bulk_load(by + st * SLOT, a.Y + tile * tile_doubles, tile_bytes, &full[st]);
    };
    if (tid == 0)
    {
        for (int j = 0; j < STAGES - 1; ++j)
        {
            const int64_t tile = blockIdx.x + static_cast<int64_t>(j) * gridDim.x;
            if (tile < n_full) load_tile(tile, j);
        }
    }

    const bool active = tid < tile_pts;
    const int cell = tid / K, k = tid % K;
    int64_t i = 0;
    for (int64_t tile = blockIdx.x; tile < n_full; tile += gridDim.x, ++i)
    {
        const int st = static_cast<int>(i % STAGES);
        const double s = (active && a.d.n_scalars > 0) ? scalar_product(a, a.first_point + tile * tile_pts + tid) : 1.0;
        if (!mbar_wait(&full[st], static_cast<uint32_t>((i / STAGES) & 1))) atomicExch(a.wait_flag, 1);

        double x[BLK], y[BLK], blk[BLK];
        if (active)
        {
#pragma unroll
            for (int j = 0; j < BLK; ++j)
            {
                x[j] = bx[st * SLOT + tid * BLK + j];
                y[j] = SAME_XY ? x[j] : by[st * SLOT + tid * BLK + j];
                blk[j] = 0.0;
            }
            point_block<DIM>(a, s, x, y, blk);
        }
        __syncthreads();         // every operand of the tile is in registers
        if (active)
        {
            double *out = bx + st * SLOT + cell * BLK * K + k;
#pragma unroll
            for (int j = 0; j < BLK; ++j)
            {
                const int pos = a.d.swapped ? (j % DIM) * DIM + j / DIM : j;
                out[pos * K] = blk[j];
            }
        }
        fence_proxy_async();
        __syncthreads();
        if (tid == 0)
        {
            bulk_store(a.D + tile * tile_doubles, bx + st * SLOT, tile_bytes);
            bulk_commit();
            const int64_t next = tile + static_cast<int64_t>(STAGES - 1) * gridDim.x;
            if (next < n_full)
            {
                bulk_wait_read<1>();
                load_tile(next, static_cast<int>((i + STAGES - 1) % STAGES));
            }
        }
    }
    if (tid == 0) bulk_wait_all<0>();
}

template <int DIM>
int launch_cell(const PointwiseArgs &args_in, cudaStream_t s)
{
    constexpr int BLK = DIM * DIM;
    PointwiseArgs args = args_in;
    const int64_t K = args.d.cell_points;
    const int tile_pts = K <= kTile ? static_cast<int>((kTile / K) * K) : 0;
    const bool pipe = args.d.op == ACRO_B200_OP_ASSIGN && tile_pts > 0 && (tile_pts * BLK) % 2 == 0 && args.points >= tile_pts &&
                      aligned16(args.X) && aligned16(args.Y) && aligned16(args.D);
    if (pipe)
    {
        const bool same_xy = args.X == args.Y;
        const int stages = (DIM == 3 && !same_xy) ? 3 : 4;
        const size_t smem = static_cast<size_t>(stages) * kTile * BLK * sizeof(double) * (same_xy ? 1 : 2);
        const int64_t n_full = args.points / tile_pts;
        int64_t grid = static_cast<int64_t>(sm_count()) * (DIM == 3 ? (same_xy ? 3 : 2) : 4);
        if (grid > n_full) grid = n_full;
        cudaError_t status;
        if (same_xy)
        {
            auto kernel = pointwise_cell_pipe_kernel<DIM, true, 4>;
            status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (status != cudaSuccess) return fail_cuda(status, "acro_b200_pointwise_sym (shared memory opt-in)");
            kernel<<<static_cast<int>(grid), kTile, smem, s>>>(args, tile_pts);
        }
        else if (DIM == 3)
        {
            auto kernel = pointwise_cell_pipe_kernel<DIM, false, 3>;
            status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (status != cudaSuccess) return fail_cuda(status, "acro_b200_pointwise_sym (shared memory opt-in)");
            kernel<<<static_cast<int>(grid), kTile, smem, s>>>(args, tile_pts);
        }
        else
        {
            auto kernel = pointwise_cell_pipe_kernel<DIM, false, 4>;
            status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (status != cudaSuccess) return fail_cuda(status, "acro_b200_pointwise_sym (shared memory opt-in)");
            kernel<<<static_cast<int>(grid), kTile, smem, s>>>(args, tile_pts);
        }
        const int rc = launch_status("acro_b200_pointwise_sym (cell-major, pipelined)");
        if (rc != ACRO_B200_OK) return rc;
        const int64_t done = n_full * tile_pts;     // a multiple of K: whole cells
        if (done == args.points) return ACRO_B200_OK;
        args.X += done * BLK;
        args.Y += done * BLK;
        args.D += done * BLK;
        args.first_point += done;
        args.points -= done;
    }
    int64_t grid = (args.points + kTile - 1) / kTile;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
    if (grid > cap) grid = cap;
    pointwise_cell_direct_kernel<DIM><<<static_cast<int>(grid), kTile, 0, s>>>(args);
    return launch_status("acro_b200_pointwise_sym (cell-major)");
}

template <int DIM>
int launch(const PointwiseArgs &args_in, cudaStream_t s)
{
    if (args_in.d.cell_points > 1 || args_in.d.swapped) return launch_cell<DIM>(args_in, s);
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
    int64_t points = 1;
    for (int j = 0; j < d->n_point_loops; ++j)
    {
        if (d->point_extent[j] < 1) return 0;
        points *= d->point_extent[j];
    }
    if (d->cell_points < 1 || points % d->cell_points != 0) return 0;
    if (d->swapped != 0 && d->swapped != 1) return 0;
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
