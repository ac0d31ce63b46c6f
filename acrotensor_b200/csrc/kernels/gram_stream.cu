// gram, streaming variant: S[a, b] = sum_n X[n, a] * Y[n, b] with a, b <= 16 (normal equations with a
// few unknowns, moments).  Bound by HBM: 8 * (a + b) bytes and a * b multiply-adds per row.
//
// A persistent CTA walks over tiles of `group` consecutive rows; the X and Y spans of a tile
// (contiguous) arrive by one asynchronous bulk copy each into a double-buffered shared-memory stage
// (8-byte cp.async when an operand is not 16-byte aligned, and for the ragged last tile) while the
// previous tile is accumulated.  S is cut into 4 x 4 blocks; a thread owns one block and every
// `lanes`-th row of each tile, and keeps its 16 sums in registers over all tiles of the CTA.  At
// the end the lanes of a CTA are added in ascending order into one a x b tile of partial sums
// (plain stores; the caller adds the tiles of all CTAs in ascending order).  The order of the sum
// is fixed by the grid, so two runs on one device give the same bits; fused multiply-add is used.
#include "common.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kThreads = 256;
constexpr int kBlock = 4;                    // S is cut into kBlock x kBlock blocks
constexpr int kStageBudget = 32 * 1024;      // bytes of one stage
constexpr int kMaxDim = 16;

struct GramArgs
{
    const double *X;
    const double *Y;
    double *partials;       // [gridDim.x][a * b]
    int64_t rows;
    int a, b;
    int group;              // rows per tile (even)
    int bulk_in;
    int *wait_flag;
};

__device__ __forceinline__ void copy_async8(double *smem_dst, const double *gmem_src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}

__global__ void __launch_bounds__(kThreads)
gram_stream_kernel(const GramArgs args)
{
    extern __shared__ __align__(128) unsigned char raw[];
    const int a = args.a, b = args.b, G = args.group;
    double *sX = reinterpret_cast<double *>(raw);                       // [2][G * a]
    double *sY = sX + 2 * G * a;                                        // [2][G * b]
    double *red = sY + 2 * G * b;                                       // [kThreads][kBlock * kBlock]
    uint64_t *full = reinterpret_cast<uint64_t *>(red + kThreads * kBlock * kBlock);
    const int tid = threadIdx.x;
    const int64_t n_tiles = (args.rows + G - 1) / G;
    const int64_t n_full = args.rows / G;

    if (tid == 0)
    {
        mbar_init(&full[0], kThreads);
        mbar_init(&full[1], kThreads);
        fence_mbar_init();
    }
    __syncthreads();

    // Fills a stage.  Every thread arrives once on the stage's barrier: thread 0 together with the byte
    // count of the two bulk copies, or every thread behind its own 8-byte copies.
    auto issue = [&](int64_t tile, int stage) {
        if (tile >= n_tiles) return;
        const int64_t r0 = tile * G;
        double *dx = sX + stage * G * a, *dy = sY + stage * G * b;
        if (args.bulk_in && tile < n_full)
        {
            if (tid == 0)
            {
                mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(G * (a + b) * 8));
                bulk_load(dx, args.X + r0 * a, static_cast<uint32_t>(G * a * 8), &full[stage]);
                bulk_load(dy, args.Y + r0 * b, static_cast<uint32_t>(G * b * 8), &full[stage]);
            }
            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&full[stage])) : "memory");
            return;
        }
        const int n_r = args.rows - r0 < G ? static_cast<int>(args.rows - r0) : G;
        for (int x = tid; x < n_r * a; x += kThreads) copy_async8(dx + x, args.X + r0 * a + x);
        for (int x = tid; x < n_r * b; x += kThreads) copy_async8(dy + x, args.Y + r0 * b + x);
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&full[stage])) : "memory");
    };

    // this thread's block of S and its rows of every tile
    const int nbb = (b + kBlock - 1) / kBlock;
    const int n_blocks = ((a + kBlock - 1) / kBlock) * nbb;
    const int lanes = kThreads / n_blocks;
    const int blk = tid % n_blocks, lane = tid / n_blocks;
    const int i0 = (blk / nbb) * kBlock, j0 = (blk % nbb) * kBlock;
    int xi[kBlock], yj[kBlock];         // entries of a row this thread reads; clamped, results outside S are dropped
#pragma unroll
    for (int u = 0; u < kBlock; ++u)
    {
        xi[u] = i0 + u < a ? i0 + u : a - 1;
        yj[u] = j0 + u < b ? j0 + u : b - 1;
    }
    double acc[kBlock][kBlock];
#pragma unroll
    for (int u = 0; u < kBlock; ++u)
#pragma unroll
        for (int v = 0; v < kBlock; ++v) acc[u][v] = 0.0;

    int64_t tile = blockIdx.x;
    issue(tile, 0);
    uint32_t phase_bits = 0;
    int stage = 0;
    for (; tile < n_tiles; tile += gridDim.x)
    {
        issue(tile + gridDim.x, stage ^ 1);      // that stage was last read before the barrier that closed the previous tile
        const int64_t r0 = tile * G;
        const int n_r = args.rows - r0 < G ? static_cast<int>(args.rows - r0) : G;
        const double *tx = sX + stage * G * a, *ty = sY + stage * G * b;
        if (!mbar_wait(&full[stage], (phase_bits >> stage) & 1u)) atomicExch(args.wait_flag, 1);
        phase_bits ^= (1u << stage);

        if (lane < lanes)
        {
            for (int r = lane; r < n_r; r += lanes)
            {
                const double *xr = tx + r * a, *yr = ty + r * b;
                double xv[kBlock], yv[kBlock];
#pragma unroll
                for (int u = 0; u < kBlock; ++u)
                {
                    xv[u] = xr[xi[u]];
                    yv[u] = yr[yj[u]];
                }
#pragma unroll
                for (int u = 0; u < kBlock; ++u)
#pragma unroll
                    for (int v = 0; v < kBlock; ++v) acc[u][v] = fma(xv[u], yv[v], acc[u][v]);
            }
        }
        __syncthreads();      // every thread is done with this stage
        stage ^= 1;
    }

    // lanes of the CTA, ascending
#pragma unroll
    for (int u = 0; u < kBlock; ++u)
#pragma unroll
        for (int v = 0; v < kBlock; ++v) red[tid * (kBlock * kBlock) + u * kBlock + v] = acc[u][v];
    __syncthreads();
    for (int e = tid; e < a * b; e += kThreads)
    {
        const int i = e / b, j = e - i * b;
        const int owner = (i / kBlock) * nbb + j / kBlock;
        const int slot = (i % kBlock) * kBlock + j % kBlock;
        double total = 0.0;
        for (int l = 0; l < lanes; ++l) total = __dadd_rn(total, red[(l * n_blocks + owner) * (kBlock * kBlock) + slot]);
        args.partials[static_cast<int64_t>(blockIdx.x) * a * b + e] = total;
    }
}

}

namespace acro_b200_detail
{

bool gram_stream_supported(int a, int b) { return a >= 1 && b >= 1 && a <= kMaxDim && b <= kMaxDim; }

int gram_stream_launch(const double *X, const double *Y, double *partials, int64_t rows, int a, int b, int max_parts, int *parts, cudaStream_t stream)
{
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_gram");
    GramArgs args;
    args.X = X;
    args.Y = Y;
    args.partials = partials;
    args.rows = rows;
    args.a = a;
    args.b = b;
    int group = kStageBudget / ((a + b) * 8);
    if (group > 2048) group = 2048;
    group &= ~1;                                  // even: the spans of a tile stay 16-byte multiples
    if (group < 2) group = 2;
    args.group = group;
    args.bulk_in = (aligned16(X) && aligned16(Y)) ? 1 : 0;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_gram (status flag)");
    const size_t smem = static_cast<size_t>(2) * group * (a + b) * 8 + static_cast<size_t>(kThreads) * kBlock * kBlock * 8 + 2 * sizeof(uint64_t);
    cudaError_t status = cudaFuncSetAttribute(gram_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_gram (shared memory opt-in)");
    int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
    if (per_sm > 4) per_sm = 4;
    if (per_sm < 1) per_sm = 1;
    const int64_t tiles = (rows + group - 1) / group;
    int64_t grid = static_cast<int64_t>(sms) * per_sm;
    if (grid > tiles) grid = tiles;
    if (grid > max_parts) grid = max_parts;
    gram_stream_kernel<<<static_cast<int>(grid), kThreads, smem, stream>>>(args);
    *parts = static_cast<int>(grid);
    return launch_status("acro_b200_gram (streaming)");
}

}
