// batched_gemm, small variant: C_e = A_e * B_e for m x k by k x n matrices with m, n, k <= 16.
// Either operand may be stored transposed (A_e as k x m, B_e as n x k): the stages keep the
// global layout, so a transposed operand only changes the strides of the shared-memory reads.
//
// These products are bound by HBM (16^3: 1.3 flop per byte), so the kernel is a streaming
// one: a persistent CTA walks over tiles of `group` consecutive matrices.  The A and B spans of
// a tile (contiguous in global memory) arrive by one asynchronous bulk copy each into a
// double-buffered shared-memory stage while the previous tile is multiplied (8-byte cp.async
// copies when the operands are not 16-byte aligned, and for the ragged last tile).  A thread
// computes a 4 x 1 strip of one C matrix (one B load feeds four rows; the lanes of a warp run
// along a row of C); the C tile is assembled in shared memory and leaves as one bulk store
// (plain stores when C is not 16-byte aligned, the tile is ragged, or the operator is "-=").
//
// Each entry is accumulated from zero in ascending k with separate multiply and add (no fused
// multiply-add): bit-identical to the reference's CPU executor for "=" and, starting from
// the old value, for "+=".
//
// Measured on B200 (1.2-1.6 GB of traffic each): 3^3 96 % of measured HBM bandwidth, 4^3 62 %, 8^3 72 %,
// 12^3 58 %, 16^3 64 % (the thread-per-entry kernel: 86 / 61 / 61 / 41 / 29 %).  An ncu capture at
// 16^3 shows the shared-memory pipe 82 % busy, much of it on bank conflicts: the matrices and row
// strips that share a warp sit multiples of 128 bytes apart.  Variants that were measured and
// were slower: entries copied one by one (8-byte cp.async) into a padded conflict-free layout
// (57 / 69 / 62 / 54 / 55 %); one bulk copy per matrix into padded slots with the lanes of a warp
// spread over matrices (41 / 43 / 59 / 60 / 45 %); 4 x 2 blocks with 16-byte B loads
// (98 / 50 / 64 / 47 / 64 %); a third stage (91 / 61 / 72 / 57 / 59 %); the k loop unrolled by four
// (94 / 54 / 64 / 52 / 61 %).  A sweep over the stage size (16 ... 64 KB) and the strips per thread (2 ... 8) moved
// nothing by more than three points.
#include "common.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kThreads = 256;
constexpr int kStrip = 4;               // C rows per thread
constexpr int kMaxDim = 16;
constexpr int kStages = 2;               // input stages: one tile in flight while one is multiplied
constexpr int kStageBudget = 40 * 1024;   // bytes of shared memory for the input stages and the C tile

struct SmallArgs
{
    const double *A;
    const double *B;
    double *C;
    int64_t batch;
    int m, n, k, op;
    int group;          // matrices per tile (even)
    int bulk_in;        // A and B are 16-byte aligned
    int bulk_out;       // C is 16-byte aligned
    int *wait_flag;
};

__device__ __forceinline__ void copy_async8(double *smem_dst, const double *gmem_src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}

template <bool TA, bool TB>
__global__ void __launch_bounds__(kThreads)
batched_gemm_small_kernel(const SmallArgs a)
{
    extern __shared__ __align__(128) unsigned char raw[];
    const int m = a.m, n = a.n, k = a.k, G = a.group;
    const int a_mat = m * k, b_mat = k * n, c_mat = m * n;
    const int sa = a_mat, sb = b_mat;              // the stage keeps the global layout
    double *sA = reinterpret_cast<double *>(raw);                 // [kStages][G * sa]
    double *sB = sA + kStages * G * sa;                           // [kStages][G * sb]
    double *sC = sB + kStages * G * sb;                           // [G * c_mat]
    uint64_t *full = reinterpret_cast<uint64_t *>(sC + G * c_mat);   // [kStages]
    const int tid = threadIdx.x;
    const int64_t n_tiles = (a.batch + G - 1) / G;
    const int64_t n_full = a.batch / G;

    if (tid == 0)
    {
        for (int st = 0; st < kStages; ++st) mbar_init(&full[st], kThreads);
        fence_mbar_init();
    }
    __syncthreads();

    // items of a tile: (matrix, row strip, column), column fastest; how a step of kThreads moves one
    const int mb = (m + kStrip - 1) / kStrip;
    const int step_j = kThreads % n, step_r = kThreads / n;
    const int step_ib = step_r % mb, step_g = step_r / mb;

    // Fills a stage.  Every thread arrives once on the stage's barrier: thread 0 together with the byte
    // count of the two bulk copies, or every thread behind its own 8-byte copies.
    auto issue = [&](int64_t tile, int stage) {
        if (tile >= n_tiles) return;
        const int64_t g0 = tile * G;
        double *da = sA + stage * G * sa, *db = sB + stage * G * sb;
        if (a.bulk_in && tile < n_full)
        {
            if (tid == 0)
            {
                mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(G * (a_mat + b_mat) * 8));
                bulk_load(da, a.A + g0 * a_mat, static_cast<uint32_t>(G * a_mat * 8), &full[stage]);
                bulk_load(db, a.B + g0 * b_mat, static_cast<uint32_t>(G * b_mat * 8), &full[stage]);
            }
            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&full[stage])) : "memory");
            return;
        }
        const int n_g = a.batch - g0 < G ? static_cast<int>(a.batch - g0) : G;
        for (int idx = tid; idx < n_g * a_mat; idx += kThreads) copy_async8(da + idx, a.A + g0 * a_mat + idx);
        for (int idx = tid; idx < n_g * b_mat; idx += kThreads) copy_async8(db + idx, a.B + g0 * b_mat + idx);
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&full[stage])) : "memory");
    };

    int64_t tile = blockIdx.x;
    for (int st = 0; st < kStages - 1; ++st) issue(tile + static_cast<int64_t>(st) * gridDim.x, st);
    uint32_t phase_bits = 0;
    int stage = 0;
    bool store_in_flight = false;

    for (; tile < n_tiles; tile += gridDim.x)
    {
        // the stage refilled here was last read before the barrier that closed the previous tile
        issue(tile + static_cast<int64_t>(kStages - 1) * gridDim.x, (stage + kStages - 1) % kStages);
        const int64_t g0 = tile * G;
        const int n_g = a.batch - g0 < G ? static_cast<int>(a.batch - g0) : G;
        const double *ta = sA + stage * G * sa, *tb = sB + stage * G * sb;

        // the previous tile's bulk store must have read the C tile before it is overwritten
        if (store_in_flight)
        {
            if (tid == 0) bulk_wait_read<0>();
            __syncthreads();
        }
        if (a.op == ACRO_B200_OP_ADD)
        {
            for (int i = tid; i < n_g * c_mat; i += kThreads) sC[i] = a.C[g0 * c_mat + i];
            __syncthreads();
        }
        if (!mbar_wait(&full[stage], (phase_bits >> stage) & 1u)) atomicExch(a.wait_flag, 1);
        phase_bits ^= (1u << stage);

        int j = tid % n, r = tid / n;
        int ib = r % mb, g = r / mb;
        while (g < n_g)
        {
            const int i0 = ib * kStrip;
            const int rows = m - i0 < kStrip ? m - i0 : kStrip;
            // entry (i, kk) of A and (kk, j) of B in the stage
            const int a_i = TA ? 1 : k, a_k = TA ? m : 1, b_k = TB ? 1 : n, b_j = TB ? k : 1;
            const double *ar = ta + g * sa + i0 * a_i;
            const double *bc = tb + g * sb + j * b_j;
            double *cc = sC + g * c_mat + i0 * n + j;
            double acc[kStrip];
#pragma unroll
            for (int x = 0; x < kStrip; ++x) acc[x] = (a.op == ACRO_B200_OP_ADD && x < rows) ? cc[x * n] : 0.0;
            for (int kk = 0; kk < k; ++kk)
            {
                const double bv = bc[kk * b_k];
#pragma unroll
                for (int x = 0; x < kStrip; ++x)
                {
                    const double av = ar[(x < rows ? x : 0) * a_i + kk * a_k];
                    acc[x] = __dadd_rn(acc[x], __dmul_rn(av, bv));
                }
            }
#pragma unroll
            for (int x = 0; x < kStrip; ++x)
            {
                if (x < rows) cc[x * n] = acc[x];
            }
            // next item of this thread
            j += step_j;
            if (j >= n) { j -= n; ++ib; }
            ib += step_ib;
            if (ib >= mb) { ib -= mb; ++g; }
            g += step_g;
        }

        double *dst = a.C + g0 * c_mat;
        if (a.bulk_out && n_g == G && a.op != ACRO_B200_OP_SUB)
        {
            fence_proxy_async();      // make the C tile visible to the asynchronous proxy
            __syncthreads();          // tile complete; inputs of this stage dead
            if (tid == 0)
            {
                bulk_store(dst, sC, static_cast<uint32_t>(G * c_mat * 8));
                bulk_commit();
            }
            store_in_flight = true;
        }
        else
        {
            __syncthreads();
            if (a.op == ACRO_B200_OP_SUB)
            {
                for (int x = tid; x < n_g * c_mat; x += kThreads) dst[x] = __dsub_rn(dst[x], sC[x]);
            }
            else
            {
                for (int x = tid; x < n_g * c_mat; x += kThreads) __stcs(dst + x, sC[x]);
            }
            __syncthreads();          // the next tile overwrites the C tile
            store_in_flight = false;
        }
        stage = (stage + 1) % kStages;
    }
    if (tid == 0) bulk_wait_all<0>();   // shared memory must outlive the stores that read it
}

int group_for(int m, int n, int k)
{
    const int per_matrix = (kStages * (m * k + k * n) + m * n) * 8;
    const int mb = (m + kStrip - 1) / kStrip;
    int group = (2 * kThreads + mb * n - 1) / (mb * n);     // about two strips per thread
    if (group * per_matrix > kStageBudget) group = kStageBudget / per_matrix;
    if (group > 512) group = 512;
    group &= ~1;                                             // even: the C tile stays a 16-byte multiple
    return group < 2 ? 2 : group;
}

}

namespace acro_b200_detail
{

bool batched_gemm_small_supported(int m, int n, int k)
{
    return m >= 1 && n >= 1 && k >= 1 && m <= kMaxDim && n <= kMaxDim && k <= kMaxDim;
}

int batched_gemm_small_launch(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k, int trans_a, int trans_b, int op,
                              cudaStream_t stream)
{
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_batched_gemm");
    SmallArgs args;
    args.A = A;
    args.B = B;
    args.C = C;
    args.batch = batch;
    args.m = m;
    args.n = n;
    args.k = k;
    args.op = op;
    args.group = group_for(m, n, k);
    args.bulk_in = (aligned16(A) && aligned16(B)) ? 1 : 0;
    args.bulk_out = aligned16(C) ? 1 : 0;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_batched_gemm (status flag)");

    const size_t smem = static_cast<size_t>(args.group) * (kStages * (m * k + k * n) + m * n) * 8 + kStages * sizeof(uint64_t);
    auto kernel = trans_a ? (trans_b ? batched_gemm_small_kernel<true, true> : batched_gemm_small_kernel<true, false>)
                          : (trans_b ? batched_gemm_small_kernel<false, true> : batched_gemm_small_kernel<false, false>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
    if (per_sm > 6) per_sm = 6;
    if (per_sm < 1) per_sm = 1;
    const int64_t tiles = (batch + args.group - 1) / args.group;
    int64_t grid = static_cast<int64_t>(sms) * per_sm;
    if (grid > tiles) grid = tiles;
    kernel<<<static_cast<int>(grid), kThreads, smem, stream>>>(args);
    return launch_status("acro_b200_batched_gemm (small)");
}

}
