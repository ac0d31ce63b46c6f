// batched_gemm for matrices of 17 .. 32 whose rows are an odd number of doubles (27 x 27 element matrices of a
// triquadratic hexahedron, 25, 21 ...):  C_e = A_e * B_e, either operand possibly stored transposed, and the
// accumulating form S = sum_e A_e^T * B_e that the Gram kernel needs.
//
// Rows of an odd length are not 16-byte multiples, so the zero-padded ring of batched_gemm.cu has to copy such
// matrices with 8-byte cp.async and run-time row bookkeeping, which makes it bound by instruction issue (ncu: 72 %
// of the issue slots, tensor pipe 32 %, DRAM 41 % at 27^3).  Two consecutive matrices together, however, are always a
// 16-byte multiple and, for an even element number and a 16-byte aligned tensor, start on a 16-byte boundary.  This
// kernel therefore works on PAIRS of elements: one asynchronous bulk copy per operand and pair into an unpadded
// shared-memory slot (odd row lengths keep the tensor-core fragment loads nearly conflict-free without padding: row g
// starts 2 * odd banks after row g - 1), fragment entries outside the matrices read as zeros by predicate, and the
// pair's two result matrices leave as one bulk store from a staging tile (two tiles, used alternately, so that one
// CTA barrier per pair is enough).  A warp owns one 8-row tile of one element of the pair over all (up to four)
// 8-column tiles.
//
// Algorithmic HBM traffic per element: 8 * (m*k + k*n + m*n) bytes; 2*m*n*k flops.
#include "common.cuh"
#include "dmma.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kStages = 3;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxDim = 32;

struct PairArgs
{
    const double *A;      // [pairs][2][rows_a][cols_a]
    const double *B;      // [pairs][2][rows_b][cols_b]
    double *C;            // [pairs][2][m][n], or (accumulating) [2 * gridDim.x][m][n] partial sums
    int64_t pairs;
    int m, n, k, op;
    int rows_a, cols_a, rows_b, cols_b;      // the operands as stored: A is m x k (k x m when transposed), B is k x n (n x k)
    int *wait_flag;
};

struct PairLayout
{
    int a_doubles, b_doubles, c_doubles;     // per pair
    int stage_doubles;                       // A pair + B pair, rounded to 16 bytes
    int c_off, bar_off, total;               // byte offsets
};

__host__ __device__ inline PairLayout pair_layout(const PairArgs &a, bool accumulate)
{
    PairLayout l;
    l.a_doubles = 2 * a.rows_a * a.cols_a;
    l.b_doubles = 2 * a.rows_b * a.cols_b;
    l.c_doubles = 2 * a.m * a.n;
    l.stage_doubles = l.a_doubles + l.b_doubles;       // both even: every slot starts on a 16-byte boundary
    l.c_off = ((kStages * l.stage_doubles * 8 + 127) / 128) * 128;
    const int c_bytes = accumulate ? 0 : ((l.c_doubles * 8 + 127) / 128) * 128;
    l.bar_off = l.c_off + 2 * c_bytes;
    l.total = l.bar_off + 2 * kStages * 8;
    return l;
}

__device__ __forceinline__ void mbar_arrive_one(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// MC, NC, KC: the extents when known at compile time (the 27-wide cases, whose inner loop then unrolls and loses its
// run-time predicates and index arithmetic), 0 = taken from the arguments.
template <bool TA, bool TB, bool ACC, int MC = 0, int NC = 0, int KC = 0>
__global__ void __launch_bounds__(kThreads, 2)
batched_gemm_pairs_kernel(const PairArgs a)
{
    extern __shared__ __align__(128) unsigned char raw[];
    const PairLayout L = pair_layout(a, ACC);
    double *ring = reinterpret_cast<double *>(raw);
    uint64_t *full = reinterpret_cast<uint64_t *>(raw + L.bar_off);
    uint64_t *empty = full + kStages;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m = MC ? MC : a.m, n = NC ? NC : a.n, k = KC ? KC : a.k;
    const int row_tiles = (m + 7) / 8;                 // per element
    const bool active = warp < 2 * row_tiles;          // this warp has a row tile of one element of the pair
    const int el = warp / row_tiles, m0 = (warp % row_tiles) * 8;
    const int k4 = (k + 3) & ~3;
    const int lda = TA ? m : k, ldb = TB ? k : n;      // row lengths of the operands as stored

    if (tid == 0)
    {
        for (int i = 0; i < kStages; ++i)
        {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], kWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();

    auto issue = [&](int64_t pair, int stage) {      // thread 0 only
        double *sa = ring + stage * L.stage_doubles, *sb = sa + L.a_doubles;
        mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(L.stage_doubles) * 8u);
        bulk_load(sa, a.A + pair * L.a_doubles, static_cast<uint32_t>(L.a_doubles) * 8u, &full[stage]);
        bulk_load(sb, a.B + pair * L.b_doubles, static_cast<uint32_t>(L.b_doubles) * 8u, &full[stage]);
    };

    double c[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) c[nt][0] = c[nt][1] = 0.0;

    constexpr int AHEAD = kStages - 1;
    int64_t pair = blockIdx.x;
    if (tid == 0)
    {
        for (int d = 0; d < AHEAD; ++d)
        {
            if (pair + static_cast<int64_t>(d) * gridDim.x < a.pairs) issue(pair + static_cast<int64_t>(d) * gridDim.x, d);
        }
    }

    int64_t it = 0;
    for (; pair < a.pairs; pair += gridDim.x, ++it)
    {
        const int stage = static_cast<int>(it % kStages);
        if (tid == 0)
        {
            const int64_t nxt = pair + static_cast<int64_t>(AHEAD) * gridDim.x;
            if (nxt < a.pairs)
            {
                const int ns = static_cast<int>((it + AHEAD) % kStages);
                const int64_t use = (it + AHEAD) / kStages;
                if (use > 0 && !mbar_wait_counted(&empty[ns], static_cast<uint32_t>((use - 1) & 1))) atomicExch(a.wait_flag, 1);
                issue(nxt, ns);
            }
        }
        if (!mbar_wait_counted(&full[stage], static_cast<uint32_t>((it / kStages) & 1))) atomicExch(a.wait_flag, 1);

        if (!ACC)
        {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) c[nt][0] = c[nt][1] = 0.0;
        }
        if (active)
        {
            const double *sa = ring + stage * L.stage_doubles + el * (L.a_doubles / 2);
            const double *sb = ring + stage * L.stage_doubles + L.a_doubles + el * (L.b_doubles / 2);
            const int i = m0 + g;
#pragma unroll (KC ? 8 : 1)
            for (int k0 = 0; k0 < k4; k0 += 4)
            {
                const int kk = k0 + t;
                const bool k_in = kk < k;
                double af = 0.0, bf[4];
                if (k_in && i < m) af = TA ? sa[kk * lda + i] : sa[i * lda + kk];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
                {
                    const int j = nt * 8 + g;
                    bf[nt] = 0.0;
                    if (k_in && j < n) bf[nt] = TB ? sb[j * ldb + kk] : sb[kk * ldb + j];
                }
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
                {
                    if (nt * 8 < n) dmma_m8n8k4(c[nt], af, bf[nt]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_one(&empty[stage]);   // this warp no longer reads the slot
        if (ACC) continue;

        // Pair `it` goes through staging tile it % 2.  The last store that read this tile belongs to pair it - 2; thread 0
        // waited for it before the barrier of pair it - 1.
        double *cst = reinterpret_cast<double *>(raw + L.c_off) + (it & 1) * ((L.c_doubles + 15) / 16 * 16);
        if (active)
        {
            const int i = m0 + g;
            const double *old = a.C + pair * L.c_doubles + el * m * n;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    const int j = nt * 8 + 2 * t + h;
                    if (i < m && j < n)
                    {
                        double v = c[nt][h];
                        if (a.op == ACRO_B200_OP_ADD) v += old[i * n + j];
                        else if (a.op == ACRO_B200_OP_SUB) v = old[i * n + j] - v;
                        cst[el * m * n + i * n + j] = v;
                    }
                }
        }
        fence_proxy_async();
        if (tid == 0) bulk_wait_read<0>();      // the store of the previous pair (the other tile) has read its tile
        __syncthreads();
        if (tid == 0)
        {
            bulk_store(a.C + pair * L.c_doubles, cst, static_cast<uint32_t>(L.c_doubles) * 8u);
            bulk_commit();
        }
    }
    if (ACC)
    {
        // partial sums of this CTA: one tile per element slot of the pairs it walked over
        if (active)
        {
            double *gc = a.C + (2 * static_cast<int64_t>(blockIdx.x) + el) * m * n;
            const int i = m0 + g;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    const int j = nt * 8 + 2 * t + h;
                    if (i < m && j < n) gc[i * n + j] = c[nt][h];
                }
        }
    }
    else if (tid == 0) bulk_wait_all<0>();   // shared memory must outlive the stores that read it
}

template <bool ACC>
int launch_pairs(const PairArgs &args, int trans_a, int trans_b, int grid, cudaStream_t stream, const char *where)
{
    typedef void (*kernel_t)(const PairArgs);
    kernel_t kernel = trans_a ? (trans_b ? batched_gemm_pairs_kernel<true, true, ACC> : batched_gemm_pairs_kernel<true, false, ACC>)
                              : (trans_b ? batched_gemm_pairs_kernel<false, true, ACC> : batched_gemm_pairs_kernel<false, false, ACC>);
    // the sizes of a triquadratic hexahedron's element matrices, compiled in
    if (args.m == 27 && args.n == 27)
    {
        if (ACC && trans_a && !trans_b && args.k == 32) kernel = batched_gemm_pairs_kernel<true, false, ACC, 27, 27, 32>;
        if (!ACC && !trans_a && !trans_b && args.k == 27) kernel = batched_gemm_pairs_kernel<false, false, ACC, 27, 27, 27>;
    }
    const PairLayout L = pair_layout(args, ACC);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total);
    if (status != cudaSuccess) return fail_cuda(status, where);
    kernel<<<grid, kThreads, L.total, stream>>>(args);
    return launch_status(where);
}

}

namespace acro_b200_detail
{

bool batched_gemm_pairs_supported(int m, int n, int k, int trans_a, int trans_b)
{
    if (m < 1 || n < 1 || k < 1 || m > kMaxDim || n > kMaxDim || k > kMaxDim) return false;
    if (m <= 16 && n <= 16 && k <= 16) return false;          // the streaming kernel's sizes
    const int cols_a = trans_a ? m : k, cols_b = trans_b ? k : n;
    return (cols_a % 2 == 1) && (cols_b % 2 == 1);            // odd rows: no padding needed, and nothing else copies them in 16-byte units
}

int batched_gemm_pairs_launch(const double *A, const double *B, double *C, int64_t pairs, int m, int n, int k, int trans_a, int trans_b, int op,
                              cudaStream_t stream)
{
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_batched_gemm (pairs)");
    PairArgs args;
    args.A = A;
    args.B = B;
    args.C = C;
    args.pairs = pairs;
    args.m = m;
    args.n = n;
    args.k = k;
    args.op = op;
    args.rows_a = trans_a ? k : m;
    args.cols_a = trans_a ? m : k;
    args.rows_b = trans_b ? n : k;
    args.cols_b = trans_b ? k : n;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_batched_gemm (status flag)");
    int64_t grid = static_cast<int64_t>(sms) * 2;
    if (grid > pairs) grid = pairs;
    return launch_pairs<false>(args, trans_a, trans_b, static_cast<int>(grid), stream, "acro_b200_batched_gemm (pairs)");
}

int gram_pairs_launch(const double *X, const double *Y, double *partials, int64_t pairs, int slab_rows, int a, int b, int max_parts, int *parts,
                      cudaStream_t stream)
{
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_gram (pairs)");
    PairArgs args;
    args.A = X;                 // a slab of X is stored k x m: first operand transposed
    args.B = Y;
    args.C = partials;
    args.pairs = pairs;
    args.m = a;
    args.n = b;
    args.k = slab_rows;
    args.op = ACRO_B200_OP_ASSIGN;
    args.rows_a = slab_rows;
    args.cols_a = a;
    args.rows_b = slab_rows;
    args.cols_b = b;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_gram (status flag)");
    int64_t grid = static_cast<int64_t>(sms) * 2;
    if (grid > pairs) grid = pairs;
    if (2 * grid > max_parts) grid = max_parts / 2;
    *parts = static_cast<int>(2 * grid);
    return launch_pairs<true>(args, 1, 0, static_cast<int>(grid), stream, "acro_b200_gram (pairs)");
}

}
