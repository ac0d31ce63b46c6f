// batched_matvec: an element matrix applied to an element vector,
//     form 0:  Y[e, i] (op)= sum_k M[e, i, k] * X[e, k]        (M is rows x cols = m x k)
//     form 1:  Y[e, j] (op)= sum_k X[e, k] * M[e, k, j]        (M is k x n)
// with rows, cols <= 64: the action of assembled element matrices on element vectors.
//
// Bound by HBM (every entry of M is used once), so it streams: a persistent CTA walks over tiles
// of `group` consecutive elements; the M and X spans of a tile (contiguous) arrive by one
// asynchronous bulk copy each into a double-buffered shared-memory stage (8-byte cp.async when an
// operand is not 16-byte aligned, and for the ragged last tile) while the previous tile is computed;
// Y goes straight to global memory.  Form 0: `split` adjacent lanes share a row of M and combine
// by shuffles; a lane starts its walk along the row at a column rotated by the row number, so
// that the rows of a warp (a multiple of 128 bytes apart when cols is even) fall into different
// banks.  The order of the sum therefore differs from the reference's and fused multiply-add is
// used: results agree within the usual 1e-12 * sum|terms|.  Form 1 walks k in order, lanes along j.
// Measured on B200: 8 x 8 100 %, 16 x 16 101 %, 27 x 27 98 %, 40 x 40 97 %, 64 x 64 98 % of measured HBM bandwidth.
#include "common.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kThreads = 256;
constexpr int kStageBudget = 32 * 1024;      // bytes of one stage

struct MatvecArgs
{
    const double *M;
    const double *X;
    double *Y;
    int64_t batch;
    int rows, cols, form, op;
    int group, split;
    int bulk_in;
    int *wait_flag;
};

__device__ __forceinline__ void copy_async8(double *smem_dst, const double *gmem_src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}

__global__ void __launch_bounds__(kThreads)
batched_matvec_kernel(const MatvecArgs a)
{
    extern __shared__ __align__(128) unsigned char raw[];
    const int rows = a.rows, cols = a.cols, G = a.group, split = a.split;
    const int mat = rows * cols;
    const int xin = a.form == 0 ? cols : rows;          // length of the input vector
    const int yout = a.form == 0 ? rows : cols;         // length of the result
    double *sM = reinterpret_cast<double *>(raw);                       // [2][G * mat]
    double *sX = sM + 2 * G * mat;                                      // [2][G * xin]
    uint64_t *full = reinterpret_cast<uint64_t *>(sX + 2 * G * xin + ((2 * G * xin) & 1));
    const int tid = threadIdx.x;
    const int64_t n_tiles = (a.batch + G - 1) / G;
    const int64_t n_full = a.batch / G;

    if (tid == 0)
    {
        mbar_init(&full[0], kThreads);
        mbar_init(&full[1], kThreads);
        fence_mbar_init();
    }
    __syncthreads();

    auto issue = [&](int64_t tile, int stage) {
        if (tile >= n_tiles) return;
        const int64_t e0 = tile * G;
        double *dm = sM + stage * G * mat, *dx = sX + stage * G * xin;
        if (a.bulk_in && tile < n_full)
        {
            if (tid == 0)
            {
                mbar_arrive_expect_tx(&full[stage], static_cast<uint32_t>(G * (mat + xin) * 8));
                bulk_load(dm, a.M + e0 * mat, static_cast<uint32_t>(G * mat * 8), &full[stage]);
                bulk_load(dx, a.X + e0 * xin, static_cast<uint32_t>(G * xin * 8), &full[stage]);
            }
            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&full[stage])) : "memory");
            return;
        }
        const int n_e = a.batch - e0 < G ? static_cast<int>(a.batch - e0) : G;
        for (int x = tid; x < n_e * mat; x += kThreads) copy_async8(dm + x, a.M + e0 * mat + x);
        for (int x = tid; x < n_e * xin; x += kThreads) copy_async8(dx + x, a.X + e0 * xin + x);
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&full[stage])) : "memory");
    };

    int64_t tile = blockIdx.x;
    issue(tile, 0);
    uint32_t phase_bits = 0;
    int stage = 0;
    // items of a tile: (element, result entry, lane of the entry), the last one fastest
    const int per_elem = yout * split;
    const int step_r = kThreads % per_elem, step_g = kThreads / per_elem;

    for (; tile < n_tiles; tile += gridDim.x)
    {
        issue(tile + gridDim.x, stage ^ 1);      // that stage was last read before the barrier that closed the previous tile
        const int64_t e0 = tile * G;
        const int n_e = a.batch - e0 < G ? static_cast<int>(a.batch - e0) : G;
        const double *tm = sM + stage * G * mat, *tx = sX + stage * G * xin;
        if (!mbar_wait(&full[stage], (phase_bits >> stage) & 1u)) atomicExch(a.wait_flag, 1);
        phase_bits ^= (1u << stage);

        // every thread runs the same number of rounds: the shuffles below need whole warps
        const int rounds = (G * per_elem + kThreads - 1) / kThreads;
        int r = tid % per_elem, g = tid / per_elem;
        for (int round = 0; round < rounds; ++round)
        {
            const bool live = g < n_e;
            const int entry = r / split, q = r - entry * split;
            double acc = 0.0;
            if (live)
            {
                const double *x = tx + g * xin;
                if (a.form == 0)
                {
                    const double *row = tm + g * mat + entry * cols;
                    const int rot = entry % cols;
                    for (int c = q; c < cols; c += split)
                    {
                        int kk = c + rot;
                        kk = kk >= cols ? kk - cols : kk;
                        acc = fma(row[kk], x[kk], acc);
                    }
                }
                else
                {
                    const double *col = tm + g * mat + entry;
                    for (int kk = q; kk < rows; kk += split) acc = fma(x[kk], col[kk * cols], acc);
                }
            }
            for (int width = split >> 1; width > 0; width >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, width);
            if (live && q == 0)
            {
                double *dst = a.Y + (e0 + g) * yout + entry;
                if (a.op == ACRO_B200_OP_ASSIGN) __stcs(dst, acc);
                else if (a.op == ACRO_B200_OP_ADD) *dst += acc;
                else *dst -= acc;
            }
            // next item of this thread
            r += step_r;
            if (r >= per_elem) { r -= per_elem; ++g; }
            g += step_g;
        }
        __syncthreads();      // every thread is done with this stage
        stage ^= 1;
    }
}

}

namespace acro_b200_detail
{

bool batched_matvec_supported(int rows, int cols) { return rows >= 1 && cols >= 1 && rows <= 64 && cols <= 64; }

int batched_matvec_launch(const double *M, const double *X, double *Y, int64_t batch, int rows, int cols, int form, int op, cudaStream_t stream)
{
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_batched_gemm");
    MatvecArgs args;
    args.M = M;
    args.X = X;
    args.Y = Y;
    args.batch = batch;
    args.rows = rows;
    args.cols = cols;
    args.form = form;
    args.op = op;
    const int xin = form == 0 ? cols : rows;
    const int per_elem_bytes = (rows * cols + xin) * 8;
    int group = kStageBudget / per_elem_bytes;
    if (group > 256) group = 256;
    if (group > 1) group &= ~1;                       // even: the spans of a tile stay 16-byte multiples
    if (group < 1) group = 1;
    args.group = group;
    // lanes per result entry (form 0; form 1 keeps one lane per entry, lanes along j).  Measured on B200 with 32 KB
    // stages: rows of 8 and 16 entries run at the HBM rate with one lane per row (two lanes: 71 % and 91 %), rows of
    // 27, 40 and 64 entries with two (one lane: 86 %, 72 %, 69 %; four lanes: 75 %, 74 %, 89 %).
    const int split = (form == 0 && cols >= 24) ? 2 : 1;
    args.split = split;
    args.bulk_in = (aligned16(M) && aligned16(X) && (static_cast<long long>(group) * rows * cols) % 2 == 0 &&
                    (static_cast<long long>(group) * xin) % 2 == 0) ? 1 : 0;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_batched_gemm (status flag)");
    const size_t smem = static_cast<size_t>(2) * group * (rows * cols + xin) * 8 + 8 + 2 * sizeof(uint64_t);
    cudaError_t status = cudaFuncSetAttribute(batched_matvec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
    if (per_sm > 8) per_sm = 8;
    if (per_sm < 1) per_sm = 1;
    const int64_t tiles = (batch + group - 1) / group;
    int64_t grid = static_cast<int64_t>(sms) * per_sm;
    if (grid > tiles) grid = tiles;
    batched_matvec_kernel<<<static_cast<int>(grid), kThreads, smem, stream>>>(args);
    return launch_status("acro_b200_batched_gemm (matrix-vector)");
}

}
