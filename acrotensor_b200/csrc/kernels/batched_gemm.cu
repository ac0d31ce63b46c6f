// batched_gemm: C_e = A_e * B_e for a batch of small dense fp64 matrices (N x N x N, N = 64 or 32).
// The description below gives the N = 64 figures.
//
// Persistent CTAs (one per SM, 8 warps) walk over the batch.  A_e and B_e (32 KB each,
// contiguous) are copied asynchronously (16-byte cp.async, one 512-byte matrix row per warp
// instruction) into a three-slot ring of shared-memory buffers whose rows are padded to 68
// doubles, which makes every DMMA fragment load bank-conflict free.  Completion of a slot
// is tracked by an mbarrier ("full", one asynchronous arrival per thread); a second mbarrier
// per slot ("empty") collects the threads that finished reading it.  The copy of element
// e+1 is issued before element e is multiplied and targets the slot that was read two
// elements ago, so neither wait normally blocks and warps drift apart by up to one element
// instead of meeting at a CTA barrier.  Each warp owns a 16 x 32 block of C: 8 accumulator
// tiles of mma.sync m8n8k4 (fp64 tensor cores), 6 shared-memory fragment loads per 8 MMAs.
// C leaves straight from the accumulator registers as full 64-byte row segments.
//
// Measured alternatives on B200 (E = 2^14): one bulk copy (TMA) per matrix row issued by a
// single warp 0.597 ms, the same copies spread over all warps 0.351 ms, cp.async 0.339 ms.
//
// Algorithmic HBM traffic: 3 * 8 * 64 * 64 = 98,304 bytes per element; 2 * 64^3 = 524,288
// flops per element (arithmetic intensity 5.33 flop/byte, the fp64 ridge of a B200).
#include "common.cuh"
#include "dmma.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int STAGES = 3;
constexpr int NT = 256;               // 8 warps

template <int N>
struct Smem
{
    static constexpr int LD = N + 4;      // padded row (N = 64: 68 doubles = 544 bytes, a 16-byte multiple)
    static constexpr int MAT = N * LD;    // doubles per padded matrix
    double A[STAGES][MAT];
    double B[STAGES][MAT];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
};

struct GemmArgs
{
    const double *A;
    const double *B;
    double *C;
    int64_t batch;
    int op;
    int *wait_flag;
    int async_copy;   // operands are 16-byte aligned: cp.async allowed
};

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// Every thread copies its 16 chunks of element e into slot `stage` and attaches an arrival
// on the slot's "full" barrier to the completion of those copies.
template <int N>
__device__ __forceinline__ void issue_element_load(Smem<N> &s, const GemmArgs &a, int64_t e, int stage)
{
    constexpr int LD = Smem<N>::LD;
    constexpr int ROW_CHUNKS = N / 2;          // 16-byte chunks per matrix row
    const int tid = threadIdx.x;
    const double *ga = a.A + e * N * N, *gb = a.B + e * N * N;
#pragma unroll
    for (int i = 0; i < N * ROW_CHUNKS / NT; ++i)
    {
        const int c = tid + i * NT;            // 16-byte chunk number inside A (and inside B)
        const int row = c / ROW_CHUNKS, col = (c % ROW_CHUNKS) * 2;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.A[stage][row * LD + col])), "l"(ga + c * 2) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.B[stage][row * LD + col])), "l"(gb + c * 2) : "memory");
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&s.full[stage])) : "memory");
}

template <int N>
__global__ void __launch_bounds__(NT, N == 64 ? 1 : 4)
batched_gemm_kernel(const GemmArgs a)
{
    constexpr int LD = Smem<N>::LD;
    constexpr int MT = N / 32, NTL = N / 16;      // 8-row / 8-column accumulator tiles per warp
    extern __shared__ __align__(128) unsigned char raw[];
    Smem<N> &s = *reinterpret_cast<Smem<N> *>(raw);
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp >> 1) * (N / 4), n0 = (warp & 1) * (N / 2);

    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i)
        {
            mbar_init(&s.full[i], NT);
            mbar_init(&s.empty[i], NT);
        }
        fence_mbar_init();
    }
    __syncthreads();

    int64_t e = blockIdx.x;
    if (a.async_copy && e < a.batch) issue_element_load(s, a, e, 0);

    int64_t it = 0;   // elements this CTA has started
    for (; e < a.batch; e += gridDim.x, ++it)
    {
        const int stage = static_cast<int>(it % STAGES);
        if (a.async_copy)
        {
            // Prefetch the next element into the slot read two elements ago.
            const int64_t nxt = e + gridDim.x;
            if (nxt < a.batch)
            {
                const int ns = static_cast<int>((it + 1) % STAGES);
                const int64_t use = (it + 1) / STAGES;      // how often that slot was filled before
                if (use > 0 && !mbar_wait(&s.empty[ns], static_cast<uint32_t>((use - 1) & 1))) atomicExch(a.wait_flag, 1);
                issue_element_load(s, a, nxt, ns);
            }
            if (!mbar_wait(&s.full[stage], static_cast<uint32_t>((it / STAGES) & 1))) atomicExch(a.wait_flag, 1);
        }
        else
        {
            // unaligned operands: plain loads into the same padded layout
            __syncthreads();
            const double *ga = a.A + e * N * N, *gb = a.B + e * N * N;
            for (int i = tid; i < N * N; i += NT)
            {
                s.A[stage][(i / N) * LD + (i % N)] = __ldcs(ga + i);
                s.B[stage][(i / N) * LD + (i % N)] = __ldcs(gb + i);
            }
            __syncthreads();
        }

        const double *sa = s.A[stage];
        const double *sb = s.B[stage];
        double c[MT][NTL][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;

#pragma unroll 4
        for (int k0 = 0; k0 < N; k0 += 4)
        {
            double af[MT], bf[NTL];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) af[mt] = sa[(m0 + mt * 8 + g) * LD + k0 + t];
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) bf[nt] = sb[(k0 + t) * LD + n0 + nt * 8 + g];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) dmma_m8n8k4(c[mt][nt], af[mt], bf[nt]);
        }
        if (a.async_copy) mbar_arrive(&s.empty[stage]);   // this thread no longer reads the slot

        // C rows leave as 64-byte segments per quad (two doubles per lane)
        double *gc = a.C + e * N * N;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
            {
                double *dst = gc + (m0 + mt * 8 + g) * N + n0 + nt * 8 + 2 * t;
                double v0 = c[mt][nt][0], v1 = c[mt][nt][1];
                if (a.op == ACRO_B200_OP_ADD) { v0 += dst[0]; v1 += dst[1]; }
                else if (a.op == ACRO_B200_OP_SUB) { v0 = dst[0] - v0; v1 = dst[1] - v1; }
                if (aligned16(a.C)) __stcs(reinterpret_cast<double2 *>(dst), make_double2(v0, v1));
                else { __stcs(dst, v0); __stcs(dst + 1, v1); }
            }
    }
}

}

extern "C" {

int acro_b200_batched_gemm_supported(int m, int n, int k)
{
    return ((m == n && n == k && (m == 64 || m == 32)) || batched_gemm_small_supported(m, n, k)) ? 1 : 0;
}

int acro_b200_batched_gemm(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k, int op, void *stream)
{
    if (A == nullptr || B == nullptr || C == nullptr) return fail_invalid("acro_b200_batched_gemm: null argument");
    if (batch < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_batched_gemm: bad batch or operator");
    if (!acro_b200_batched_gemm_supported(m, n, k)) return fail_unsupported("acro_b200_batched_gemm: built for 64^3, 32^3 and every m, n, k <= 16");
    if (batched_gemm_small_supported(m, n, k)) return batched_gemm_small_launch(A, B, C, batch, m, n, k, op, as_stream(stream));
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_batched_gemm");

    GemmArgs args;
    args.A = A;
    args.B = B;
    args.C = C;
    args.batch = batch;
    args.op = op;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_batched_gemm (status flag)");
    args.async_copy = (aligned16(A) && aligned16(B)) ? 1 : 0;

    auto kernel = m == 64 ? batched_gemm_kernel<64> : batched_gemm_kernel<32>;
    const size_t smem = m == 64 ? sizeof(Smem<64>) : sizeof(Smem<32>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int64_t grid = static_cast<int64_t>(sms) * (m == 64 ? 1 : 4);
    if (grid > batch) grid = batch;
    kernel<<<static_cast<int>(grid), NT, smem, as_stream(stream)>>>(args);
    return launch_status("acro_b200_batched_gemm");
}

}
