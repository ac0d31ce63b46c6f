// batched_gemm: C_e = A_e * B_e for a batch of small dense fp64 matrices (64 x 64 x 64).
//
// Persistent CTAs (one per SM, 8 warps) walk over the batch.  A_e and B_e (32 KB each,
// contiguous) arrive through a three-stage ring of asynchronous bulk copies, one copy per
// matrix row into rows padded to 68 doubles so that DMMA fragment loads are bank-conflict
// free; the copies of elements e+1 and e+2 are in flight while element e is multiplied.
// Each warp owns a 16 x 32 block of C: 8 accumulator tiles of mma.sync m8n8k4 (fp64 tensor
// cores), 6 shared-memory fragment loads per 8 MMAs.  C leaves straight from the
// accumulator registers as full 64-byte row segments.
//
// Algorithmic HBM traffic: 3 * 8 * 64 * 64 = 98,304 bytes per element; 2 * 64^3 = 524,288
// flops per element (arithmetic intensity 5.33 flop/byte, the fp64 ridge of a B200).
#include "common.cuh"
#include "dmma.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int N = 64;                 // matrix extent
constexpr int LD = N + 4;             // padded row: 68 doubles (544 bytes, a 16-byte multiple)
constexpr int STAGES = 3;
constexpr int NT = 256;               // 8 warps
constexpr int MAT = N * LD;           // doubles per padded matrix

struct Smem
{
    double A[STAGES][MAT];
    double B[STAGES][MAT];
    uint64_t full[STAGES];
};

struct GemmArgs
{
    const double *A;
    const double *B;
    double *C;
    int64_t batch;
    int op;
    int *wait_flag;
    int use_bulk;
};

__device__ __forceinline__ void issue_element_load(Smem &s, const GemmArgs &a, int64_t e, int stage)
{
    if (e >= a.batch) return;
    const int tid = threadIdx.x;
    if (a.use_bulk && tid < 32)
    {
        // warp 0 issues all 128 row copies; the byte count is announced first
        if (tid == 0) mbar_arrive_expect_tx(&s.full[stage], 2 * N * N * 8);
        __syncwarp();
#pragma unroll
        for (int r = tid; r < N; r += 32)
        {
            bulk_load(&s.A[stage][r * LD], a.A + e * N * N + r * N, N * 8, &s.full[stage]);
            bulk_load(&s.B[stage][r * LD], a.B + e * N * N + r * N, N * 8, &s.full[stage]);
        }
    }
}

__global__ void __launch_bounds__(NT, 1)
batched_gemm64_kernel(const GemmArgs a)
{
    extern __shared__ __align__(128) unsigned char raw[];
    Smem &s = *reinterpret_cast<Smem *>(raw);
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp >> 1) * 16, n0 = (warp & 1) * 32;

    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i) mbar_init(&s.full[i], 1);
        fence_mbar_init();
    }
    __syncthreads();

    // prologue: fill the ring
    int64_t e = blockIdx.x;
    for (int i = 0; i < STAGES - 1; ++i) issue_element_load(s, a, e + static_cast<int64_t>(i) * gridDim.x, i);

    uint32_t phase_bits = 0;   // bit i = parity to wait for on stage i
    int stage = 0;
    for (; e < a.batch; e += gridDim.x)
    {
        // keep the ring full: the slot two elements ahead was released by the barrier that
        // closed the previous iteration
        issue_element_load(s, a, e + static_cast<int64_t>(STAGES - 1) * gridDim.x, (stage + STAGES - 1) % STAGES);

        if (a.use_bulk)
        {
            if (!mbar_wait(&s.full[stage], (phase_bits >> stage) & 1u)) atomicExch(a.wait_flag, 1);
            phase_bits ^= (1u << stage);
        }
        else
        {
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
        double c[2][4][2];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;

#pragma unroll 4
        for (int k0 = 0; k0 < N; k0 += 4)
        {
            double af[2], bf[4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) af[mt] = sa[(m0 + mt * 8 + g) * LD + k0 + t];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) bf[nt] = sb[(k0 + t) * LD + n0 + nt * 8 + g];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) dmma_m8n8k4(c[mt][nt], af[mt], bf[nt]);
        }

        // C rows leave as 64-byte segments per quad (two doubles per lane)
        double *gc = a.C + e * N * N;
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
            {
                double *dst = gc + (m0 + mt * 8 + g) * N + n0 + nt * 8 + 2 * t;
                double v0 = c[mt][nt][0], v1 = c[mt][nt][1];
                if (a.op == ACRO_B200_OP_ADD) { v0 += dst[0]; v1 += dst[1]; }
                else if (a.op == ACRO_B200_OP_SUB) { v0 = dst[0] - v0; v1 = dst[1] - v1; }
                if (aligned16(a.C)) __stcs(reinterpret_cast<double2 *>(dst), make_double2(v0, v1));
                else { __stcs(dst, v0); __stcs(dst + 1, v1); }
            }

        __syncthreads();   // every warp is done with this stage: it may be refilled
        stage = (stage + 1) % STAGES;
    }
}

}

extern "C" {

int acro_b200_batched_gemm_supported(int m, int n, int k) { return (m == N && n == N && k == N) ? 1 : 0; }

int acro_b200_batched_gemm(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k, int op, void *stream)
{
    if (A == nullptr || B == nullptr || C == nullptr) return fail_invalid("acro_b200_batched_gemm: null argument");
    if (batch < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_batched_gemm: bad batch or operator");
    if (!acro_b200_batched_gemm_supported(m, n, k)) return fail_unsupported("acro_b200_batched_gemm: only 64 x 64 x 64 is instantiated");
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
    args.use_bulk = (aligned16(A) && aligned16(B)) ? 1 : 0;

    const size_t smem = sizeof(Smem);
    cudaError_t status = cudaFuncSetAttribute(batched_gemm64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int64_t grid = sms;
    if (grid > batch) grid = batch;
    batched_gemm64_kernel<<<static_cast<int>(grid), NT, smem, as_stream(stream)>>>(args);
    return launch_status("acro_b200_batched_gemm");
}

}
