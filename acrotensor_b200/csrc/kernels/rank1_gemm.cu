// rank1_gemm: M[e,i,j] (op)= sum_q W[e,q] * B1[q,i] * B2[q,j]   (element mass-matrix assembly).
//
// Viewed as one GEMM  M[e,(i,j)] = sum_q W[e,q] * BB[q,(i,j)],  BB[q,(i,j)] = B1[q,i]*B2[q,j]:
// E x 64 times 64 x (NI*NJ).  It is compute bound on fp64 (2*64*NI*NJ flops against
// 8*(64 + NI*NJ) bytes per element: 14.7 flop/byte for 27 x 27), so it runs on the fp64
// tensor cores (mma.sync m8n8k4).  A CTA owns 32 elements: their W rows arrive by
// asynchronous bulk copies into rows padded to 68 doubles (conflict-free fragment loads),
// double buffered; B1, B2 sit in shared memory for the whole kernel and the BB operand is
// formed on the fly (one multiply per fragment entry, reused by the four 8-element row
// tiles of the warp: 3 % extra fp64 work).  A warp computes 32 elements x 32 columns at a
// time (16 accumulator tiles), then routes each 8 x 32 block through a small per-warp
// staging area so that rows leave as contiguous 256-byte stores.
//
// Algorithmic HBM traffic per element: 8*64 (W) + 8*NI*NJ (M) bytes.
#include "common.cuh"
#include "dmma.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int QN = 64;                 // contracted extent
constexpr int ET = 32;                 // elements per CTA tile (4 row tiles of 8)
constexpr int LDW = QN + 4;            // padded W row
constexpr int NTHREADS = 256;
constexpr int WARPS = NTHREADS / 32;
constexpr int MAXN = 32;               // NI, NJ <= 32
constexpr int LDS_STAGE = 40;          // staging row (doubles)

struct Smem
{
    double W[2][ET * LDW];
    double B1[QN * MAXN];
    double B2[QN * MAXN];
    double stage[WARPS][8 * LDS_STAGE];
    uint64_t full[2];
};

struct Rank1Args
{
    const double *W;
    const double *B1;
    const double *B2;
    double *M;
    int64_t elements;
    int ni, nj;
    int op;
    int *wait_flag;
    int use_bulk;
};

__device__ __forceinline__ void issue_w_load(Smem &s, const Rank1Args &a, int64_t tile, int buf)
{
    const int64_t e0 = tile * ET;
    if (!a.use_bulk || e0 >= a.elements) return;
    if (threadIdx.x < 32)
    {
        const int64_t left = a.elements - e0;
        const int n_e = left < ET ? static_cast<int>(left) : ET;
        if (threadIdx.x == 0) mbar_arrive_expect_tx(&s.full[buf], n_e * QN * 8);
        __syncwarp();
        if (static_cast<int>(threadIdx.x) < n_e)
            bulk_load(&s.W[buf][threadIdx.x * LDW], a.W + (e0 + threadIdx.x) * QN, QN * 8, &s.full[buf]);
    }
}

__global__ void __launch_bounds__(NTHREADS, 2)
rank1_gemm_kernel(const Rank1Args a)
{
    extern __shared__ __align__(128) unsigned char raw[];
    Smem &s = *reinterpret_cast<Smem *>(raw);
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ni = a.ni, nj = a.nj, nc = ni * nj;
    const int n_groups = (nc + 31) / 32;
    const int64_t n_tiles = (a.elements + ET - 1) / ET;

    if (tid == 0)
    {
        mbar_init(&s.full[0], 1);
        mbar_init(&s.full[1], 1);
        fence_mbar_init();
    }
    for (int i = tid; i < QN * ni; i += NTHREADS) s.B1[i] = a.B1[i];
    for (int i = tid; i < QN * nj; i += NTHREADS) s.B2[i] = a.B2[i];
    __syncthreads();

    int64_t tile = blockIdx.x;
    issue_w_load(s, a, tile, 0);
    uint32_t phase_bits = 0;
    int buf = 0;
    double *stg = s.stage[warp];

    for (; tile < n_tiles; tile += gridDim.x)
    {
        issue_w_load(s, a, tile + gridDim.x, buf ^ 1);   // released by the barrier that closed the previous tile
        const int64_t e0 = tile * ET;
        const int64_t left = a.elements - e0;
        const int n_e = left < ET ? static_cast<int>(left) : ET;
        if (a.use_bulk)
        {
            if (!mbar_wait(&s.full[buf], (phase_bits >> buf) & 1u)) atomicExch(a.wait_flag, 1);
            phase_bits ^= (1u << buf);
        }
        else
        {
            for (int i = tid; i < n_e * QN; i += NTHREADS) s.W[buf][(i / QN) * LDW + (i % QN)] = __ldcs(a.W + e0 * QN + i);
            __syncthreads();
        }
        const double *sw = s.W[buf];

        for (int grp = warp; grp < n_groups; grp += WARPS)
        {
            const int c0 = grp * 32;
            // column -> (i, j) of this lane's B-fragment column in each of the 4 column tiles
            int off1[4], off2[4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
            {
                int c = c0 + nt * 8 + g;
                c = c < nc ? c : nc - 1;          // padded columns compute a copy that is never stored
                off1[nt] = c / nj;
                off2[nt] = c - off1[nt] * nj;
            }
            double acc[4][4][2];
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = 0.0;

#pragma unroll 2
            for (int k0 = 0; k0 < QN; k0 += 4)
            {
                double af[4], bf[4];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) af[mt] = sw[(mt * 8 + g) * LDW + k0 + t];
                const double *b1 = s.B1 + (k0 + t) * ni;
                const double *b2 = s.B2 + (k0 + t) * nj;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) bf[nt] = b1[off1[nt]] * b2[off2[nt]];
#pragma unroll
                for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) dmma_m8n8k4(acc[mt][nt], af[mt], bf[nt]);
            }

            // epilogue: 8 x 32 blocks through the warp's staging rows, then contiguous row stores
            const int col = c0 + lane;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
            {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
                    *reinterpret_cast<double2 *>(stg + g * LDS_STAGE + nt * 8 + 2 * t) = make_double2(acc[mt][nt][0], acc[mt][nt][1]);
                __syncwarp();
                if (col < nc)
                {
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                    {
                        const int el = mt * 8 + r;
                        if (el < n_e)
                        {
                            double *dst = a.M + (e0 + el) * nc + col;
                            double v = stg[r * LDS_STAGE + lane];
                            if (a.op == ACRO_B200_OP_ADD) v += *dst;
                            else if (a.op == ACRO_B200_OP_SUB) v = *dst - v;
                            __stcs(dst, v);
                        }
                    }
                }
                __syncwarp();
            }
        }
        __syncthreads();   // every warp is done with this W buffer
        buf ^= 1;
    }
}

}

extern "C" {

int acro_b200_rank1_gemm_supported(int q, int ni, int nj)
{
    return (q == QN && ni >= 1 && ni <= MAXN && nj >= 1 && nj <= MAXN) ? 1 : 0;
}

int acro_b200_rank1_gemm(const double *W, const double *B1, const double *B2, double *M, int64_t elements, int q, int ni, int nj,
                         int op, void *stream)
{
    if (W == nullptr || B1 == nullptr || B2 == nullptr || M == nullptr) return fail_invalid("acro_b200_rank1_gemm: null argument");
    if (elements < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_rank1_gemm: bad element count or operator");
    if (!acro_b200_rank1_gemm_supported(q, ni, nj)) return fail_unsupported("acro_b200_rank1_gemm: needs q = 64 and 1 <= ni, nj <= 32");
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_rank1_gemm");

    Rank1Args args;
    args.W = W;
    args.B1 = B1;
    args.B2 = B2;
    args.M = M;
    args.elements = elements;
    args.ni = ni;
    args.nj = nj;
    args.op = op;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_rank1_gemm (status flag)");
    args.use_bulk = aligned16(W) ? 1 : 0;

    const size_t smem = sizeof(Smem);
    cudaError_t status = cudaFuncSetAttribute(rank1_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_rank1_gemm (shared memory opt-in)");
    const int64_t n_tiles = (elements + ET - 1) / ET;
    int64_t grid = static_cast<int64_t>(sms) * 2;
    if (grid > n_tiles) grid = n_tiles;
    rank1_gemm_kernel<<<static_cast<int>(grid), NTHREADS, smem, as_stream(stream)>>>(args);
    return launch_status("acro_b200_rank1_gemm");
}

}
