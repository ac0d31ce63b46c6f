// gemm: C[M x N] (op)= A[M x K] * P[K x N], row-major fp64 with leading dimensions, on the fp64
// tensor cores (mma.sync m8n8k4).
//
// It serves contractions in which exactly one input carries the batch index and all of that
// input's other indices are contracted ("assembly" strings such as
// M_e_i1_i2_j1_j2 = B_k1_i1 B_k1_j1 B_k2_i2 B_k2_j2 D_e_k1_k2): the batch-invariant inputs are
// multiplied out once into P[(contracted indices) x (output indices)] and the contraction becomes
// one GEMM with the batch as its row dimension.
//
// Persistent CTAs (8 warps, two or three per SM) walk over 64 x 64 tiles of C; for every tile the K
// extent is walked in slabs of 32 (16 when K is that small) through a three-slot ring of shared-memory buffers (rows padded by four doubles:
// conflict-free fragment loads), filled by cp.async (16-byte chunks when rows are 16-byte
// multiples on 16-byte boundaries, else 8-byte) with completion on "full" mbarriers and reuse
// gated by "empty" mbarriers, so warps do not meet at a CTA barrier.  Only the valid part of a
// slab is copied; the up to three columns of A (rows of P) that pad K to a multiple of four are
// written as zeros by the copy itself (source size 0), rows of A beyond M and columns of P beyond
// N are left as they are: they only reach entries of C that are never stored.  A warp owns a
// 16 x 32 block of the tile (8 accumulator tiles, kept in registers across the slabs).
#include "common.cuh"
#include "dmma.cuh"
#include "tma.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int T = 64;                  // tile edge and slab depth
constexpr int LD = T + 4;              // padded shared-memory row
constexpr int STAGES = 3;
constexpr int NT = 256;

// KT: slab depth, 32 (16 when K is that small): the ring then leaves room for two (three) CTAs per SM, so that
// one CTA's copies and stores overlap another's tensor-core loop
template <int KT>
struct Smem
{
    static constexpr int LDA = KT + 4;      // padded row of the A slot (4 mod 16 doubles: conflict-free fragment loads)
    double A[STAGES][T * LDA];
    double P[STAGES][KT * LD];
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
};

struct GemmArgs
{
    const double *A;
    const double *P;
    double *C;
    int64_t M, N, K, lda, ldp, ldc;
    int64_t batch, stride_a, stride_p, stride_c;      // independent products: element e starts stride_* doubles further on
    int op;
    int wide_a, wide_p;       // 16-byte copies allowed for the operand
    int shift_a;              // lda is odd: rows of A that start on an odd element sit one column to the right in shared memory
    int *wait_flag;
};

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// `bytes` of the chunk come from global memory, the rest is written as zeros.  The form with a source
// size is kept for the chunks that need it: whole chunks take the plain form.
__device__ __forceinline__ void copy16(double *dst, const double *src, int bytes)
{
    if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
    else asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void copy8(double *dst, const double *src, int bytes)
{
    if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}

// Copies slab `kt` of tile (tm, tn) into slot `stage`; k4 = slab depth padded to a multiple of four.
template <int KT>
__device__ __forceinline__ void issue_slab(Smem<KT> &s, const GemmArgs &a, int64_t e, int64_t tm, int64_t tn, int64_t kt, int k4, int stage)
{
    const double *A = a.A + e * a.stride_a, *P = a.P + e * a.stride_p;
    const int par_e = static_cast<int>((e & a.stride_a) & 1);      // parity of the element's first entry (the base of a.A is 16-byte aligned)
    constexpr int LDA = Smem<KT>::LDA;
    constexpr int CPR = KT / 2;                 // 16-byte chunks per row of the A tile
    const int tid = threadIdx.x;
    const int64_t row0 = tm * T, col0 = tn * T, k0 = kt * KT;
    const int rows = a.M - row0 < T ? static_cast<int>(a.M - row0) : T;         // valid rows of the A tile
    const int cols = a.N - col0 < T ? static_cast<int>(a.N - col0) : T;         // valid columns of the P tile
    const int depth = a.K - k0 < KT ? static_cast<int>(a.K - k0) : KT;          // valid depth of the slab (k4 - depth in 0..3)

    if (a.wide_a && !a.shift_a && a.wide_p && rows == T && cols == T && depth == KT)
    {
        // interior slab: whole 16-byte chunks only, addresses by shifts
        const double *ga = A + row0 * a.lda + k0, *gp = P + k0 * a.ldp + col0;
#pragma unroll
        for (int i = 0; i < T * CPR / NT; ++i)
        {
            const int c = tid + i * NT;
            const int r = c / CPR, col = (c % CPR) * 2;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.A[stage][r * LDA + col])), "l"(ga + r * a.lda + col) : "memory");
        }
#pragma unroll
        for (int i = 0; i < KT * (T / 2) / NT; ++i)
        {
            const int c = tid + i * NT;
            const int r = c >> 5, col = (c & 31) * 2;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.P[stage][r * LD + col])), "l"(gp + r * a.ldp + col) : "memory");
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&s.full[stage])) : "memory");
        return;
    }
    // Edge slabs, odd leading dimensions, unaligned operands: the same fixed assignment of chunks to threads,
    // every copy guarded by what is valid.  The passes are unrolled and independent of one another (a loop with
    // run-time bounds made the address arithmetic one long dependent chain, which two warps per scheduler
    // cannot hide: measured 30 % slower at K = 60 than at K = 64).
    // A tile: rows x k4.  With an odd lda every other row starts on an odd element; such a row is stored one
    // column to the right (sh = 1), so that pairs that are 16-byte aligned in global memory are so in shared
    // memory too; its first entry travels alone and its last chunk is number 32.
    if (a.wide_a)
    {
#pragma unroll
        for (int i = 0; i < T * CPR / NT; ++i)
        {
            const int c = tid + i * NT;
            const int r = c / CPR, cc = c % CPR;
            const int sh = a.shift_a ? (par_e ^ static_cast<int>((row0 + r) & a.lda & 1)) : 0;
            if (r < rows && 2 * cc < k4 + sh)
            {
                const double *src = A + (row0 + r) * a.lda + k0;
                const int c0 = 2 * cc - sh;           // slab column of the chunk's first slot
                double *dst = &s.A[stage][r * LDA + 2 * cc];
                const int left = depth - c0;          // valid doubles from this chunk on
                if (c0 < 0) copy8(dst + 1, src, 8);
                else copy16(dst, left > 0 ? src + c0 : a.A, left >= 2 ? 16 : (left == 1 ? 8 : 0));
            }
        }
        if (a.shift_a && k4 == KT && tid < rows && (par_e ^ static_cast<int>((row0 + tid) & a.lda & 1)))
        {
            // the extra chunk of a shifted row: slab column KT - 1 and one slot of padding
            const int left = depth - (KT - 1);
            copy16(&s.A[stage][tid * LDA + KT], left > 0 ? A + (row0 + tid) * a.lda + k0 + KT - 1 : a.A, left > 0 ? 8 : 0);
        }
    }
    else
    {
#pragma unroll
        for (int i = 0; i < T * KT / NT; ++i)
        {
            const int c = tid + i * NT;
            const int r = c / KT, col = c % KT;
            if (r < rows && col < k4) copy8(&s.A[stage][r * LDA + col], A + (row0 + r) * a.lda + k0 + (col < depth ? col : 0), col < depth ? 8 : 0);
        }
    }
    // P tile: k4 x cols; rows of the padding are written as zeros
    if (a.wide_p)
    {
#pragma unroll
        for (int i = 0; i < KT * (T / 2) / NT; ++i)
        {
            const int c = tid + i * NT;
            const int r = c >> 5, cc = c & 31;
            if (r < k4 && 2 * cc < cols)
            {
                const int left = r < depth ? cols - 2 * cc : 0;
                copy16(&s.P[stage][r * LD + 2 * cc], left > 0 ? P + (k0 + r) * a.ldp + col0 + 2 * cc : a.P, left >= 2 ? 16 : (left == 1 ? 8 : 0));
            }
        }
    }
    else
    {
#pragma unroll
        for (int i = 0; i < KT * T / NT; ++i)
        {
            const int c = tid + i * NT;
            const int r = c >> 6, col = c & 63;
            if (r < k4 && col < cols) copy8(&s.P[stage][r * LD + col], r < depth ? P + (k0 + r) * a.ldp + col0 + col : a.P, r < depth ? 8 : 0);
        }
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&s.full[stage])) : "memory");
}

template <int KT>
__global__ void __launch_bounds__(NT, KT == 32 ? 2 : 3)
gemm_f64_kernel(const GemmArgs a)
{
    constexpr int LDA = Smem<KT>::LDA;
    extern __shared__ __align__(128) unsigned char raw[];
    Smem<KT> &s = *reinterpret_cast<Smem<KT> *>(raw);
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp >> 1) * 16, n0 = (warp & 1) * 32;
    constexpr int MT = 2, NTL = 4;
    const bool pairs = aligned16(a.C) && a.ldc % 2 == 0 && a.stride_c % 2 == 0;      // entry pairs of C sit on 16-byte boundaries

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

    // 32-bit bookkeeping (the launcher checks the tile count): 64-bit divisions per step would cost
    // more than the step's tensor-core loop
    const int tiles_m = static_cast<int>((a.M + T - 1) / T), tiles_n = static_cast<int>((a.N + T - 1) / T);
    const int slabs = static_cast<int>((a.K + KT - 1) / KT);
    const int per_matrix = tiles_m * tiles_n;
    const int n_tiles = per_matrix * static_cast<int>(a.batch);
    const int last_k4 = (static_cast<int>(a.K - static_cast<int64_t>(slabs - 1) * KT) + 3) & ~3;

    // position of the slab being multiplied and of the slab being fetched (one step ahead); tiles run
    // down the rows of C first, so that CTAs working side by side share the same slabs of P
    // tile number -> (element, column tile, row tile), row tile fastest
    int tile = blockIdx.x, kt = 0, te = tile / per_matrix, tm = (tile % per_matrix) % tiles_m, tn = (tile % per_matrix) / tiles_m;
    int f_tile = tile, f_kt = 0, f_te = te, f_tm = tm, f_tn = tn;
    unsigned int fetched = 0;      // slabs fetched so far: slab number `fetched` goes to slot fetched % STAGES

    auto fetch = [&]() {
        const unsigned int slot = fetched % STAGES, use = fetched / STAGES;      // use: how often the slot was filled before
        if (use > 0 && !mbar_wait(&s.empty[slot], (use - 1) & 1u)) atomicExch(a.wait_flag, 1);
        issue_slab<KT>(s, a, f_te, f_tm, f_tn, f_kt, f_kt == slabs - 1 ? last_k4 : KT, static_cast<int>(slot));
        ++fetched;
        if (++f_kt == slabs)
        {
            f_kt = 0;
            f_tile += gridDim.x;
            f_te = f_tile / per_matrix;
            f_tm = (f_tile % per_matrix) % tiles_m;
            f_tn = (f_tile % per_matrix) / tiles_m;
        }
    };

    if (tile < n_tiles) fetch();
    double c[MT][NTL][2];
    for (unsigned int step = 0; tile < n_tiles; ++step)
    {
        const int stage = static_cast<int>(step % STAGES);
        if (f_tile < n_tiles) fetch();          // one slab ahead, into the slot read two steps ago
        if (!mbar_wait(&s.full[stage], (step / STAGES) & 1u)) atomicExch(a.wait_flag, 1);

        if (kt == 0)
        {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;
        }
        const double *sa = s.A[stage];
        const double *sp = s.P[stage];
        const int k4 = kt == slabs - 1 ? last_k4 : KT;
        // rows of A stored one column to the right (odd lda): m0 + mt * 8 is even, so the parity is that of tile row g
        const int sh = a.shift_a ? (static_cast<int>((te & a.stride_a) & 1) ^ static_cast<int>(g & a.lda & 1)) : 0;
#pragma unroll 4
        for (int k0 = 0; k0 < k4; k0 += 4)
        {
            double af[MT], bf[NTL];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) af[mt] = sa[(m0 + mt * 8 + g) * LDA + sh + k0 + t];
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) bf[nt] = sp[(k0 + t) * LD + n0 + nt * 8 + g];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) dmma_m8n8k4(c[mt][nt], af[mt], bf[nt]);
        }
        mbar_arrive(&s.empty[stage]);   // this thread no longer reads the slot

        if (kt == slabs - 1)
        {
            const int64_t row0 = static_cast<int64_t>(tm) * T, col0 = static_cast<int64_t>(tn) * T;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
            {
                const int64_t i = row0 + m0 + mt * 8 + g;
                if (i >= a.M) continue;
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt)
                {
                    const int64_t j = col0 + n0 + nt * 8 + 2 * t;
                    double *dst = a.C + te * a.stride_c + i * a.ldc + j;
                    if (pairs && j + 1 < a.N)
                    {
                        // both entries of the lane as one 16-byte store: a quad writes a 64-byte row segment
                        double v0 = c[mt][nt][0], v1 = c[mt][nt][1];
                        if (a.op == ACRO_B200_OP_ADD) { v0 += dst[0]; v1 += dst[1]; }
                        else if (a.op == ACRO_B200_OP_SUB) { v0 = dst[0] - v0; v1 = dst[1] - v1; }
                        __stcs(reinterpret_cast<double2 *>(dst), make_double2(v0, v1));
                        continue;
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                    {
                        if (j + h >= a.N) continue;
                        double v = c[mt][nt][h];
                        if (a.op == ACRO_B200_OP_ADD) v += dst[h];
                        else if (a.op == ACRO_B200_OP_SUB) v = dst[h] - v;
                        __stcs(dst + h, v);
                    }
                }
            }
        }
        if (++kt == slabs)
        {
            kt = 0;
            tile += gridDim.x;
            te = tile / per_matrix;
            tm = (tile % per_matrix) % tiles_m;
            tn = (tile % per_matrix) / tiles_m;
        }
    }
}

}

extern "C" int acro_b200_gemm_batched(const double *A, const double *P, double *C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                                      int64_t ldp, int64_t ldc, int64_t stride_a, int64_t stride_p, int64_t stride_c, int op, void *stream)
{
    if (A == nullptr || P == nullptr || C == nullptr) return fail_invalid("acro_b200_gemm: null argument");
    if (batch < 1 || M < 1 || N < 1 || K < 1 || lda < K || ldp < N || ldc < N || op < 0 || op > 2 || stride_a < 0 || stride_p < 0 || stride_c < 0)
        return fail_invalid("acro_b200_gemm: bad sizes, leading dimensions, strides or operator");
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_gemm");
    GemmArgs args;
    args.A = A;
    args.P = P;
    args.C = C;
    args.M = M;
    args.N = N;
    args.K = K;
    args.lda = lda;
    args.ldp = ldp;
    args.ldc = ldc;
    args.batch = batch;
    args.stride_a = stride_a;
    args.stride_p = stride_p;
    args.stride_c = stride_c;
    args.op = op;
    args.wide_a = aligned16(A) ? 1 : 0;
    args.shift_a = (args.wide_a && (lda % 2 != 0 || stride_a % 2 != 0)) ? 1 : 0;
    args.wide_p = (aligned16(P) && ldp % 2 == 0 && stride_p % 2 == 0) ? 1 : 0;
    args.wait_flag = wait_flag_device_ptr();
    if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_gemm (status flag)");
    const int64_t tiles = batch * ((M + T - 1) / T) * ((N + T - 1) / T);
    if (tiles > (int64_t(1) << 30) || K > (int64_t(1) << 30)) return fail_unsupported("acro_b200_gemm: more than 2^30 tiles of C or K above 2^30");
    auto launch = [&](auto kernel, size_t smem, int per_sm) {
        cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_gemm (shared memory opt-in)");
        int64_t grid = static_cast<int64_t>(sms) * per_sm;
        if (grid > tiles) grid = tiles;
        kernel<<<static_cast<int>(grid), NT, smem, as_stream(stream)>>>(args);
        return ACRO_B200_OK;
    };
    // Slab depth 32 with two CTAs per SM beats depth 64 with one for every K measured (K = 60 ... 1125: 24.7-30.4
    // against 16.0-30.0 TFLOP/s): one CTA's copies and stores overlap the other's tensor-core loop.
    int status;
    if (K <= 16) status = launch(gemm_f64_kernel<16>, sizeof(Smem<16>), 3);
    else status = launch(gemm_f64_kernel<32>, sizeof(Smem<32>), 2);
    if (status != ACRO_B200_OK) return status;
    return launch_status("acro_b200_gemm");
}

extern "C" int acro_b200_gemm(const double *A, const double *P, double *C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldp,
                              int64_t ldc, int op, void *stream)
{
    return acro_b200_gemm_batched(A, P, C, 1, M, N, K, lda, ldp, ldc, 0, 0, 0, op, stream);
}
