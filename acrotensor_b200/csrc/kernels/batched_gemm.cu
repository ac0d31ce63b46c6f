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
// Transposed operands (A_e stored as k x m, B_e stored as n x k; template flags TA, TB): the copies
// are the same, only the fragment loads swap their two strides; with rows padded to 4 (mod 16)
// doubles both orientations are free of bank conflicts.
//
// Algorithmic HBM traffic: 3 * 8 * 64 * 64 = 98,304 bytes per element; 2 * 64^3 = 524,288
// flops per element (arithmetic intensity 5.33 flop/byte, the fp64 ridge of a B200).
#include "common.cuh"
#include "dmma.cuh"
#include "tma.cuh"
#include "tensormap.cuh"

#include <cstdlib>

using namespace acro_b200_detail;

namespace
{

constexpr int STAGES = 3;
constexpr int NT = 256;               // 8 warps
constexpr int kGramMaxParts = 1024;   // partial tiles of the Gram form: one per CTA, plus one for the last rows

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

// Fragments of mma.sync m8n8k4 from a padded slot: A(i, kk) and B(kk, j) in either storage order.
template <int LD, bool T>
__device__ __forceinline__ double frag_a(const double *sa, int i, int kk) { return T ? sa[kk * LD + i] : sa[i * LD + kk]; }
template <int LD, bool T>
__device__ __forceinline__ double frag_b(const double *sb, int kk, int j) { return T ? sb[j * LD + kk] : sb[kk * LD + j]; }

template <int N, bool TA, bool TB>
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
            for (int mt = 0; mt < MT; ++mt) af[mt] = frag_a<LD, TA>(sa, m0 + mt * 8 + g, k0 + t);
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) bf[nt] = frag_b<LD, TB>(sb, k0 + t, n0 + nt * 8 + g);
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


// ------------------------------------------------------------------ any m, n, k up to N
// The same ring and the same warp tiling for matrices that do not fill the N x N slots: the slots are
// zeroed once, every element's entries are copied to the top-left corner of its slots (16-byte cp.async
// when rows are 16-byte multiples on 16-byte boundaries, else 8-byte), so the padding rows and columns
// stay zero and add nothing; the contracted extent is walked in steps of four up to its padded value,
// accumulator tiles that lie entirely outside C are skipped, and only the valid entries of C are stored.
struct PaddedArgs
{
    const double *A;
    const double *B;
    double *C;
    int64_t batch;
    int m, n, k, op;
    int rows_a, cols_a, rows_b, cols_b;      // the operands as stored: A is m x k (k x m when transposed), B is k x n (n x k)
    int *wait_flag;
    int wide;        // rows of A and B are 16-byte multiples on 16-byte boundaries: 16-byte copies
};

template <int N>
__device__ __forceinline__ void issue_padded_load(Smem<N> &s, const PaddedArgs &a, int64_t e, int stage)
{
    constexpr int LD = Smem<N>::LD;
    const int tid = threadIdx.x;
    const double *ga = a.A + e * a.m * a.k, *gb = a.B + e * a.k * a.n;
    if (a.wide)
    {
        const int ca = a.cols_a / 2, cb = a.cols_b / 2;          // 16-byte chunks per row
        int col = tid % ca, row = tid / ca;
        const int sc = NT % ca, sr = NT / ca;
        for (int c = tid; row < a.rows_a; c += NT)
        {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.A[stage][row * LD + col * 2])), "l"(ga + c * 2) : "memory");
            col += sc;
            if (col >= ca) { col -= ca; ++row; }
            row += sr;
        }
        col = tid % cb, row = tid / cb;
        const int tc = NT % cb, tr = NT / cb;
        for (int c = tid; row < a.rows_b; c += NT)
        {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.B[stage][row * LD + col * 2])), "l"(gb + c * 2) : "memory");
            col += tc;
            if (col >= cb) { col -= cb; ++row; }
            row += tr;
        }
    }
    else
    {
        int col = tid % a.cols_a, row = tid / a.cols_a;
        const int sc = NT % a.cols_a, sr = NT / a.cols_a;
        for (int c = tid; row < a.rows_a; c += NT)
        {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr(&s.A[stage][row * LD + col])), "l"(ga + c) : "memory");
            col += sc;
            if (col >= a.cols_a) { col -= a.cols_a; ++row; }
            row += sr;
        }
        col = tid % a.cols_b, row = tid / a.cols_b;
        const int tc = NT % a.cols_b, tr = NT / a.cols_b;
        for (int c = tid; row < a.rows_b; c += NT)
        {
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_addr(&s.B[stage][row * LD + col])), "l"(gb + c) : "memory");
            col += tc;
            if (col >= a.cols_b) { col -= a.cols_b; ++row; }
            row += tr;
        }
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&s.full[stage])) : "memory");
}

// ACC: the products of all elements a CTA walks over are summed in its accumulators and the CTA stores one
// m x n tile of partial sums at C + blockIdx.x * m * n when it is done (the Gram form below).
template <int N, bool TA, bool TB, bool ACC = false>
__global__ void __launch_bounds__(NT, N == 64 ? 1 : 4)
batched_gemm_padded_kernel(const PaddedArgs a)
{
    constexpr int LD = Smem<N>::LD;
    constexpr int MT = N / 32, NTL = N / 16;
    extern __shared__ __align__(128) unsigned char raw[];
    Smem<N> &s = *reinterpret_cast<Smem<N> *>(raw);
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = (warp >> 1) * (N / 4), n0 = (warp & 1) * (N / 2);
    const int m = a.m, n = a.n;
    const int k4 = (a.k + 3) & ~3;

    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i)
        {
            mbar_init(&s.full[i], NT);
            mbar_init(&s.empty[i], NT);
        }
        fence_mbar_init();
    }
    for (int i = tid; i < STAGES * Smem<N>::MAT; i += NT)
    {
        (&s.A[0][0])[i] = 0.0;
        (&s.B[0][0])[i] = 0.0;
    }
    __syncthreads();

    double c[MT][NTL][2];
    bool row_live[MT], col_live[NTL];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) row_live[mt] = m0 + mt * 8 < m;
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) col_live[nt] = n0 + nt * 8 < n;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;

    // Elements in flight ahead of the one being multiplied.  One leaves a slot of slack, so that warps may drift
    // apart by an element; the Gram form has short elements and nothing to store per element, and fills every slot.
    constexpr int AHEAD = ACC ? STAGES - 1 : 1;
    int64_t e = blockIdx.x;
#pragma unroll
    for (int d = 0; d < AHEAD; ++d)
    {
        if (e + static_cast<int64_t>(d) * gridDim.x < a.batch) issue_padded_load(s, a, e + static_cast<int64_t>(d) * gridDim.x, d);
    }

    int64_t it = 0;
    for (; e < a.batch; e += gridDim.x, ++it)
    {
        const int stage = static_cast<int>(it % STAGES);
        const int64_t nxt = e + static_cast<int64_t>(AHEAD) * gridDim.x;
        if (nxt < a.batch)
        {
            const int ns = static_cast<int>((it + AHEAD) % STAGES);
            const int64_t use = (it + AHEAD) / STAGES;      // how often that slot was filled before
            if (use > 0 && !mbar_wait(&s.empty[ns], static_cast<uint32_t>((use - 1) & 1))) atomicExch(a.wait_flag, 1);
            issue_padded_load(s, a, nxt, ns);
        }
        if (!mbar_wait(&s.full[stage], static_cast<uint32_t>((it / STAGES) & 1))) atomicExch(a.wait_flag, 1);

        const double *sa = s.A[stage];
        const double *sb = s.B[stage];
        if (!ACC)
        {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;
        }

        if (row_live[0] && col_live[0])
        {
            for (int k0 = 0; k0 < k4; k0 += 4)
            {
                double af[MT], bf[NTL];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) af[mt] = frag_a<LD, TA>(sa, m0 + mt * 8 + g, k0 + t);
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) bf[nt] = frag_b<LD, TB>(sb, k0 + t, n0 + nt * 8 + g);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NTL; ++nt)
                    {
                        if (row_live[mt] && col_live[nt]) dmma_m8n8k4(c[mt][nt], af[mt], bf[nt]);
                    }
            }
        }
        mbar_arrive(&s.empty[stage]);   // this thread no longer reads the slot

        if (ACC) continue;
        double *gc = a.C + e * m * n;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
            {
                const int i = m0 + mt * 8 + g, j = n0 + nt * 8 + 2 * t;
                if (i >= m) continue;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    if (j + h >= n) continue;
                    double *dst = gc + i * n + j + h;
                    double v = c[mt][nt][h];
                    if (a.op == ACRO_B200_OP_ADD) v += *dst;
                    else if (a.op == ACRO_B200_OP_SUB) v = *dst - v;
                    __stcs(dst, v);
                }
            }
    }
    if (ACC)
    {
        // this CTA's partial sums (the grid never exceeds the batch: every CTA had at least one element)
        double *gc = a.C + static_cast<int64_t>(blockIdx.x) * m * n;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
            {
                const int i = m0 + mt * 8 + g, j = n0 + nt * 8 + 2 * t;
                if (i >= m) continue;
#pragma unroll
                for (int h = 0; h < 2; ++h)
                {
                    if (j + h < n) gc[i * n + j + h] = c[mt][nt][h];
                }
            }
    }
}

// Sum of `parts` partial tiles (ascending order: the same bits on every run with the same grid), applied to out.
__global__ void __launch_bounds__(256)
gram_combine_kernel(double *__restrict__ out, const double *__restrict__ partials, int parts, int entries, int op)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= entries) return;
    double acc = 0.0;
    for (int p = 0; p < parts; ++p) acc = __dadd_rn(acc, __ldcg(partials + static_cast<int64_t>(p) * entries + i));
    if (op == ACRO_B200_OP_ASSIGN) out[i] = acc;
    else if (op == ACRO_B200_OP_ADD) out[i] = __dadd_rn(out[i], acc);
    else out[i] = __dsub_rn(out[i], acc);
}

template <int N>
int launch_padded(const PaddedArgs &args, int trans_a, int trans_b, int sms, cudaStream_t stream)
{
    const size_t smem = sizeof(Smem<N>);
    auto kernel = trans_a ? (trans_b ? batched_gemm_padded_kernel<N, true, true> : batched_gemm_padded_kernel<N, true, false>)
                          : (trans_b ? batched_gemm_padded_kernel<N, false, true> : batched_gemm_padded_kernel<N, false, false>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int64_t grid = static_cast<int64_t>(sms) * (N == 64 ? 1 : 4);
    if (grid > args.batch) grid = args.batch;
    kernel<<<static_cast<int>(grid), NT, smem, stream>>>(args);
    return launch_status("acro_b200_batched_gemm (padded)");
}

template <int N>
int launch_ring(const GemmArgs &args, int trans_a, int trans_b, int sms, cudaStream_t stream)
{
    const size_t smem = sizeof(Smem<N>);
    auto kernel = trans_a ? (trans_b ? batched_gemm_kernel<N, true, true> : batched_gemm_kernel<N, true, false>)
                          : (trans_b ? batched_gemm_kernel<N, false, true> : batched_gemm_kernel<N, false, false>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int64_t grid = static_cast<int64_t>(sms) * (N == 64 ? 1 : 4);
    if (grid > args.batch) grid = args.batch;
    kernel<<<static_cast<int>(grid), NT, smem, stream>>>(args);
    return launch_status("acro_b200_batched_gemm");
}

// ------------------------------------------------------------------ 64 x 64 x 64 through tiled bulk copies
// The same persistent CTA, ring and warp tiling as batched_gemm_kernel<64>, with every copy done by the copy
// engine instead of by the threads.  An operand matrix arrives as eight tiled copies (tensor maps, boxes of
// 8 columns x 64 rows = 4 KB) issued by one thread; the map's 64-byte swizzle takes the place of the padded rows:
// a box is stored as 64 rows of 64 bytes and the 16-byte unit u of row r sits at unit u ^ ((r / 2) % 4), which
// makes both fragment patterns of mma.sync m8n8k4 (8 rows x 4 consecutive doubles, 4 rows x 8 consecutive
// doubles) free of bank conflicts, in either storage order of the operand.  The unpadded ring leaves room for a
// staging area: every warp writes its 16 x 32 block of C there in the same swizzled layout and sends it off as
// four tiled stores of its own, so warps still never meet at a CTA barrier.  What this removes from the
// threads, per element: 32 sixteen-byte copy instructions with their address arithmetic, and 16 sixteen-byte
// global stores.
constexpr int T64 = 64;
constexpr int T64_BOX = 8;                                   // columns per box (64 bytes: the swizzle span)
constexpr int T64_MATRIX = T64 * T64;                        // doubles per operand matrix in the ring (unpadded)
constexpr int T64_CHUNK = T64 * T64_BOX;                     // doubles per box of an operand
constexpr int T64_RING_BYTES = STAGES * 2 * T64_MATRIX * 8;  // 196,608
constexpr int T64_SMEM_BYTES = T64_RING_BYTES + 2 * STAGES * 8 + 1024;   // + barriers + alignment slack

struct Tiled64Args
{
    double *C;
    int64_t batch;
    int op;
    int *wait_flag;
};

// Offset (doubles) of entry (r, c) of a matrix stored as boxes of 8 columns, rows of 64 bytes, 64-byte swizzle.
template <int ROWS>
__device__ __forceinline__ int swz(int r, int c)
{
    return (c >> 3) * (ROWS * T64_BOX) + r * T64_BOX + ((((c >> 1) & 3) ^ ((r >> 1) & 3)) << 1) + (c & 1);
}

// Sixteen warps in two groups of eight.  The elements a CTA walks over go alternately to the two groups, each of
// which tiles its element like the eight warps of batched_gemm_kernel<64> (16 x 32 of C per warp); the groups run
// half an element apart, so that while one drains its accumulators, stores C and waits for its next operands the
// other is in the middle of its tensor-core loop (with a single group the pipe idled 22 % of the time whatever the
// copy mechanism, the number of warps or the depth of the prefetch).  Holding group 1 back by half an element at the
// start, so that short launches begin in that rhythm, changed nothing measurable here and is not done.  The ring's three slots hold the two elements
// being multiplied and the one in flight; a group's first thread refills the slot its own group read two elements
// earlier, so neither group ever waits for the other.
constexpr int T64_GROUPS = 2, T64_GROUP_WARPS = 8, T64_THREADS = T64_GROUPS * T64_GROUP_WARPS * 32;

template <bool TA, bool TB>
__global__ void __launch_bounds__(T64_THREADS, 1)
batched_gemm64_tiled_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Tiled64Args a)
{
    constexpr int N = T64, MT = 2, NTL = 4;
    extern __shared__ unsigned char raw_unaligned[];
    // the swizzle is a function of the shared-memory address: boxes must start on multiples of 512 bytes
    unsigned char *raw = raw_unaligned + ((1024u - (smem_addr(raw_unaligned) & 1023u)) & 1023u);
    double *ring = reinterpret_cast<double *>(raw);                                      // [STAGES][A | B][T64_MATRIX]
    uint64_t *full = reinterpret_cast<uint64_t *>(raw + T64_RING_BYTES);
    uint64_t *empty = full + STAGES;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = warp / T64_GROUP_WARPS, wg = warp % T64_GROUP_WARPS;
    const int m0 = (wg >> 1) * 16, n0 = (wg & 1) * 32;
    const bool issuer = (wg == 0 && lane == 0);      // the thread of this group that starts copies

    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i)
        {
            mbar_init(&full[i], 1);                   // the issuing thread's arrival, which also announces the bytes
            mbar_init(&empty[i], T64_GROUP_WARPS);    // one arrival per warp of the group that read the slot
        }
        fence_mbar_init();
    }
    __syncthreads();

    auto issue = [&](int64_t j) {      // element number j of this CTA into slot j % STAGES
        const int64_t e = blockIdx.x + j * gridDim.x;
        if (e >= a.batch) return;
        const int stage = static_cast<int>(j % STAGES);
        mbar_arrive_expect_tx(&full[stage], 2 * T64_MATRIX * 8);
        double *sa = ring + stage * 2 * T64_MATRIX, *sb = sa + T64_MATRIX;
        const int y = static_cast<int>(e * N);
#pragma unroll
        for (int c = 0; c < N / T64_BOX; ++c) tensor_load_2d(sa + c * T64_CHUNK, &map_a, c * T64_BOX, y, &full[stage]);
#pragma unroll
        for (int c = 0; c < N / T64_BOX; ++c) tensor_load_2d(sb + c * T64_CHUNK, &map_b, c * T64_BOX, y, &full[stage]);
    };
    if (tid == 0)
    {
        issue(0);
        issue(1);
    }

    // this group takes elements j = group, group + 2, ... of the CTA
    for (int64_t j = group; blockIdx.x + j * gridDim.x < a.batch; j += T64_GROUPS)
    {
        const int64_t e = blockIdx.x + j * gridDim.x;
        const int stage = static_cast<int>(j % STAGES);
        if (issuer && j >= 1)
        {
            // element j + 1 (the other group's next one) goes to the slot this group read two elements ago
            const int ns = static_cast<int>((j + 1) % STAGES);
            const int64_t use = (j + 1) / STAGES;      // how often that slot was filled before
            if (use > 0 && !mbar_wait(&empty[ns], static_cast<uint32_t>((use - 1) & 1))) atomicExch(a.wait_flag, 1);
            issue(j + 1);
        }
        if (!mbar_wait(&full[stage], static_cast<uint32_t>((j / STAGES) & 1))) atomicExch(a.wait_flag, 1);

        const double *sa = ring + stage * 2 * T64_MATRIX;
        const double *sb = sa + T64_MATRIX;
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
            for (int mt = 0; mt < MT; ++mt) af[mt] = TA ? sa[swz<N>(k0 + t, m0 + mt * 8 + g)] : sa[swz<N>(m0 + mt * 8 + g, k0 + t)];
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) bf[nt] = TB ? sb[swz<N>(n0 + nt * 8 + g, k0 + t)] : sb[swz<N>(k0 + t, n0 + nt * 8 + g)];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) dmma_m8n8k4(c[mt][nt], af[mt], bf[nt]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);   // this warp no longer reads the slot

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
                __stcs(reinterpret_cast<double2 *>(dst), make_double2(v0, v1));
            }
    }
}

template <bool TA, bool TB>
int launch_tiled64_as(const CUtensorMap &ma, const CUtensorMap &mb, const Tiled64Args &args, int sms, cudaStream_t stream)
{
    auto kernel = batched_gemm64_tiled_kernel<TA, TB>;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T64_SMEM_BYTES);
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int64_t grid = sms;
    if (grid > args.batch) grid = args.batch;
    kernel<<<static_cast<int>(grid), T64_THREADS, T64_SMEM_BYTES, stream>>>(ma, mb, args);
    return launch_status("acro_b200_batched_gemm (tiled copies)");
}

// Returns 1 when the tiled-copy kernel cannot be used for this call (the caller then takes the ring of thread copies).
int launch_tiled64(const double *A, const double *B, double *C, int64_t batch, int trans_a, int trans_b, int op, int *wait_flag, int sms,
                   cudaStream_t stream, int *status)
{
    if (!aligned16(A) || !aligned16(B) || !aligned16(C) || batch * T64 >= (int64_t(1) << 31)) return 1;
    CUtensorMap ma, mb;
    const uint64_t rows = static_cast<uint64_t>(batch) * T64;
    if (!encode_matrix_map(&ma, A, rows, T64, T64_BOX, T64) || !encode_matrix_map(&mb, B, rows, T64, T64_BOX, T64)) return 1;
    Tiled64Args args;
    args.C = C;
    args.batch = batch;
    args.op = op;
    args.wait_flag = wait_flag;
    *status = trans_a ? (trans_b ? launch_tiled64_as<true, true>(ma, mb, args, sms, stream) : launch_tiled64_as<true, false>(ma, mb, args, sms, stream))
                      : (trans_b ? launch_tiled64_as<false, true>(ma, mb, args, sms, stream) : launch_tiled64_as<false, false>(ma, mb, args, sms, stream));
    return 0;
}

}

extern "C" {

int acro_b200_batched_gemm_t_supported(int m, int n, int k, int trans_a, int trans_b)
{
    if (m < 1 || n < 1 || k < 1 || m > 4096 || n > 4096 || k > 4096) return 0;
    // a single row or column is a matrix-vector product: streamed for matrices up to 64 x 64, else left to the generic kernel
    if ((m == 1 || n == 1) && (m > 64 || n > 64 || k > 64)) return 0;
    // transposed operands: the kernels that stage whole matrices in shared memory (up to 64 x 64)
    if ((trans_a || trans_b) && (m > 64 || n > 64 || k > 64)) return 0;
    return 1;
}

int acro_b200_batched_gemm_supported(int m, int n, int k) { return acro_b200_batched_gemm_t_supported(m, n, k, 0, 0); }

int acro_b200_batched_gemm_t(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k, int trans_a, int trans_b, int op,
                             void *stream)
{
    if (A == nullptr || B == nullptr || C == nullptr) return fail_invalid("acro_b200_batched_gemm: null argument");
    if (batch < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_batched_gemm: bad batch or operator");
    trans_a = trans_a ? 1 : 0;
    trans_b = trans_b ? 1 : 0;
    if (m == 1) trans_a = 0;      // a row or a column is stored the same way in both orders
    if (n == 1) trans_b = 0;
    if (!acro_b200_batched_gemm_t_supported(m, n, k, trans_a, trans_b))
        return fail_unsupported("acro_b200_batched_gemm: m, n, k must be in 1..4096 (1..64 with a transposed operand or a single row or column)");
    // one column or one row: a matrix-vector product per element; a transposed matrix swaps the two forms
    if (n == 1 && batched_matvec_supported(m, k))
        return trans_a ? batched_matvec_launch(A, B, C, batch, k, m, 1, op, as_stream(stream)) : batched_matvec_launch(A, B, C, batch, m, k, 0, op, as_stream(stream));
    if (m == 1 && batched_matvec_supported(k, n))
        return trans_b ? batched_matvec_launch(B, A, C, batch, n, k, 0, op, as_stream(stream)) : batched_matvec_launch(B, A, C, batch, k, n, 1, op, as_stream(stream));
    const bool plain = !trans_a && !trans_b;
    if (plain && (m > 32 || n > 32 || k > 32) && !(m == 64 && n == 64 && k == 64))
    {
        // 64 x 64 tiles of every product through the tensor-core GEMM kernel (measured 11-12 % faster than zero-padding
        // 40^3 and 48^3 into the 64-wide slots of the ring below)
        return acro_b200_gemm_batched(A, B, C, batch, m, n, k, k, n, n, static_cast<int64_t>(m) * k, static_cast<int64_t>(k) * n,
                                      static_cast<int64_t>(m) * n, op, stream);
    }
    if (batched_gemm_small_supported(m, n, k)) return batched_gemm_small_launch(A, B, C, batch, m, n, k, trans_a, trans_b, op, as_stream(stream));
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

    if (!(m == n && n == k && (m == 64 || m == 32)))
    {
        PaddedArgs pa;
        pa.A = A;
        pa.B = B;
        pa.C = C;
        pa.batch = batch;
        pa.m = m;
        pa.n = n;
        pa.k = k;
        pa.op = op;
        pa.rows_a = trans_a ? k : m;
        pa.cols_a = trans_a ? m : k;
        pa.rows_b = trans_b ? n : k;
        pa.cols_b = trans_b ? k : n;
        pa.wait_flag = args.wait_flag;
        pa.wide = (aligned16(A) && aligned16(B) && pa.cols_a % 2 == 0 && pa.cols_b % 2 == 0 && (m * k) % 2 == 0 && (k * n) % 2 == 0) ? 1 : 0;
        // sizes 17..32; plain products with a larger extent went to the GEMM kernel above, transposed ones use the 64-wide slots
        if (m <= 32 && n <= 32 && k <= 32) return launch_padded<32>(pa, trans_a, trans_b, sms, as_stream(stream));
        return launch_padded<64>(pa, trans_a, trans_b, sms, as_stream(stream));
    }
    static const bool thread_copies = [] { const char *e = std::getenv("ACRO_B200_GEMM64_OLD"); return e != nullptr && e[0] == '1'; }();
    if (m == 64 && !thread_copies)
    {
        int status = ACRO_B200_OK;
        if (launch_tiled64(A, B, C, batch, trans_a, trans_b, op, args.wait_flag, sms, as_stream(stream), &status) == 0) return status;
    }
    return m == 64 ? launch_ring<64>(args, trans_a, trans_b, sms, as_stream(stream)) : launch_ring<32>(args, trans_a, trans_b, sms, as_stream(stream));
}

int acro_b200_batched_gemm(const double *A, const double *B, double *C, int64_t batch, int m, int n, int k, int op, void *stream)
{
    return acro_b200_batched_gemm_t(A, B, C, batch, m, n, k, 0, 0, op, stream);
}

// ------------------------------------------------------------------ Gram form
// S[a, b] (op)= sum_n X[n, a] * Y[n, b].  Up to 16 x 16 the streaming kernel of gram_stream.cu; above that
// the rows of X and Y are cut into slabs of 32 or 64; a slab is one
// "element" of the zero-padded ring kernel with the first operand transposed (m = a, n = b, k = slab rows),
// whose CTAs keep summing into their accumulators instead of storing a product per element.
int acro_b200_gram_supported(int a, int b) { return (a >= 1 && b >= 1 && a <= 64 && b <= 64) ? 1 : 0; }

size_t acro_b200_gram_scratch_bytes(int a, int b)
{
    if (!acro_b200_gram_supported(a, b)) return 0;
    return static_cast<size_t>(kGramMaxParts) * a * b * sizeof(double);
}

int acro_b200_gram(const double *X, const double *Y, double *S, int64_t rows, int a, int b, int op, double *scratch, size_t scratch_bytes,
                   void *stream)
{
    if (X == nullptr || Y == nullptr || S == nullptr || scratch == nullptr) return fail_invalid("acro_b200_gram: null argument");
    if (rows < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_gram: bad row count or operator");
    if (!acro_b200_gram_supported(a, b)) return fail_unsupported("acro_b200_gram: a, b must be in 1..64");
    if (scratch_bytes < acro_b200_gram_scratch_bytes(a, b)) return fail_invalid("acro_b200_gram: scratch smaller than acro_b200_gram_scratch_bytes");
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_gram");
    int *wait_flag = wait_flag_device_ptr();
    if (wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_gram (status flag)");
    cudaStream_t st = as_stream(stream);
    const int entries = a * b;

    if (gram_stream_supported(a, b))
    {
        // a, b <= 16: bound by HBM, streamed with plain fused multiply-adds (gram_stream.cu)
        int tiles_written = 0;
        const int rc = gram_stream_launch(X, Y, scratch, rows, a, b, kGramMaxParts, &tiles_written, st);
        if (rc != ACRO_B200_OK) return rc;
        gram_combine_kernel<<<(entries + 255) / 256, 256, 0, st>>>(S, scratch, tiles_written, entries, op);
        return launch_status("acro_b200_gram (combine)");
    }

    const bool big = a > 32 || b > 32;
    const int slab = big ? 64 : 32;
    const int64_t slabs = rows / slab;
    const int tail = static_cast<int>(rows - slabs * slab);
    auto kernel = big ? batched_gemm_padded_kernel<64, true, false, true> : batched_gemm_padded_kernel<32, true, false, true>;
    const size_t smem = big ? sizeof(Smem<64>) : sizeof(Smem<32>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_gram (shared memory opt-in)");

    PaddedArgs pa;
    pa.m = a;
    pa.n = b;
    pa.op = ACRO_B200_OP_ASSIGN;
    pa.cols_a = a;
    pa.cols_b = b;
    pa.wait_flag = wait_flag;
    int parts = 0;
    if (slabs > 0)
    {
        int64_t grid = static_cast<int64_t>(sms) * (big ? 1 : 4);
        if (grid > slabs) grid = slabs;
        if (grid > kGramMaxParts - 1) grid = kGramMaxParts - 1;
        pa.A = X;
        pa.B = Y;
        pa.C = scratch;
        pa.batch = slabs;
        pa.k = pa.rows_a = pa.rows_b = slab;
        pa.wide = (aligned16(X) && aligned16(Y) && a % 2 == 0 && b % 2 == 0) ? 1 : 0;
        kernel<<<static_cast<int>(grid), NT, smem, st>>>(pa);
        const int launched = launch_status("acro_b200_gram");
        if (launched != ACRO_B200_OK) return launched;
        parts = static_cast<int>(grid);
    }
    if (tail > 0)
    {
        pa.A = X + slabs * slab * a;
        pa.B = Y + slabs * slab * b;
        pa.C = scratch + static_cast<int64_t>(parts) * entries;
        pa.batch = 1;
        pa.k = pa.rows_a = pa.rows_b = tail;
        pa.wide = (aligned16(pa.A) && aligned16(pa.B) && a % 2 == 0 && b % 2 == 0) ? 1 : 0;
        kernel<<<1, NT, smem, st>>>(pa);
        const int launched = launch_status("acro_b200_gram (last rows)");
        if (launched != ACRO_B200_OK) return launched;
        ++parts;
    }
    gram_combine_kernel<<<(entries + 255) / 256, 256, 0, st>>>(S, scratch, parts, entries, op);
    return launch_status("acro_b200_gram (combine)");
}

}
