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

// Sum of `parts` partial tiles, applied to out.  A CTA takes 32 consecutive entries; its 16 rows of threads each sum
// every sixteenth tile (eight loads in flight, each a warp-wide row of 256 contiguous bytes), then the first row adds
// the 16 sums in ascending order: the order is fixed by `parts` alone, so the bits are the same on every run.  (One
// thread per entry walking all the tiles took 50-100 us for 300-600 tiles, a chain of dependent L2 round trips.)
constexpr int kCombineRows = 16;

__global__ void __launch_bounds__(32 * kCombineRows)
gram_combine_kernel(double *__restrict__ out, const double *__restrict__ partials, int parts, int entries, int op)
{
    __shared__ double sums[kCombineRows][33];
    const int i = blockIdx.x * 32 + threadIdx.x;
    const int row = threadIdx.y;
    double acc = 0.0;
    if (i < entries)
    {
        const double *src = partials + i;
        int p = row;
        for (; p + 7 * kCombineRows < parts; p += 8 * kCombineRows)
        {
            double v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __ldcg(src + static_cast<int64_t>(p + u * kCombineRows) * entries);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = __dadd_rn(acc, v[u]);
        }
        for (; p < parts; p += kCombineRows) acc = __dadd_rn(acc, __ldcg(src + static_cast<int64_t>(p) * entries));
    }
    sums[row][threadIdx.x] = acc;
    __syncthreads();
    if (row != 0 || i >= entries) return;
    double total = sums[0][threadIdx.x];
#pragma unroll
    for (int r = 1; r < kCombineRows; ++r) total = __dadd_rn(total, sums[r][threadIdx.x]);
    if (op == ACRO_B200_OP_ASSIGN) out[i] = total;
    else if (op == ACRO_B200_OP_ADD) out[i] = __dadd_rn(out[i], total);
    else out[i] = __dsub_rn(out[i], total);
}

void launch_gram_combine(double *out, const double *partials, int parts, int entries, int op, cudaStream_t stream)
{
    gram_combine_kernel<<<(entries + 31) / 32, dim3(32, kCombineRows), 0, stream>>>(out, partials, parts, entries, op);
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

// ------------------------------------------------------------------ 64 x 64 x 64, two warp groups
// Sixteen warps in two groups of eight over the same three-slot ring as batched_gemm_kernel<64>.  The elements a
// CTA walks over go alternately to the two groups, each of which tiles its element like the eight warps of that
// kernel (16 x 32 of C per warp); the groups run half an element apart, so that while one drains its accumulators,
// stores C and waits for its next operands the other is in the middle of its tensor-core loop.  With a single
// group the tensor pipe idled 22 % of the time whatever the copy mechanism (thread copies or tiled bulk copies),
// the number of warps (8 or 16 on one element) or the depth of the prefetch (one or two elements ahead): all of
// those measured 0.293-0.295 ms at 2^14 elements, this 0.273 ms.  The ring's three slots hold the two elements
// being multiplied and the one in flight; the threads of a group copy the element the OTHER group needs next into
// the slot their own group read two elements earlier, so neither group ever waits for the other.
//
// Measured alternatives for the copies (2^14 elements / 2^11 elements; this kernel: 0.273 / 0.0455 ms): tiled bulk
// copies through tensor maps into an unpadded ring, boxes of 8 columns x 64 rows with the 64-byte swizzle in place of
// the padded rows: 0.267-0.271 / 0.0476 ms, with two-way bank conflicts left in the fragment loads (the hardware
// serves an 8-byte load per half-warp, and rows g and g + 2 of a half-warp fall on the same banks; ncu: shared-memory
// pipe 74 % busy); boxes of 4 columns x 64 rows without swizzle, which both fragment patterns read without conflicts:
// 0.282 / 0.0516 ms (32-byte rows are too narrow for the copy engine).  Within 2 % of each other on long launches and
// this one best on short ones, so the thread copies into padded rows stayed.
constexpr int G2_GROUPS = 2, G2_GROUP_THREADS = NT, G2_THREADS = G2_GROUPS * G2_GROUP_THREADS;

// The threads of one group copy element e into slot `stage` (16 chunks of 16 bytes each per thread and operand)
// and attach their arrivals on the slot's "full" barrier to the completion of those copies.
__device__ __forceinline__ void issue_group_load(Smem<64> &s, const GemmArgs &a, int64_t e, int stage, int gtid)
{
    constexpr int N = 64, LD = Smem<N>::LD, ROW_CHUNKS = N / 2;
    const double *ga = a.A + e * N * N, *gb = a.B + e * N * N;
#pragma unroll
    for (int i = 0; i < N * ROW_CHUNKS / G2_GROUP_THREADS; ++i)
    {
        const int c = gtid + i * G2_GROUP_THREADS;
        const int row = c / ROW_CHUNKS, col = (c % ROW_CHUNKS) * 2;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.A[stage][row * LD + col])), "l"(ga + c * 2) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&s.B[stage][row * LD + col])), "l"(gb + c * 2) : "memory");
    }
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_addr(&s.full[stage])) : "memory");
}

// ACC: the products of all elements a group walks over are summed in its accumulators and the group stores one
// 64 x 64 tile of partial sums at C + (2 * blockIdx.x + group) * 64 * 64 when it is done (the Gram form; every group
// of every CTA writes its tile, zeros if it had no element).
template <bool TA, bool TB, bool ACC = false>
__global__ void __launch_bounds__(G2_THREADS, 1)
batched_gemm64_groups_kernel(const GemmArgs a)
{
    constexpr int N = 64, LD = Smem<N>::LD, MT = 2, NTL = 4;
    extern __shared__ __align__(128) unsigned char raw[];
    Smem<N> &s = *reinterpret_cast<Smem<N> *>(raw);
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int group = tid / G2_GROUP_THREADS, gtid = tid % G2_GROUP_THREADS, wg = gtid >> 5;
    const int m0 = (wg >> 1) * 16, n0 = (wg & 1) * 32;

    if (tid == 0)
    {
        for (int i = 0; i < STAGES; ++i)
        {
            mbar_init(&s.full[i], G2_GROUP_THREADS);    // the copying group's threads
            mbar_init(&s.empty[i], G2_GROUP_THREADS);   // the reading group's threads
        }
        fence_mbar_init();
    }
    __syncthreads();

    // element number j of this CTA is element blockIdx.x + j * gridDim.x of the batch, lives in slot j % STAGES and
    // belongs to group j % 2; the first two are copied by the groups that will read them
    auto element_of = [&](int64_t j) { return blockIdx.x + j * gridDim.x; };
    if (element_of(group) < a.batch) issue_group_load(s, a, element_of(group), group, gtid);

    double c[MT][NTL][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;

    for (int64_t j = group; element_of(j) < a.batch; j += G2_GROUPS)
    {
        const int64_t e = element_of(j);
        const int stage = static_cast<int>(j % STAGES);
        if (j >= 1 && element_of(j + 1) < a.batch)
        {
            // element j + 1 (the other group's next one) goes to the slot this group read two elements ago
            const int ns = static_cast<int>((j + 1) % STAGES);
            const int64_t use = (j + 1) / STAGES;      // how often that slot was filled before
            if (use > 0 && !mbar_wait(&s.empty[ns], static_cast<uint32_t>((use - 1) & 1))) atomicExch(a.wait_flag, 1);
            issue_group_load(s, a, element_of(j + 1), ns, gtid);
        }
        if (!mbar_wait(&s.full[stage], static_cast<uint32_t>((j / STAGES) & 1))) atomicExch(a.wait_flag, 1);

        const double *sa = s.A[stage];
        const double *sb = s.B[stage];
        if (!ACC)
        {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int nt = 0; nt < NTL; ++nt) c[mt][nt][0] = c[mt][nt][1] = 0.0;
        }

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
        mbar_arrive(&s.empty[stage]);   // this thread no longer reads the slot
        if (ACC) continue;

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
    if (ACC)
    {
        double *gc = a.C + (static_cast<int64_t>(G2_GROUPS) * blockIdx.x + group) * N * N;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt)
            {
                double *dst = gc + (m0 + mt * 8 + g) * N + n0 + nt * 8 + 2 * t;
                dst[0] = c[mt][nt][0];
                dst[1] = c[mt][nt][1];
            }
    }
}

int launch_groups64(const GemmArgs &args, int trans_a, int trans_b, int sms, cudaStream_t stream)
{
    const size_t smem = sizeof(Smem<64>);
    auto kernel = trans_a ? (trans_b ? batched_gemm64_groups_kernel<true, true> : batched_gemm64_groups_kernel<true, false>)
                          : (trans_b ? batched_gemm64_groups_kernel<false, true> : batched_gemm64_groups_kernel<false, false>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_batched_gemm (shared memory opt-in)");
    int64_t grid = sms;
    if (grid > args.batch) grid = args.batch;
    kernel<<<static_cast<int>(grid), G2_THREADS, smem, stream>>>(args);
    return launch_status("acro_b200_batched_gemm (two groups)");
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

int acro_b200_batched_gemm_by_pairs(int m, int n, int k, int trans_a, int trans_b)
{
    return batched_gemm_pairs_supported(m, n, k, trans_a ? 1 : 0, trans_b ? 1 : 0) ? 1 : 0;
}

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
    if (batch >= 2 && batched_gemm_pairs_supported(m, n, k, trans_a, trans_b) && aligned16(A) && aligned16(B) && aligned16(C))
    {
        // rows of an odd length: pairs of elements travel by bulk copy; an odd last element goes through the padded ring below
        const int rc = batched_gemm_pairs_launch(A, B, C, batch / 2, m, n, k, trans_a, trans_b, op, as_stream(stream));
        if (rc != ACRO_B200_OK || batch % 2 == 0) return rc;
        const int64_t done = batch - 1;
        return acro_b200_batched_gemm_t(A + done * m * k, B + done * k * n, C + done * m * n, 1, m, n, k, trans_a, trans_b, op, stream);
    }
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
    // 64^3 with 16-byte aligned operands: two warp groups per CTA; unaligned operands keep the one-group kernel and its plain loads
    if (m == 64 && args.async_copy) return launch_groups64(args, trans_a, trans_b, sms, as_stream(stream));
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
        launch_gram_combine(S, scratch, tiles_written, entries, op, st);
        return launch_status("acro_b200_gram (combine)");
    }

    const bool big = a > 32 || b > 32;
    const int slab = big ? 64 : 32;
    int parts = 0;
    if (!big && rows >= 2 * slab && batched_gemm_pairs_supported(a, b, slab, 1, 0) && aligned16(X) && aligned16(Y))
    {
        // odd row lengths (27 x 27 ...): pairs of 32-row slabs by bulk copy; what is left (fewer than 64 rows) goes through the ring below
        const int64_t pairs = rows / (2 * slab);
        const int rc = gram_pairs_launch(X, Y, scratch, pairs, slab, a, b, kGramMaxParts - 3, &parts, st);
        if (rc != ACRO_B200_OK) return rc;
        X += pairs * 2 * slab * a;
        Y += pairs * 2 * slab * b;
        rows -= pairs * 2 * slab;
        if (rows == 0)
        {
            launch_gram_combine(S, scratch, parts, entries, op, st);
            return launch_status("acro_b200_gram (combine)");
        }
    }
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
    if (slabs > 0 && a == 64 && b == 64 && aligned16(X) && aligned16(Y))
    {
        // full 64 x 64 slabs fill the ring's slots exactly: the two-group kernel of the batched 64^3 product, accumulating
        // (X_slab stored k x m: first operand transposed); one tile of partial sums per group
        auto gk = batched_gemm64_groups_kernel<true, false, true>;
        status = cudaFuncSetAttribute(gk, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(Smem<64>)));
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_gram (shared memory opt-in)");
        int64_t grid = sms;
        if (grid > slabs) grid = slabs;
        if (G2_GROUPS * grid > kGramMaxParts - 1) grid = (kGramMaxParts - 1) / G2_GROUPS;
        GemmArgs ga;
        ga.A = X;
        ga.B = Y;
        ga.C = scratch;
        ga.batch = slabs;
        ga.op = ACRO_B200_OP_ASSIGN;
        ga.wait_flag = wait_flag;
        ga.async_copy = 1;
        gk<<<static_cast<int>(grid), G2_THREADS, sizeof(Smem<64>), st>>>(ga);
        const int launched = launch_status("acro_b200_gram (two groups)");
        if (launched != ACRO_B200_OK) return launched;
        parts = static_cast<int>(G2_GROUPS * grid);
    }
    else if (slabs > 0)
    {
        int64_t grid = static_cast<int64_t>(sms) * (big ? 1 : 4);
        if (grid > slabs) grid = slabs;
        if (grid > kGramMaxParts - 1) grid = kGramMaxParts - 1;
        pa.A = X;
        pa.B = Y;
        pa.C = scratch + static_cast<int64_t>(parts) * entries;
        pa.batch = slabs;
        pa.k = pa.rows_a = pa.rows_b = slab;
        pa.wide = (aligned16(X) && aligned16(Y) && a % 2 == 0 && b % 2 == 0) ? 1 : 0;
        kernel<<<static_cast<int>(grid), NT, smem, st>>>(pa);
        const int launched = launch_status("acro_b200_gram");
        if (launched != ACRO_B200_OK) return launched;
        parts += static_cast<int>(grid);
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
    launch_gram_combine(S, scratch, parts, entries, op, st);
    return launch_status("acro_b200_gram (combine)");
}

}
