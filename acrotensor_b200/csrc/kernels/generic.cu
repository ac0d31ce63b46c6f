// Generic contraction kernel: one thread per output entry, contracted loops run
// serially in the reference's summation order, without fused multiply-add.
#include "common.cuh"
#include <cstring>

using namespace acro_b200_detail;

namespace
{

struct InputPointers
{
    const double *p[ACRO_B200_MAX_INPUTS];
};

// Left-to-right product of the inputs at their current offsets (no fused multiply-add).
template <int N_IN>
__device__ __forceinline__ double product_at(const InputPointers &ins, const int64_t *off, int n_in)
{
    double prod = ins.p[0][off[0]];
#pragma unroll
    for (int v = 1; v < ACRO_B200_MAX_INPUTS; ++v)
    {
        if (v < (N_IN > 0 ? N_IN : n_in)) prod = __dmul_rn(prod, ins.p[v][off[v]]);
    }
    return prod;
}

template <int N_IN>
__device__ __forceinline__ void advance(int64_t *off, const acro_b200_generic_desc &d, int loop, int64_t times, int n_in)
{
#pragma unroll
    for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v)
    {
        if (v < (N_IN > 0 ? N_IN : n_in)) off[v] += times * d.in_step[v][loop];
    }
}

// N_IN: input count (0 = run time).  N_CONTR: contracted loops handled by plain nested loops
// (0..3), or -1 for any depth through an odometer.  One thread per output entry.
template <int N_IN, int N_CONTR>
__global__ void __launch_bounds__(256)
generic_contract_kernel(const __grid_constant__ acro_b200_generic_desc d, double *__restrict__ out,
                        const __grid_constant__ InputPointers ins, int64_t outer_points, int64_t terms)
{
    const int n_in = N_IN > 0 ? N_IN : d.n_inputs;
    const int n_outer = d.n_outer;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool narrow = outer_points <= 0x7fffffffLL;     // 32-bit index arithmetic is much cheaper

    for (int64_t point = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; point < outer_points; point += stride)
    {
        // Unflatten the output entry (last outer loop fastest) into per-variable offsets.
        int64_t out_off = 0;
        int64_t off[ACRO_B200_MAX_INPUTS];
#pragma unroll
        for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v) off[v] = 0;
        if (narrow)
        {
            uint32_t rest = static_cast<uint32_t>(point);
            for (int l = n_outer - 1; l >= 0; --l)
            {
                const uint32_t ext = static_cast<uint32_t>(d.extent[l]);
                const uint32_t q = rest / ext;
                const int64_t idx = rest - q * ext;
                rest = q;
                out_off += idx * d.out_step[l];
                advance<N_IN>(off, d, l, idx, n_in);
            }
        }
        else
        {
            int64_t rest = point;
            for (int l = n_outer - 1; l >= 0; --l)
            {
                const int64_t ext = d.extent[l];
                const int64_t idx = rest % ext;
                rest /= ext;
                out_off += idx * d.out_step[l];
                advance<N_IN>(off, d, l, idx, n_in);
            }
        }

        double acc = (d.op == ACRO_B200_OP_ADD) ? out[out_off] : 0.0;
        if (N_CONTR == 0)
        {
            acc = __dadd_rn(acc, product_at<N_IN>(ins, off, n_in));
        }
        else if (N_CONTR == 1)
        {
            const int l0 = n_outer;
            const int e0 = static_cast<int>(d.extent[l0]);
            for (int i = 0; i < e0; ++i)
            {
                acc = __dadd_rn(acc, product_at<N_IN>(ins, off, n_in));
                advance<N_IN>(off, d, l0, 1, n_in);
            }
        }
        else if (N_CONTR == 2)
        {
            const int l0 = n_outer, l1 = n_outer + 1;
            const int e0 = static_cast<int>(d.extent[l0]), e1 = static_cast<int>(d.extent[l1]);
            for (int i = 0; i < e0; ++i)
            {
                for (int j = 0; j < e1; ++j)
                {
                    acc = __dadd_rn(acc, product_at<N_IN>(ins, off, n_in));
                    advance<N_IN>(off, d, l1, 1, n_in);
                }
                advance<N_IN>(off, d, l1, -static_cast<int64_t>(e1), n_in);
                advance<N_IN>(off, d, l0, 1, n_in);
            }
        }
        else if (N_CONTR == 3)
        {
            const int l0 = n_outer, l1 = n_outer + 1, l2 = n_outer + 2;
            const int e0 = static_cast<int>(d.extent[l0]), e1 = static_cast<int>(d.extent[l1]), e2 = static_cast<int>(d.extent[l2]);
            for (int i = 0; i < e0; ++i)
            {
                for (int j = 0; j < e1; ++j)
                {
                    for (int k = 0; k < e2; ++k)
                    {
                        acc = __dadd_rn(acc, product_at<N_IN>(ins, off, n_in));
                        advance<N_IN>(off, d, l2, 1, n_in);
                    }
                    advance<N_IN>(off, d, l2, -static_cast<int64_t>(e2), n_in);
                    advance<N_IN>(off, d, l1, 1, n_in);
                }
                advance<N_IN>(off, d, l1, -static_cast<int64_t>(e1), n_in);
                advance<N_IN>(off, d, l0, 1, n_in);
            }
        }
        else
        {
            // any depth: odometer over the contracted loops, innermost fastest
            const int n_contr = d.n_loops - d.n_outer;
            int32_t counter[ACRO_B200_MAX_LOOPS];
            for (int c = 0; c < n_contr; ++c) counter[c] = 0;
            for (int64_t term = 0; term < terms; ++term)
            {
                acc = __dadd_rn(acc, product_at<N_IN>(ins, off, n_in));
                for (int c = n_contr - 1; c >= 0; --c)
                {
                    const int l = n_outer + c;
                    if (++counter[c] < d.extent[l])
                    {
                        advance<N_IN>(off, d, l, 1, n_in);
                        break;
                    }
                    counter[c] = 0;
                    advance<N_IN>(off, d, l, -(d.extent[l] - 1), n_in);
                }
            }
        }

        if (d.op == ACRO_B200_OP_SUB) out[out_off] = __dsub_rn(out[out_off], acc);
        else out[out_off] = acc;
    }
}

// Register-blocked variant: one thread owns R output entries that differ only in one outer
// index (entry r sits r * (extent / R) steps along that loop, so neighbouring lanes still touch
// neighbouring addresses).  An input that does not carry the blocked index is loaded once and
// used for all R entries; the leading inputs that do not carry the innermost contracted index
// are multiplied once per pass of that loop.  Every entry still sees the reference's
// left-to-right products and sequential sum, without fused multiply-add: results are
// bit-identical to the thread-per-entry kernel.  32-bit offsets throughout (the launcher checks).
constexpr int kBlockedMaxInputs = 5;

struct BlockedArgs
{
    int n_outer, n_loops, op;
    int hoist;                 // leading inputs without the innermost contracted index
    unsigned int dep_mask;     // bit v: input v carries the blocked index
    int mid_terms;             // product of the contracted extents but the innermost
    int blk_out;               // offset between a thread's consecutive entries
    int blk_in[kBlockedMaxInputs];
    int extent[ACRO_B200_MAX_LOOPS];      // blocked loop already divided by R
    int out_step[ACRO_B200_MAX_LOOPS];
    int in_step[kBlockedMaxInputs][ACRO_B200_MAX_LOOPS];
};

// One pass of the innermost contracted index for the R entries of a thread.  H leading inputs do
// not carry that index: their product is formed once, before the loop.
template <int N_IN, int R, int H>
__device__ __forceinline__ void inner_pass(const BlockedArgs &a, const InputPointers &ins, const int (&off)[N_IN], int e_in, int inner,
                                           double (&acc)[R])
{
    double pre[R];
#pragma unroll
    for (int r = 0; r < R; ++r) pre[r] = 0.0;
#pragma unroll
    for (int v = 0; v < H; ++v)
    {
        if ((a.dep_mask >> v) & 1u)
        {
#pragma unroll
            for (int r = 0; r < R; ++r)
            {
                const double x = ins.p[v][off[v] + r * a.blk_in[v]];
                pre[r] = (v == 0) ? x : __dmul_rn(pre[r], x);
            }
        }
        else
        {
            const double x = ins.p[v][off[v]];
#pragma unroll
            for (int r = 0; r < R; ++r) pre[r] = (v == 0) ? x : __dmul_rn(pre[r], x);
        }
    }

    int o[N_IN];
#pragma unroll
    for (int v = 0; v < N_IN; ++v) o[v] = off[v];
    for (int i = 0; i < e_in; ++i)
    {
        double prod[R];
#pragma unroll
        for (int r = 0; r < R; ++r) prod[r] = pre[r];
#pragma unroll
        for (int v = H; v < N_IN; ++v)
        {
            if ((a.dep_mask >> v) & 1u)
            {
#pragma unroll
                for (int r = 0; r < R; ++r)
                {
                    const double x = ins.p[v][o[v] + r * a.blk_in[v]];
                    prod[r] = (v == 0) ? x : __dmul_rn(prod[r], x);
                }
            }
            else
            {
                const double x = ins.p[v][o[v]];
#pragma unroll
                for (int r = 0; r < R; ++r) prod[r] = (v == 0) ? x : __dmul_rn(prod[r], x);
            }
            o[v] += a.in_step[v][inner];
        }
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = __dadd_rn(acc[r], prod[r]);
    }
}

template <int N_IN, int R>
__global__ void __launch_bounds__(256)
generic_blocked_kernel(const __grid_constant__ BlockedArgs a, double *__restrict__ out,
                       const __grid_constant__ InputPointers ins, unsigned int coarse_points)
{
    const unsigned int stride = gridDim.x * blockDim.x;
    const int n_outer = a.n_outer;
    const int n_contr = a.n_loops - n_outer;
    const int inner = a.n_loops - 1;
    const int e_in = n_contr > 0 ? a.extent[inner] : 1;
    const int hoist = n_contr > 0 ? a.hoist : 0;

    for (unsigned int point = blockIdx.x * blockDim.x + threadIdx.x; point < coarse_points; point += stride)
    {
        int out_off = 0;
        int off[N_IN];
#pragma unroll
        for (int v = 0; v < N_IN; ++v) off[v] = 0;
        unsigned int rest = point;
        for (int l = n_outer - 1; l >= 0; --l)
        {
            const unsigned int ext = static_cast<unsigned int>(a.extent[l]);
            const unsigned int q = rest / ext;
            const int idx = static_cast<int>(rest - q * ext);
            rest = q;
            out_off += idx * a.out_step[l];
#pragma unroll
            for (int v = 0; v < N_IN; ++v) off[v] += idx * a.in_step[v][l];
        }

        double acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = (a.op == ACRO_B200_OP_ADD) ? out[out_off + r * a.blk_out] : 0.0;

        int counter[ACRO_B200_MAX_LOOPS];
        for (int c = 0; c < n_contr - 1; ++c) counter[c] = 0;

        for (int mid = 0; mid < a.mid_terms; ++mid)
        {
            // one pass of the innermost contracted index, with the hoisted input count as a compile-time constant
            switch (hoist)
            {
                case 0: inner_pass<N_IN, R, 0>(a, ins, off, e_in, inner, acc); break;
                case 1: inner_pass<N_IN, R, 1>(a, ins, off, e_in, inner, acc); break;
                case 2: inner_pass<N_IN, R, (N_IN >= 2 ? 2 : N_IN)>(a, ins, off, e_in, inner, acc); break;
                case 3: inner_pass<N_IN, R, (N_IN >= 3 ? 3 : N_IN)>(a, ins, off, e_in, inner, acc); break;
                case 4: inner_pass<N_IN, R, (N_IN >= 4 ? 4 : N_IN)>(a, ins, off, e_in, inner, acc); break;
                default: inner_pass<N_IN, R, N_IN>(a, ins, off, e_in, inner, acc); break;
            }

            // next combination of the other contracted indices (innermost of them fastest)
            for (int c = n_contr - 2; c >= 0; --c)
            {
                const int l = n_outer + c;
                if (++counter[c] < a.extent[l])
                {
#pragma unroll
                    for (int v = 0; v < N_IN; ++v) off[v] += a.in_step[v][l];
                    break;
                }
                counter[c] = 0;
#pragma unroll
                for (int v = 0; v < N_IN; ++v) off[v] -= (a.extent[l] - 1) * a.in_step[v][l];
            }
        }

#pragma unroll
        for (int r = 0; r < R; ++r)
        {
            double *dst = out + out_off + r * a.blk_out;
            *dst = (a.op == ACRO_B200_OP_SUB) ? __dsub_rn(*dst, acc[r]) : acc[r];
        }
    }
}

// Picks the outer loop to block and the entries per thread.  entries = 1: leave the launch to
// the thread-per-entry kernel.
struct BlockedPlan
{
    int loop = -1;
    int entries = 1;
};

BlockedPlan blocked_plan(const acro_b200_generic_desc &d)
{
    BlockedPlan p;
    const int n_contr = d.n_loops - d.n_outer;
    if (d.n_inputs < 2 || d.n_inputs > kBlockedMaxInputs || n_contr < 0) return p;      // entry-wise products (no contraction) too
    int64_t outer_points = 1, terms = 1;
    for (int l = 0; l < d.n_loops; ++l) (l < d.n_outer ? outer_points : terms) *= d.extent[l];
    if (terms >= 0x7fffffffLL) return p;
    // every offset must fit 31 bits
    for (int v = -1; v < d.n_inputs; ++v)
    {
        int64_t reach = 0;
        for (int l = 0; l < d.n_loops; ++l)
        {
            const int64_t step = v < 0 ? d.out_step[l] : d.in_step[v][l];
            if (step < 0) return p;
            reach += (d.extent[l] - 1) * step;
        }
        if (reach >= 0x7fffffffLL) return p;
    }
    // Loads per term: an input carrying the blocked index is loaded per entry, the others once per
    // thread; the leading inputs without the innermost contracted index only once per pass of it.
    // Take the cheapest loop; on ties rather not the fastest output index (whose inputs are the
    // ones read with unit stride across a warp), and rather an inner loop than an outer one.
    const int inner = d.n_loops - 1;
    int hoist = 0;
    while (n_contr > 0 && hoist < d.n_inputs && d.in_step[hoist][inner] == 0) ++hoist;
    double best = 0.0;
    for (int v = 0; v < d.n_inputs; ++v) best += v < hoist ? 1.0 / static_cast<double>(d.extent[inner]) : 1.0;
    static const int kEntries[4] = {4, 5, 3, 2};
    for (int turn = 0; turn < d.n_outer; ++turn)
    {
        const int l = turn < d.n_outer - 1 ? d.n_outer - 2 - turn : d.n_outer - 1;
        for (int e = 0; e < 4; ++e)
        {
            const int r = kEntries[e];
            if (d.extent[l] % r != 0 || outer_points / r < 148 * 512) continue;
            double loads = 0.0;
            for (int v = 0; v < d.n_inputs; ++v)
            {
                const double weight = v < hoist ? 1.0 / static_cast<double>(d.extent[inner]) : 1.0;
                loads += d.in_step[v][l] != 0 ? weight : weight / r;
            }
            if (loads < best - 1e-9)
            {
                best = loads;
                p.loop = l;
                p.entries = r;
            }
        }
    }
    return p;
}

template <int N_IN>
void launch_blocked(const BlockedArgs &a, int entries, double *out, const InputPointers &ins, unsigned int coarse_points,
                    int grid, cudaStream_t s)
{
    switch (entries)
    {
        case 2: generic_blocked_kernel<N_IN, 2><<<grid, 256, 0, s>>>(a, out, ins, coarse_points); break;
        case 3: generic_blocked_kernel<N_IN, 3><<<grid, 256, 0, s>>>(a, out, ins, coarse_points); break;
        case 4: generic_blocked_kernel<N_IN, 4><<<grid, 256, 0, s>>>(a, out, ins, coarse_points); break;
        default: generic_blocked_kernel<N_IN, 5><<<grid, 256, 0, s>>>(a, out, ins, coarse_points); break;
    }
}

// Same layout on both sides and nothing contracted ("A_i = B_i", "A_i_j += B_i_j"): a flat stream,
// two entries per access where both pointers are 16-byte aligned.
__global__ void __launch_bounds__(256)
generic_flat_kernel(double *__restrict__ out, const double *__restrict__ in, int64_t n, int op, int vec2)
{
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vec2)
    {
        double2 *o2 = reinterpret_cast<double2 *>(out);
        const double2 *i2 = reinterpret_cast<const double2 *>(in);
        for (int64_t p = first; p < n / 2; p += stride)
        {
            double2 v = __ldcs(i2 + p);
            if (op != ACRO_B200_OP_ASSIGN)
            {
                const double2 old = o2[p];
                v.x = op == ACRO_B200_OP_ADD ? __dadd_rn(old.x, v.x) : __dsub_rn(old.x, v.x);
                v.y = op == ACRO_B200_OP_ADD ? __dadd_rn(old.y, v.y) : __dsub_rn(old.y, v.y);
            }
            __stcs(o2 + p, v);
        }
        if (first == 0 && (n & 1))
        {
            const double v = in[n - 1];
            out[n - 1] = op == ACRO_B200_OP_ASSIGN ? v : (op == ACRO_B200_OP_ADD ? __dadd_rn(out[n - 1], v) : __dsub_rn(out[n - 1], v));
        }
        return;
    }
    for (int64_t p = first; p < n; p += stride)
    {
        const double v = __ldcs(in + p);
        out[p] = op == ACRO_B200_OP_ASSIGN ? v : (op == ACRO_B200_OP_ADD ? __dadd_rn(out[p], v) : __dsub_rn(out[p], v));
    }
}

// Few output entries but a long contraction (for example "S_a = X_n_a Y_n_a"): the terms of
// every output entry are cut into `chunks` contiguous ranges, one CTA per (entry, range); the
// threads of a CTA take interleaved terms (coalesced for a unit-stride innermost index) and
// combine in a fixed tree order; the CTA that finishes last for an entry (ticket counter in
// scratch) adds the range sums in ascending order.  The sum order differs from the
// reference's sequential one (results agree to rounding and are reproducible run to run);
// the one-thread-per-entry kernel above would leave the GPU idle on such shapes.
constexpr int kWideThreads = 256;
constexpr int kWideMaxChunks = 256;
constexpr int kWideMaxOuter = 2048;

struct WideScratch
{
    unsigned int *counters;   // [outer_points]
    double *partials;         // [outer_points][chunks]
    int chunks;
    int64_t chunk_terms;
};

__device__ __forceinline__ double block_tree_sum(double v, double *partial)
{
    partial[threadIdx.x] = v;
    __syncthreads();
    for (int width = kWideThreads / 2; width > 0; width >>= 1)
    {
        if (threadIdx.x < width) partial[threadIdx.x] = __dadd_rn(partial[threadIdx.x], partial[threadIdx.x + width]);
        __syncthreads();
    }
    const double total = partial[0];
    __syncthreads();
    return total;
}

template <int N_IN>
__global__ void __launch_bounds__(kWideThreads)
generic_wide_kernel(const __grid_constant__ acro_b200_generic_desc d, double *__restrict__ out,
                    const __grid_constant__ InputPointers ins, int64_t terms, const WideScratch ws)
{
    __shared__ double partial[kWideThreads];
    __shared__ bool is_last;
    const int n_in = N_IN > 0 ? N_IN : d.n_inputs;
    const int n_outer = d.n_outer, n_loops = d.n_loops;
    const int64_t point = blockIdx.x / ws.chunks;
    const int chunk = blockIdx.x % ws.chunks;

    int64_t out_off = 0;
    int64_t base[ACRO_B200_MAX_INPUTS];
#pragma unroll
    for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v) base[v] = 0;
    int64_t rest = point;
    for (int l = n_outer - 1; l >= 0; --l)
    {
        const int64_t idx = rest % d.extent[l];
        rest /= d.extent[l];
        out_off += idx * d.out_step[l];
        advance<N_IN>(base, d, l, idx, n_in);
    }

    const int64_t t_begin = chunk * ws.chunk_terms;
    const int64_t t_end = t_begin + ws.chunk_terms < terms ? t_begin + ws.chunk_terms : terms;
    double acc = 0.0;
    for (int64_t term = t_begin + threadIdx.x; term < t_end; term += kWideThreads)
    {
        int64_t off[ACRO_B200_MAX_INPUTS];
#pragma unroll
        for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v) off[v] = base[v];
        uint32_t r = static_cast<uint32_t>(term);            // the launcher guarantees terms < 2^31
        for (int l = n_loops - 1; l > n_outer; --l)
        {
            const uint32_t ext = static_cast<uint32_t>(d.extent[l]);
            const uint32_t q = r / ext;
            advance<N_IN>(off, d, l, static_cast<int64_t>(r - q * ext), n_in);
            r = q;
        }
        advance<N_IN>(off, d, n_outer, static_cast<int64_t>(r), n_in);   // outermost contracted loop: no division
        acc = __dadd_rn(acc, product_at<N_IN>(ins, off, n_in));
    }
    const double chunk_sum = block_tree_sum(acc, partial);

    if (threadIdx.x == 0)
    {
        ws.partials[point * ws.chunks + chunk] = chunk_sum;
        __threadfence();
        is_last = (atomicAdd(ws.counters + point, 1u) == static_cast<unsigned int>(ws.chunks - 1));
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // chunks <= kWideThreads: thread c fetches range sum c; ascending-index tree
    const double mine = threadIdx.x < ws.chunks ? __ldcg(ws.partials + point * ws.chunks + threadIdx.x) : 0.0;
    const double total = block_tree_sum(mine, partial);
    if (threadIdx.x == 0)
    {
        if (d.op == ACRO_B200_OP_ASSIGN) out[out_off] = total;
        else if (d.op == ACRO_B200_OP_ADD) out[out_off] = __dadd_rn(out[out_off], total);
        else out[out_off] = __dsub_rn(out[out_off], total);
        ws.counters[point] = 0u;
    }
}

// How the wide kernel cuts the work: 0 chunks = use the thread-per-entry kernel.
struct WidePlan
{
    int chunks = 0;
    int64_t chunk_terms = 0;
    int64_t outer_points = 1, terms = 1;
    size_t counter_bytes = 0, total_bytes = 0;
};

WidePlan wide_plan(const acro_b200_generic_desc &d)
{
    WidePlan p;
    for (int l = 0; l < d.n_loops && l < ACRO_B200_MAX_LOOPS; ++l) (l < d.n_outer ? p.outer_points : p.terms) *= d.extent[l];
    if (d.n_loops <= d.n_outer || p.outer_points > kWideMaxOuter || p.terms < 16384 || p.terms >= 0x7fffffffLL) return p;
    // enough CTAs to fill the machine, at least 4096 terms each
    int64_t want = (4 * 148 + p.outer_points - 1) / p.outer_points;
    const int64_t by_size = p.terms / 4096;
    if (want > by_size) want = by_size;
    if (want > kWideMaxChunks) want = kWideMaxChunks;
    if (want < 1) want = 1;
    p.chunk_terms = (p.terms + want - 1) / want;
    p.chunks = static_cast<int>((p.terms + p.chunk_terms - 1) / p.chunk_terms);
    p.counter_bytes = ((static_cast<size_t>(p.outer_points) * sizeof(unsigned int) + 255) / 256) * 256;
    p.total_bytes = p.counter_bytes + static_cast<size_t>(p.outer_points) * p.chunks * sizeof(double);
    return p;
}

template <int N_IN>
void launch_thread_per_entry(const acro_b200_generic_desc &d, double *out, const InputPointers &ins, int64_t outer_points,
                             int64_t terms, int grid, cudaStream_t s)
{
    switch (d.n_loops - d.n_outer)
    {
        case 0: generic_contract_kernel<N_IN, 0><<<grid, 256, 0, s>>>(d, out, ins, outer_points, terms); break;
        case 1: generic_contract_kernel<N_IN, 1><<<grid, 256, 0, s>>>(d, out, ins, outer_points, terms); break;
        case 2: generic_contract_kernel<N_IN, 2><<<grid, 256, 0, s>>>(d, out, ins, outer_points, terms); break;
        case 3: generic_contract_kernel<N_IN, 3><<<grid, 256, 0, s>>>(d, out, ins, outer_points, terms); break;
        default: generic_contract_kernel<N_IN, -1><<<grid, 256, 0, s>>>(d, out, ins, outer_points, terms); break;
    }
}

}

// 1 when the launch would use the CTA-per-range kernel: few output entries, long contraction.
extern "C" int acro_b200_generic_uses_wide_kernel(const acro_b200_generic_desc *desc)
{
    return (desc != nullptr && wide_plan(*desc).chunks > 0) ? 1 : 0;
}

// Entries per thread (1 = no blocking) and the blocked outer loop that the launch would use.
extern "C" int acro_b200_generic_blocking(const acro_b200_generic_desc *desc, int *loop)
{
    if (desc == nullptr || wide_plan(*desc).chunks > 0) return 1;
    const BlockedPlan bp = blocked_plan(*desc);
    if (loop != nullptr) *loop = bp.loop;
    return bp.entries;
}

extern "C" size_t acro_b200_generic_scratch_bytes(const acro_b200_generic_desc *desc)
{
    return desc != nullptr ? wide_plan(*desc).total_bytes : 0;
}

extern "C" int acro_b200_generic_launch(const acro_b200_generic_desc *desc, double *out, const double *const *inputs,
                                        double *scratch, size_t scratch_bytes, void *stream)
{
    if (desc == nullptr || out == nullptr || inputs == nullptr) return fail_invalid("acro_b200_generic_launch: null argument");
    if (desc->n_loops < 1 || desc->n_loops > ACRO_B200_MAX_LOOPS || desc->n_outer < 0 || desc->n_outer > desc->n_loops ||
        desc->n_inputs < 1 || desc->n_inputs > ACRO_B200_MAX_INPUTS || desc->op < 0 || desc->op > 2)
    {
        return fail_invalid("acro_b200_generic_launch: descriptor out of range");
    }
    int64_t outer_points = 1, terms = 1;
    for (int l = 0; l < desc->n_loops; ++l)
    {
        if (desc->extent[l] < 1 || desc->extent[l] > INT32_MAX) return fail_invalid("acro_b200_generic_launch: bad loop extent");
        (l < desc->n_outer ? outer_points : terms) *= desc->extent[l];
    }
    InputPointers ins;
    for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v)
    {
        ins.p[v] = v < desc->n_inputs ? inputs[v] : nullptr;
        if (v < desc->n_inputs && inputs[v] == nullptr) return fail_invalid("acro_b200_generic_launch: null input pointer");
    }
    if (sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_generic_launch");

    cudaStream_t s = as_stream(stream);
    const WidePlan wp = wide_plan(*desc);
    if (wp.chunks > 0)
    {
        if (scratch == nullptr || scratch_bytes < wp.total_bytes) return fail_invalid("acro_b200_generic_launch: scratch buffer missing or too small (see acro_b200_generic_scratch_bytes)");
        if ((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return fail_invalid("acro_b200_generic_launch: scratch must be 256-byte aligned");
        WideScratch ws;
        ws.counters = reinterpret_cast<unsigned int *>(scratch);
        ws.partials = reinterpret_cast<double *>(reinterpret_cast<char *>(scratch) + wp.counter_bytes);
        ws.chunks = wp.chunks;
        ws.chunk_terms = wp.chunk_terms;
        cudaError_t status = cudaMemsetAsync(ws.counters, 0, wp.counter_bytes, s);
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_generic_launch (counter reset)");
        const int grid = static_cast<int>(outer_points * wp.chunks);
        switch (desc->n_inputs)
        {
            case 1: generic_wide_kernel<1><<<grid, kWideThreads, 0, s>>>(*desc, out, ins, terms, ws); break;
            case 2: generic_wide_kernel<2><<<grid, kWideThreads, 0, s>>>(*desc, out, ins, terms, ws); break;
            case 3: generic_wide_kernel<3><<<grid, kWideThreads, 0, s>>>(*desc, out, ins, terms, ws); break;
            default: generic_wide_kernel<0><<<grid, kWideThreads, 0, s>>>(*desc, out, ins, terms, ws); break;
        }
        return launch_status("acro_b200_generic_launch (wide)");
    }
    if (desc->n_inputs == 1 && desc->n_loops == desc->n_outer)
    {
        // one input, nothing contracted, the same step in both tensors for every loop: a flat stream
        bool flat = true;
        for (int l = 0; l < desc->n_loops; ++l) flat = flat && (desc->extent[l] == 1 || desc->in_step[0][l] == desc->out_step[l]);
        int64_t expect = 1;
        for (int l = desc->n_loops - 1; l >= 0 && flat; --l)
        {
            if (desc->extent[l] == 1) continue;
            flat = desc->out_step[l] == expect;          // dense, in loop order
            expect *= desc->extent[l];
        }
        if (flat)
        {
            const int vec2 = (aligned16(out) && aligned16(ins.p[0])) ? 1 : 0;
            const int64_t work = vec2 ? (outer_points + 1) / 2 : outer_points;
            const int64_t need = (work + 255) / 256, most = static_cast<int64_t>(sm_count()) * 16;
            generic_flat_kernel<<<static_cast<int>(need < most ? need : most), 256, 0, s>>>(out, ins.p[0], outer_points, desc->op, vec2);
            return launch_status("acro_b200_generic_launch (flat)");
        }
    }
    const BlockedPlan bp = blocked_plan(*desc);
    if (bp.entries > 1)
    {
        BlockedArgs a;
        std::memset(&a, 0, sizeof a);
        a.n_outer = desc->n_outer;
        a.n_loops = desc->n_loops;
        a.op = desc->op;
        const int inner = desc->n_loops - 1;
        a.mid_terms = desc->n_loops > desc->n_outer ? static_cast<int>(terms / desc->extent[inner]) : 1;
        for (int l = 0; l < desc->n_loops; ++l)
        {
            a.extent[l] = static_cast<int>(l == bp.loop ? desc->extent[l] / bp.entries : desc->extent[l]);
            a.out_step[l] = static_cast<int>(desc->out_step[l]);
            for (int v = 0; v < desc->n_inputs; ++v) a.in_step[v][l] = static_cast<int>(desc->in_step[v][l]);
        }
        a.blk_out = static_cast<int>(a.extent[bp.loop] * desc->out_step[bp.loop]);
        bool leading = true;
        for (int v = 0; v < desc->n_inputs; ++v)
        {
            a.blk_in[v] = static_cast<int>(a.extent[bp.loop] * desc->in_step[v][bp.loop]);
            if (desc->in_step[v][bp.loop] != 0) a.dep_mask |= 1u << v;
            leading = leading && desc->n_loops > desc->n_outer && desc->in_step[v][inner] == 0;
            if (leading) a.hoist = v + 1;
        }
        const int64_t coarse = outer_points / bp.entries;
        const int64_t blocks = (coarse + 255) / 256;
        const int64_t most = static_cast<int64_t>(sm_count()) * 32;
        const int grid_b = static_cast<int>(blocks < most ? blocks : most);
        switch (desc->n_inputs)
        {
            case 2: launch_blocked<2>(a, bp.entries, out, ins, static_cast<unsigned int>(coarse), grid_b, s); break;
            case 3: launch_blocked<3>(a, bp.entries, out, ins, static_cast<unsigned int>(coarse), grid_b, s); break;
            case 4: launch_blocked<4>(a, bp.entries, out, ins, static_cast<unsigned int>(coarse), grid_b, s); break;
            default: launch_blocked<5>(a, bp.entries, out, ins, static_cast<unsigned int>(coarse), grid_b, s); break;
        }
        return launch_status("acro_b200_generic_launch (blocked)");
    }
    const int64_t blocks_needed = (outer_points + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const int grid = static_cast<int>(blocks_needed < cap ? blocks_needed : cap);
    switch (desc->n_inputs)
    {
        case 1: launch_thread_per_entry<1>(*desc, out, ins, outer_points, terms, grid, s); break;
        case 2: launch_thread_per_entry<2>(*desc, out, ins, outer_points, terms, grid, s); break;
        case 3: launch_thread_per_entry<3>(*desc, out, ins, outer_points, terms, grid, s); break;
        case 4: launch_thread_per_entry<4>(*desc, out, ins, outer_points, terms, grid, s); break;
        case 5: launch_thread_per_entry<5>(*desc, out, ins, outer_points, terms, grid, s); break;
        default: launch_thread_per_entry<0>(*desc, out, ins, outer_points, terms, grid, s); break;
    }
    return launch_status("acro_b200_generic_launch");
}
