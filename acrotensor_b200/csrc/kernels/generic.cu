// Generic contraction kernel: one thread per output entry, contracted loops run
// serially in the reference's summation order, without fused multiply-add.
#include "common.cuh"

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
