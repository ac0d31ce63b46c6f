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

template <int N_IN>   // 0 = run-time input count
__global__ void __launch_bounds__(256)
generic_contract_kernel(const __grid_constant__ acro_b200_generic_desc d, double *__restrict__ out,
                        const __grid_constant__ InputPointers ins, int64_t outer_points, int64_t terms)
{
    const int n_in = N_IN > 0 ? N_IN : d.n_inputs;
    const int n_outer = d.n_outer;
    const int n_contr = d.n_loops - d.n_outer;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;

    for (int64_t point = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; point < outer_points; point += stride)
    {
        // Unflatten the output entry (last outer loop fastest) into per-variable offsets.
        int64_t out_off = 0;
        int64_t in_off[ACRO_B200_MAX_INPUTS];
#pragma unroll
        for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v) in_off[v] = 0;
        int64_t rest = point;
        for (int l = n_outer - 1; l >= 0; --l)
        {
            const int64_t ext = d.extent[l];
            const int64_t idx = rest % ext;
            rest /= ext;
            out_off += idx * d.out_step[l];
#pragma unroll
            for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v)
            {
                if (v < n_in) in_off[v] += idx * d.in_step[v][l];
            }
        }

        double acc = (d.op == ACRO_B200_OP_ADD) ? out[out_off] : 0.0;
        int32_t counter[ACRO_B200_MAX_LOOPS];
        for (int c = 0; c < n_contr; ++c) counter[c] = 0;

        for (int64_t term = 0; term < terms; ++term)
        {
            double prod = ins.p[0][in_off[0]];
#pragma unroll
            for (int v = 1; v < ACRO_B200_MAX_INPUTS; ++v)
            {
                if (v < n_in) prod = __dmul_rn(prod, ins.p[v][in_off[v]]);
            }
            acc = __dadd_rn(acc, prod);

            // Odometer over the contracted loops, innermost fastest.
            for (int c = n_contr - 1; c >= 0; --c)
            {
                const int l = n_outer + c;
                if (++counter[c] < d.extent[l])
                {
#pragma unroll
                    for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v)
                    {
                        if (v < n_in) in_off[v] += d.in_step[v][l];
                    }
                    break;
                }
                counter[c] = 0;
#pragma unroll
                for (int v = 0; v < ACRO_B200_MAX_INPUTS; ++v)
                {
                    if (v < n_in) in_off[v] -= d.in_step[v][l] * (d.extent[l] - 1);
                }
            }
        }

        if (d.op == ACRO_B200_OP_SUB) out[out_off] = __dsub_rn(out[out_off], acc);
        else out[out_off] = acc;
    }
}

}

extern "C" int acro_b200_generic_launch(const acro_b200_generic_desc *desc, double *out, const double *const *inputs, void *stream)
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

    const int64_t blocks_needed = (outer_points + 255) / 256;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
    const int grid = static_cast<int>(blocks_needed < cap ? blocks_needed : cap);
    cudaStream_t s = as_stream(stream);
    switch (desc->n_inputs)
    {
        case 1: generic_contract_kernel<1><<<grid, 256, 0, s>>>(*desc, out, ins, outer_points, terms); break;
        case 2: generic_contract_kernel<2><<<grid, 256, 0, s>>>(*desc, out, ins, outer_points, terms); break;
        case 3: generic_contract_kernel<3><<<grid, 256, 0, s>>>(*desc, out, ins, outer_points, terms); break;
        case 4: generic_contract_kernel<4><<<grid, 256, 0, s>>>(*desc, out, ins, outer_points, terms); break;
        default: generic_contract_kernel<0><<<grid, 256, 0, s>>>(*desc, out, ins, outer_points, terms); break;
    }
    return launch_status("acro_b200_generic_launch");
}
