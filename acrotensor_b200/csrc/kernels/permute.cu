// permute: Out (op)= In with the indices in another order ("A_i_j = B_j_i", "Z_m_e_k = D_e_k_m").
//
// When the fastest index of the input is not the fastest index of the output, one side of a
// thread-per-entry copy is strided.  Here 64 x 64 tiles over (fastest output index, fastest input
// index) go through shared memory (rows padded to 65), so that both the loads and the stores of a
// warp are contiguous runs; the other indices are flattened into the grid.  Pure data movement:
// bit-identical by construction.
#include "common.cuh"

using namespace acro_b200_detail;

namespace
{

constexpr int kTile = 64;
constexpr int kLanes = 32;
constexpr int kRows = 8;        // block = 32 x 8 threads; a thread moves 16 entries of a tile, all loads in flight before the barrier

struct PermuteArgs
{
    const double *in;
    double *out;
    int n_rest;                              // loops other than the two tiled ones
    int op;
    long long rest_extent[ACRO_B200_MAX_LOOPS], rest_in[ACRO_B200_MAX_LOOPS], rest_out[ACRO_B200_MAX_LOOPS];
    long long ext_fo, ext_fi;                // extents of the fastest output / fastest input index
    long long in_fo, out_fi;                 // stride of the fastest output index in the input, of the fastest input index in the output
    long long tiles_fo, tiles_fi;
};

__global__ void __launch_bounds__(kLanes * kRows)
permute_kernel(const PermuteArgs a)
{
    __shared__ double tile[kTile][kTile + 1];
    const long long tiles_per_slice = a.tiles_fo * a.tiles_fi;
    long long block = blockIdx.x;
    const long long slice = block / tiles_per_slice;
    block -= slice * tiles_per_slice;
    const long long tfo = block / a.tiles_fi, tfi = block - tfo * a.tiles_fi;

    long long base_in = 0, base_out = 0, rest = slice;
    for (int l = a.n_rest - 1; l >= 0; --l)
    {
        const long long idx = rest % a.rest_extent[l];
        rest /= a.rest_extent[l];
        base_in += idx * a.rest_in[l];
        base_out += idx * a.rest_out[l];
    }
    const long long fo0 = tfo * kTile, fi0 = tfi * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;

    // load: lanes along the input's fastest index
#pragma unroll
    for (int r = ty; r < kTile; r += kRows)
    {
#pragma unroll
        for (int c = tx; c < kTile; c += kLanes)
        {
            const long long fo = fo0 + r, fi = fi0 + c;
            if (fo < a.ext_fo && fi < a.ext_fi) tile[r][c] = a.in[base_in + fo * a.in_fo + fi];
        }
    }
    __syncthreads();
    // store: lanes along the output's fastest index
#pragma unroll
    for (int r = ty; r < kTile; r += kRows)
    {
#pragma unroll
        for (int c = tx; c < kTile; c += kLanes)
        {
            const long long fi = fi0 + r, fo = fo0 + c;
            if (fo < a.ext_fo && fi < a.ext_fi)
            {
                double *dst = a.out + base_out + fi * a.out_fi + fo;
                const double v = tile[c][r];
                if (a.op == ACRO_B200_OP_ASSIGN) *dst = v;
                else if (a.op == ACRO_B200_OP_ADD) *dst = __dadd_rn(*dst, v);
                else *dst = __dsub_rn(*dst, v);
            }
        }
    }
}

}

extern "C" {

int acro_b200_permute_supported(const acro_b200_generic_desc *d)
{
    if (d == nullptr || d->n_inputs != 1 || d->n_loops != d->n_outer || d->n_loops < 2 || d->n_loops > ACRO_B200_MAX_LOOPS) return 0;
    if (d->op < 0 || d->op > 2) return 0;
    int fo = -1, fi = -1;
    for (int l = 0; l < d->n_loops; ++l)
    {
        if (d->extent[l] < 1 || d->out_step[l] < 1 || d->in_step[0][l] < 1) return 0;     // every index in both tensors
        if (d->out_step[l] == 1 && d->extent[l] > 1) fo = l;
        if (d->in_step[0][l] == 1 && d->extent[l] > 1) fi = l;
    }
    return (fo >= 0 && fi >= 0 && fo != fi) ? 1 : 0;
}

int acro_b200_permute(const acro_b200_generic_desc *d, double *out, const double *in, void *stream)
{
    if (d == nullptr || out == nullptr || in == nullptr) return fail_invalid("acro_b200_permute: null argument");
    if (!acro_b200_permute_supported(d)) return fail_unsupported("acro_b200_permute: needs one input carrying every output index, with different fastest indices");
    if (sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_permute");
    PermuteArgs a;
    a.in = in;
    a.out = out;
    a.op = d->op;
    a.n_rest = 0;
    int fo = -1, fi = -1;
    for (int l = 0; l < d->n_loops; ++l)
    {
        if (d->out_step[l] == 1 && d->extent[l] > 1) fo = l;
        if (d->in_step[0][l] == 1 && d->extent[l] > 1) fi = l;
    }
    long long slices = 1;
    for (int l = 0; l < d->n_loops; ++l)
    {
        if (l == fo || l == fi) continue;
        a.rest_extent[a.n_rest] = d->extent[l];
        a.rest_in[a.n_rest] = d->in_step[0][l];
        a.rest_out[a.n_rest] = d->out_step[l];
        slices *= d->extent[l];
        ++a.n_rest;
    }
    a.ext_fo = d->extent[fo];
    a.ext_fi = d->extent[fi];
    a.in_fo = d->in_step[0][fo];
    a.out_fi = d->out_step[fi];
    a.tiles_fo = (a.ext_fo + kTile - 1) / kTile;
    a.tiles_fi = (a.ext_fi + kTile - 1) / kTile;
    const long long blocks = slices * a.tiles_fo * a.tiles_fi;
    if (blocks > 0x7fffffffLL) return fail_unsupported("acro_b200_permute: more than 2^31 tiles");
    permute_kernel<<<static_cast<unsigned int>(blocks), dim3(kLanes, kRows), 0, as_stream(stream)>>>(a);
    return launch_status("acro_b200_permute");
}

}
