// Internal: the launch plan the "Cuda" back end derives from a bound kernel group.
// A Program is a list of Steps; each Step names a kernel family of the C ABI
// (acro_b200.h), the launch parameters computed once at planning time and the
// call-site tensors (by member kernel and variable number) it reads and writes.
#ifndef ACRO_B200_PLAN_HPP
#define ACRO_B200_PLAN_HPP

#include <cstdint>
#include <string>
#include <vector>
#include "DimensionedMultiKernel.hpp"
#include "acro_b200.h"

namespace acro
{
namespace plan
{

enum class Family
{
    Generic,
    ReduceBatch,
    PointwiseSym,
    Rank1Gemm,
    BatchedGemm,
    SumfactMass,
    InvariantGemm,
    Permute,
    Gram
};

const char *FamilyName(Family f);

// A tensor of the call: variable vari (-1 = output) of member kernel ki.
struct TensorRef
{
    int ki = 0;
    int vari = -1;
};

struct Step
{
    Family family = Family::Generic;
    std::vector<int> kernels;        // member kernels this step computes
    std::string note;                // human-readable parameters for GetImplementation
    std::int64_t bytes = 0;          // algorithmic HBM traffic of the step
    std::int64_t flops = 0;          // algorithmic floating point operations

    TensorRef out;
    std::vector<TensorRef> ins;      // meaning depends on the family (see Plan.cpp)
    int op = ACRO_B200_OP_ASSIGN;
    bool zero_fill_first = false;    // "=" into an output with a repeated index

    acro_b200_generic_desc generic;
    acro_b200_pointwise_desc pointwise;
    std::int64_t rows = 0;           // reduce_batch / batch count of the GEMM families
    int sizes[5] = {0, 0, 0, 0, 0};  // family-specific sizes and flags
    std::vector<TensorRef> elided;   // transient outputs this step keeps on chip
    // Inputs whose leading (slowest) index is contracted.  When the engine has a peer group and one of
    // these tensors is a rank's slab (Tensor::IsSharded), the step's result is summed over the ranks.
    std::vector<TensorRef> lead_contracted;
};

struct Program
{
    std::vector<Step> steps;
    std::size_t scratch_bytes = 0;
    bool elides = false;             // true when some output is not materialised
    std::string Describe(DimensionedMultiKernel &mk) const;
};

// allow_elision: transient intermediates of a recognised chain may stay on chip.
Program BuildProgram(DimensionedMultiKernel &mk, bool allow_elision);

}
}

#endif
