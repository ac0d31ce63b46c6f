// acro::SlabTensor: a leading-range view with its own device mirror, and the slab arithmetic.
#include "SlabTensor.hpp"
#include "acro_b200.h"

namespace acro
{

BatchSlab SlabOf(std::int64_t batch, int rank, int world)
{
    ACROBATIC_ASSERT(batch >= 0 && world >= 1 && rank >= 0 && rank < world, "SlabOf: need batch >= 0 and 0 <= rank < world.");
    BatchSlab s;
    ACROBATIC_ASSERT(acro_b200_batch_slab(batch, rank, world, &s.begin, &s.end) == ACRO_B200_OK, "SlabOf: the slab arithmetic overflowed.");
    return s;
}

void SlabTensor::SlabInit(Tensor &T, std::int64_t begin, std::int64_t end)
{
    ACROBATIC_ASSERT(T.IsInitialized(), "Can't take a slab of an uninitilized tensor.");
    ACROBATIC_ASSERT(!IsInitialized(), "Can't initilize a slab a second time.");
    ACROBATIC_ASSERT(begin >= 0 && begin < end && end <= T.GetDim(0), "Slab range must be a non-empty part of the leading dimension.");
    ACROBATIC_ASSERT(T.GetData() != nullptr, "Can't take a slab of a tensor without host data.");
    Begin = begin;
    End = end;
    std::vector<int> dims = T.GetDims();
    dims[0] = static_cast<int>(end - begin);
    const std::int64_t row = T.GetSize64() / T.GetDim(0);
    Init(dims, T.GetData() + begin * row);
    SetSharded(true);
}

}
