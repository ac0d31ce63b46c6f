// acro::BatchSlab and acro::SlabTensor — the cut of a batch (element) index into one contiguous
// slab per rank, for the multi-GPU model "one process per GPU, batch index sharded".
//
// No counterpart in LLNL/acrotensor, which is single-device (exec/CudaExecutor.cpp:21); the view
// is the leading-range sibling of acro::SliceTensor, whose offset arithmetic it shares
// (tensor/SliceTensor.cpp:142-168): a SliceTensor fixes a prefix of leading indices, a SlabTensor
// keeps a range [begin, end) of the first one.
#ifndef ACRO_B200_SLAB_TENSOR_HPP
#define ACRO_B200_SLAB_TENSOR_HPP

#include <cstdint>
#include "Tensor.hpp"

namespace acro
{

// Range [begin, end) of a batch index of extent `batch` that rank `rank` of `world` owns:
// contiguous, in rank order, sizes differing by at most one, empty ranges only when world > batch.
struct BatchSlab
{
    std::int64_t begin;
    std::int64_t end;
    std::int64_t size() const { return end - begin; }
};
BatchSlab SlabOf(std::int64_t batch, int rank, int world);

// Rows [begin, end) of the leading dimension of a parent tensor.  The view shares the parent's HOST
// buffer (results copied back with MoveFromGPU land in the parent's rows) but owns a device mirror
// of its own that holds the slab only, so a rank never uploads the rows of other ranks.  It is
// flagged IsSharded(): an engine with a peer group sums a contraction over the leading index across
// the ranks.  The parent must outlive the view and is not touched by the view's GPU motion.
class SlabTensor : public Tensor
{
    public:
    SlabTensor() : Begin(0), End(0) {}
    SlabTensor(Tensor &T, std::int64_t begin, std::int64_t end) : SlabTensor() { SlabInit(T, begin, end); }
    // this rank's slab of T:  SlabTensor mine(T, SlabOf(T.GetDim(0), rank, world));
    SlabTensor(Tensor &T, const BatchSlab &slab) : SlabTensor() { SlabInit(T, slab.begin, slab.end); }
    ~SlabTensor() override {}

    void SlabInit(Tensor &T, std::int64_t begin, std::int64_t end);
    std::int64_t GetBegin() const { return Begin; }
    std::int64_t GetEnd() const { return End; }

    void Retarget(double *, double * = nullptr) override
    {
        ACROBATIC_ASSERT(false, "Retarget not supported on SlabTensors");
    }

    private:
    std::int64_t Begin, End;
};

}

#endif
