// acro::SliceTensor — a view of the trailing dimensions of a parent Tensor at a
// fixed prefix of leading indices, sharing the parent's host and device
// buffers.  Follows tensor/SliceTensor.hpp:14-57 of LLNL/acrotensor: all data
// motion is forwarded to the parent (tensor/SliceTensor.cpp:171-232).
#ifndef ACRO_B200_SLICE_TENSOR_HPP
#define ACRO_B200_SLICE_TENSOR_HPP

#include "Tensor.hpp"

namespace acro
{

class SliceTensor : public Tensor
{
    public:
    SliceTensor() : FullT(nullptr), Offset(0) {}
    SliceTensor(Tensor &T, std::vector<int> &sind) : SliceTensor() { SliceInit(T, sind); }
    template <class... I>
    SliceTensor(Tensor &T, int i0, I... rest) : SliceTensor()
    {
        std::vector<int> sind = {i0, static_cast<int>(rest)...};
        SliceInit(T, sind);
    }
    ~SliceTensor() override {}

    void SliceInit(Tensor &T, std::vector<int> &sind);
    template <class... I>
    void SliceInit(Tensor &T, int i0, I... rest)
    {
        std::vector<int> sind = {i0, static_cast<int>(rest)...};
        SliceInit(T, sind);
    }

    void Retarget(double *, double * = nullptr) override
    {
        ACROBATIC_ASSERT(false, "Retarget not supported on SliceTensors");
    }

    double *GetData() const override;
    double *GetDeviceData() const override;
    void MapToGPU() override;
    void MoveToGPU() override;
    void SwitchToGPU() override;
    void UnmapFromGPU() override;
    void MoveFromGPU() override;
    void SwitchFromGPU() override;
    bool IsMappedToGPU() const override;
    bool IsOnGPU() const override;

    private:
    Tensor *FullT;
    std::int64_t Offset;
};

}

#endif
