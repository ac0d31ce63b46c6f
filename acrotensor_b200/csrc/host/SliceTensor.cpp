// acro::SliceTensor: a prefix-indexed view that forwards all data motion to its parent.
#include "SliceTensor.hpp"

namespace acro
{

void SliceTensor::SliceInit(Tensor &T, std::vector<int> &sind)
{
    ACROBATIC_ASSERT(T.IsInitialized(), "Can't slice an uninitilized tensor.");
    ACROBATIC_ASSERT(T.GetRank() > static_cast<int>(sind.size()), "Can't slice more dimensions than the tensor rank.");
    ACROBATIC_ASSERT(!IsInitialized(), "Can't initilize a slice a second time.");
    // Like the reference, the prefix indices are not range-checked: its own unit tests
    // construct (and never touch) slices past the end (unittest/tensor/test_SliceTensor.cpp:25-27).
    FullT = &T;
    Offset = T.GetRawIndex(sind);

    std::vector<int> dims(T.GetDims().begin() + sind.size(), T.GetDims().end());
    double *hdata = T.GetData();
    double *ddata = T.GetDeviceData();
    Init(dims, hdata ? hdata + Offset : nullptr, ddata ? ddata + Offset : nullptr, T.IsOnGPU());
}

double *SliceTensor::GetData() const { return FullT->GetData() + Offset; }

double *SliceTensor::GetDeviceData() const
{
    double *base = FullT->GetDeviceData();
    return base ? base + Offset : nullptr;
}

void SliceTensor::MapToGPU()
{
    FullT->MapToGPU();
    DeviceData = GetDeviceData();
}

void SliceTensor::MoveToGPU()
{
    FullT->MoveToGPU();
    DeviceData = GetDeviceData();
}

void SliceTensor::SwitchToGPU()
{
    FullT->SwitchToGPU();
    DeviceData = GetDeviceData();
}

void SliceTensor::UnmapFromGPU() {}   // the parent owns the mirror

void SliceTensor::MoveFromGPU() { FullT->MoveFromGPU(); }
void SliceTensor::SwitchFromGPU() { FullT->SwitchFromGPU(); }
bool SliceTensor::IsMappedToGPU() const { return FullT->IsMappedToGPU(); }
bool SliceTensor::IsOnGPU() const { return FullT->IsOnGPU(); }

}
