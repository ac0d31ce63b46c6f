// acro::IndexVector storage and host<->device motion.
#include "IndexVector.hpp"

#include <cuda_runtime_api.h>
#include <iostream>

namespace acro
{

namespace
{
cudaStream_t stream() { return static_cast<cudaStream_t>(getCudaStream()); }
}

IndexVector::IndexVector()
    : Size(0), Initialized(false), OwnsData(false), OwnsDeviceData(false), MappedToGPU(false), OnGPU(false), Data(nullptr),
      DeviceData(nullptr)
{
}

IndexVector::IndexVector(int dim, int *hdata, int *ddata, bool ongpu) : IndexVector() { Init(dim, hdata, ddata, ongpu); }

void IndexVector::Init(int dim, int *hdata, int *ddata, bool ongpu)
{
    ACROBATIC_ASSERT(!IsInitialized(), "Can't initilize a vector a second time.");
    ACROBATIC_ASSERT(dim > 0, "Cant initilize vector with dim <= 0.");
    ACROBATIC_ASSERT(ddata == nullptr || hdata != nullptr, "GPU only index vectors are not supported: pass a host buffer too.");
    ACROBATIC_ASSERT(ddata != nullptr || !ongpu, "Cannot mark external data as on the GPU if no GPU pointer is provided.");
    Size = dim;
    OwnsData = (hdata == nullptr);
    Data = OwnsData ? new int[static_cast<std::size_t>(dim)] : hdata;
    DeviceData = ddata;
    MappedToGPU = (ddata != nullptr);
    OwnsDeviceData = false;
    OnGPU = ongpu;
    Initialized = true;
}

IndexVector::~IndexVector()
{
    if (OwnsDeviceData && DeviceData != nullptr) cudaFree(DeviceData);
    if (OwnsData) delete[] Data;
}

void IndexVector::Retarget(int *hdata, int *ddata)
{
    ACROBATIC_ASSERT(!OwnsData, "Only index vectors over external data can be retargeted.");
    ACROBATIC_ASSERT(!OwnsDeviceData, "Can't retarget a vector whose device mirror the library allocated.");
    Data = hdata;
    DeviceData = ddata;
    MappedToGPU = (ddata != nullptr);
    if (!MappedToGPU) OnGPU = false;
}

void IndexVector::MapToGPU()
{
    ACROBATIC_ASSERT(!IsMappedToGPU(), "Trying to map data to the GPU a second time.");
    void *p = nullptr;
    acroCudaErrorCheck(cudaMalloc(&p, Bytes()));
    DeviceData = static_cast<int *>(p);
    OwnsDeviceData = true;
    MappedToGPU = true;
}

void IndexVector::MoveToGPU()
{
    if (!IsMappedToGPU()) MapToGPU();
    if (!IsOnGPU())
    {
        acroCudaErrorCheck(cudaMemcpyAsync(DeviceData, Data, Bytes(), cudaMemcpyHostToDevice, stream()));
        acroCudaErrorCheck(cudaStreamSynchronize(stream()));
        OnGPU = true;
    }
}

void IndexVector::SwitchToGPU()
{
    if (!IsMappedToGPU()) MapToGPU();
    OnGPU = true;
}

void IndexVector::UnmapFromGPU()
{
    ACROBATIC_ASSERT(IsMappedToGPU(), "Can't unmap data that is not mapped to the GPU.");
    if (OwnsDeviceData) acroCudaErrorCheck(cudaFree(DeviceData));
    DeviceData = nullptr;
    OwnsDeviceData = false;
    MappedToGPU = false;
    OnGPU = false;
}

void IndexVector::MoveFromGPU()
{
    if (IsOnGPU())
    {
        acroCudaErrorCheck(cudaMemcpyAsync(Data, DeviceData, Bytes(), cudaMemcpyDeviceToHost, stream()));
        acroCudaErrorCheck(cudaStreamSynchronize(stream()));
        OnGPU = false;
    }
}

void IndexVector::SwitchFromGPU() { OnGPU = false; }

void IndexVector::Print()
{
    for (int i = 0; i < Size; ++i) std::cout << Data[i] << "\n";
    std::cout << std::endl;
}

}
