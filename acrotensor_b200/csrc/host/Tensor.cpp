// acro::Tensor storage and host<->device motion.
#include "Tensor.hpp"
#include "acro_b200.h"

#include <cuda_runtime_api.h>
#include <iostream>

namespace acro
{

namespace
{
cudaStream_t stream() { return static_cast<cudaStream_t>(getCudaStream()); }

void check_abi(int status)
{
    if (status != ACRO_B200_OK) throw_error(std::string("acro_b200: ") + acro_b200_last_error());
}
}

Tensor::Tensor()
    : Size(0), Initialized(false), OwnsData(false), OwnsDeviceData(false), MappedToGPU(false), OnGPU(false),
      Transient(false), Sharded(false), Data(nullptr), DeviceData(nullptr)
{
}

Tensor::Tensor(std::vector<int> &dims, double *hdata, double *ddata, bool ongpu) : Tensor()
{
    Init(dims, hdata, ddata, ongpu);
}

void Tensor::Init(std::vector<int> &dims, double *hdata, double *ddata, bool ongpu)
{
    ACROBATIC_ASSERT(!IsInitialized(), "Can't initilize a tensor a second time.");
    ACROBATIC_ASSERT(dims.size() > 0, "Cant initilize tensor without any dimensions.");
    std::int64_t count = 1;
    for (int extent : dims)
    {
        ACROBATIC_ASSERT(extent > 0, "Can't initilize tensor with non-positive dimensions.");
        count *= extent;
    }
    ACROBATIC_ASSERT(ddata == nullptr || hdata != nullptr, "GPU only tensors are not supported: pass a host buffer too.");
    ACROBATIC_ASSERT(ddata != nullptr || !ongpu,
                     "Cannot mark external data as on the GPU if no GPU pointer is provided.");

    Dims = dims;
    Size = count;
    UpdateStrides();
    OwnsData = (hdata == nullptr);
    Data = OwnsData ? new double[static_cast<std::size_t>(Size)] : hdata;
    DeviceData = ddata;
    MappedToGPU = (ddata != nullptr);
    OwnsDeviceData = false;
    OnGPU = ongpu;
    Initialized = true;
}

Tensor::~Tensor()
{
    if (OwnsDeviceData && DeviceData != nullptr)
    {
        cudaFree(DeviceData);   // never throw from a destructor
    }
    if (OwnsData)
    {
        delete[] Data;
    }
}

void Tensor::UpdateStrides()
{
    Strides.assign(Dims.size(), 1);
    for (int d = static_cast<int>(Dims.size()) - 2; d >= 0; --d)
    {
        Strides[d] = Strides[d + 1] * Dims[d + 1];
    }
}

void Tensor::Reshape(std::vector<int> &dims)
{
    ACROBATIC_ASSERT(dims.size() > 0, "Can't reshape a tensor to no dimensions.");
    std::int64_t count = 1;
    for (int extent : dims)
    {
        ACROBATIC_ASSERT(extent > 0, "Can't reshape a tensor to non-positive dimensions.");
        count *= extent;
    }
    ACROBATIC_ASSERT(count == Size, "Reshape must keep the number of entries.");
    Dims = dims;
    UpdateStrides();
}

void Tensor::Retarget(double *hdata, double *ddata)
{
    ACROBATIC_ASSERT(!OwnsData, "Only tensors over external data can be retargeted.");
    ACROBATIC_ASSERT(!OwnsDeviceData, "Can't retarget a tensor whose device mirror the library allocated.");
    Data = hdata;
    DeviceData = ddata;
    MappedToGPU = (ddata != nullptr);
    if (!MappedToGPU) OnGPU = false;
}

void Tensor::Set(double val)
{
    if (!IsOnGPU())
    {
        double *p = GetData();
        for (std::int64_t i = 0; i < Size; ++i) p[i] = val;
    }
    else
    {
        check_abi(acro_b200_fill(GetDeviceData(), Size, val, stream()));
    }
}

void Tensor::Mult(double c)
{
    if (!IsOnGPU())
    {
        double *p = GetData();
        for (std::int64_t i = 0; i < Size; ++i) p[i] *= c;
    }
    else
    {
        check_abi(acro_b200_scale(GetDeviceData(), Size, c, stream()));
    }
}

void Tensor::MapToGPU()
{
    ACROBATIC_ASSERT(!IsMappedToGPU(), "Trying to map data to the GPU a second time.");
    void *p = nullptr;
    acroCudaErrorCheck(cudaMalloc(&p, GetByteSize()));
    DeviceData = static_cast<double *>(p);
    OwnsDeviceData = true;
    MappedToGPU = true;
}

void Tensor::MoveToGPU()
{
    if (!IsMappedToGPU()) MapToGPU();
    if (!IsOnGPU())
    {
        acroCudaErrorCheck(cudaMemcpyAsync(DeviceData, Data, GetByteSize(), cudaMemcpyHostToDevice, stream()));
        acroCudaErrorCheck(cudaStreamSynchronize(stream()));
        OnGPU = true;
    }
}

void Tensor::SwitchToGPU()
{
    if (!IsMappedToGPU()) MapToGPU();
    OnGPU = true;
}

void Tensor::UnmapFromGPU()
{
    ACROBATIC_ASSERT(IsMappedToGPU(), "Can't unmap data that is not mapped to the GPU.");
    if (OwnsDeviceData)
    {
        acroCudaErrorCheck(cudaFree(DeviceData));
    }
    DeviceData = nullptr;
    OwnsDeviceData = false;
    MappedToGPU = false;
    OnGPU = false;
}

void Tensor::MoveFromGPU()
{
    if (IsOnGPU())
    {
        acroCudaErrorCheck(cudaMemcpyAsync(Data, DeviceData, GetByteSize(), cudaMemcpyDeviceToHost, stream()));
        acroCudaErrorCheck(cudaStreamSynchronize(stream()));
        OnGPU = false;
    }
}

void Tensor::SwitchFromGPU() { OnGPU = false; }

void Tensor::Print()
{
    std::cout << "Dims:  ";
    for (int extent : Dims) std::cout << extent << "  ";
    std::cout << "\nStrides:  ";
    for (std::int64_t s : Strides) std::cout << s << "  ";
    std::cout << "\n";
    const double *p = GetData();
    for (std::int64_t i = 0; i < Size; ++i) std::cout << p[i] << "\n";
    std::cout << std::endl;
}

}
