// acro::IndexVector — an int buffer with the same host / device mirroring rules as
// acro::Tensor (tensor/IndexVector.hpp:14-58 of LLNL/acrotensor).  It carries the index
// maps of FlatIndexedScatter / FlatIndexedSumGather.
#ifndef ACRO_B200_INDEX_VECTOR_HPP
#define ACRO_B200_INDEX_VECTOR_HPP

#include <cstddef>
#include "Util.hpp"

namespace acro
{

class IndexVector
{
    public:
    IndexVector();
    IndexVector(int dim, int *hdata = nullptr, int *ddata = nullptr, bool ongpu = false);
    IndexVector(const IndexVector &) = delete;
    IndexVector &operator=(const IndexVector &) = delete;
    ~IndexVector();
    void Init(int dim, int *hdata = nullptr, int *ddata = nullptr, bool ongpu = false);

    int GetSize() const { return Size; }
    int *GetData() const { return Data; }
    int *GetDeviceData() const { return DeviceData; }
    int *GetCurrentData() const { return IsOnGPU() ? DeviceData : Data; }
    int &operator[](int raw_index) { return Data[raw_index]; }

    void Retarget(int *hdata, int *ddata);

    void MapToGPU();
    void MoveToGPU();
    void SwitchToGPU();
    void UnmapFromGPU();
    void MoveFromGPU();
    void SwitchFromGPU();
    bool IsMappedToGPU() const { return MappedToGPU; }
    bool IsOnGPU() const { return OnGPU; }
    bool IsInitialized() const { return Initialized; }

    void Print();

    private:
    std::size_t Bytes() const { return static_cast<std::size_t>(Size) * sizeof(int); }
    int Size;
    bool Initialized;
    bool OwnsData;
    bool OwnsDeviceData;
    bool MappedToGPU;
    bool OnGPU;
    int *Data;
    int *DeviceData;
};

}

#endif
