// acro::Tensor — dense row-major fp64 N-d array with a host buffer and an
// optional device mirror plus one "which side is fresh" bit.
//
// Public surface follows tensor/Tensor.hpp:15-127 of LLNL/acrotensor
// (constructors / Init for rank 1..9 or a vector of dims, optional external
// host and device pointers, operator[] / operator(), Reshape, Retarget,
// MapToGPU / MoveToGPU / SwitchToGPU / UnmapFromGPU / MoveFromGPU /
// SwitchFromGPU, Set, Mult, Print).  Differences, all deliberate:
//   * sizes and byte counts are 64-bit internally (the 4.8 GB tensors of the
//     benchmark configurations overflow a 32-bit byte count);
//   * device memory this object allocated is always released by it;
//   * SetTransient() lets a tensor that only links two kernels of a
//     multi-kernel launch stay on chip (see TensorEngine);
//   * SetSharded() says that this tensor is one rank's slab of a larger tensor
//     cut along its leading dimension (see SlabTensor and TensorEngine::SetPeerGroup).
#ifndef ACRO_B200_TENSOR_HPP
#define ACRO_B200_TENSOR_HPP

#include <cstddef>
#include <cstdint>
#include <type_traits>
#include <vector>
#include "Util.hpp"

namespace acro
{

namespace detail
{
// Collects "d0, d1, ..., [hdata, [ddata, [ongpu]]]" argument packs.
struct ShapeArgs
{
    std::vector<int> dims;
    double *host = nullptr;
    double *device = nullptr;
    bool on_gpu = false;
    int pointers_seen = 0;

    template <class I, typename std::enable_if<std::is_integral<I>::value && !std::is_same<I, bool>::value, int>::type = 0>
    void take(I extent)
    {
        ACROBATIC_ASSERT(pointers_seen == 0, "Tensor dimensions must precede the data pointers.");
        dims.push_back(static_cast<int>(extent));
    }
    void take(double *p)
    {
        ACROBATIC_ASSERT(pointers_seen < 2, "Too many data pointers for a Tensor.");
        (pointers_seen == 0 ? host : device) = p;
        ++pointers_seen;
    }
    void take(std::nullptr_t) { take(static_cast<double *>(nullptr)); }
    void take(bool flag) { on_gpu = flag; pointers_seen = 2; }

    void absorb() {}
    template <class H, class... T>
    void absorb(H head, T... tail)
    {
        take(head);
        absorb(tail...);
    }
};
}

class Tensor
{
    public:
    // An empty tensor to be initialised later with Init().
    Tensor();

    Tensor(std::vector<int> &dims, double *hdata = nullptr, double *ddata = nullptr, bool ongpu = false);

    // Tensor(d0, ..., d8, hdata = nullptr, ddata = nullptr, ongpu = false)
    template <class... Tail>
    explicit Tensor(int d0, Tail... tail) : Tensor()
    {
        detail::ShapeArgs a;
        a.absorb(d0, tail...);
        Init(a.dims, a.host, a.device, a.on_gpu);
    }

    Tensor(const Tensor &) = delete;
    Tensor &operator=(const Tensor &) = delete;
    virtual ~Tensor();

    void Init(std::vector<int> &dims, double *hdata = nullptr, double *ddata = nullptr, bool ongpu = false);
    template <class... Tail>
    void Init(int d0, Tail... tail)
    {
        detail::ShapeArgs a;
        a.absorb(d0, tail...);
        Init(a.dims, a.host, a.device, a.on_gpu);
    }

    // Linear access into the host buffer.
    double &operator[](std::int64_t raw_index) { return Data[raw_index]; }

    // Row-major linear index of a multi-index.
    std::int64_t GetRawIndex(const std::vector<int> &indices) const
    {
        std::int64_t raw = 0;
        for (std::size_t d = 0; d < indices.size(); ++d) raw += static_cast<std::int64_t>(indices[d]) * Strides[d];
        return raw;
    }
    template <class... I>
    std::int64_t GetRawIndex(int i0, I... rest) const
    {
        const int idx[] = {i0, static_cast<int>(rest)...};
        std::int64_t raw = 0;
        for (std::size_t d = 0; d < sizeof...(rest) + 1; ++d) raw += static_cast<std::int64_t>(idx[d]) * Strides[d];
        return raw;
    }

    // Multi-index access into the host buffer.
    double &operator()(std::vector<int> &indices) { return Data[GetRawIndex(indices)]; }
    template <class... I>
    double &operator()(int i0, I... rest) { return Data[GetRawIndex(i0, rest...)]; }

    // Change the dimensions without touching the data; the element count must match.
    void Reshape(std::vector<int> &dims);
    template <class... I>
    void Reshape(int d0, I... rest)
    {
        std::vector<int> dims = {d0, static_cast<int>(rest)...};
        Reshape(dims);
    }

    int GetRank() const { return static_cast<int>(Dims.size()); }
    int GetSize() const { return static_cast<int>(Size); }
    std::int64_t GetSize64() const { return Size; }
    std::size_t GetByteSize() const { return static_cast<std::size_t>(Size) * sizeof(double); }
    int GetDim(int d) const { return Dims[d]; }
    int GetStride(int d) const { return static_cast<int>(Strides[d]); }
    const std::vector<int> &GetDims() const { return Dims; }
    virtual double *GetData() const { return Data; }
    virtual double *GetDeviceData() const { return DeviceData; }
    double *GetCurrentData() const { return IsOnGPU() ? GetDeviceData() : GetData(); }

    // Re-point a tensor over externally owned buffers.
    virtual void Retarget(double *hdata, double *ddata = nullptr);

    virtual void MapToGPU();       // allocate the device mirror
    virtual void MoveToGPU();      // copy host -> device (if the host copy is the fresh one), mark device fresh
    virtual void SwitchToGPU();    // mark the device copy fresh without copying (outputs)
    virtual void UnmapFromGPU();   // release the device mirror
    virtual void MoveFromGPU();    // copy device -> host (if the device copy is the fresh one), mark host fresh
    virtual void SwitchFromGPU();  // mark the host copy fresh without copying
    virtual bool IsMappedToGPU() const { return MappedToGPU; }
    virtual bool IsOnGPU() const { return OnGPU; }
    virtual bool IsInitialized() const { return Initialized; }

    void Set(double val);   // every entry := val, on whichever side is fresh
    void Mult(double c);    // every entry *= c, on whichever side is fresh
    void Print();

    // A transient tensor may be elided by a multi-kernel launch that both
    // produces and consumes it: its contents afterwards are unspecified.
    void SetTransient(bool transient) { Transient = transient; }
    bool IsTransient() const { return Transient; }

    // Multi-GPU, one process per GPU: this tensor holds this rank's slab of a tensor whose leading
    // (slowest) dimension is cut over the ranks of the engine's peer group.  A contraction that sums
    // over that dimension then returns the sum over every rank's slab (TensorEngine::SetPeerGroup).
    void SetSharded(bool sharded) { Sharded = sharded; }
    bool IsSharded() const { return Sharded; }

    protected:
    void UpdateStrides();

    std::vector<int> Dims;
    std::vector<std::int64_t> Strides;
    std::int64_t Size;

    bool Initialized;
    bool OwnsData;
    bool OwnsDeviceData;
    bool MappedToGPU;
    bool OnGPU;
    bool Transient;
    bool Sharded;
    double *Data;
    double *DeviceData;
};

}

#endif
