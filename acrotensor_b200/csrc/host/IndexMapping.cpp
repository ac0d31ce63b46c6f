// acro::IndexMapping: the map, and its inverse in CSR form.
#include "IndexMapping.hpp"

#include <algorithm>
#include <numeric>

namespace acro
{

IndexMapping::IndexMapping(int domain_size, int range_size)
    : InverseComputed(false), MappedToGPU(false), OnGPU(false), DomainSize(domain_size), RangeSize(range_size), M(range_size),
      InvM(range_size), InvMOff(domain_size + 1)
{
}

IndexVector &IndexMapping::GetInvMap()
{
    ACROBATIC_ASSERT(InverseComputed, "Trying to access inverse mapping before the inverse is computed.");
    return InvM;
}

IndexVector &IndexMapping::GetInvMapOffsets()
{
    ACROBATIC_ASSERT(InverseComputed, "Trying to access inverse mapping offsets before the inverse is computed.");
    return InvMOff;
}

void IndexMapping::ComputeInverse()
{
    ACROBATIC_ASSERT(!InverseComputed, "Can't compute the inverse mapping twice.");
    if (M.IsOnGPU()) M.MoveFromGPU();
    const int *map = M.GetData();
    for (int i = 0; i < RangeSize; ++i)
    {
        ACROBATIC_ASSERT(map[i] >= 0 && map[i] < DomainSize, "IndexMapping entry outside the domain.");
    }
    // Counting sort by domain entry; positions inside a group stay in ascending order,
    // which is what a stable sort of the positions by M gives.
    int *offsets = InvMOff.GetData();
    std::fill(offsets, offsets + DomainSize + 1, 0);
    for (int i = 0; i < RangeSize; ++i) ++offsets[map[i] + 1];
    std::partial_sum(offsets, offsets + DomainSize + 1, offsets);
    std::vector<int> cursor(offsets, offsets + DomainSize);
    int *inv = InvM.GetData();
    for (int i = 0; i < RangeSize; ++i) inv[cursor[map[i]]++] = i;
    InverseComputed = true;
    if (OnGPU)
    {
        M.MoveToGPU();
        InvM.SwitchFromGPU();
        InvM.MoveToGPU();
        InvMOff.SwitchFromGPU();
        InvMOff.MoveToGPU();
    }
}

void IndexMapping::MapToGPU()
{
    M.MapToGPU();
    InvM.MapToGPU();
    InvMOff.MapToGPU();
    MappedToGPU = true;
}

void IndexMapping::MoveToGPU()
{
    M.MoveToGPU();
    if (InverseComputed)
    {
        InvM.MoveToGPU();
        InvMOff.MoveToGPU();
    }
    MappedToGPU = true;
    OnGPU = true;
}

void IndexMapping::SwitchToGPU()
{
    M.SwitchToGPU();
    InvM.SwitchToGPU();
    InvMOff.SwitchToGPU();
    MappedToGPU = true;
    OnGPU = true;
}

void IndexMapping::UnmapFromGPU()
{
    if (M.IsMappedToGPU()) M.UnmapFromGPU();
    if (InvM.IsMappedToGPU()) InvM.UnmapFromGPU();
    if (InvMOff.IsMappedToGPU()) InvMOff.UnmapFromGPU();
    MappedToGPU = false;
    OnGPU = false;
}

void IndexMapping::MoveFromGPU()
{
    M.MoveFromGPU();
    InvM.MoveFromGPU();
    InvMOff.MoveFromGPU();
    OnGPU = false;
}

void IndexMapping::SwitchFromGPU()
{
    M.SwitchFromGPU();
    InvM.SwitchFromGPU();
    InvMOff.SwitchFromGPU();
    OnGPU = false;
}

}
