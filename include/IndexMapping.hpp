// acro::IndexMapping — a map M from a "range" of flat positions (size range_size) into a
// "domain" (size domain_size), M[i] in [0, domain_size), plus its inverse in CSR form:
// InvMap lists the range positions grouped by domain entry (stable: ascending position
// inside a group) and InvMapOffsets[d] .. InvMapOffsets[d+1] delimits group d.
// Follows tensor/IndexMapping.hpp:14-48 and tensor/IndexMapping.cpp:27-62 of LLNL/acrotensor.
#ifndef ACRO_B200_INDEX_MAPPING_HPP
#define ACRO_B200_INDEX_MAPPING_HPP

#include <vector>
#include "IndexVector.hpp"

namespace acro
{

class IndexMapping
{
    public:
    IndexMapping(int domain_size, int range_size);

    int GetDomainSize() { return DomainSize; }
    int GetRangeSize() { return RangeSize; }
    bool IsInverseComputed() { return InverseComputed; }

    int &operator[](int raw_index) { return M[raw_index]; }
    void ComputeInverse();

    IndexVector &GetMap() { return M; }
    IndexVector &GetInvMap();
    IndexVector &GetInvMapOffsets();

    void MapToGPU();
    void MoveToGPU();
    void SwitchToGPU();
    void UnmapFromGPU();
    void MoveFromGPU();
    void SwitchFromGPU();
    bool IsMappedToGPU() const { return MappedToGPU; }
    bool IsOnGPU() const { return OnGPU; }

    private:
    bool InverseComputed;
    bool MappedToGPU;
    bool OnGPU;
    int DomainSize;
    int RangeSize;
    IndexVector M;
    IndexVector InvM, InvMOff;
};

}

#endif
