// A group of bound kernels executed as one unit.
#include "DimensionedMultiKernel.hpp"

#include <algorithm>

namespace acro
{

namespace
{
template <class C, class V>
bool contains(const C &c, const V &v)
{
    return std::find(c.begin(), c.end(), v) != c.end();
}
}

DimensionedMultiKernel::DimensionedMultiKernel(std::vector<DimensionedKernel *> &kernels) { Adopt(kernels); }

DimensionedMultiKernel::DimensionedMultiKernel(DimensionedKernel *kernel)
{
    std::vector<DimensionedKernel *> one = {kernel};
    Adopt(one);
}

void DimensionedMultiKernel::Adopt(std::vector<DimensionedKernel *> &kernels)
{
    for (DimensionedKernel *k : kernels)
    {
        Owned.emplace_back(new DimensionedKernel(*k));   // private copy: loop re-ordering stays local
        Kernels.push_back(Owned.back().get());
    }
    Analyse();
}

void DimensionedMultiKernel::Analyse()
{
    std::vector<std::string> var_names;
    for (int ki = 0; ki < GetNumKernels(); ++ki)
    {
        DimensionedKernel *k = Kernels[ki];
        for (std::string &idx : k->AllIndexNames)
        {
            if (!contains(AllIndexNames, idx)) AllIndexNames.push_back(idx);
        }
        for (std::string &idx : k->ContractionIndexNames)
        {
            if (!contains(ContractionIndexNames, idx)) ContractionIndexNames.push_back(idx);
        }
        for (int vari = -1; vari < k->GetNumInputVars(); ++vari)
        {
            auto it = std::find(var_names.begin(), var_names.end(), k->GetVarName(vari));
            if (it == var_names.end())
            {
                KiVariToUVari[std::make_pair(ki, vari)] = static_cast<int>(var_names.size());
                UVariToFirstKiVari.push_back(std::make_pair(ki, vari));
                var_names.push_back(k->GetVarName(vari));
            }
            else
            {
                KiVariToUVari[std::make_pair(ki, vari)] = static_cast<int>(it - var_names.begin());
            }
        }
    }

    // Shared outer = a non-contracted loop of every member.
    std::vector<std::string> shared;
    for (std::string &idx : AllIndexNames)
    {
        bool everywhere = true;
        for (DimensionedKernel *k : Kernels)
        {
            everywhere = everywhere && k->IsDependentOnIndex(idx) && !k->IsContractionIndex(idx);
        }
        if (everywhere) shared.push_back(idx);
    }

    // Extents are needed to rank the shared loops: bind any complete order first.
    std::vector<std::string> order = shared;
    for (std::string &idx : AllIndexNames)
    {
        if (!contains(order, idx)) order.push_back(idx);
    }
    SetLoopIndices(order);

    // Largest extent first; equal extents keep alphabetical order.
    std::sort(shared.begin(), shared.end());
    std::stable_sort(shared.begin(), shared.end(),
                     [this](const std::string &a, const std::string &b) {
                         std::string aa = a, bb = b;
                         return GetLoopDim(aa) > GetLoopDim(bb);
                     });
    SharedOuterIndexNames = shared;
    order = shared;
    for (std::string &idx : AllIndexNames)
    {
        if (!contains(order, idx)) order.push_back(idx);
    }
    SetLoopIndices(order);
}

void DimensionedMultiKernel::SetLoopIndices(std::vector<std::string> &idx_list)
{
    LoopDims.assign(idx_list.size(), 1);
    for (DimensionedKernel *k : Kernels)
    {
        k->SetLoopIndices(idx_list);
        for (std::size_t l = 0; l < idx_list.size(); ++l) LoopDims[l] = std::max(LoopDims[l], k->GetLoopDim(static_cast<int>(l)));
    }
    LoopStrides.assign(idx_list.size(), 1);
    for (int l = static_cast<int>(idx_list.size()) - 2; l >= 0; --l) LoopStrides[l] = LoopStrides[l + 1] * LoopDims[l + 1];
    LoopIndices = idx_list;
}

int DimensionedMultiKernel::GetNumInputVars()
{
    int n = 0;
    for (DimensionedKernel *k : Kernels) n += k->GetNumInputVars();
    return n;
}

std::string DimensionedMultiKernel::GetDimensionedNameString()
{
    std::string s;
    for (DimensionedKernel *k : Kernels) s += k->GetDimensionedNameString() + ";";
    return s;
}

int DimensionedMultiKernel::GetIndexLoopNum(std::string &idx)
{
    auto it = std::find(LoopIndices.begin(), LoopIndices.end(), idx);
    return it == LoopIndices.end() ? -1 : static_cast<int>(it - LoopIndices.begin());
}

bool DimensionedMultiKernel::IsContractionLoop(int loop_num) { return contains(ContractionIndexNames, LoopIndices[loop_num]); }
bool DimensionedMultiKernel::IsSharedOuterLoop(int loop_num) { return contains(SharedOuterIndexNames, LoopIndices[loop_num]); }

bool DimensionedMultiKernel::IsOutputUVar(int uvari)
{
    for (int ki = 0; ki < GetNumKernels(); ++ki)
    {
        if (GetUVari(ki, -1) == uvari) return true;
    }
    return false;
}

bool DimensionedMultiKernel::IsInputUVar(int uvari)
{
    for (int ki = 0; ki < GetNumKernels(); ++ki)
    {
        for (int vari = 0; vari < Kernels[ki]->GetNumInputVars(); ++vari)
        {
            if (GetUVari(ki, vari) == uvari) return true;
        }
    }
    return false;
}

std::int64_t DimensionedMultiKernel::GetFlatIdxSize64()
{
    std::int64_t n = 1;
    for (int extent : LoopDims) n *= extent;
    return n;
}

int DimensionedMultiKernel::GetSharedOuterIdxSize() { return GetIdxSizeForFirstNumLoops(GetNumOuterIndices()); }

int DimensionedMultiKernel::GetIdxSizeForFirstNumLoops(int num_loops)
{
    ACROBATIC_ASSERT(num_loops <= GetNumIndices(), "More loops requested than the kernel group has.");
    std::int64_t n = 1;
    for (int l = 0; l < num_loops; ++l) n *= LoopDims[l];
    return static_cast<int>(n);
}

int DimensionedMultiKernel::GetVarSize(int uvari)
{
    std::pair<int, int> first = GetFirstKiVariForUVari(uvari);
    return Kernels[first.first]->GetVarSize(first.second);
}

}
