// A parsed kernel bound to concrete extents.
#include "DimensionedKernel.hpp"

#include <algorithm>

namespace acro
{

DimensionedKernel::DimensionedKernel(TensorKernel *kernel, Tensor *output, std::vector<Tensor *> &inputs)
{
    KernelStr = kernel->KernelStr;
    OutputVar = kernel->OutputVar;
    EqOperator = kernel->EqOperator;
    InputVars = kernel->InputVars;
    AllIndexNames = kernel->AllIndexNames;
    ContractionIndexNames = kernel->ContractionIndexNames;
    LoopIndices = kernel->LoopIndices;
    LoopDims = kernel->GetLoopIdxSizes(output, inputs);
    RebuildLoopStrides();
}

void DimensionedKernel::RebuildLoopStrides()
{
    LoopStrides.assign(LoopDims.size(), 1);
    for (int l = static_cast<int>(LoopDims.size()) - 2; l >= 0; --l)
    {
        LoopStrides[l] = LoopStrides[l + 1] * LoopDims[l + 1];
    }
}

void DimensionedKernel::SetLoopIndices(std::vector<std::string> &idx_list)
{
    // Carry each known index's extent to its new position; foreign indices get extent 1.
    std::vector<int> dims(idx_list.size(), 1);
    for (std::size_t l = 0; l < idx_list.size(); ++l)
    {
        auto it = std::find(LoopIndices.begin(), LoopIndices.end(), idx_list[l]);
        if (it != LoopIndices.end()) dims[l] = LoopDims[it - LoopIndices.begin()];
    }
    LoopDims.swap(dims);
    RebuildLoopStrides();
    TensorKernel::SetLoopIndices(idx_list);
}

std::string DimensionedKernel::GetLoopDimsString()
{
    std::string s = "__dim";
    for (std::string &idx : AllIndexNames) s += "_" + std::to_string(GetLoopDim(idx));
    return s;
}

std::int64_t DimensionedKernel::GetFlatIdxSize64()
{
    std::int64_t n = 1;
    for (int extent : LoopDims) n *= extent;
    return n;
}

int DimensionedKernel::GetOutIdxSize()
{
    std::int64_t n = 1;
    for (int l = 0; l < static_cast<int>(LoopDims.size()); ++l)
    {
        if (!IsContractionLoop(l)) n *= LoopDims[l];
    }
    return static_cast<int>(n);
}

int DimensionedKernel::GetContIdxSize()
{
    std::int64_t n = 1;
    for (int l = 0; l < static_cast<int>(LoopDims.size()); ++l)
    {
        if (IsContractionLoop(l)) n *= LoopDims[l];
    }
    return static_cast<int>(n);
}

int DimensionedKernel::GetLoopsIdxSize(std::vector<int> loops)
{
    std::int64_t n = 1;
    for (int l : loops) n *= LoopDims[l];
    return static_cast<int>(n);
}

int DimensionedKernel::GetIdxSizeForFirstNumLoops(int num_loops)
{
    ACROBATIC_ASSERT(num_loops <= GetNumIndices(), "More loops requested than the kernel has.");
    std::int64_t n = 1;
    for (int l = 0; l < num_loops; ++l) n *= LoopDims[l];
    return static_cast<int>(n);
}

std::int64_t DimensionedKernel::GetVarDimStride64(int vari, int dim)
{
    // Variables are dense row-major over their own dimensions.
    std::int64_t stride = 1;
    for (int d = GetVarRank(vari) - 1; d > dim; --d) stride *= LoopDims[GetVarDimLoopNum(vari, d)];
    return stride;
}

std::int64_t DimensionedKernel::GetVarSize64(int vari)
{
    std::int64_t n = 1;
    for (int d = 0; d < GetVarRank(vari); ++d) n *= LoopDims[GetVarDimLoopNum(vari, d)];
    return n;
}

int DimensionedKernel::GetVarStorageReqForInnerLoops(int vari, int num_loops)
{
    ACROBATIC_ASSERT(num_loops >= 0 && num_loops <= GetNumIndices(), "Inner loop count out of range.");
    std::int64_t entries = 1;
    for (int l = GetNumIndices() - num_loops; l < GetNumIndices(); ++l)
    {
        if (IsVarDependentOnLoop(vari, l)) entries *= LoopDims[l];
    }
    return static_cast<int>(entries);
}

int DimensionedKernel::GetInputStorageReqForInnerLoops(int num_loops)
{
    int entries = 0;
    for (int vari = 0; vari < GetNumInputVars(); ++vari) entries += GetVarStorageReqForInnerLoops(vari, num_loops);
    return entries;
}

int DimensionedKernel::GetOutputStorageReqForInnerLoops(int num_loops)
{
    return GetVarStorageReqForInnerLoops(-1, num_loops);
}

int DimensionedKernel::GetTotalStorageReqForInnerLoops(int num_loops)
{
    return GetInputStorageReqForInnerLoops(num_loops) + GetOutputStorageReqForInnerLoops(num_loops);
}

int DimensionedKernel::GetIndexSpaceSizeForInnerLoops(int num_loops)
{
    std::int64_t n = 1;
    for (int l = GetNumIndices() - num_loops; l < GetNumIndices(); ++l) n *= LoopDims[l];
    return static_cast<int>(n);
}

}
