// acro::DimensionedMultiKernel — one or more bound kernels that execute as a
// unit: variables with the same name are one tensor ("uvar"), indices that are
// a non-contracted loop of every member are "shared outer" loops, and the
// common loop order puts those first, largest extent first (ties by name),
// followed by the remaining indices in order of first appearance.
// Follows kernel/DimensionedMultiKernel.hpp:17-120 and
// kernel/DimensionedMultiKernel.cpp:25-135 of LLNL/acrotensor.  Unlike the
// reference this object owns private copies of its member kernels, so
// re-ordering loops here never disturbs kernels cached elsewhere.
#ifndef ACRO_B200_DIMENSIONED_MULTI_KERNEL_HPP
#define ACRO_B200_DIMENSIONED_MULTI_KERNEL_HPP

#include <map>
#include <memory>
#include <utility>
#include "DimensionedKernel.hpp"

namespace acro
{

class DimensionedMultiKernel
{
    public:
    DimensionedMultiKernel(std::vector<DimensionedKernel *> &kernels);
    DimensionedMultiKernel(DimensionedKernel *kernel);

    int GetNumKernels() { return static_cast<int>(Kernels.size()); }
    int GetNumIndices() { return static_cast<int>(AllIndexNames.size()); }
    int GetNumOuterIndices() { return static_cast<int>(SharedOuterIndexNames.size()); }
    int GetNumContractionIndices() { return static_cast<int>(ContractionIndexNames.size()); }
    int GetNumVars() { return GetNumInputVars() + GetNumOutputVars(); }
    int GetNumUVars() { return static_cast<int>(UVariToFirstKiVari.size()); }
    int GetNumInputVars();
    int GetNumOutputVars() { return GetNumKernels(); }

    std::string GetDimensionedNameString();
    std::string GetLoopIndex(int loopi) { return LoopIndices[loopi]; }
    int GetIndexLoopNum(std::string &idx);
    void SetLoopIndices(std::vector<std::string> &idx_list);

    // (ki, vari) addresses variable vari (-1 = output) of member kernel ki.
    int GetVarRank(int ki, int vari) { return Kernels[ki]->GetVarRank(vari); }
    int GetVarDimLoopNum(int ki, int vari, int dim) { return Kernels[ki]->GetVarDimLoopNum(vari, dim); }
    int GetLoopNumVarDim(int loop_num, int ki, int vari) { return Kernels[ki]->GetLoopNumVarDim(loop_num, vari); }
    bool IsVarDependentOnLoop(int ki, int vari, int loop_num) { return Kernels[ki]->IsVarDependentOnLoop(vari, loop_num); }
    bool IsContractionLoop(int loop_num);
    bool IsSharedOuterLoop(int loop_num);
    bool IsOutputUVar(int uvari);
    bool IsInputUVar(int uvari);

    const std::vector<int> &GetLoopDims() { return LoopDims; }
    int GetLoopDim(int i) { return LoopDims[i]; }
    int GetLoopDim(std::string &idx) { return LoopDims[GetIndexLoopNum(idx)]; }
    int GetLoopStride(int i) { return LoopStrides[i]; }
    std::int64_t GetFlatIdxSize64();
    int GetFlatIdxSize() { return static_cast<int>(GetFlatIdxSize64()); }
    int GetSharedOuterIdxSize();
    int GetIdxSizeForFirstNumLoops(int num_loops);
    int GetVarDimStride(int ki, int vari, int dim) { return Kernels[ki]->GetVarDimStride(vari, dim); }
    int GetVarSize(int ki, int vari) { return Kernels[ki]->GetVarSize(vari); }
    int GetVarSize(int uvari);
    int GetVarLoopDepth(int ki, int vari) { return Kernels[ki]->GetVarLoopDepth(vari); }

    // Unique variables are numbered in order of first appearance.
    int GetUVari(int ki, int vari) { return KiVariToUVari[std::make_pair(ki, vari)]; }
    std::pair<int, int> GetFirstKiVariForUVari(int uvari) { return UVariToFirstKiVari[uvari]; }

    std::vector<DimensionedKernel *> Kernels;   // private copies, owned by this object
    std::vector<std::string> AllIndexNames;
    std::vector<std::string> ContractionIndexNames;
    std::vector<std::string> SharedOuterIndexNames;
    std::vector<std::string> LoopIndices;

    private:
    void Adopt(std::vector<DimensionedKernel *> &kernels);
    void Analyse();

    std::vector<std::unique_ptr<DimensionedKernel>> Owned;
    std::map<std::pair<int, int>, int> KiVariToUVari;
    std::vector<std::pair<int, int>> UVariToFirstKiVari;
    std::vector<int> LoopDims;
    std::vector<int> LoopStrides;
};

}

#endif
