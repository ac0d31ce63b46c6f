// acro::DimensionedKernel — a parsed kernel bound to concrete tensor extents:
// per-loop extents and strides, dense per-variable strides and sizes.
// Follows kernel/DimensionedKernel.hpp:19-67 of LLNL/acrotensor; counts that
// can exceed 2^31 (the flat index space of the benchmark kernels does) are
// also available as 64-bit values.
#ifndef ACRO_B200_DIMENSIONED_KERNEL_HPP
#define ACRO_B200_DIMENSIONED_KERNEL_HPP

#include <cstdint>
#include "TensorKernel.hpp"

namespace acro
{

class DimensionedKernel : public TensorKernel
{
    public:
    DimensionedKernel(TensorKernel *kernel, Tensor *output, std::vector<Tensor *> &inputs);

    const std::vector<int> &GetLoopDims() { return LoopDims; }
    const std::vector<int> &GetLoopStrides() { return LoopStrides; }
    int GetLoopDim(std::string &idx) { return LoopDims[GetLoopNum(idx)]; }
    int GetLoopStride(std::string &idx) { return LoopStrides[GetLoopNum(idx)]; }
    int GetLoopDim(int i) { return LoopDims[i]; }
    int GetLoopStride(int i) { return LoopStrides[i]; }
    void SetLoopIndices(std::vector<std::string> &idx_list) override;

    std::string GetLoopDimsString();
    std::string GetDimensionedNameString() override { return GetNameString() + GetLoopDimsString(); }
    std::string GetDimensionedNameString(Tensor *, std::vector<Tensor *> &) override { return GetDimensionedNameString(); }

    int GetFlatIdxSize() { return static_cast<int>(GetFlatIdxSize64()); }
    std::int64_t GetFlatIdxSize64();
    int GetOutIdxSize();
    int GetContIdxSize();
    int GetIdxSizeForFirstNumLoops(int num_loops);
    int GetLoopsIdxSize(std::vector<int> loops);

    int GetVarDimSize(int vari, int dim) { return LoopDims[GetVarDimLoopNum(vari, dim)]; }
    int GetVarDimStride(int vari, int dim) { return static_cast<int>(GetVarDimStride64(vari, dim)); }
    std::int64_t GetVarDimStride64(int vari, int dim);
    int GetVarSize(int vari) { return static_cast<int>(GetVarSize64(vari)); }
    std::int64_t GetVarSize64(int vari);

    // Storage touched by the innermost num_loops loops (entries, not bytes).
    int GetVarStorageReqForInnerLoops(int vari, int num_loops);
    int GetInputStorageReqForInnerLoops(int num_loops);
    int GetOutputStorageReqForInnerLoops(int num_loops);
    int GetTotalStorageReqForInnerLoops(int num_loops);
    int GetIndexSpaceSizeForInnerLoops(int num_loops);

    private:
    void RebuildLoopStrides();
    std::vector<int> LoopDims;
    std::vector<int> LoopStrides;
};

}

#endif
