// acro::TensorKernel — the parsed form of one contraction string such as
// "S_i_j = A_n_i_j B_n".
//
// Grammar (kernel/TensorKernel.cpp:26-139 of LLNL/acrotensor):
//     kernel := var op var+          op := "=" | "+=" | "-="
//     var    := Upper alnum* ("_" (lower|digit)+)+
// Whitespace is ignored.  AllIndexNames lists the output indices first and
// then the contracted indices in order of first appearance; that order fixes
// the order in which terms are summed (kernel/TensorKernel.cpp:45-63).
// The public data members and queries keep the reference's names
// (kernel/TensorKernel.hpp:15-104) so code written against it compiles.
#ifndef ACRO_B200_TENSOR_KERNEL_HPP
#define ACRO_B200_TENSOR_KERNEL_HPP

#include <string>
#include <vector>
#include "Tensor.hpp"

namespace acro
{

class KernelVar
{
    public:
    std::string Name;
    std::vector<std::string> IndexNames;
    std::vector<int> LoopNums;   // loop number bound to each dimension
};

class TensorKernel
{
    protected:
    TensorKernel() {}

    public:
    TensorKernel(const char *kernel);
    TensorKernel(std::string &kernel);
    virtual ~TensorKernel() {}

    int GetNumIndices() { return static_cast<int>(AllIndexNames.size()); }
    int GetNumOuterIndices() { return static_cast<int>(AllIndexNames.size() - ContractionIndexNames.size()); }
    int GetNumContractionIndices() { return static_cast<int>(ContractionIndexNames.size()); }
    int GetNumVars() { return static_cast<int>(InputVars.size()) + 1; }
    int GetNumInputVars() { return static_cast<int>(InputVars.size()); }

    // vari = -1 addresses the output variable, 0.. the inputs.
    int GetVarRank(int vari);
    std::string &GetVarName(int vari);

    std::string GetLoopIndex(int loopi) { return LoopIndices[loopi]; }
    int GetLoopNum(std::string &idx);
    virtual void SetLoopIndices(std::vector<std::string> &idx_list);

    int GetVarDimLoopNum(int vari, int dim);
    int GetLoopNumVarDim(int loop_num, int vari);   // -1 when the variable does not carry that loop
    bool IsVarDependentOnLoop(int vari, int loop_num);
    bool IsDependentOnIndex(std::string &idx);
    bool IsDependentOnLoop(int loop_num);
    bool IsContractionIndex(std::string &idx);
    bool IsContractionLoop(int loop_num);
    bool IsContractionVar(int vari);
    int GetLoopDepth();
    int GetVarLoopDepth(int vari);

    // Canonical text of the parsed kernel, used as a cache key.
    std::string GetNameString();
    virtual std::string GetDimensionedNameString()
    {
        ACROBATIC_ASSERT(false, "A TensorKernel has no dimensions yet.");
        return "";
    }
    virtual std::string GetDimensionedNameString(Tensor *output, std::vector<Tensor *> &inputs);

    // Extent of every loop given the attached tensors; throws when two tensors disagree.
    std::vector<int> GetLoopIdxSizes(Tensor *output, std::vector<Tensor *> &inputs);

    std::string KernelStr;
    KernelVar OutputVar;
    std::string EqOperator;
    std::vector<KernelVar> InputVars;
    std::vector<std::string> AllIndexNames;
    std::vector<std::string> ContractionIndexNames;
    std::vector<std::string> LoopIndices;

    protected:
    KernelVar &Var(int vari);
    void BindLoopNums();

    private:
    void Parse();
};

}

#endif
