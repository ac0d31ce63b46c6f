// Parser and index bookkeeping for contraction strings.
#include "TensorKernel.hpp"

#include <algorithm>
#include <cctype>

namespace acro
{

namespace
{

// A cursor over the whitespace-free kernel text; peeking past the end yields '\0'.
struct Cursor
{
    const std::string &text;
    std::size_t pos;
    char peek() const { return pos < text.size() ? text[pos] : '\0'; }
    char next() { return pos < text.size() ? text[pos++] : '\0'; }
    bool done() const { return pos >= text.size(); }
};

bool is_upper(char c) { return std::isupper(static_cast<unsigned char>(c)) != 0; }
bool is_index_char(char c)
{
    return std::islower(static_cast<unsigned char>(c)) != 0 || std::isdigit(static_cast<unsigned char>(c)) != 0;
}
bool is_name_char(char c) { return std::isalnum(static_cast<unsigned char>(c)) != 0; }

// var := Upper alnum* ("_" index_char+)+
KernelVar read_var(Cursor &cur, const std::string &whole)
{
    KernelVar var;
    ACROBATIC_ASSERT(is_upper(cur.peek()), "Variable names start with an upper case letter in kernel:  " + whole);
    while (is_name_char(cur.peek())) var.Name += cur.next();
    ACROBATIC_ASSERT(cur.peek() == '_', "Variable " + var.Name + " has no index in kernel:  " + whole);
    while (cur.peek() == '_')
    {
        cur.next();
        ACROBATIC_ASSERT(is_index_char(cur.peek()), "Empty or malformed index on " + var.Name + " in kernel:  " + whole);
        std::string idx;
        while (is_index_char(cur.peek())) idx += cur.next();
        var.IndexNames.push_back(idx);
    }
    var.LoopNums.assign(var.IndexNames.size(), -1);
    return var;
}

std::string read_operator(Cursor &cur, const std::string &whole)
{
    std::string op;
    if (cur.peek() == '+' || cur.peek() == '-') op += cur.next();
    ACROBATIC_ASSERT(cur.peek() == '=', "Expected =, += or -= in kernel:  " + whole);
    op += cur.next();
    return op;
}

template <class C, class V>
bool contains(const C &c, const V &v)
{
    return std::find(c.begin(), c.end(), v) != c.end();
}

}

TensorKernel::TensorKernel(const char *kernel) : KernelStr(kernel) { Parse(); }
TensorKernel::TensorKernel(std::string &kernel) : KernelStr(kernel) { Parse(); }

void TensorKernel::Parse()
{
    std::string squeezed;
    for (char c : KernelStr)
    {
        if (!std::isspace(static_cast<unsigned char>(c))) squeezed += c;
    }
    Cursor cur{squeezed, 0};
    OutputVar = read_var(cur, KernelStr);
    EqOperator = read_operator(cur, KernelStr);
    do
    {
        InputVars.push_back(read_var(cur, KernelStr));
    } while (!cur.done());

    // Output indices come first; what only the inputs carry is contracted, in
    // order of first appearance.  This order is the summation order.
    for (const std::string &idx : OutputVar.IndexNames)
    {
        if (!contains(AllIndexNames, idx)) AllIndexNames.push_back(idx);
    }
    for (const KernelVar &var : InputVars)
    {
        for (const std::string &idx : var.IndexNames)
        {
            if (!contains(AllIndexNames, idx))
            {
                ContractionIndexNames.push_back(idx);
                AllIndexNames.push_back(idx);
            }
        }
    }
    LoopIndices = AllIndexNames;
    BindLoopNums();
}

KernelVar &TensorKernel::Var(int vari)
{
    ACROBATIC_ASSERT(vari >= -1 && vari < GetNumInputVars(), "Variable number out of range.");
    return vari < 0 ? OutputVar : InputVars[vari];
}

void TensorKernel::BindLoopNums()
{
    for (int vari = -1; vari < GetNumInputVars(); ++vari)
    {
        KernelVar &var = Var(vari);
        var.LoopNums.resize(var.IndexNames.size());
        for (std::size_t d = 0; d < var.IndexNames.size(); ++d)
        {
            auto it = std::find(LoopIndices.begin(), LoopIndices.end(), var.IndexNames[d]);
            var.LoopNums[d] = static_cast<int>(it - LoopIndices.begin());
        }
    }
}

int TensorKernel::GetVarRank(int vari) { return static_cast<int>(Var(vari).IndexNames.size()); }
std::string &TensorKernel::GetVarName(int vari) { return Var(vari).Name; }

int TensorKernel::GetLoopNum(std::string &idx)
{
    auto it = std::find(LoopIndices.begin(), LoopIndices.end(), idx);
    ACROBATIC_ASSERT(it != LoopIndices.end(), "Loop index (" + idx + ") not found in kernel:\n" + KernelStr + "\n");
    return static_cast<int>(it - LoopIndices.begin());
}

void TensorKernel::SetLoopIndices(std::vector<std::string> &idx_list)
{
    LoopIndices = idx_list;
    BindLoopNums();
}

int TensorKernel::GetVarDimLoopNum(int vari, int dim)
{
    KernelVar &var = Var(vari);
    ACROBATIC_ASSERT(dim >= 0 && dim < static_cast<int>(var.LoopNums.size()), "Dimension out of range.");
    return var.LoopNums[dim];
}

int TensorKernel::GetLoopNumVarDim(int loop_num, int vari)
{
    ACROBATIC_ASSERT(loop_num >= 0 && loop_num < static_cast<int>(LoopIndices.size()), "Loop number out of range.");
    KernelVar &var = Var(vari);
    for (std::size_t d = 0; d < var.IndexNames.size(); ++d)
    {
        if (var.IndexNames[d] == LoopIndices[loop_num]) return static_cast<int>(d);
    }
    return -1;
}

bool TensorKernel::IsVarDependentOnLoop(int vari, int loop_num) { return GetLoopNumVarDim(loop_num, vari) >= 0; }
bool TensorKernel::IsDependentOnIndex(std::string &idx) { return contains(AllIndexNames, idx); }
bool TensorKernel::IsDependentOnLoop(int loop_num) { return IsDependentOnIndex(LoopIndices[loop_num]); }
bool TensorKernel::IsContractionIndex(std::string &idx) { return contains(ContractionIndexNames, idx); }
bool TensorKernel::IsContractionLoop(int loop_num) { return IsContractionIndex(LoopIndices[loop_num]); }

bool TensorKernel::IsContractionVar(int vari)
{
    if (vari < 0) return false;
    for (std::string &idx : Var(vari).IndexNames)
    {
        if (IsContractionIndex(idx)) return true;
    }
    return false;
}

int TensorKernel::GetVarLoopDepth(int vari)
{
    int depth = -1;
    for (int loop = 0; loop < static_cast<int>(LoopIndices.size()); ++loop)
    {
        if (IsVarDependentOnLoop(vari, loop)) depth = loop;
    }
    return depth;
}

int TensorKernel::GetLoopDepth()
{
    int depth = -1;
    for (int vari = -1; vari < GetNumInputVars(); ++vari) depth = std::max(depth, GetVarLoopDepth(vari));
    return depth;
}

std::string TensorKernel::GetNameString()
{
    auto spell = [](const KernelVar &var) {
        std::string s = var.Name;
        for (const std::string &idx : var.IndexNames) s += "_" + idx;
        return s;
    };
    std::string name = spell(OutputVar);
    name += (EqOperator == "=") ? "eq" : (EqOperator == "+=") ? "pe" : "me";
    for (const KernelVar &var : InputVars) name += spell(var);
    return name;
}

std::string TensorKernel::GetDimensionedNameString(Tensor *output, std::vector<Tensor *> &inputs)
{
    std::string name = GetNameString() + "_";
    for (int extent : GetLoopIdxSizes(output, inputs)) name += "_" + std::to_string(extent);
    return name;
}

std::vector<int> TensorKernel::GetLoopIdxSizes(Tensor *output, std::vector<Tensor *> &inputs)
{
    ACROBATIC_ASSERT(output->GetRank() == GetVarRank(-1),
                     "Tensor rank of the output var in the kernel does not match the rank of the actual tensor.\nKernel:  " + KernelStr);
    ACROBATIC_ASSERT(static_cast<int>(inputs.size()) == GetNumInputVars(),
                     "Number of input tensors does not match the kernel:  " + KernelStr);
    std::vector<int> sizes(LoopIndices.size(), 1);   // loops this kernel does not use have extent 1
    std::vector<bool> fixed(LoopIndices.size(), false);
    for (int vari = 0; vari < GetNumInputVars(); ++vari)
    {
        ACROBATIC_ASSERT(inputs[vari]->GetRank() == GetVarRank(vari),
                         "Tensor rank of input var " + std::to_string(vari) +
                             " does not match the rank of the actual tensor.\nKernel:  " + KernelStr);
        for (int d = 0; d < GetVarRank(vari); ++d)
        {
            int loop = GetVarDimLoopNum(vari, d);
            ACROBATIC_ASSERT(!fixed[loop] || sizes[loop] == inputs[vari]->GetDim(d),
                             "Incompatible tensor dimensions for kernel:  " + KernelStr);
            sizes[loop] = inputs[vari]->GetDim(d);
            fixed[loop] = true;
        }
    }
    // The output must agree with the inputs too (the reference leaves this unchecked and
    // would write out of bounds); an index only the output carries takes the output's extent.
    for (int d = 0; d < GetVarRank(-1); ++d)
    {
        int loop = GetVarDimLoopNum(-1, d);
        ACROBATIC_ASSERT(!fixed[loop] || sizes[loop] == output->GetDim(d),
                         "Incompatible output tensor dimensions for kernel:  " + KernelStr);
        sizes[loop] = output->GetDim(d);
        fixed[loop] = true;
    }
    return sizes;
}

}
