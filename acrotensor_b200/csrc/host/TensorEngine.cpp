// acro::TensorEngine: parse / bind / plan caches and single or recorded multi-kernel execution.
#include "TensorEngine.hpp"

namespace acro
{

TensorEngine::TensorEngine() : IsMultiKernelLaunch(false), TheCudaStream(nullptr)
{
    SetExecutorType("Cuda");
}

TensorEngine::TensorEngine(const char *bare_exec_type) : IsMultiKernelLaunch(false), TheCudaStream(nullptr)
{
    SetExecutorType(bare_exec_type);
}

TensorEngine::TensorEngine(std::string &exec_type) : IsMultiKernelLaunch(false), TheCudaStream(nullptr)
{
    SetExecutorType(exec_type);
}

TensorEngine::~TensorEngine() {}

void TensorEngine::SetExecutorType(const char *bare_exec_type)
{
    std::string exec_type(bare_exec_type ? bare_exec_type : "");
    SetExecutorType(exec_type);
}

void TensorEngine::SetExecutorType(std::string &exec_type)
{
    ACROBATIC_ASSERT(exec_type == "Cuda" || exec_type == "CPUInterpreted", "Unknown Executor type:  " + exec_type);
    Clear();
    ExecutorType = exec_type;
}

void TensorEngine::Clear()
{
    ExecutorMap.clear();
    DimensionedKernelMap.clear();
    KernelMap.clear();
    MKLKernels.clear();
    MKLOutputT.clear();
    MKLInputT.clear();
}

void TensorEngine::operator()(const char *bare_kernel_str, Tensor *out, std::vector<Tensor *> &inputs)
{
    std::string kernel_str(bare_kernel_str);
    (*this)(kernel_str, out, inputs);
}

void TensorEngine::Record(std::string &kernel_str, Tensor *output, std::vector<Tensor *> &inputs)
{
    ACROBATIC_ASSERT(output != nullptr && output->IsInitialized(), "Output variable not initilized in:  " + kernel_str);
    for (Tensor *t : inputs)
    {
        ACROBATIC_ASSERT(t != nullptr && t->IsInitialized(), "Input variable not initilized in:  " + kernel_str);
    }
    if (!IsMultiKernelLaunch)
    {
        MKLKernels.clear();
        MKLOutputT.clear();
        MKLInputT.clear();
    }
    TensorKernel *kernel = GetAddTensorKernel(kernel_str);
    DimensionedKernel *bound = GetAddDimensionedKernel(kernel, output, inputs);
    MKLKernels.push_back(bound);
    MKLOutputT.push_back(output);
    MKLInputT.push_back(inputs);
}

void TensorEngine::operator()(std::string &kernel_str, Tensor *output, std::vector<Tensor *> &inputs)
{
    Record(kernel_str, output, inputs);
    if (!IsMultiKernelLaunch)
    {
        KernelExecutor *executor = GetAddKernelExecutor();
        executor->SetCudaStream(TheCudaStream);
        executor->ExecuteSingle(output, inputs);
    }
}

std::string TensorEngine::GetImplementation(const char *bare_kernel_str, Tensor *out, std::vector<Tensor *> &inputs)
{
    std::string kernel_str(bare_kernel_str);
    return GetImplementation(kernel_str, out, inputs);
}

std::string TensorEngine::GetImplementation(std::string &kernel_str, Tensor *output, std::vector<Tensor *> &inputs)
{
    ACROBATIC_ASSERT(!IsMultiKernelLaunch, "GetImplementation can't be used inside a multi kernel launch.");
    Record(kernel_str, output, inputs);
    return GetAddKernelExecutor()->GetImplementation();
}

void TensorEngine::BeginMultiKernelLaunch()
{
    ACROBATIC_ASSERT(!IsMultiKernelLaunch, "Trying to BeginMultiKernelLaunch twice.");
    IsMultiKernelLaunch = true;
    MKLKernels.clear();
    MKLOutputT.clear();
    MKLInputT.clear();
}

void TensorEngine::EndMultiKernelLaunch()
{
    ACROBATIC_ASSERT(IsMultiKernelLaunch, "Found an EndMultiKernelLaunch before a BeginMultiKernelLaunch!");
    IsMultiKernelLaunch = false;
    if (MKLKernels.empty()) return;
    KernelExecutor *executor = GetAddKernelExecutor();
    executor->SetCudaStream(TheCudaStream);
    executor->ExecuteMulti(MKLOutputT, MKLInputT);
}

std::string TensorEngine::EndMultiKernelLaunchDescribe()
{
    ACROBATIC_ASSERT(IsMultiKernelLaunch, "Found an EndMultiKernelLaunch before a BeginMultiKernelLaunch!");
    IsMultiKernelLaunch = false;
    if (MKLKernels.empty()) return "";
    return GetAddKernelExecutor()->GetImplementation();
}

TensorKernel *TensorEngine::GetAddTensorKernel(std::string &kernel_str)
{
    auto it = KernelMap.find(kernel_str);
    if (it == KernelMap.end())
    {
        it = KernelMap.emplace(kernel_str, std::unique_ptr<TensorKernel>(new TensorKernel(kernel_str))).first;
    }
    return it->second.get();
}

DimensionedKernel *TensorEngine::GetAddDimensionedKernel(TensorKernel *kernel, Tensor *output, std::vector<Tensor *> &inputs)
{
    // The key spells the kernel and every loop extent, so equal keys mean equal bindings.
    std::string key = kernel->GetDimensionedNameString(output, inputs);
    auto it = DimensionedKernelMap.find(key);
    if (it == DimensionedKernelMap.end())
    {
        it = DimensionedKernelMap.emplace(key, std::unique_ptr<DimensionedKernel>(new DimensionedKernel(kernel, output, inputs))).first;
    }
    return it->second.get();
}

KernelExecutor *TensorEngine::GetAddKernelExecutor()
{
    std::string key;
    for (DimensionedKernel *k : MKLKernels) key += k->GetDimensionedNameString() + ";";
    auto it = ExecutorMap.find(key);
    if (it == ExecutorMap.end())
    {
        KernelExecutor *executor = KernelExecutor::Create(ExecutorType, new DimensionedMultiKernel(MKLKernels));
        it = ExecutorMap.emplace(key, std::unique_ptr<KernelExecutor>(executor)).first;
    }
    return it->second.get();
}

}
