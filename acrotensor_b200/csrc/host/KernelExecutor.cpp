// Executor base: ownership, tensor placement helpers, factory.
#include "KernelExecutor.hpp"
#include "B200Executor.hpp"

namespace acro
{

KernelExecutor::KernelExecutor(DimensionedMultiKernel *multi_kernel)
    : OwnedMultiKernel(multi_kernel), MultiKernel(multi_kernel), FirstKernel(nullptr), TheCudaStream(nullptr), ThePeerGroup(nullptr)
{
    ACROBATIC_ASSERT(multi_kernel != nullptr, "An executor needs a kernel group.");
    if (MultiKernel->GetNumKernels() > 0) FirstKernel = MultiKernel->Kernels[0];
}

KernelExecutor::~KernelExecutor() {}

void *KernelExecutor::Stream() const { return TheCudaStream ? TheCudaStream : getCudaStream(); }

void KernelExecutor::MoveTensorsFromGPU(Tensor *output, std::vector<Tensor *> &inputs)
{
    if (output->IsOnGPU()) output->MoveFromGPU();
    for (Tensor *t : inputs)
    {
        if (t->IsOnGPU()) t->MoveFromGPU();
    }
}

void KernelExecutor::MoveTensorsToGPU(Tensor *output, std::vector<Tensor *> &inputs)
{
    // MoveToGPU maps on demand and copies only when the host side is the fresh one.
    if (!output->IsOnGPU()) output->MoveToGPU();
    for (Tensor *t : inputs)
    {
        if (!t->IsOnGPU()) t->MoveToGPU();
    }
}

void KernelExecutor::MoveTensorsToOutputLocation(Tensor *output, std::vector<Tensor *> &inputs)
{
    if (output->IsOnGPU()) MoveTensorsToGPU(output, inputs);
    else MoveTensorsFromGPU(output, inputs);
}

void KernelExecutor::ExecuteMulti(std::vector<Tensor *> &output, std::vector<std::vector<Tensor *>> &inputs)
{
    const int n = MultiKernel->GetNumKernels();
    if (static_cast<int>(SubExecutors.size()) != n)
    {
        SubExecutors.clear();
        for (int ki = 0; ki < n; ++ki)
        {
            SubExecutors.emplace_back(Create(GetExecType(), new DimensionedMultiKernel(MultiKernel->Kernels[ki])));
        }
    }
    for (int ki = 0; ki < n; ++ki)
    {
        SubExecutors[ki]->SetCudaStream(TheCudaStream);
        SubExecutors[ki]->SetPeerGroup(ThePeerGroup);
        SubExecutors[ki]->ExecuteSingle(output[ki], inputs[ki]);
    }
}

KernelExecutor *KernelExecutor::Create(std::string exec_type, DimensionedMultiKernel *multi_kernel)
{
    std::unique_ptr<DimensionedMultiKernel> guard(multi_kernel);
    if (exec_type == "Cuda")
    {
        return new B200Executor(guard.release());
    }
    ACROBATIC_ASSERT(exec_type != "CPUInterpreted",
                     "The CPUInterpreted executor is not part of this library: it is a GPU-only "
                     "replacement for the Cuda execution policy.");
    ACROBATIC_ASSERT(false, "Executor type does not exist:  " + exec_type);
    return nullptr;
}

}
