// acro::KernelExecutor — the plug-in interface every execution back end sits
// behind (exec/KernelExecutor.hpp:16-45 of LLNL/acrotensor): built from a
// DimensionedMultiKernel, it runs one kernel (ExecuteSingle) or the whole
// group (ExecuteMulti) on the tensors it is handed, and can describe what it
// would run (GetImplementation).  KernelExecutor::Create("Cuda", ...) returns
// the sm_100a back end of this library (B200Executor).  The reference's
// "CPUInterpreted" type is recognised by name but not provided: this library
// is a GPU-only replacement for the "Cuda" policy and has no CPU code path.
#ifndef ACRO_B200_KERNEL_EXECUTOR_HPP
#define ACRO_B200_KERNEL_EXECUTOR_HPP

#include <memory>
#include <string>
#include <vector>
#include "DimensionedMultiKernel.hpp"
#include "Tensor.hpp"

namespace acro
{

class KernelExecutor
{
    public:
    // The executor takes ownership of multi_kernel.
    KernelExecutor(DimensionedMultiKernel *multi_kernel);
    static KernelExecutor *Create(std::string exec_type, DimensionedMultiKernel *multi_kernel);
    virtual ~KernelExecutor();

    virtual std::string GetImplementation() = 0;
    virtual std::string GetExecType() = 0;
    virtual void ExecuteSingle(Tensor *output, std::vector<Tensor *> &inputs) = 0;
    // Default: every member kernel through its own single-kernel executor, in order
    // (exec/KernelExecutor.cpp:86-103).
    virtual void ExecuteMulti(std::vector<Tensor *> &output, std::vector<std::vector<Tensor *>> &inputs);

    // cudaStream_t passed as void*; nullptr selects the library-wide stream (setCudaStream).
    void SetCudaStream(void *cuda_stream) { TheCudaStream = cuda_stream; }
    // acro_b200_peer_group* passed as void*: ranks that share a contracted batch index (nullptr = none).
    void SetPeerGroup(void *peer_group) { ThePeerGroup = peer_group; }

    protected:
    void MoveTensorsFromGPU(Tensor *output, std::vector<Tensor *> &inputs);
    void MoveTensorsToGPU(Tensor *output, std::vector<Tensor *> &inputs);
    void MoveTensorsToOutputLocation(Tensor *output, std::vector<Tensor *> &inputs);
    void *Stream() const;

    std::unique_ptr<DimensionedMultiKernel> OwnedMultiKernel;
    DimensionedMultiKernel *MultiKernel;
    DimensionedKernel *FirstKernel;
    std::vector<std::unique_ptr<KernelExecutor>> SubExecutors;
    void *TheCudaStream;
    void *ThePeerGroup;
};

}

#endif
