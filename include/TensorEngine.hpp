// acro::TensorEngine — the user entry point: TE("S_i_j = A_n_i_j B_n", S, A, B).
//
// Keeps the public surface of kernel/TensorEngine.hpp:26-86 of LLNL/acrotensor for
// the contraction path: construction from an execution-policy string,
// SetExecutorType / GetExecType, operator() and GetImplementation with 1..N
// inputs (by reference, or as Tensor* + vector<Tensor*>), Clear,
// IsGPUAvailable and Begin/EndMultiKernelLaunch, with the same three-level
// caching (parsed kernel by string, bound kernel by string + extents,
// executor by the group's bound names; kernel/TensorEngine.cpp:557-623).
//
// Only the "Cuda" policy executes here.  "CPUInterpreted" is accepted as a
// name (the reference's default) but asking it to run a kernel throws: this
// library deliberately contains no CPU execution path.
#ifndef ACRO_B200_TENSOR_ENGINE_HPP
#define ACRO_B200_TENSOR_ENGINE_HPP

#include <memory>
#include <string>
#include <unordered_map>
#include <vector>
#include "DimensionedMultiKernel.hpp"
#include "Executor.hpp"
#include "IndexMapping.hpp"

namespace acro
{

class TensorEngine
{
    public:
    TensorEngine();                             // "Cuda"
    TensorEngine(const char *bare_exec_type);
    TensorEngine(std::string &exec_type);
    ~TensorEngine();
    TensorEngine(const TensorEngine &) = delete;
    TensorEngine &operator=(const TensorEngine &) = delete;

    void SetExecutorType(const char *bare_exec_type);
    void SetExecutorType(std::string &exec_type);
    std::string GetExecType() { return ExecutorType; }

    // TE(kernel, out, in1, ..., inN)
    template <class... In>
    void operator()(const char *bare_kernel_str, Tensor &out, Tensor &in1, In &...more)
    {
        std::string kernel_str(bare_kernel_str);
        std::vector<Tensor *> inputs = {&in1, static_cast<Tensor *>(&more)...};
        (*this)(kernel_str, &out, inputs);
    }
    template <class... In>
    void operator()(std::string &kernel_str, Tensor &out, Tensor &in1, In &...more)
    {
        std::vector<Tensor *> inputs = {&in1, static_cast<Tensor *>(&more)...};
        (*this)(kernel_str, &out, inputs);
    }
    void operator()(const char *bare_kernel_str, Tensor *out, std::vector<Tensor *> &inputs);
    void operator()(std::string &kernel_str, Tensor *out, std::vector<Tensor *> &inputs);

    // Text describing how the kernel would run (family, tile, grid, traffic model).
    template <class... In>
    std::string GetImplementation(const char *bare_kernel_str, Tensor &out, Tensor &in1, In &...more)
    {
        std::string kernel_str(bare_kernel_str);
        std::vector<Tensor *> inputs = {&in1, static_cast<Tensor *>(&more)...};
        return GetImplementation(kernel_str, &out, inputs);
    }
    template <class... In>
    std::string GetImplementation(std::string &kernel_str, Tensor &out, Tensor &in1, In &...more)
    {
        std::vector<Tensor *> inputs = {&in1, static_cast<Tensor *>(&more)...};
        return GetImplementation(kernel_str, &out, inputs);
    }
    std::string GetImplementation(const char *bare_kernel_str, Tensor *out, std::vector<Tensor *> &inputs);
    std::string GetImplementation(std::string &kernel_str, Tensor *out, std::vector<Tensor *> &inputs);

    // Non-contraction operations (kernel/TensorEngine.hpp:74-78 of the reference).
    // The trailing two dimensions of A are a square matrix of extent <= 3; everything before is batch.
    void BatchMatrixInverse(Tensor &Ainv, Tensor &A);
    void BatchMatrixDet(Tensor &Adet, Tensor &A);
    void BatchMatrixInvDet(Tensor &Ainv, Tensor &Adet, Tensor &A);
    // Aout[i] = Ain[M[i]]   /   Aout[M[i]] += Ain[i] (Aout zeroed first)
    void FlatIndexedScatter(Tensor &Aout, Tensor &Ain, IndexMapping &M);
    void FlatIndexedSumGather(Tensor &Aout, Tensor &Ain, IndexMapping &M);
    // Sharded form (no counterpart in the reference): M maps this rank's slab of the range; after the
    // local sum the domain entries shared with other ranks are summed over them through `halo`
    // (an acro_b200_halo, see acro_b200.h, or a SharedEntryExchange).  Collective over the ranks.
    void FlatIndexedSumGather(Tensor &Aout, Tensor &Ain, IndexMapping &M, void *halo);

    void Clear();
    bool IsGPUAvailable() { return isCudaReady(); }

    // Kernels issued between Begin and End are recorded and run as one unit at End.
    void BeginMultiKernelLaunch();
    void EndMultiKernelLaunch();
    // Text describing how the recorded group would run; ends the recording without running it.
    std::string EndMultiKernelLaunchDescribe();

    // cudaStream_t (as void*) used by this engine's launches; nullptr = library-wide stream.
    void SetCudaStream(void *cuda_stream) { TheCudaStream = cuda_stream; }

    // Multi-GPU, one process per GPU: attach the acro_b200_peer_group (as void*) of the ranks that
    // hold slabs of a contracted batch index.  A contraction such as "S_i_j = A_n_i_j B_n" then
    // returns, on every rank, the sum over all ranks' slabs (reduction and all-reduce in one kernel).
    void SetPeerGroup(void *peer_group) { ThePeerGroup = peer_group; }

    private:
    TensorKernel *GetAddTensorKernel(std::string &kernel_str);
    DimensionedKernel *GetAddDimensionedKernel(TensorKernel *kernel, Tensor *output, std::vector<Tensor *> &inputs);
    KernelExecutor *GetAddKernelExecutor();
    void RequireCuda(const char *what);
    void *Stream();
    void Record(std::string &kernel_str, Tensor *output, std::vector<Tensor *> &inputs);

    std::string ExecutorType;
    std::unordered_map<std::string, std::unique_ptr<TensorKernel>> KernelMap;
    std::unordered_map<std::string, std::unique_ptr<DimensionedKernel>> DimensionedKernelMap;
    std::unordered_map<std::string, std::unique_ptr<KernelExecutor>> ExecutorMap;

    bool IsMultiKernelLaunch;
    std::vector<DimensionedKernel *> MKLKernels;
    std::vector<Tensor *> MKLOutputT;
    std::vector<std::vector<Tensor *>> MKLInputT;
    void *TheCudaStream;
    void *ThePeerGroup;
};

}

#endif
