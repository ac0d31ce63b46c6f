// acro::TensorEngine: parse / bind / plan caches and single or recorded multi-kernel execution.
#include "TensorEngine.hpp"
#include "acro_b200.h"

namespace acro
{

TensorEngine::TensorEngine() : IsMultiKernelLaunch(false), TheCudaStream(nullptr), ThePeerGroup(nullptr)
{
    SetExecutorType("Cuda");
}

TensorEngine::TensorEngine(const char *bare_exec_type) : IsMultiKernelLaunch(false), TheCudaStream(nullptr), ThePeerGroup(nullptr)
{
    SetExecutorType(bare_exec_type);
}

TensorEngine::TensorEngine(std::string &exec_type) : IsMultiKernelLaunch(false), TheCudaStream(nullptr), ThePeerGroup(nullptr)
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
        executor->SetPeerGroup(ThePeerGroup);
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
    executor->SetPeerGroup(ThePeerGroup);
    executor->ExecuteMulti(MKLOutputT, MKLInputT);
}

std::string TensorEngine::EndMultiKernelLaunchDescribe()
{
    ACROBATIC_ASSERT(IsMultiKernelLaunch, "Found an EndMultiKernelLaunch before a BeginMultiKernelLaunch!");
    IsMultiKernelLaunch = false;
    if (MKLKernels.empty()) return "";
    return GetAddKernelExecutor()->GetImplementation();
}

void TensorEngine::RequireCuda(const char *what)
{
    ACROBATIC_ASSERT(ExecutorType == "Cuda", std::string(what) + ": the CPUInterpreted executor is not part of this library.");
    ACROBATIC_ASSERT(isCudaReady(), std::string(what) + ": No CUDA device is available; this library has no CPU execution path.");
}

void *TensorEngine::Stream() { return TheCudaStream ? TheCudaStream : getCudaStream(); }

namespace
{
void check_abi(int status, const char *what)
{
    if (status != ACRO_B200_OK) throw_error(std::string("acro_b200 ") + what + " failed: " + acro_b200_last_error());
}

// Shape checks shared by the batched matrix operations (kernel/TensorEngine.cpp:627-690).
void check_matrix_batch(Tensor &A, Tensor *Ainv, Tensor *Adet)
{
    const int rank = A.GetRank();
    ACROBATIC_ASSERT(A.IsInitialized(), "Batched matrix operation on an uninitialized tensor.");
    ACROBATIC_ASSERT(rank >= 2, "Can't treat a tensor of rank < 2 as a batch of matrices.");
    ACROBATIC_ASSERT(A.GetDim(rank - 1) == A.GetDim(rank - 2), "Batched matrix operations need square matrices in the last two dims.");
    ACROBATIC_ASSERT(A.GetDim(rank - 1) <= 3, "Batched matrix operations support matrix dims <= 3.");
    if (Ainv != nullptr)
    {
        ACROBATIC_ASSERT(Ainv->IsInitialized() && Ainv->GetRank() == rank, "Can't BatchMatrixInverse with mismatched ranks for Ainv and A.");
        for (int d = 0; d < rank; ++d) ACROBATIC_ASSERT(Ainv->GetDim(d) == A.GetDim(d), "Can't BatchMatrixInverse with mismatched dims for Ainv and A.");
    }
    if (Adet != nullptr)
    {
        ACROBATIC_ASSERT(rank >= 3, "Can't BatchMatrixDet a tensor of rank < 3.");
        ACROBATIC_ASSERT(Adet->IsInitialized() && Adet->GetRank() == rank - 2, "Can't BatchMatrixDet with mismatched ranks for Adet and A.");
        for (int d = 0; d < rank - 2; ++d) ACROBATIC_ASSERT(Adet->GetDim(d) == A.GetDim(d), "Can't BatchMatrixDet with mismatched dims for Adet and A.");
    }
}
}

void TensorEngine::BatchMatrixInverse(Tensor &Ainv, Tensor &A)
{
    check_matrix_batch(A, &Ainv, nullptr);
    RequireCuda("BatchMatrixInverse");
    A.MoveToGPU();
    if (&Ainv != &A) Ainv.SwitchToGPU();
    const int dim = A.GetDim(A.GetRank() - 1);
    check_abi(acro_b200_batch_inv_det(A.GetDeviceData(), Ainv.GetDeviceData(), nullptr, A.GetSize64() / (dim * dim), dim, Stream()),
              "batch_inv_det");
}

void TensorEngine::BatchMatrixDet(Tensor &Adet, Tensor &A)
{
    check_matrix_batch(A, nullptr, &Adet);
    RequireCuda("BatchMatrixDet");
    A.MoveToGPU();
    Adet.SwitchToGPU();
    const int dim = A.GetDim(A.GetRank() - 1);
    check_abi(acro_b200_batch_inv_det(A.GetDeviceData(), nullptr, Adet.GetDeviceData(), A.GetSize64() / (dim * dim), dim, Stream()),
              "batch_inv_det");
}

void TensorEngine::BatchMatrixInvDet(Tensor &Ainv, Tensor &Adet, Tensor &A)
{
    check_matrix_batch(A, &Ainv, &Adet);
    RequireCuda("BatchMatrixInvDet");
    A.MoveToGPU();
    if (&Ainv != &A) Ainv.SwitchToGPU();
    Adet.SwitchToGPU();
    const int dim = A.GetDim(A.GetRank() - 1);
    check_abi(acro_b200_batch_inv_det(A.GetDeviceData(), Ainv.GetDeviceData(), Adet.GetDeviceData(), A.GetSize64() / (dim * dim), dim, Stream()),
              "batch_inv_det");
}

void TensorEngine::FlatIndexedScatter(Tensor &Aout, Tensor &Ain, IndexMapping &M)
{
    ACROBATIC_ASSERT(Aout.IsInitialized() && Ain.IsInitialized(), "FlatIndexedScatter on an uninitialized tensor.");
    ACROBATIC_ASSERT(Aout.GetSize64() == M.GetRangeSize(), "IndexMapping RangeSize does not match the output Tensor size.");
    ACROBATIC_ASSERT(Ain.GetSize64() == M.GetDomainSize(), "IndexMapping DomainSize does not match the input Tensor size.");
    RequireCuda("FlatIndexedScatter");
    Aout.SwitchToGPU();
    Ain.MoveToGPU();
    M.MoveToGPU();
    check_abi(acro_b200_flat_scatter(Aout.GetDeviceData(), Ain.GetDeviceData(), M.GetMap().GetDeviceData(), M.GetRangeSize(), Stream()),
              "flat_scatter");
}

void TensorEngine::FlatIndexedSumGather(Tensor &Aout, Tensor &Ain, IndexMapping &M)
{
    ACROBATIC_ASSERT(Aout.IsInitialized() && Ain.IsInitialized(), "FlatIndexedSumGather on an uninitialized tensor.");
    ACROBATIC_ASSERT(Aout.GetSize64() == M.GetDomainSize(), "IndexMapping DomainSize does not match the output Tensor size.");
    ACROBATIC_ASSERT(Ain.GetSize64() == M.GetRangeSize(), "IndexMapping RangeSize does not match the input Tensor size.");
    RequireCuda("FlatIndexedSumGather");
    if (!M.IsInverseComputed()) M.ComputeInverse();
    Aout.SwitchToGPU();
    Ain.MoveToGPU();
    M.MoveToGPU();
    check_abi(acro_b200_flat_sum_gather(Aout.GetDeviceData(), Ain.GetDeviceData(), M.GetInvMap().GetDeviceData(),
                                        M.GetInvMapOffsets().GetDeviceData(), M.GetDomainSize(), Stream()),
              "flat_sum_gather");
}

void TensorEngine::FlatIndexedSumGather(Tensor &Aout, Tensor &Ain, IndexMapping &M, void *halo)
{
    ACROBATIC_ASSERT(halo != nullptr, "FlatIndexedSumGather over a sharded range needs a shared-entry exchange.");
    FlatIndexedSumGather(Aout, Ain, M);
    check_abi(acro_b200_halo_exchange_sum(static_cast<acro_b200_halo *>(halo), Aout.GetDeviceData(), Stream()), "halo_exchange_sum");
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
