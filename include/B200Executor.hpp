// acro::B200Executor — the "Cuda" execution policy of this library.
//
// It takes the place of exec/CudaExecutor.{hpp,cpp} of LLNL/acrotensor (a CUDA C
// string generator compiled at run time with NVRTC, exec/CudaExecutor.cpp:111-190)
// with a planner that maps the bound kernel group onto hand-written, ahead-of-time
// compiled sm_100a kernel families reached through the C ABI in acro_b200.h:
//   reduce_batch     out_f      = sum_n A_n_f [w_n]             (streaming reduction)
//   pointwise_sym    D_p_m_n    = s_p sum_l X_p_m_l Y_p_n_l      (per-point small product)
//   rank1_gemm       M_e_i_j    = sum_q W_e_q B_q_i B_q_j        (batched rank-1 updates)
//   batched_gemm     C_e_i_j    = sum_k A_e_i_k B_e_k_j          (batched small GEMM)
//   sumfact_mass     six-stage sum-factorised mass operator, fused, on-chip intermediates
//   generic          any other string: one thread per output entry, terms summed in the
//                    reference CPU executor's order (bit-identical results for "=")
// There is no CPU fallback: a shape no family covers runs on the generic GPU kernel.
// Multi-GPU (one process per GPU): with a peer group attached, a step that contracts the leading
// index of an input flagged Tensor::IsSharded() is completed by the sum over the ranks, inside the
// kernel for reduce_batch and by the all-reduce kernel acro_b200_peer_allreduce for every other family.
#ifndef ACRO_B200_EXECUTOR_HPP
#define ACRO_B200_EXECUTOR_HPP

#include <string>
#include <vector>
#include "KernelExecutor.hpp"

namespace acro
{

namespace plan { struct Program; }

class B200Executor : public KernelExecutor
{
    public:
    B200Executor(DimensionedMultiKernel *multi_kernel);
    ~B200Executor() override;

    std::string GetImplementation() override;
    std::string GetExecType() override { return "Cuda"; }
    void ExecuteSingle(Tensor *output, std::vector<Tensor *> &inputs) override;
    void ExecuteMulti(std::vector<Tensor *> &outputs, std::vector<std::vector<Tensor *>> &inputs) override;

    private:
    void Run(std::vector<Tensor *> &outputs, std::vector<std::vector<Tensor *>> &inputs);
    std::unique_ptr<plan::Program> Fused;      // plan that may elide transient intermediates
    std::unique_ptr<plan::Program> Unfused;    // plan that materialises every output
    double *Scratch;            // work space of the step that is running (shared by the families)
    std::size_t ScratchBytes;
    double *ReduceScratch;      // ticket counter and CTA partial sums of reduce_batch, kept zeroed between launches
    std::size_t ReduceScratchBytes;
    double *RankSum;            // this rank's partial result of a "+=" / "-=" contraction that is summed over ranks
    std::size_t RankSumBytes;
};

}

#endif
