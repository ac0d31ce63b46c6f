// The "Cuda" execution policy: plan once, then launch ahead-of-time compiled
// sm_100a kernels through the C ABI.  No code in this file computes on the host.
#include "B200Executor.hpp"
#include "Plan.hpp"
#include "SliceTensor.hpp"
#include "acro_b200.h"

#include <cuda_runtime_api.h>

namespace acro
{

namespace
{
void check_abi(int status, const std::string &what)
{
    if (status != ACRO_B200_OK)
    {
        throw_error("acro_b200 " + what + " failed (" + std::to_string(status) + "): " + acro_b200_last_error());
    }
}

Tensor *resolve(const plan::TensorRef &r, std::vector<Tensor *> &outputs, std::vector<std::vector<Tensor *>> &inputs)
{
    return r.vari < 0 ? outputs[r.ki] : inputs[r.ki][r.vari];
}
}

B200Executor::B200Executor(DimensionedMultiKernel *multi_kernel)
    : KernelExecutor(multi_kernel), Scratch(nullptr), ScratchBytes(0), ReduceScratch(nullptr), ReduceScratchBytes(0), RankSum(nullptr),
      RankSumBytes(0)
{
    Unfused.reset(new plan::Program(plan::BuildProgram(*MultiKernel, false)));
    Fused.reset(new plan::Program(plan::BuildProgram(*MultiKernel, true)));
}

B200Executor::~B200Executor()
{
    if (Scratch != nullptr) cudaFree(Scratch);
    if (ReduceScratch != nullptr) cudaFree(ReduceScratch);
    if (RankSum != nullptr) cudaFree(RankSum);
}

namespace
{
// Grows a device buffer owned by the executor (contents are not kept).
void reserve(double *&buffer, std::size_t &have, std::size_t need)
{
    if (need <= have) return;
    if (buffer != nullptr) acroCudaErrorCheck(cudaFree(buffer));
    buffer = nullptr;
    have = 0;
    void *p = nullptr;
    acroCudaErrorCheck(cudaMalloc(&p, need));
    buffer = static_cast<double *>(p);
    have = need;
}
}

std::string B200Executor::GetImplementation()
{
    std::string text = Unfused->Describe(*MultiKernel);
    if (Fused->elides)
    {
        text += "--- when every intermediate is transient ---\n" + Fused->Describe(*MultiKernel);
    }
    return text;
}

void B200Executor::ExecuteSingle(Tensor *output, std::vector<Tensor *> &inputs)
{
    std::vector<Tensor *> outs = {output};
    std::vector<std::vector<Tensor *>> ins = {inputs};
    Run(outs, ins);
}

void B200Executor::ExecuteMulti(std::vector<Tensor *> &outputs, std::vector<std::vector<Tensor *>> &inputs)
{
    Run(outputs, inputs);
}

void B200Executor::Run(std::vector<Tensor *> &outputs, std::vector<std::vector<Tensor *>> &inputs)
{
    ACROBATIC_ASSERT(static_cast<int>(outputs.size()) == MultiKernel->GetNumKernels() && outputs.size() == inputs.size(),
                     "Tensor lists do not match the kernel group.");
    ACROBATIC_ASSERT(isCudaReady(), "No CUDA device is available; this library has no CPU execution path.");

    // The fused plan may skip transient intermediates; it is used only when every
    // output it would elide is flagged transient by the caller.
    const plan::Program *program = Unfused.get();
    if (Fused->elides)
    {
        bool all_transient = true;
        for (const plan::Step &s : Fused->steps)
        {
            for (const plan::TensorRef &r : s.elided) all_transient = all_transient && resolve(r, outputs, inputs)->IsTransient();
        }
        if (all_transient) program = Fused.get();
    }

    void *stream = Stream();
    reserve(Scratch, ScratchBytes, program->scratch_bytes);
    acro_b200_peer_group *group = static_cast<acro_b200_peer_group *>(ThePeerGroup);

    for (const plan::Step &planned : program->steps)
    {
        Tensor *out = resolve(planned.out, outputs, inputs);
        std::vector<Tensor *> ins;
        for (const plan::TensorRef &r : planned.ins) ins.push_back(resolve(r, outputs, inputs));

        // Bring operands to the device (allocating / copying only where the host side is
        // fresh).  A "=" output is overwritten, so its old contents are not uploaded,
        // unless it is a slice: its parent holds other entries that must survive.
        if (planned.op == ACRO_B200_OP_ASSIGN && !out->IsOnGPU() && dynamic_cast<SliceTensor *>(out) == nullptr) out->SwitchToGPU();
        MoveTensorsToGPU(out, ins);

        // Multi-GPU: when an input whose leading index is contracted is this rank's slab of a sharded
        // tensor, the kernel leaves a partial sum on every rank and the result is their sum.  reduce_batch
        // exchanges inside its own kernel; every other family is followed by the all-reduce kernel.  With
        // "+=" / "-=" the partial sum goes to a buffer of its own first, so that the old contents of the
        // output are counted once and not once per rank.
        bool sum_over_ranks = false;
        if (group != nullptr)
        {
            for (const plan::TensorRef &r : planned.lead_contracted) sum_over_ranks = sum_over_ranks || resolve(r, outputs, inputs)->IsSharded();
        }
        const bool fused_rank_sum = sum_over_ranks && planned.family == plan::Family::ReduceBatch;
        const bool separate_rank_sum = sum_over_ranks && !fused_rank_sum;
        const bool to_buffer = separate_rank_sum && planned.op != ACRO_B200_OP_ASSIGN;
        plan::Step redirected;
        double *out_data = out->GetDeviceData();
        if (to_buffer)
        {
            redirected = planned;
            redirected.op = redirected.generic.op = redirected.pointwise.op = ACRO_B200_OP_ASSIGN;
            redirected.zero_fill_first = (planned.family == plan::Family::Generic);
            reserve(RankSum, RankSumBytes, out->GetByteSize());
            out_data = RankSum;
        }
        const plan::Step &s = to_buffer ? redirected : planned;
        const std::int64_t out_size = out->GetSize64();

        switch (s.family)
        {
            case plan::Family::Generic:
            {
                if (s.zero_fill_first) check_abi(acro_b200_fill(out_data, out_size, 0.0, stream), "fill");
                const double *ptrs[ACRO_B200_MAX_INPUTS];
                for (std::size_t i = 0; i < ins.size(); ++i) ptrs[i] = ins[i]->GetDeviceData();
                check_abi(acro_b200_generic_launch(&s.generic, out_data, ptrs, Scratch, ScratchBytes, stream), "generic_launch");
                break;
            }
            case plan::Family::ReduceBatch:
            {
                const double *w = ins.size() > 1 ? ins[1]->GetDeviceData() : nullptr;
                // A buffer of its own for the ticket counter and the CTA partial sums: zeroed once here, left
                // zeroed by every launch, touched by nothing else, so no clear precedes the launches.
                const std::size_t need = acro_b200_reduce_batch_scratch_bytes(s.sizes[0]);
                if (need > ReduceScratchBytes)
                {
                    reserve(ReduceScratch, ReduceScratchBytes, need);
                    acroCudaErrorCheck(cudaMemsetAsync(ReduceScratch, 0, 256, static_cast<cudaStream_t>(stream)));
                }
                if (fused_rank_sum)
                {
                    check_abi(acro_b200_reduce_batch_allreduce(ins[0]->GetDeviceData(), w, out_data, s.rows, s.sizes[0], s.op | ACRO_B200_SCRATCH_READY,
                                                               ReduceScratch, ReduceScratchBytes, group, stream),
                              "reduce_batch_allreduce");
                }
                else
                {
                    check_abi(acro_b200_reduce_batch(ins[0]->GetDeviceData(), w, out_data, s.rows, s.sizes[0], s.op | ACRO_B200_SCRATCH_READY,
                                                     ReduceScratch, ReduceScratchBytes, stream),
                              "reduce_batch");
                }
                break;
            }
            case plan::Family::PointwiseSym:
            {
                const int ns = s.pointwise.n_scalars;
                const double *scalars[ACRO_B200_MAX_SCALARS] = {nullptr};
                for (int i = 0; i < ns; ++i) scalars[i] = ins[i]->GetDeviceData();
                check_abi(acro_b200_pointwise_sym(&s.pointwise, scalars, ins[ns]->GetDeviceData(), ins[ns + 1]->GetDeviceData(),
                                                  out_data, stream),
                          "pointwise_sym");
                break;
            }
            case plan::Family::Rank1Gemm:
            {
                check_abi(acro_b200_rank1_gemm(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), ins[2]->GetDeviceData(),
                                               out_data, s.rows, s.sizes[0], s.sizes[1], s.sizes[2], s.op, stream),
                          "rank1_gemm");
                break;
            }
            case plan::Family::BatchedGemm:
            {
                check_abi(acro_b200_batched_gemm_t(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), out_data, s.rows,
                                                   s.sizes[0], s.sizes[1], s.sizes[2], s.sizes[3], s.sizes[4], s.op, stream),
                          "batched_gemm");
                break;
            }
            case plan::Family::SumfactMass:
            {
                check_abi(acro_b200_sumfact_mass(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), ins[2]->GetDeviceData(),
                                                 out_data, s.rows, s.sizes[0], s.sizes[1], stream),
                          "sumfact_mass");
                break;
            }
            case plan::Family::Gram:
            {
                check_abi(acro_b200_gram(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), out_data, s.rows, s.sizes[0], s.sizes[1],
                                         s.op, Scratch, ScratchBytes, stream),
                          "gram");
                break;
            }
            case plan::Family::InvariantGemm:
            {
                const double *ptrs[ACRO_B200_MAX_INPUTS];
                for (std::size_t i = 1; i < ins.size(); ++i) ptrs[i - 1] = ins[i]->GetDeviceData();
                check_abi(acro_b200_generic_launch(&s.generic, Scratch, ptrs, nullptr, 0, stream), "generic_launch (invariant product)");
                check_abi(acro_b200_gemm(ins[0]->GetDeviceData(), Scratch, out_data, s.rows, s.sizes[1], s.sizes[0], s.sizes[0],
                                         s.sizes[2], s.sizes[1], s.op, stream),
                          "gemm");
                break;
            }
            case plan::Family::Permute:
            {
                check_abi(acro_b200_permute(&s.generic, out_data, ins[0]->GetDeviceData(), stream), "permute");
                break;
            }
            default:
                ACROBATIC_ASSERT(false, "Planned a kernel family that is not built into this library.");
        }
        if (separate_rank_sum)
        {
            check_abi(acro_b200_peer_allreduce(out->GetDeviceData(), out_data, out_size, planned.op, group, stream), "peer_allreduce");
        }
    }
}

}
