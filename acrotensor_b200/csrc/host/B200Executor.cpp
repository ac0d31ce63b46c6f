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
    : KernelExecutor(multi_kernel), Scratch(nullptr), ScratchBytes(0)
{
    Unfused.reset(new plan::Program(plan::BuildProgram(*MultiKernel, false)));
    Fused.reset(new plan::Program(plan::BuildProgram(*MultiKernel, true)));
}

B200Executor::~B200Executor()
{
    if (Scratch != nullptr) cudaFree(Scratch);
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
    if (program->scratch_bytes > ScratchBytes)
    {
        if (Scratch != nullptr) acroCudaErrorCheck(cudaFree(Scratch));
        Scratch = nullptr;
        void *p = nullptr;
        acroCudaErrorCheck(cudaMalloc(&p, program->scratch_bytes));
        Scratch = static_cast<double *>(p);
        ScratchBytes = program->scratch_bytes;
    }

    for (const plan::Step &s : program->steps)
    {
        Tensor *out = resolve(s.out, outputs, inputs);
        std::vector<Tensor *> ins;
        for (const plan::TensorRef &r : s.ins) ins.push_back(resolve(r, outputs, inputs));

        // Bring operands to the device (allocating / copying only where the host side is
        // fresh).  A "=" output is overwritten, so its old contents are not uploaded,
        // unless it is a slice: its parent holds other entries that must survive.
        if (s.op == ACRO_B200_OP_ASSIGN && !out->IsOnGPU() && dynamic_cast<SliceTensor *>(out) == nullptr) out->SwitchToGPU();
        MoveTensorsToGPU(out, ins);

        switch (s.family)
        {
            case plan::Family::Generic:
            {
                if (s.zero_fill_first) check_abi(acro_b200_fill(out->GetDeviceData(), out->GetSize64(), 0.0, stream), "fill");
                const double *ptrs[ACRO_B200_MAX_INPUTS];
                for (std::size_t i = 0; i < ins.size(); ++i) ptrs[i] = ins[i]->GetDeviceData();
                check_abi(acro_b200_generic_launch(&s.generic, out->GetDeviceData(), ptrs, Scratch, ScratchBytes, stream), "generic_launch");
                break;
            }
            case plan::Family::ReduceBatch:
            {
                const double *w = ins.size() > 1 ? ins[1]->GetDeviceData() : nullptr;
                if (ThePeerGroup != nullptr)
                {
                    // the batch index is sharded over the ranks of the group: fused all-reduce
                    check_abi(acro_b200_reduce_batch_allreduce(ins[0]->GetDeviceData(), w, out->GetDeviceData(), s.rows, s.sizes[0], s.op,
                                                               Scratch, ScratchBytes, static_cast<acro_b200_peer_group *>(ThePeerGroup), stream),
                              "reduce_batch_allreduce");
                }
                else
                {
                    check_abi(acro_b200_reduce_batch(ins[0]->GetDeviceData(), w, out->GetDeviceData(), s.rows, s.sizes[0], s.op,
                                                     Scratch, ScratchBytes, stream),
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
                                                  out->GetDeviceData(), stream),
                          "pointwise_sym");
                break;
            }
            case plan::Family::Rank1Gemm:
            {
                check_abi(acro_b200_rank1_gemm(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), ins[2]->GetDeviceData(),
                                               out->GetDeviceData(), s.rows, s.sizes[0], s.sizes[1], s.sizes[2], s.op, stream),
                          "rank1_gemm");
                break;
            }
            case plan::Family::BatchedGemm:
            {
                check_abi(acro_b200_batched_gemm_t(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), out->GetDeviceData(), s.rows,
                                                   s.sizes[0], s.sizes[1], s.sizes[2], s.sizes[3], s.sizes[4], s.op, stream),
                          "batched_gemm");
                break;
            }
            case plan::Family::SumfactMass:
            {
                check_abi(acro_b200_sumfact_mass(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), ins[2]->GetDeviceData(),
                                                 out->GetDeviceData(), s.rows, s.sizes[0], s.sizes[1], stream),
                          "sumfact_mass");
                break;
            }
            case plan::Family::Gram:
            {
                check_abi(acro_b200_gram(ins[0]->GetDeviceData(), ins[1]->GetDeviceData(), out->GetDeviceData(), s.rows, s.sizes[0], s.sizes[1],
                                         s.op, Scratch, ScratchBytes, stream),
                          "gram");
                break;
            }
            case plan::Family::InvariantGemm:
            {
                const double *ptrs[ACRO_B200_MAX_INPUTS];
                for (std::size_t i = 1; i < ins.size(); ++i) ptrs[i - 1] = ins[i]->GetDeviceData();
                check_abi(acro_b200_generic_launch(&s.generic, Scratch, ptrs, nullptr, 0, stream), "generic_launch (invariant product)");
                check_abi(acro_b200_gemm(ins[0]->GetDeviceData(), Scratch, out->GetDeviceData(), s.rows, s.sizes[1], s.sizes[0], s.sizes[0],
                                         s.sizes[2], s.sizes[1], s.op, stream),
                          "gemm");
                break;
            }
            case plan::Family::Permute:
            {
                check_abi(acro_b200_permute(&s.generic, out->GetDeviceData(), ins[0]->GetDeviceData(), stream), "permute");
                break;
            }
            default:
                ACROBATIC_ASSERT(false, "Planned a kernel family that is not built into this library.");
        }
    }
}

}
