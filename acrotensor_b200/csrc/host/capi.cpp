// Engine layer of the C ABI: handle-based access to acro::Tensor and
// acro::TensorEngine for hosts that cannot include the C++ headers, plus
// host-only introspection of the parser and planner.
#include "acro_b200.h"

#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "AcroTensor.hpp"
#include "Plan.hpp"

namespace acro_b200_detail
{
void set_last_error(const std::string &text);   // defined with the kernel layer
}

struct acro_tensor
{
    std::unique_ptr<acro::Tensor> t;
};

struct acro_index_mapping
{
    acro::IndexMapping m;
    acro_index_mapping(int domain, int range) : m(domain, range) {}
};

struct acro_engine
{
    acro::TensorEngine te;
    explicit acro_engine(const char *type) : te(type) {}
};

namespace
{

template <class F>
int guarded(F &&body)
{
    try
    {
        body();
        return ACRO_B200_OK;
    }
    catch (const std::exception &e)
    {
        acro_b200_detail::set_last_error(e.what());
        std::string what = e.what();
        return what.find("CUDA error") != std::string::npos || what.find("No CUDA device") != std::string::npos
                   ? ACRO_B200_ECUDA
                   : ACRO_B200_EINVAL;
    }
}

int copy_out(const std::string &text, char *buf, size_t buf_len)
{
    if (buf == nullptr || buf_len == 0) return ACRO_B200_OK;
    size_t n = text.size() < buf_len - 1 ? text.size() : buf_len - 1;
    std::memcpy(buf, text.data(), n);
    buf[n] = '\0';
    return ACRO_B200_OK;
}

std::vector<acro::Tensor *> unwrap(int n, acro_tensor *const *handles)
{
    std::vector<acro::Tensor *> v;
    for (int i = 0; i < n; ++i)
    {
        if (handles == nullptr || handles[i] == nullptr) acro::throw_error("null tensor handle");
        v.push_back(handles[i]->t.get());
    }
    return v;
}

std::string join(const std::vector<std::string> &names)
{
    std::string s;
    for (std::size_t i = 0; i < names.size(); ++i) s += (i ? " " : "") + names[i];
    return s;
}

}

extern "C" {

int acro_tensor_create(int rank, const int *dims, double *hdata, double *ddata, int ongpu, acro_tensor **out)
{
    return guarded([&] {
        if (out == nullptr || dims == nullptr || rank < 0) acro::throw_error("acro_tensor_create: bad arguments");
        std::vector<int> d(dims, dims + rank);
        std::unique_ptr<acro_tensor> h(new acro_tensor);
        h->t.reset(new acro::Tensor(d, hdata, ddata, ongpu != 0));
        *out = h.release();
    });
}

int acro_tensor_slice(acro_tensor *parent, int n_indices, const int *indices, acro_tensor **out)
{
    return guarded([&] {
        if (parent == nullptr || out == nullptr || indices == nullptr) acro::throw_error("acro_tensor_slice: bad arguments");
        std::vector<int> idx(indices, indices + n_indices);
        std::unique_ptr<acro_tensor> h(new acro_tensor);
        h->t.reset(new acro::SliceTensor(*parent->t, idx));
        *out = h.release();
    });
}

int acro_tensor_destroy(acro_tensor *t)
{
    delete t;
    return ACRO_B200_OK;
}

int acro_tensor_rank(const acro_tensor *t) { return t ? t->t->GetRank() : ACRO_B200_EINVAL; }
int64_t acro_tensor_size(const acro_tensor *t) { return t ? t->t->GetSize64() : ACRO_B200_EINVAL; }
int acro_tensor_dim(const acro_tensor *t, int d) { return (t && d >= 0 && d < t->t->GetRank()) ? t->t->GetDim(d) : ACRO_B200_EINVAL; }
double *acro_tensor_data(const acro_tensor *t) { return t ? t->t->GetData() : nullptr; }
double *acro_tensor_device_data(const acro_tensor *t) { return t ? t->t->GetDeviceData() : nullptr; }
int acro_tensor_is_on_gpu(const acro_tensor *t) { return t ? (t->t->IsOnGPU() ? 1 : 0) : ACRO_B200_EINVAL; }
int acro_tensor_is_mapped_to_gpu(const acro_tensor *t) { return t ? (t->t->IsMappedToGPU() ? 1 : 0) : ACRO_B200_EINVAL; }

#define ACRO_TENSOR_CALL(name, expr)                                                   \
    int name(acro_tensor *t)                                                           \
    {                                                                                  \
        return guarded([&] {                                                           \
            if (t == nullptr) acro::throw_error(#name ": null tensor handle");        \
            t->t->expr;                                                                \
        });                                                                            \
    }
ACRO_TENSOR_CALL(acro_tensor_map_to_gpu, MapToGPU())
ACRO_TENSOR_CALL(acro_tensor_move_to_gpu, MoveToGPU())
ACRO_TENSOR_CALL(acro_tensor_switch_to_gpu, SwitchToGPU())
ACRO_TENSOR_CALL(acro_tensor_unmap_from_gpu, UnmapFromGPU())
ACRO_TENSOR_CALL(acro_tensor_move_from_gpu, MoveFromGPU())
ACRO_TENSOR_CALL(acro_tensor_switch_from_gpu, SwitchFromGPU())
#undef ACRO_TENSOR_CALL

int acro_tensor_set(acro_tensor *t, double val)
{
    return guarded([&] {
        if (t == nullptr) acro::throw_error("acro_tensor_set: null tensor handle");
        t->t->Set(val);
    });
}

int acro_tensor_mult(acro_tensor *t, double c)
{
    return guarded([&] {
        if (t == nullptr) acro::throw_error("acro_tensor_mult: null tensor handle");
        t->t->Mult(c);
    });
}

int acro_tensor_reshape(acro_tensor *t, int rank, const int *dims)
{
    return guarded([&] {
        if (t == nullptr || dims == nullptr) acro::throw_error("acro_tensor_reshape: bad arguments");
        std::vector<int> d(dims, dims + rank);
        t->t->Reshape(d);
    });
}

int acro_tensor_retarget(acro_tensor *t, double *hdata, double *ddata)
{
    return guarded([&] {
        if (t == nullptr) acro::throw_error("acro_tensor_retarget: null tensor handle");
        t->t->Retarget(hdata, ddata);
    });
}

int acro_tensor_set_transient(acro_tensor *t, int transient)
{
    return guarded([&] {
        if (t == nullptr) acro::throw_error("acro_tensor_set_transient: null tensor handle");
        t->t->SetTransient(transient != 0);
    });
}

int acro_b200_batch_slab(int64_t batch, int rank, int world, int64_t *begin, int64_t *end)
{
    if (begin == nullptr || end == nullptr || batch < 0 || world < 1 || rank < 0 || rank >= world)
    {
        acro_b200_detail::set_last_error("acro_b200_batch_slab: need batch >= 0, 0 <= rank < world and result pointers");
        return ACRO_B200_EINVAL;
    }
    // 128-bit products: batch * world may pass 2^63
    *begin = static_cast<int64_t>(static_cast<__int128>(batch) * rank / world);
    *end = static_cast<int64_t>(static_cast<__int128>(batch) * (rank + 1) / world);
    return ACRO_B200_OK;
}

int acro_tensor_slab(acro_tensor *parent, int64_t begin, int64_t end, acro_tensor **out)
{
    return guarded([&] {
        if (parent == nullptr || out == nullptr) acro::throw_error("acro_tensor_slab: bad arguments");
        std::unique_ptr<acro_tensor> h(new acro_tensor);
        h->t.reset(new acro::SlabTensor(*parent->t, begin, end));
        *out = h.release();
    });
}

int acro_tensor_set_sharded(acro_tensor *t, int sharded)
{
    return guarded([&] {
        if (t == nullptr) acro::throw_error("acro_tensor_set_sharded: null tensor handle");
        t->t->SetSharded(sharded != 0);
    });
}

int acro_tensor_is_sharded(const acro_tensor *t) { return t ? (t->t->IsSharded() ? 1 : 0) : ACRO_B200_EINVAL; }

int acro_engine_create(const char *exec_type, acro_engine **out)
{
    return guarded([&] {
        if (out == nullptr) acro::throw_error("acro_engine_create: null result pointer");
        *out = new acro_engine(exec_type ? exec_type : "Cuda");
    });
}

int acro_engine_destroy(acro_engine *e)
{
    delete e;
    return ACRO_B200_OK;
}

int acro_engine_set_executor_type(acro_engine *e, const char *exec_type)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        e->te.SetExecutorType(exec_type);
    });
}

int acro_engine_exec_type(acro_engine *e, char *buf, size_t buf_len)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        copy_out(e->te.GetExecType(), buf, buf_len);
    });
}

int acro_engine_contract(acro_engine *e, const char *kernel, acro_tensor *out, int n_inputs, acro_tensor *const *inputs)
{
    return guarded([&] {
        if (e == nullptr || kernel == nullptr || out == nullptr) acro::throw_error("acro_engine_contract: bad arguments");
        std::vector<acro::Tensor *> ins = unwrap(n_inputs, inputs);
        std::string k(kernel);
        e->te(k, out->t.get(), ins);
    });
}

int acro_engine_implementation(acro_engine *e, const char *kernel, acro_tensor *out, int n_inputs,
                               acro_tensor *const *inputs, char *buf, size_t buf_len)
{
    return guarded([&] {
        if (e == nullptr || kernel == nullptr || out == nullptr) acro::throw_error("acro_engine_implementation: bad arguments");
        std::vector<acro::Tensor *> ins = unwrap(n_inputs, inputs);
        std::string k(kernel);
        copy_out(e->te.GetImplementation(k, out->t.get(), ins), buf, buf_len);
    });
}

int acro_engine_begin_multi(acro_engine *e)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        e->te.BeginMultiKernelLaunch();
    });
}

int acro_engine_end_multi(acro_engine *e)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        e->te.EndMultiKernelLaunch();
    });
}

int acro_engine_end_multi_describe(acro_engine *e, char *buf, size_t buf_len)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        copy_out(e->te.EndMultiKernelLaunchDescribe(), buf, buf_len);
    });
}

int acro_engine_clear(acro_engine *e)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        e->te.Clear();
    });
}

int acro_engine_set_peer_group(acro_engine *e, acro_b200_peer_group *group)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        e->te.SetPeerGroup(group);
    });
}

int acro_engine_set_stream(acro_engine *e, void *stream)
{
    return guarded([&] {
        if (e == nullptr) acro::throw_error("null engine handle");
        e->te.SetCudaStream(stream);
    });
}

int acro_index_mapping_create(int domain_size, int range_size, acro_index_mapping **out)
{
    return guarded([&] {
        if (out == nullptr || domain_size < 1 || range_size < 1) acro::throw_error("acro_index_mapping_create: bad arguments");
        *out = new acro_index_mapping(domain_size, range_size);
    });
}

int acro_index_mapping_destroy(acro_index_mapping *m)
{
    delete m;
    return ACRO_B200_OK;
}

int *acro_index_mapping_data(acro_index_mapping *m) { return m ? m->m.GetMap().GetData() : nullptr; }

int acro_index_mapping_compute_inverse(acro_index_mapping *m)
{
    return guarded([&] {
        if (m == nullptr) acro::throw_error("null index mapping handle");
        m->m.ComputeInverse();
    });
}

const int *acro_index_mapping_inverse(acro_index_mapping *m)
{
    return (m && m->m.IsInverseComputed()) ? m->m.GetInvMap().GetData() : nullptr;
}

const int *acro_index_mapping_inverse_offsets(acro_index_mapping *m)
{
    return (m && m->m.IsInverseComputed()) ? m->m.GetInvMapOffsets().GetData() : nullptr;
}

int acro_engine_batch_matrix_inverse(acro_engine *e, acro_tensor *Ainv, acro_tensor *A)
{
    return guarded([&] {
        if (e == nullptr || Ainv == nullptr || A == nullptr) acro::throw_error("acro_engine_batch_matrix_inverse: null handle");
        e->te.BatchMatrixInverse(*Ainv->t, *A->t);
    });
}

int acro_engine_batch_matrix_det(acro_engine *e, acro_tensor *Adet, acro_tensor *A)
{
    return guarded([&] {
        if (e == nullptr || Adet == nullptr || A == nullptr) acro::throw_error("acro_engine_batch_matrix_det: null handle");
        e->te.BatchMatrixDet(*Adet->t, *A->t);
    });
}

int acro_engine_batch_matrix_inv_det(acro_engine *e, acro_tensor *Ainv, acro_tensor *Adet, acro_tensor *A)
{
    return guarded([&] {
        if (e == nullptr || Ainv == nullptr || Adet == nullptr || A == nullptr) acro::throw_error("acro_engine_batch_matrix_inv_det: null handle");
        e->te.BatchMatrixInvDet(*Ainv->t, *Adet->t, *A->t);
    });
}

int acro_engine_flat_indexed_scatter(acro_engine *e, acro_tensor *Aout, acro_tensor *Ain, acro_index_mapping *m)
{
    return guarded([&] {
        if (e == nullptr || Aout == nullptr || Ain == nullptr || m == nullptr) acro::throw_error("acro_engine_flat_indexed_scatter: null handle");
        e->te.FlatIndexedScatter(*Aout->t, *Ain->t, m->m);
    });
}

int acro_engine_flat_indexed_sum_gather(acro_engine *e, acro_tensor *Aout, acro_tensor *Ain, acro_index_mapping *m)
{
    return guarded([&] {
        if (e == nullptr || Aout == nullptr || Ain == nullptr || m == nullptr) acro::throw_error("acro_engine_flat_indexed_sum_gather: null handle");
        e->te.FlatIndexedSumGather(*Aout->t, *Ain->t, m->m);
    });
}

int acro_engine_flat_indexed_sum_gather_shared(acro_engine *e, acro_tensor *Aout, acro_tensor *Ain, acro_index_mapping *m,
                                               acro_b200_halo *halo)
{
    return guarded([&] {
        if (e == nullptr || Aout == nullptr || Ain == nullptr || m == nullptr || halo == nullptr)
            acro::throw_error("acro_engine_flat_indexed_sum_gather_shared: null handle");
        e->te.FlatIndexedSumGather(*Aout->t, *Ain->t, m->m, halo);
    });
}

int acro_b200_set_stream(void *stream)
{
    acro::setCudaStream(stream);
    return ACRO_B200_OK;
}

int acro_b200_describe_kernel(const char *kernel, char *buf, size_t buf_len)
{
    return guarded([&] {
        if (kernel == nullptr) acro::throw_error("acro_b200_describe_kernel: null kernel string");
        acro::TensorKernel k(kernel);
        std::ostringstream os;
        os << "name: " << k.GetNameString() << "\n";
        os << "op: " << k.EqOperator << "\n";
        os << "output: " << k.OutputVar.Name << " [" << join(k.OutputVar.IndexNames) << "]\n";
        for (acro::KernelVar &v : k.InputVars) os << "input: " << v.Name << " [" << join(v.IndexNames) << "]\n";
        os << "all: " << join(k.AllIndexNames) << "\n";
        os << "contraction: " << join(k.ContractionIndexNames) << "\n";
        for (int vari = -1; vari < k.GetNumInputVars(); ++vari)
        {
            os << "loopnums " << k.GetVarName(vari) << ":";
            for (int d = 0; d < k.GetVarRank(vari); ++d) os << " " << k.GetVarDimLoopNum(vari, d);
            os << "\n";
        }
        copy_out(os.str(), buf, buf_len);
    });
}

int acro_b200_describe_plan(int n_kernels, const char *const *kernels, const int *dims_flat, int transient_intermediates,
                            char *buf, size_t buf_len)
{
    return guarded([&] {
        if (n_kernels < 1 || kernels == nullptr || dims_flat == nullptr) acro::throw_error("acro_b200_describe_plan: bad arguments");
        // Shape-only tensors: they point at one dummy double that is never dereferenced,
        // because nothing is executed here.
        static double dummy = 0.0;
        std::vector<std::unique_ptr<acro::TensorKernel>> parsed;
        std::vector<std::unique_ptr<acro::Tensor>> tensors;
        std::vector<std::unique_ptr<acro::DimensionedKernel>> bound;
        const int *d = dims_flat;
        for (int ki = 0; ki < n_kernels; ++ki)
        {
            parsed.emplace_back(new acro::TensorKernel(kernels[ki]));
            acro::TensorKernel &k = *parsed.back();
            std::vector<acro::Tensor *> vars;
            for (int vari = -1; vari < k.GetNumInputVars(); ++vari)
            {
                std::vector<int> dims(d, d + k.GetVarRank(vari));
                d += k.GetVarRank(vari);
                tensors.emplace_back(new acro::Tensor(dims, &dummy));
                vars.push_back(tensors.back().get());
            }
            std::vector<acro::Tensor *> ins(vars.begin() + 1, vars.end());
            bound.emplace_back(new acro::DimensionedKernel(&k, vars[0], ins));
        }
        std::vector<acro::DimensionedKernel *> group;
        for (auto &b : bound) group.push_back(b.get());
        acro::DimensionedMultiKernel mk(group);
        acro::plan::Program p = acro::plan::BuildProgram(mk, transient_intermediates != 0);
        std::ostringstream os;
        os << p.Describe(mk);
        os << "shared outer:";
        for (std::string &idx : mk.SharedOuterIndexNames) os << " " << idx;
        os << "\nuvars:";
        for (int u = 0; u < mk.GetNumUVars(); ++u)
        {
            std::pair<int, int> kv = mk.GetFirstKiVariForUVari(u);
            os << " " << mk.Kernels[kv.first]->GetVarName(kv.second) << (mk.IsOutputUVar(u) ? "(out)" : "") << (mk.IsInputUVar(u) ? "(in)" : "");
        }
        os << "\n";
        copy_out(os.str(), buf, buf_len);
    });
}

}  // extern "C"
