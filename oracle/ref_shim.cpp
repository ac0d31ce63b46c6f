// TEST INFRASTRUCTURE — not part of the product.
//
// C-callable shim over the UNMODIFIED reference library (LLNL/acrotensor),
// compiled CPU-only (no ACRO_HAVE_CUDA) from the reference's own sources by
// oracle/Makefile.  It drives the reference's public API exactly as a user
// would: acro::Tensor views over caller-owned host arrays, then
// acro::TensorEngine("CPUInterpreted") (kernel/TensorEngine.cpp:290-336 ->
// exec/CPUInterpretedExecutor.cpp:59-91).  Nothing here restates the
// algorithm; the arithmetic is the reference's.
//
// Only tests/, the smoke check and bench.py's CPU-baseline legs may load the
// library built from this file.
#include "AcroTensor.hpp"

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#define SHIM_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_err;

struct TensorTable {
    std::vector<std::unique_ptr<acro::Tensor>> t;
};

// Build non-owning reference Tensors over caller memory.  `row_begin` /
// `row_count` restrict tensors flagged as batched to a slab of their leading
// dimension (used by the threaded driver below).
void make_views(TensorTable &tab, int n_tensors, double *const *data, const int *ranks,
                const int *dims_flat, const int *batched, int64_t row_begin, int64_t row_count) {
    const int *d = dims_flat;
    for (int i = 0; i < n_tensors; ++i) {
        std::vector<int> dims(d, d + ranks[i]);
        d += ranks[i];
        double *base = data[i];
        if (batched && batched[i]) {
            int64_t row = 1;
            for (int k = 1; k < ranks[i]; ++k) row *= dims[k];
            base += row_begin * row;
            dims[0] = (int)row_count;
        }
        tab.t.emplace_back(new acro::Tensor(dims, base));
    }
}

void run_program(TensorTable &tab, int n_kernels, const char *const *kernels, const int *out_idx,
                 const int *n_in, const int *in_idx_flat, bool as_multi_launch) {
    acro::TensorEngine TE("CPUInterpreted");
    if (as_multi_launch) TE.BeginMultiKernelLaunch();
    const int *ii = in_idx_flat;
    for (int k = 0; k < n_kernels; ++k) {
        std::vector<acro::Tensor *> ins;
        for (int j = 0; j < n_in[k]; ++j) ins.push_back(tab.t[ii[j]].get());
        ii += n_in[k];
        std::string s(kernels[k]);
        TE(s, tab.t[out_idx[k]].get(), ins);
    }
    if (as_multi_launch) TE.EndMultiKernelLaunch();
}

}  // namespace

SHIM_API const char *acro_ref_last_error() { return g_err.c_str(); }

// Run a program of one or more contraction strings over a table of tensors.
//   data/ranks/dims_flat : the tensor table (dims concatenated)
//   kernels[k], out_idx[k], n_in[k], in_idx_flat : per contraction, indices into the table
//   as_multi_launch      : wrap in Begin/EndMultiKernelLaunch
// Returns 0, or -1 with acro_ref_last_error() set when the reference throws.
SHIM_API int acro_ref_run(int n_tensors, double *const *data, const int *ranks, const int *dims_flat,
                          int n_kernels, const char *const *kernels, const int *out_idx,
                          const int *n_in, const int *in_idx_flat, int as_multi_launch) {
    try {
        TensorTable tab;
        make_views(tab, n_tensors, data, ranks, dims_flat, nullptr, 0, 0);
        run_program(tab, n_kernels, kernels, out_idx, n_in, in_idx_flat, as_multi_launch != 0);
        return 0;
    } catch (const std::exception &e) {
        g_err = e.what();
        return -1;
    }
}

// Same program, but the leading ("batch") dimension of every tensor flagged in
// `batched` is cut into `n_threads` contiguous slabs and each slab is run by
// its own std::thread with its own reference TensorEngine (the reference
// itself is single-threaded; engines are independent objects).  Tensors that
// are written but not batched (the batch index is contracted away) get a
// private copy per thread and the copies are summed in thread order at the end.
// This is the "all host cores" CPU baseline; n_threads = 1 is the reference as shipped.
SHIM_API int acro_ref_run_slabs(int n_tensors, double *const *data, const int *ranks,
                                const int *dims_flat, const int *batched, int64_t batch,
                                int n_kernels, const char *const *kernels, const int *out_idx,
                                const int *n_in, const int *in_idx_flat, int as_multi_launch,
                                int n_threads) {
    if (n_threads < 1) n_threads = 1;
    if ((int64_t)n_threads > batch) n_threads = (int)batch;
    std::vector<int64_t> sizes(n_tensors, 1);
    {
        const int *d = dims_flat;
        for (int i = 0; i < n_tensors; ++i) {
            for (int k = 0; k < ranks[i]; ++k) sizes[i] *= d[k];
            d += ranks[i];
        }
    }
    std::vector<char> written(n_tensors, 0);
    for (int k = 0; k < n_kernels; ++k) written[out_idx[k]] = 1;

    std::vector<std::vector<std::vector<double>>> priv(n_threads);
    std::vector<std::string> errs(n_threads);
    std::vector<std::thread> pool;
    for (int t = 0; t < n_threads; ++t) {
        priv[t].resize(n_tensors);
        pool.emplace_back([&, t]() {
            try {
                int64_t b0 = batch * t / n_threads, b1 = batch * (t + 1) / n_threads;
                std::vector<double *> ptrs(data, data + n_tensors);
                for (int i = 0; i < n_tensors; ++i) {
                    if (written[i] && !batched[i] && n_threads > 1) {
                        priv[t][i].assign(sizes[i], 0.0);
                        ptrs[i] = priv[t][i].data();
                    }
                }
                TensorTable tab;
                make_views(tab, n_tensors, ptrs.data(), ranks, dims_flat, batched, b0, b1 - b0);
                run_program(tab, n_kernels, kernels, out_idx, n_in, in_idx_flat, as_multi_launch != 0);
            } catch (const std::exception &e) {
                errs[t] = e.what();
            }
        });
    }
    for (auto &th : pool) th.join();
    for (int t = 0; t < n_threads; ++t) {
        if (!errs[t].empty()) {
            g_err = errs[t];
            return -1;
        }
    }
    if (n_threads > 1) {
        for (int i = 0; i < n_tensors; ++i) {
            if (!(written[i] && !batched[i])) continue;
            std::fill(data[i], data[i] + sizes[i], 0.0);
            for (int t = 0; t < n_threads; ++t)
                for (int64_t j = 0; j < sizes[i]; ++j) data[i][j] += priv[t][i][j];
        }
    }
    return 0;
}

// Batched inverse / determinant through the reference's TensorEngine("CPUInterpreted")
// (kernel/TensorEngine.cpp:627-690 -> ops/NativeCPUOps.cpp:11-120).  Ainv or Adet may be null.
SHIM_API int acro_ref_batch_inv_det(double *A, double *Ainv, double *Adet, int rank, const int *dims)
{
    try
    {
        std::vector<int> d(dims, dims + rank), dd(dims, dims + (rank > 2 ? rank - 2 : 0));
        acro::TensorEngine TE("CPUInterpreted");
        acro::Tensor a(d, A);
        if (Ainv && Adet)
        {
            acro::Tensor inv(d, Ainv), det(dd, Adet);
            TE.BatchMatrixInvDet(inv, det, a);
        }
        else if (Ainv)
        {
            acro::Tensor inv(d, Ainv);
            TE.BatchMatrixInverse(inv, a);
        }
        else
        {
            acro::Tensor det(dd, Adet);
            TE.BatchMatrixDet(det, a);
        }
        return 0;
    }
    catch (const std::exception &e)
    {
        g_err = e.what();
        return -1;
    }
}

// FlatIndexedScatter (gather == 0) or FlatIndexedSumGather (gather != 0) through the
// reference's CPU engine (kernel/TensorEngine.cpp:693-716 -> ops/NativeCPUOps.cpp:123-144).
// When inv / inv_off are given they receive the reference's ComputeInverse() result.
SHIM_API int acro_ref_flat_indexed(double *Aout, double *Ain, const int *map, int domain, int range, int gather, int *inv, int *inv_off)
{
    try
    {
        acro::TensorEngine TE("CPUInterpreted");
        acro::IndexMapping M(domain, range);
        for (int i = 0; i < range; ++i) M[i] = map[i];
        acro::Tensor out(gather ? domain : range, Aout), in(gather ? range : domain, Ain);
        if (gather) TE.FlatIndexedSumGather(out, in, M);
        else TE.FlatIndexedScatter(out, in, M);
        if (inv && inv_off)
        {
            if (!M.IsInverseComputed()) M.ComputeInverse();
            for (int i = 0; i < range; ++i) inv[i] = M.GetInvMap()[i];
            for (int i = 0; i <= domain; ++i) inv_off[i] = M.GetInvMapOffsets()[i];
        }
        return 0;
    }
    catch (const std::exception &e)
    {
        g_err = e.what();
        return -1;
    }
}

SHIM_API int acro_ref_hardware_threads() {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}
