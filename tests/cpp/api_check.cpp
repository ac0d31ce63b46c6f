// Exercises the C++ API exactly as user code written against LLNL/acrotensor would:
// AcroTensor.hpp, acro::Tensor / SliceTensor / TensorEngine / TensorKernel / DimensionedKernel.
// Host-only checks always run; device checks run when a GPU is present (pass "gpu" to require one).
// Prints "OK <n> checks" and returns 0 on success.
#include "AcroTensor.hpp"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <string>
#include <vector>

static int checks = 0, failures = 0;
#define CHECK(cond)                                                                  \
    do {                                                                             \
        ++checks;                                                                    \
        if (!(cond)) { ++failures; std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)
#define CHECK_THROWS(expr)                                                           \
    do {                                                                             \
        ++checks;                                                                    \
        bool threw = false;                                                          \
        try { expr; } catch (const std::exception &) { threw = true; }               \
        if (!threw) { ++failures; std::printf("FAILED %s:%d  no throw: %s\n", __FILE__, __LINE__, #expr); } \
    } while (0)

using namespace acro;

static void host_checks()
{
    // construction sugar: rank 1..9, vector of dims, external data
    Tensor t1(5), t3(2, 3, 4), t9(1, 2, 1, 2, 1, 2, 1, 2, 3);
    CHECK(t1.GetRank() == 1 && t3.GetRank() == 3 && t9.GetRank() == 9);
    CHECK(t3.GetSize() == 24 && t3.GetDim(1) == 3 && t3.GetStride(0) == 12 && t3.GetStride(2) == 1);
    CHECK(t9.GetSize() == 48);
    std::vector<int> dims = {1000, 3, 3};
    Tensor A(dims);
    CHECK(A.GetSize() == 9000);
    CHECK_THROWS(Tensor(0));
    CHECK_THROWS(Tensor(3, -2));
    std::vector<int> none;
    CHECK_THROWS(Tensor bad(none));
    Tensor late;
    CHECK(!late.IsInitialized());
    late.Init(4, 4);
    CHECK(late.IsInitialized());
    CHECK_THROWS(late.Init(4, 4));

    // indexing
    for (int i = 0; i < 24; ++i) t3[i] = i;
    CHECK(t3(1, 2, 3) == 23.0 && t3(0, 1, 0) == 4.0 && t3.GetRawIndex(1, 0, 2) == 14);
    std::vector<int> idx = {1, 1, 1};
    CHECK(t3(idx) == 17.0);
    t3.Reshape(6, 4);
    CHECK(t3.GetRank() == 2 && t3(5, 3) == 23.0);
    CHECK_THROWS(t3.Reshape(5, 5));

    // external buffers, Set / Mult
    double buf[12];
    Tensor ext(3, 4, buf);
    ext.Set(2.0);
    ext.Mult(1.5);
    CHECK(buf[0] == 3.0 && buf[11] == 3.0 && ext.GetData() == buf);
    CHECK_THROWS(Tensor(3, 4, buf, nullptr, true));   // "on GPU" without a device pointer
    CHECK(ext.GetCurrentData() == buf && !ext.IsOnGPU() && !ext.IsMappedToGPU());

    // slices
    Tensor T(2, 3, 4);
    for (int i = 0; i < 24; ++i) T[i] = i;
    SliceTensor S1(T, 1), S12(T, 1, 2);
    CHECK(S1.GetRank() == 2 && S1.GetDim(0) == 3 && S1(0, 0) == 12.0 && S12(3) == 23.0);
    S1.Set(-1.0);
    CHECK(T(1, 2, 3) == -1.0 && T(0, 2, 3) == 11.0);
    CHECK_THROWS(SliceTensor(T, 0, 0, 0));
    CHECK_THROWS(S1.Retarget(buf));

    // batch slabs: the cut of a batch index over ranks, and the leading-range view
    {
        std::int64_t covered = 0;
        for (int r = 0; r < 3; ++r)
        {
            const BatchSlab sl = SlabOf(10, r, 3);
            CHECK(sl.begin == covered && sl.size() >= 3 && sl.size() <= 4);
            covered = sl.end;
        }
        CHECK(covered == 10);
        CHECK(SlabOf((std::int64_t(1) << 62) + 5, 7, 8).end == (std::int64_t(1) << 62) + 5);
        CHECK_THROWS(SlabOf(10, 3, 3));
        SlabTensor mid(T, 1, 2), mine(T, SlabOf(T.GetDim(0), 1, 2));
        CHECK(mine.GetBegin() == 1 && mine.GetEnd() == 2 && mine.GetData() == mid.GetData());
        CHECK(mid.GetRank() == 3 && mid.GetDim(0) == 1 && mid.GetDim(2) == 4 && mid.IsSharded() && !T.IsSharded());
        CHECK(mid.GetData() == T.GetData() + 12 && mid.GetBegin() == 1 && mid.GetEnd() == 2);
        mid(0, 0, 1) = 77.0;
        CHECK(T(1, 0, 1) == 77.0);
        T(1, 0, 1) = -1.0;
        SlabTensor whole(T, 0, 2);
        CHECK(whole.GetSize() == 24 && !whole.IsMappedToGPU());
        CHECK_THROWS(SlabTensor(T, 1, 1));
        CHECK_THROWS(SlabTensor(T, 0, 3));
        CHECK_THROWS(mid.Retarget(buf));
    }

    // parser: accept / reject, names, index bookkeeping
    CHECK_THROWS(TensorKernel("Blah"));
    CHECK_THROWS(TensorKernel("Blah="));
    CHECK_THROWS(TensorKernel("B_lah=A_lah_"));
    CHECK_THROWS(TensorKernel("a_lah_=A_lah"));
    TensorKernel K("A_i=B_s_iC_i_s");
    CHECK(K.AllIndexNames.size() == 2 && K.AllIndexNames[1] == "s" && K.ContractionIndexNames.size() == 1);
    CHECK(K.GetNumIndices() == 2 && K.GetNumVars() == 3 && K.GetNumInputVars() == 2);
    CHECK(K.GetVarDimLoopNum(0, 0) == 1 && K.GetVarDimLoopNum(0, 1) == 0 && K.GetVarDimLoopNum(1, 1) == 1);
    CHECK(K.IsVarDependentOnLoop(-1, 0) && !K.IsVarDependentOnLoop(-1, 1) && K.IsContractionLoop(1));
    CHECK(K.GetNameString() == "A_ieqB_s_iC_i_s");

    // bound kernels
    Tensor o3(3), m33(3, 3), v3(3);
    std::vector<Tensor *> ins = {&m33, &m33};
    DimensionedKernel DK(&K, &o3, ins);
    CHECK(DK.GetFlatIdxSize() == 9 && DK.GetOutIdxSize() == 3 && DK.GetContIdxSize() == 3);
    CHECK(DK.GetOutputStorageReqForInnerLoops(1) == 1 && DK.GetOutputStorageReqForInnerLoops(2) == 3);
    CHECK(DK.GetInputStorageReqForInnerLoops(1) == 6 && DK.GetInputStorageReqForInnerLoops(2) == 18);
    std::string big = "S_e_i1_i2_i3_j1_j2_j3 =B_i1_j1_k1_m_nB_i2_j2_k2_m_nB_i3_j3_k3_m_n D_e_k1_k2_k3_m_n";
    TensorKernel KB(big);
    Tensor S(10, 5, 5, 5, 5, 5, 5), B1(5, 5, 5, 3, 3), D(10, 5, 5, 5, 3, 3);
    std::vector<Tensor *> bins = {&B1, &B1, &B1, &D};
    DimensionedKernel DKB(&KB, &S, bins);
    CHECK(DKB.GetFlatIdxSize() == 175781250 && DKB.GetOutIdxSize() == 156250 && DKB.GetContIdxSize() == 1125);

    // grouping: loop order and unique variables
    std::vector<DimensionedKernel *> group = {&DKB};
    DimensionedMultiKernel MK(group);
    CHECK(MK.GetNumUVars() == 3 && MK.GetNumOuterIndices() == 7 && MK.GetLoopIndex(0) == "e");

    // engine: policy names, dimension errors, plan text without a device
    TensorEngine TE("Cuda");
    CHECK(TE.GetExecType() == "Cuda");
    CHECK_THROWS(TensorEngine("Fortran"));
    Tensor v2(2), uninit;
    CHECK_THROWS(TE.GetImplementation("A_i=B_iC_i", o3, v3, v2));
    CHECK_THROWS(TE.GetImplementation("A_i=B_i_jC_i", uninit, m33, v3));
    std::string plan = TE.GetImplementation("A_i=B_i_jC_i", o3, m33, v3);
    CHECK(plan.find("family=generic") != std::string::npos);
    Tensor bigA(1 << 20, 3, 3, buf), bigB(1 << 20, buf), s33(3, 3);   // shape-only: never dereferenced here
    plan = TE.GetImplementation("S_i_j = A_n_i_j B_n", s33, bigA, bigB);
    CHECK(plan.find("family=reduce_batch") != std::string::npos);
    CHECK(plan.find("summed over the ranks of a peer group when one of these inputs is a rank's slab: A B") != std::string::npos);
    TE.BeginMultiKernelLaunch();
    CHECK_THROWS(TE.BeginMultiKernelLaunch());
    TE("A_i = B_i", o3, v3);     // recorded only
    CHECK(TE.EndMultiKernelLaunchDescribe().find("step 0") != std::string::npos);
    CHECK_THROWS(TE.EndMultiKernelLaunch());
}

static void device_checks()
{
    // README example
    std::vector<int> dims = {1000, 3, 3};
    Tensor A(dims), B(1000), S(3, 3);
    for (int i = 0; i < 9000; ++i) A[i] = (i % 7) * 0.25;
    B.Set(1.0);
    A.MapToGPU(); B.MapToGPU(); S.MapToGPU();
    A.MoveToGPU(); B.MoveToGPU(); S.SwitchToGPU();
    TensorEngine TE("Cuda");
    TE("S_i_j = A_n_i_j B_n", S, A, B);
    S.MoveFromGPU();
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j)
        {
            double sum = 0.0;
            for (int n = 0; n < 1000; ++n) sum += A(n, i, j);
            CHECK(std::fabs(S(i, j) - sum) <= 1e-12 * std::fabs(sum));
        }
    TE("S_i_j = A_n_i_j", S, A);
    S.MoveFromGPU();
    CHECK(std::fabs(S(0, 0) - 0.25 * ([&] { double s = 0; for (int n = 0; n < 1000; ++n) s += (n * 9) % 7; return s; })()) <= 1e-9);

    // flag semantics
    Tensor T(2);
    T.Set(3.0);
    T.MapToGPU();
    CHECK(T.IsMappedToGPU() && !T.IsOnGPU());
    T.SwitchToGPU();
    T.Set(9.0);
    CHECK(T(0) == 3.0);
    T.MoveFromGPU();
    CHECK(T(0) == 9.0 && T(1) == 9.0 && !T.IsOnGPU());

    // slices as outputs, multi-kernel launch where the last kernel wins
    Tensor U(2, 5), X(5);
    U.Set(7.0);
    for (int i = 0; i < 5; ++i) X(i) = i;
    SliceTensor U0(U, 0);
    TE("U0_i = X_i", U0, X);
    U.MoveFromGPU();
    CHECK(U(0, 3) == 3.0 && U(1, 3) == 7.0);
    Tensor Aout(3), B1(3), B2(3), C(3, 3);
    B1(0) = 1; B1(1) = 2; B1(2) = 3;
    B2.Set(1.0); C.Set(1.0);
    TE.BeginMultiKernelLaunch();
    TE("A_i = B1_i", Aout, B1);
    TE("A_i = C_i_j B2_j", Aout, C, B2);
    TE.EndMultiKernelLaunch();
    Aout.MoveFromGPU();
    CHECK(Aout(0) == 3.0 && Aout(1) == 3.0 && Aout(2) == 3.0);

    // sum-gather over a sharded range: one rank shares nothing, the result is the plain one
    IndexMapping Map(4, 6);
    const int targets[6] = {0, 1, 1, 3, 0, 1};
    for (int i = 0; i < 6; ++i) Map[i] = targets[i];
    SharedEntryExchange Exchange(Map, 1, 0, [](const SharedEntryExchange::Bytes &mine) {
        return std::vector<SharedEntryExchange::Bytes>(1, mine);
    });
    CHECK(Exchange.GetNumShared() == 0);
    Tensor In(6), Out(4);
    for (int i = 0; i < 6; ++i) In(i) = i + 1;
    TE.FlatIndexedSumGather(Out, In, Map, Exchange);
    Out.MoveFromGPU();
    CHECK(Out(0) == 6.0 && Out(1) == 11.0 && Out(2) == 0.0 && Out(3) == 4.0);
}

int main(int argc, char **argv)
{
    try
    {
        host_checks();
        const bool want_gpu = argc > 1 && std::strcmp(argv[1], "gpu") == 0;
        if (isCudaReady()) device_checks();
        else if (want_gpu) { std::printf("FAILED: a GPU was required but none is usable\n"); return 2; }
    }
    catch (const std::exception &e)
    {
        std::printf("FAILED with exception: %s\n", e.what());
        return 1;
    }
    if (failures) { std::printf("%d of %d checks failed\n", failures, checks); return 1; }
    std::printf("OK %d checks%s\n", checks, isCudaReady() ? " (with device)" : " (host only)");
    return 0;
}
