// TEST INFRASTRUCTURE — not part of the product.
//
// Force-included (-include) in front of the reference's unittest/kernel/test_TensorEngine.cpp when
// oracle/Makefile builds the reference's own unit tests against THIS library.  That test runs its
// suite on TensorEngine("CPUInterpreted") first and on TensorEngine("Cuda") second
// (unittest/kernel/test_TensorEngine.cpp:16-27).  This library has no CPU executor, so the first
// engine is created as "Cuda" too; the suite then runs once, on the device (the second engine's
// sections carry the same names and the test framework skips them as already done).
//
// One section ("Scatters and Gathers" / "FlatIndexedSumGather", :734-743) reads the result through
// Tensor::operator[] on the host without MoveFromGPU(): its name has no engine prefix, so in the
// reference it only ever runs on the CPU engine, and on the reference's own "Cuda" engine it would
// read stale host data just the same (TensorEngine::FlatIndexedSumGather leaves the result on the
// device, kernel/TensorEngine.cpp:703-714, as this library does).  The engine below brings that one
// result back so that the section's six checks see what the device computed.
//
// Every line of the reference's tests is compiled as it is.
#ifndef ACRO_B200_REF_UNIT_TESTS_ENGINE_HPP
#define ACRO_B200_REF_UNIT_TESTS_ENGINE_HPP

#include "AcroTensor.hpp"
#include <cstring>

namespace acro
{
class DeviceOnlyEngine : public TensorEngine
{
    public:
    DeviceOnlyEngine(const char *exec_type)
        : TensorEngine(std::strcmp(exec_type, "CPUInterpreted") == 0 ? "Cuda" : exec_type) {}

    void FlatIndexedSumGather(Tensor &Aout, Tensor &Ain, IndexMapping &M)
    {
        TensorEngine::FlatIndexedSumGather(Aout, Ain, M);
        Aout.MoveFromGPU();
    }
};
}

#define TensorEngine DeviceOnlyEngine

#endif
