// Umbrella header of the acro:: API (same name as LLNL/acrotensor's AcroTensor.hpp:6-9).
#ifndef ACRO_B200_ACROTENSOR_HPP
#define ACRO_B200_ACROTENSOR_HPP
#include "TensorEngine.hpp"
#include "Executor.hpp"
#include "SliceTensor.hpp"
#include "SlabTensor.hpp"
#include "IndexMapping.hpp"
#include "SharedEntryExchange.hpp"
#endif
