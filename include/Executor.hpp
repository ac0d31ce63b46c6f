#ifndef ACRO_B200_EXECUTOR_UMBRELLA_HPP
#define ACRO_B200_EXECUTOR_UMBRELLA_HPP
#include "KernelExecutor.hpp"
#include "B200Executor.hpp"
#endif
