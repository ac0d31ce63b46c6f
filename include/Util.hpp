#ifndef ACRO_B200_UTIL_HPP
#define ACRO_B200_UTIL_HPP
#include "Error.hpp"
#include "CudaUtil.hpp"
#endif
