// Placeholder for the tuning-build controls of ROCm/aotriton
// (include/aotriton/cpp_tune.h:16-70).  This library has one hand-written
// kernel per operator and no tuning database, so there is nothing to steer;
// the header exists so that `#include <aotriton/cpp_tune.h>` keeps compiling.
#ifndef AOTRITON_V3_API_CPP_TUNE_H
#define AOTRITON_V3_API_CPP_TUNE_H

#include <aotriton/config.h>

#define AOTRITON_BUILD_FOR_TUNING 0

#endif
