// Build configuration of the B200 drop-in for the aotriton operator API.
// Plays the role of the cmake-generated config.h of ROCm/aotriton
// (include/aotriton/config.h.in:1-30): namespace name, optional suffix,
// version numbers and the export attribute.
#ifndef AOTRITON_V2_CONFIG_H
#define AOTRITON_V2_CONFIG_H

// Compile with -DAOTRITON_NAME_SUFFIX=foo to get namespace aotritonfoo, the
// way the reference's tests require for side-by-side installs.
#ifdef AOTRITON_NAME_SUFFIX
#define AOTRITON_ENABLE_SUFFIX 1
#define AOTRITON_B200_CAT_(a, b) a##b
#define AOTRITON_B200_CAT(a, b) AOTRITON_B200_CAT_(a, b)
#define AOTRITON_NS AOTRITON_B200_CAT(aotriton, AOTRITON_NAME_SUFFIX)
#else
#define AOTRITON_ENABLE_SUFFIX 0
#define AOTRITON_NAME_SUFFIX
#define AOTRITON_NS aotriton
#endif

// API level mirrored from the reference (CMakeLists.txt:9-11).
#define AOTRITON_VERSION_MAJOR 0
#define AOTRITON_VERSION_MINOR 14
#define AOTRITON_VERSION_PATCH 0
#define AOTRITON_GIT_SHA1 "b200-native"

#ifdef _MSC_VER
#define AOTRITON_API __declspec(dllexport)
#else
#define AOTRITON_API __attribute__((visibility("default")))
#endif

#endif
