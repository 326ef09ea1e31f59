// Host-side helpers shared by the translation units of the library:
// thread-local error text, the device-wait deadline, and the driver entry
// point for tensor-map encoding (resolved at run time so that the library
// links against the CUDA runtime only).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/dynaflow_b200.h"

namespace df {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Returns NULL (and sets the error text) when the driver has no such entry point.
PFN_encodeTiled get_encode_tiled();

// printf-style error text for df_last_error().
void set_error(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// set_error + return code, for one-line early exits.
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// Current value (0 / 1) of a launch-form option set with df_set_launch_option.
int launch_option_value(int option);

// Fills `attr` with the programmatic-serialization attribute when the DF_OPT_DEPENDENT_LAUNCH
// option is on and returns how many attributes were written (0 or 1).
inline int dependent_launch_attr(cudaLaunchAttribute* attr) {
  if (launch_option_value(DF_OPT_DEPENDENT_LAUNCH) == 0) return 0;
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
  return 1;
}

// Deadline for device-side waits, in nanoseconds from kernel start.
unsigned long long timeout_ns();

}  // namespace df
