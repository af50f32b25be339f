// Shared helpers of the flyvec_b200 library: status/error plumbing and small
// device utilities.  Nothing here allocates.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// the public header: in include/ of the source tree, beside this file in an installed package
#if __has_include("../../include/flyvec_b200.h")
#include "../../include/flyvec_b200.h"
#else
#include "flyvec_b200.h"
#endif

namespace fv {

// Stores a printf-style message for fv_last_error() of the calling thread and
// returns `code`, so that `return fail(...)` reads naturally.
int fail(int code, const char* fmt, ...);
void clear_error();

// RAII: make `device` current for the scope, restore the previous one after.
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    ok = (cudaSetDevice(device) == cudaSuccess);
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace fv

#define FV_CUDA(call)                                                                                  \
  do {                                                                                                 \
    cudaError_t fv_e_ = (call);                                                                        \
    if (fv_e_ != cudaSuccess)                                                                          \
      return fv::fail(FV_ERR_CUDA, "%s:%d: %s failed: %s", __FILE__, __LINE__, #call,                  \
                      cudaGetErrorString(fv_e_));                                                      \
  } while (0)

#define FV_REQUIRE(cond, code, ...)                 \
  do {                                              \
    if (!(cond)) return fv::fail(code, __VA_ARGS__); \
  } while (0)

// Bits of the device-side error word (fv_run_stats.device_error).
#define FV_DEVERR_TOKEN_RANGE 1u  // a token id was >= V
#define FV_DEVERR_WINDOW_RANGE 2u // a window start or permutation entry was out of range
#define FV_DEVERR_SLOT_RANGE 4u   // a scatter slot id did not fit its tag
#define FV_DEVERR_NAN_WEIGHT 8u   // a NaN was found where a weight was expected
#define FV_DEVERR_TIMEOUT 16u     // a bounded wait on a peer's flag ran out
