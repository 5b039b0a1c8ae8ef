// Error convention of the C ABI: every entry point returns 0 on success and a non-zero code
// otherwise; the message of the last failure on the calling thread is kept for
// eisen_last_error().  Nothing aborts or throws across the boundary.
#pragma once
#include <cuda_runtime.h>

#include "../../include/eisen_b200.h"  // EISEN_OK / EISEN_ERR_* codes

namespace eisen {


void set_error(const char* msg);
int fail(int code, const char* msg);
int check_launch(const char* what);  // also counts the launch
void count_launch();

// Index of the current device for per-device one-time set-up (kernel attributes and occupancy
// are properties of a device, not of the process).  Devices beyond 63 share the last slot.
inline int device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
  return dev < 63 ? dev : 63;
}
constexpr int MAX_DEVICE_SLOTS = 64;

// eisen_set_deterministic: kernels whose result depends on the order of floating-point adds (split-K
// weight gradients, the dQ accumulation of the attention backward) switch to fixed-order forms
bool deterministic();

}  // namespace eisen
