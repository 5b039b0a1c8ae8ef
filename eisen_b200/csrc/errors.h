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

}  // namespace eisen
