// Error convention of the C ABI: every entry point returns 0 on success and a non-zero code
// otherwise; the message of the last failure on the calling thread is kept for
// eisen_last_error().  Nothing aborts or throws across the boundary.
#pragma once
#include <cuda_runtime.h>

namespace eisen {

enum Status : int {
  EISEN_OK = 0,
  EISEN_ERR_INVALID = 1,   // bad argument (shape, alignment, dtype)
  EISEN_ERR_CUDA = 2,      // a CUDA runtime / driver call failed
  EISEN_ERR_KERNEL = 3,    // a kernel recorded a fault in its status word (a bounded wait ran out)
  EISEN_ERR_OOM = 4,       // device allocation failed
  EISEN_ERR_LIMIT = 5,     // a stated size limit of an entry point was exceeded
};

void set_error(const char* msg);
int fail(int code, const char* msg);
int check_launch(const char* what);

}  // namespace eisen
