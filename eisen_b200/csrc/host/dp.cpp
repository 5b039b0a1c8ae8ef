// Data-parallel exchange step behind the C ABI: a thin, checked layer over NCCL (eisen_dp_*).
//
// The reference is single-GPU; this is the one exchange the data-parallel training step adds
// (gradient buckets summed across ranks while the backward pass is still running, or, sharded,
// reduce-scatter -> optimizer on the rank's slice -> all-gather of the updated weights).  A Rust
// host binds these entry points the same way as the kernel-level ones; it needs no torch.
//
// NCCL is bound at run time (dlopen of libnccl.so.2): the library has no link-time dependency on
// it, loads on machines without it, and shares the copy a process has already loaded.  Every
// call returns a status; nothing blocks without a limit: eisen_dp_wait polls the stream and the
// communicator's asynchronous error state until a host-side deadline and aborts the communicator
// when the deadline passes, so a peer that never arrives ends in an error code, not in a hang.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <thread>

#include "../../../include/eisen_b200.h"
#include "../errors.h"

namespace {

// the part of NCCL's public C API used here (nccl.h: types and constants of the stable ABI)
typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
enum { kNcclSuccess = 0, kNcclInProgress = 7 };
enum { kNcclInt64 = 4, kNcclFloat32 = 7, kNcclFloat64 = 8, kNcclBfloat16 = 9 };
enum { kNcclSum = 0 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  const char* load_error = nullptr;
};

NcclApi& api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (a.handle) break;
    }
    if (!a.handle) { a.load_error = "libnccl.so.2 not found (dlopen)"; return; }
    bool ok = true;
    auto sym = [&](const char* name) { void* p = dlsym(a.handle, name); if (!p) ok = false; return p; };
    a.GetUniqueId = (int (*)(NcclUniqueId*))sym("ncclGetUniqueId");
    a.CommInitRank = (int (*)(ncclComm_t*, int, NcclUniqueId, int))sym("ncclCommInitRank");
    a.CommDestroy = (int (*)(ncclComm_t))sym("ncclCommDestroy");
    a.CommAbort = (int (*)(ncclComm_t))sym("ncclCommAbort");
    a.CommGetAsyncError = (int (*)(ncclComm_t, int*))sym("ncclCommGetAsyncError");
    a.AllReduce = (int (*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))sym("ncclAllReduce");
    a.ReduceScatter = (int (*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))sym("ncclReduceScatter");
    a.AllGather = (int (*)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t))sym("ncclAllGather");
    a.Broadcast = (int (*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))sym("ncclBroadcast");
    a.GroupStart = (int (*)())sym("ncclGroupStart");
    a.GroupEnd = (int (*)())sym("ncclGroupEnd");
    a.GetErrorString = (const char* (*)(int))sym("ncclGetErrorString");
    if (!ok) a.load_error = "libnccl.so.2 lacks a required symbol";
  });
  return a;
}

struct DpComm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  bool aborted = false;
  long long launched = 0;  // collectives enqueued since init (the sequence a host-side handshake compares)
};

int nccl_fail(int rc, const char* what) {
  char buf[400];
  const char* s = api().GetErrorString ? api().GetErrorString(rc) : "?";
  std::snprintf(buf, sizeof(buf), "%s: NCCL error %d (%s)", what, rc, s);
  return eisen::fail(EISEN_ERR_COMM, buf);
}

int ready(void* h, DpComm** out, const char* who) {
  if (api().load_error) return eisen::fail(EISEN_ERR_COMM, api().load_error);
  if (!h) return eisen::fail(EISEN_ERR_INVALID, "eisen_dp: null communicator handle");
  DpComm* c = static_cast<DpComm*>(h);
  if (c->aborted || !c->comm) {
    char buf[200];
    std::snprintf(buf, sizeof(buf), "%s: the communicator was aborted", who);
    return eisen::fail(EISEN_ERR_COMM, buf);
  }
  *out = c;
  return 0;
}

int nccl_dtype(int dt, int* out) {
  switch (dt) {
    case EISEN_F32: *out = kNcclFloat32; return 0;
    case EISEN_BF16: *out = kNcclBfloat16; return 0;
    case EISEN_F64: *out = kNcclFloat64; return 0;
    case EISEN_I64: *out = kNcclInt64; return 0;
  }
  return eisen::fail(EISEN_ERR_INVALID, "eisen_dp: dtype must be EISEN_F32, EISEN_BF16, EISEN_F64 or EISEN_I64");
}

}  // namespace

extern "C" {

int eisen_dp_available(void) { return api().load_error ? 0 : 1; }

int eisen_dp_unique_id(void* out128) {
  if (api().load_error) return eisen::fail(EISEN_ERR_COMM, api().load_error);
  if (!out128) return eisen::fail(EISEN_ERR_INVALID, "dp_unique_id: null output");
  NcclUniqueId id;
  int rc = api().GetUniqueId(&id);
  if (rc != kNcclSuccess) return nccl_fail(rc, "dp_unique_id");
  std::memcpy(out128, id.internal, 128);
  return 0;
}

int eisen_dp_init(int rank, int world, const void* unique_id128, void** comm_out) {
  if (api().load_error) return eisen::fail(EISEN_ERR_COMM, api().load_error);
  if (!unique_id128 || !comm_out) return eisen::fail(EISEN_ERR_INVALID, "dp_init: null argument");
  if (world < 1 || rank < 0 || rank >= world) return eisen::fail(EISEN_ERR_INVALID, "dp_init: need 0 <= rank < world");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
    cudaGetLastError();
    return eisen::fail(EISEN_ERR_CUDA, "dp_init: no CUDA device (NCCL communicators live on GPUs)");
  }
  NcclUniqueId id;
  std::memcpy(id.internal, unique_id128, 128);
  DpComm* c = new DpComm();
  c->rank = rank;
  c->world = world;
  int rc = api().CommInitRank(&c->comm, world, id, rank);
  if (rc != kNcclSuccess) {
    delete c;
    return nccl_fail(rc, "dp_init(ncclCommInitRank)");
  }
  *comm_out = c;
  return 0;
}

int eisen_dp_destroy(void* h) {
  if (!h) return 0;
  DpComm* c = static_cast<DpComm*>(h);
  if (c->comm && !c->aborted && !api().load_error) api().CommDestroy(c->comm);
  delete c;
  return 0;
}

int eisen_dp_rank_world(void* h, int* rank, int* world, long long* launched) {
  if (!h) return eisen::fail(EISEN_ERR_INVALID, "eisen_dp: null communicator handle");
  DpComm* c = static_cast<DpComm*>(h);
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (launched) *launched = c->launched;
  return 0;
}

int eisen_dp_allreduce_bucket(void* h, void* ptr, long long n, int dtype, void* stream) {
  DpComm* c;
  if (int rc = ready(h, &c, "dp_allreduce_bucket")) return rc;
  int ndt;
  if (int rc = nccl_dtype(dtype, &ndt)) return rc;
  if (n <= 0) return 0;
  int rc = api().AllReduce(ptr, ptr, (size_t)n, ndt, kNcclSum, c->comm, (cudaStream_t)stream);
  if (rc != kNcclSuccess) return nccl_fail(rc, "dp_allreduce_bucket");
  ++c->launched;
  return 0;
}

int eisen_dp_reduce_scatter(void* h, const void* send, void* recv, long long recv_n, int dtype, void* stream) {
  DpComm* c;
  if (int rc = ready(h, &c, "dp_reduce_scatter")) return rc;
  int ndt;
  if (int rc = nccl_dtype(dtype, &ndt)) return rc;
  if (recv_n <= 0) return 0;
  int rc = api().ReduceScatter(send, recv, (size_t)recv_n, ndt, kNcclSum, c->comm, (cudaStream_t)stream);
  if (rc != kNcclSuccess) return nccl_fail(rc, "dp_reduce_scatter");
  ++c->launched;
  return 0;
}

int eisen_dp_all_gather(void* h, const void* send, void* recv, long long send_n, int dtype, void* stream) {
  DpComm* c;
  if (int rc = ready(h, &c, "dp_all_gather")) return rc;
  int ndt;
  if (int rc = nccl_dtype(dtype, &ndt)) return rc;
  if (send_n <= 0) return 0;
  int rc = api().AllGather(send, recv, (size_t)send_n, ndt, c->comm, (cudaStream_t)stream);
  if (rc != kNcclSuccess) return nccl_fail(rc, "dp_all_gather");
  ++c->launched;
  return 0;
}

int eisen_dp_broadcast(void* h, void* ptr, long long n, int dtype, int root, void* stream) {
  DpComm* c;
  if (int rc = ready(h, &c, "dp_broadcast")) return rc;
  int ndt;
  if (int rc = nccl_dtype(dtype, &ndt)) return rc;
  if (root < 0 || root >= c->world) return eisen::fail(EISEN_ERR_INVALID, "dp_broadcast: root out of range");
  if (n <= 0) return 0;
  int rc = api().Broadcast(ptr, ptr, (size_t)n, ndt, root, c->comm, (cudaStream_t)stream);
  if (rc != kNcclSuccess) return nccl_fail(rc, "dp_broadcast");
  ++c->launched;
  return 0;
}

int eisen_dp_group_begin(void) {
  if (api().load_error) return eisen::fail(EISEN_ERR_COMM, api().load_error);
  int rc = api().GroupStart();
  return rc == kNcclSuccess ? 0 : nccl_fail(rc, "dp_group_begin");
}
int eisen_dp_group_end(void) {
  if (api().load_error) return eisen::fail(EISEN_ERR_COMM, api().load_error);
  int rc = api().GroupEnd();
  return rc == kNcclSuccess ? 0 : nccl_fail(rc, "dp_group_end");
}

int eisen_dp_poll_error(void* h) {
  DpComm* c;
  if (int rc = ready(h, &c, "dp_poll_error")) return rc;
  int st = kNcclSuccess;
  int rc = api().CommGetAsyncError(c->comm, &st);
  if (rc != kNcclSuccess) return nccl_fail(rc, "dp_poll_error");
  if (st != kNcclSuccess && st != kNcclInProgress) return nccl_fail(st, "dp_poll_error(async)");
  return 0;
}

int eisen_dp_abort(void* h) {
  if (!h) return eisen::fail(EISEN_ERR_INVALID, "eisen_dp: null communicator handle");
  DpComm* c = static_cast<DpComm*>(h);
  if (c->comm && !c->aborted && !api().load_error) api().CommAbort(c->comm);
  c->aborted = true;
  c->comm = nullptr;
  return 0;
}

int eisen_dp_wait(void* h, void* stream, long long deadline_ms) {
  DpComm* c;
  if (int rc = ready(h, &c, "dp_wait")) return rc;
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    cudaError_t q = cudaStreamQuery((cudaStream_t)stream);
    if (q == cudaSuccess) return eisen_dp_poll_error(h);
    if (q != cudaErrorNotReady) {
      cudaGetLastError();
      return eisen::fail(EISEN_ERR_CUDA, "dp_wait: the stream reported a CUDA error");
    }
    if (int rc = eisen_dp_poll_error(h)) {
      eisen_dp_abort(h);
      return rc;
    }
    const long long ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if (deadline_ms >= 0 && ms > deadline_ms) {
      eisen_dp_abort(h);
      return eisen::fail(EISEN_ERR_TIMEOUT, "dp_wait: the exchange did not finish before the deadline; communicator aborted");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

}  // extern "C"
