// Embedding row gather and its backward scatter-add (src/graph/ops/transform.rs:287-324;
// kernels/ops_f32.cu:513-537 scatter with one atomicAdd per element).
//
// Token ids are int32 on the device (the reference keeps them as f32 and, in bf16 mode, rounds
// them through bf16).  The backward is deterministic and free of floating-point atomics:
//   1. rank[i]   = number of earlier positions j < i with ids[j] == ids[i]   (integer)
//      count[v]  = occurrences of id v                                       (integer atomics)
//   2. offset[v] = exclusive prefix sum of count                             (one CTA)
//   3. perm[offset[ids[i]] + rank[i]] = i      -> positions grouped by id, in position order
//   4. one warp per vocabulary row sums its positions' gradient rows in that fixed order and
//      adds the sum to the f32 weight gradient.
// Steps 1-3 are exact integer bookkeeping (identical to a stable sort of the ids).
#include "common.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

template <typename TW, typename TO>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const TW* __restrict__ w, const int* __restrict__ ids, TO* __restrict__ out, long long n_ids,
                   int dim, int vocab, int* __restrict__ bad_id_flag) {
  // one warp per output row
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = warp0; i < n_ids; i += wstride) {
    int id = ids[i];
    if (id < 0 || id >= vocab) {  // out-of-range ids are recorded, the row reads id 0
      if (lane == 0 && bad_id_flag) atomicExch(bad_id_flag, 1);
      id = 0;
    }
    const TW* src = w + (long long)id * dim;
    TO* dst = out + i * dim;
    for (int c = lane; c < dim; c += 32) dst[c] = from_f32<TO>(to_f32(src[c]));
  }
}

// vectorised same-dtype gather (16 bytes per lane)
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_vec_kernel(const T* __restrict__ w, const int* __restrict__ ids, T* __restrict__ out,
                       long long n_ids, int dim, int vocab, int* __restrict__ bad_id_flag) {
  constexpr int V = VecOf<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = warp0; i < n_ids; i += wstride) {
    int id = ids[i];
    if (id < 0 || id >= vocab) {
      if (lane == 0 && bad_id_flag) atomicExch(bad_id_flag, 1);
      id = 0;
    }
    const uint4* src = reinterpret_cast<const uint4*>(w + (long long)id * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + i * dim);
    for (int c = lane; c < dim / V; c += 32) dst[c] = src[c];
  }
}

constexpr int RANK_TILE = 1024;

// rank[i] = #{ j < i : ids[j] == ids[i] }; count[ids[i]] += 1
__global__ void __launch_bounds__(256)
rank_kernel(const int* __restrict__ ids, int* __restrict__ rank, int* __restrict__ count, int n, int vocab) {
  __shared__ int tile[RANK_TILE];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int my = (i < n) ? ids[i] : -1;
  const int last = min(n, (int)((blockIdx.x + 1) * blockDim.x));  // ids at or after `last` cannot precede
  int r = 0;
  for (int base = 0; base < last; base += RANK_TILE) {
    __syncthreads();
    for (int t = threadIdx.x; t < RANK_TILE; t += blockDim.x) tile[t] = (base + t < n) ? ids[base + t] : -2;
    __syncthreads();
    const int lim = min(RANK_TILE, i - base);  // only j < i
    for (int t = 0; t < lim; ++t) r += (tile[t] == my);
  }
  if (i < n) {
    rank[i] = r;
    if (my >= 0 && my < vocab) atomicAdd(&count[my], 1);
  }
}

// exclusive scan of count[0..vocab) by one CTA of 1024 threads
__global__ void __launch_bounds__(1024) scan_kernel(const int* __restrict__ count, int* __restrict__ offset, int vocab) {
  __shared__ int warp_tot[32];
  __shared__ int carry_sh;
  if (threadIdx.x == 0) carry_sh = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int base = 0; base < vocab; base += 1024) {
    const int idx = base + threadIdx.x;
    const int v = (idx < vocab) ? count[idx] : 0;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = warp_tot[lane];
      int winc = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
      }
      warp_tot[lane] = winc - w;  // exclusive prefix of warp totals
    }
    __syncthreads();
    const int carry = carry_sh;
    if (idx < vocab) offset[idx] = carry + warp_tot[warp] + inc - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_sh = carry + warp_tot[warp] + inc;
    __syncthreads();
  }
}

__global__ void place_kernel(const int* __restrict__ ids, const int* __restrict__ rank,
                             const int* __restrict__ offset, int* __restrict__ perm, int n, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id < 0 || id >= vocab) return;
  perm[offset[id] + rank[i]] = i;
}

// one warp per vocabulary row: dW[v,:] += sum over its positions (fixed order) of g[pos,:]
template <typename TG>
__global__ void __launch_bounds__(256)
scatter_rows_kernel(const TG* __restrict__ g, const int* __restrict__ perm, const int* __restrict__ offset,
                    const int* __restrict__ count, float* __restrict__ dw, int vocab, int dim) {
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int wstride = gridDim.x * (blockDim.x >> 5);
  for (int v = warp0; v < vocab; v += wstride) {
    const int cnt = count[v];
    if (cnt == 0) continue;
    const int off = offset[v];
    float* drow = dw + (long long)v * dim;
    for (int c0 = 0; c0 < dim; c0 += 128) {  // 4 columns per lane per sweep
      float a[4] = {0.f, 0.f, 0.f, 0.f};
      const int c = c0 + lane * 4;
      for (int k = 0; k < cnt; ++k) {
        const TG* grow = g + (long long)perm[off + k] * dim;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < dim) a[e] += to_f32(grow[c + e]);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + e < dim) drow[c + e] += a[e];
    }
  }
}

}  // namespace
}  // namespace eisen

using namespace eisen;

extern "C" {

// out[i,:] = W[ids[i],:].  w_dt / out_dt may differ (f32 table -> bf16 activations).
// bad_id_flag (device int, may be null) is set to 1 when an id falls outside [0, vocab).
int eisen_embedding_fwd(void* stream, const void* w, int w_dt, const int* ids, void* out, int out_dt,
                        long long n_ids, long long dim, long long vocab, int* bad_id_flag) {
  if (n_ids <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = grid_for(n_ids, 8, 8);
  if (w_dt == out_dt) {
    EISEN_DISPATCH_DTYPE(w_dt, T, {
      if (dim % VecOf<T>::N == 0 && aligned16(w) && aligned16(out)) {
        gather_rows_vec_kernel<T><<<grid, 256, 0, s>>>((const T*)w, ids, (T*)out, n_ids, (int)dim, (int)vocab, bad_id_flag);
      } else {
        gather_rows_kernel<T, T><<<grid, 256, 0, s>>>((const T*)w, ids, (T*)out, n_ids, (int)dim, (int)vocab, bad_id_flag);
      }
      return check_launch("embedding_fwd");
    });
  }
  if (w_dt == DT_F32)
    gather_rows_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>((const float*)w, ids, (__nv_bfloat16*)out, n_ids, (int)dim, (int)vocab, bad_id_flag);
  else
    gather_rows_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>((const __nv_bfloat16*)w, ids, (float*)out, n_ids, (int)dim, (int)vocab, bad_id_flag);
  return check_launch("embedding_fwd");
}

// scratch: count[vocab], offset[vocab], rank[n_ids], perm[n_ids] (int32 each)
long long eisen_embedding_bwd_workspace_bytes(long long n_ids, long long vocab) {
  return (2 * vocab + 2 * n_ids) * 4 + 64;
}

// dW[ids[i],:] += g[i,:] for all i, deterministically.  perm_out (may be null) receives the
// positions grouped by id (a stable sort of the ids), for bookkeeping checks.
int eisen_embedding_bwd(void* stream, const void* g, int g_dt, const int* ids, float* dw, void* workspace,
                        long long n_ids, long long dim, long long vocab) {
  if (n_ids <= 0) return 0;
  if (n_ids > 0x7fffffffLL || vocab > 0x7fffffffLL) return fail(EISEN_ERR_LIMIT, "embedding_bwd: more than 2^31 ids or rows");
  if (!workspace) return fail(EISEN_ERR_INVALID, "embedding_bwd: workspace is null");
  cudaStream_t s = (cudaStream_t)stream;
  int* count = (int*)workspace;
  int* offset = count + vocab;
  int* rank = offset + vocab;
  int* perm = rank + n_ids;
  if (cudaMemsetAsync(count, 0, (size_t)vocab * 4, s) != cudaSuccess) return fail(EISEN_ERR_CUDA, "embedding_bwd: memset failed");
  const int n = (int)n_ids;
  rank_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, rank, count, n, (int)vocab);
  scan_kernel<<<1, 1024, 0, s>>>(count, offset, (int)vocab);
  place_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, rank, offset, perm, n, (int)vocab);
  const int grid = grid_for(vocab, 8, 8);
  if (g_dt == DT_F32)
    scatter_rows_kernel<float><<<grid, 256, 0, s>>>((const float*)g, perm, offset, count, dw, (int)vocab, (int)dim);
  else
    scatter_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)g, perm, offset, count, dw, (int)vocab, (int)dim);
  return check_launch("embedding_bwd");
}

// copies the grouping computed by the last eisen_embedding_bwd on this workspace:
// perm[n_ids] (positions grouped by id), offset[vocab], count[vocab]
int eisen_embedding_bwd_bookkeeping(void* stream, const void* workspace, long long n_ids, long long vocab,
                                    int* count_out, int* offset_out, int* perm_out) {
  cudaStream_t s = (cudaStream_t)stream;
  const int* count = (const int*)workspace;
  const int* offset = count + vocab;
  const int* perm = offset + vocab + n_ids;
  if (count_out && cudaMemcpyAsync(count_out, count, (size_t)vocab * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return fail(EISEN_ERR_CUDA, "bookkeeping copy failed");
  if (offset_out && cudaMemcpyAsync(offset_out, offset, (size_t)vocab * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return fail(EISEN_ERR_CUDA, "bookkeeping copy failed");
  if (perm_out && cudaMemcpyAsync(perm_out, perm, (size_t)n_ids * 4, cudaMemcpyDeviceToDevice, s) != cudaSuccess) return fail(EISEN_ERR_CUDA, "bookkeeping copy failed");
  return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Embedding backward without any allocation by the caller or by this library.
//
// Some hosts of this library own every byte of device memory themselves and cannot hand out a
// workspace on demand: an engine that runs under a fixed VRAM budget and accounts each buffer
// in its own pool (the way the reference's Graph does with EISEN_VRAM_BUDGET_MB), or a training
// loop that must not call cudaMalloc in the middle of a step because the call synchronises the
// device.  For them the integer bookkeeping of the scatter (count, offset, rank, perm) lives in
// a fixed array inside the library image instead of a caller-provided workspace.
//
// The array is part of the module: every GPU that loads the library holds
// (2 * 131072 + 2 * 65536) * 4 bytes = 1.5 MB of it until the process exits.
// ---------------------------------------------------------------------------------------
namespace {
constexpr long long kStaticMaxIds = 65536;     // token positions per call
constexpr long long kStaticMaxVocab = 131072;  // rows of the embedding table
static __device__ __align__(256) int g_embedding_static_scratch[2 * kStaticMaxVocab + 2 * kStaticMaxIds];

// Device address of the array, looked up once per device.  In host code the array's name is only
// a handle for the runtime, not an address a kernel could use, so it goes through
// cudaGetSymbolAddress with the target device current.
int* static_scratch_for_current_device(const char** err) {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    *err = "embedding_bwd_static: cannot identify the current device";
    return nullptr;
  }
  if (!ptrs[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_embedding_static_scratch);
    if (e != cudaSuccess || !p) {
      *err = "embedding_bwd_static: cudaGetSymbolAddress failed for the scratch array";
      return nullptr;
    }
    ptrs[dev] = static_cast<int*>(p);
  }
  return ptrs[dev];
}
}  // namespace

extern "C" int eisen_embedding_bwd_static(void* stream, const void* g, int g_dt, const int* ids, float* dw,
                                          long long n_ids, long long dim, long long vocab) {
  if (n_ids > kStaticMaxIds || vocab > kStaticMaxVocab)
    return fail(EISEN_ERR_LIMIT,
                "embedding_bwd_static: at most 65536 ids and 131072 table rows fit the built-in scratch; "
                "use eisen_embedding_bwd with a workspace for larger sizes");
  const char* err = nullptr;
  int* scratch = static_scratch_for_current_device(&err);
  if (!scratch) return fail(EISEN_ERR_CUDA, err);
  // same kernels as eisen_embedding_bwd; its first step clears count[0..vocab), the only part of
  // the scratch that has to start at zero (offset, rank and perm are fully rewritten)
  return eisen_embedding_bwd(stream, g, g_dt, ids, dw, scratch, n_ids, dim, vocab);
}
