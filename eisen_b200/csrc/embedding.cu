// Embedding row gather and its backward scatter-add (src/graph/ops/transform.rs:287-324;
// kernels/ops_f32.cu:513-537 scatter with one atomicAdd per element).
//
// Token ids are int32 on the device (the reference keeps them as f32 and, in bf16 mode, rounds
// them through bf16).  The backward is deterministic and free of floating-point atomics:
//   1. count[v]  = occurrences of id v                                       (integer atomics)
//   2. offset[v] = exclusive prefix sum of count; cursor = offset            (one CTA)
//   3. slot[cursor[ids[i]]++] = i     -> positions grouped by id, in arrival order
//   4. perm[offset[id] + #{slots of the same id holding a smaller position}] = position
//      -> positions grouped by id, in position order: whatever order step 3 ran in, the
//      result is the stable sort of the ids
//   5. one warp per vocabulary row sums its positions' gradient rows in that fixed order and
//      adds the sum to the f32 weight gradient.
// Steps 1-4 are exact integer bookkeeping; their cost is O(n + vocab + sum of count^2).
#include <algorithm>
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

__global__ void __launch_bounds__(256)
count_kernel(const int* __restrict__ ids, int* __restrict__ count, int n, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id >= 0 && id < vocab) atomicAdd(&count[id], 1);
}

// exclusive scan of count[0..vocab): CTA b owns entries [4096 b, 4096 (b + 1)), four per thread as
// one 16-byte vector.  It first adds up everything before its chunk itself (coalesced, from L2),
// which keeps the scan a single launch without a cross-CTA handshake.  The arrays are 16-byte
// aligned and padded to a multiple of four entries; the padding of count is zero.
constexpr int SCAN_CHUNK = 4096;
__global__ void __launch_bounds__(1024)
scan_kernel(const int* __restrict__ count, int* __restrict__ offset, int* __restrict__ cursor, int vocab_pad) {
  __shared__ int warp_tot[32], warp_pre[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int base = blockIdx.x * SCAN_CHUNK;
  int pre = 0;
  for (int i = threadIdx.x * 4; i < base; i += SCAN_CHUNK) {
    const int4 c = *reinterpret_cast<const int4*>(count + i);
    pre += c.x + c.y + c.z + c.w;
  }
  const int idx0 = base + threadIdx.x * 4;
  int4 v = make_int4(0, 0, 0, 0);
  if (idx0 < vocab_pad) v = *reinterpret_cast<const int4*>(count + idx0);
  const int tsum = v.x + v.y + v.z + v.w;
  int inc = tsum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) pre += __shfl_xor_sync(0xffffffffu, pre, o);
  if (lane == 31) warp_tot[warp] = inc;
  if (lane == 0) warp_pre[warp] = pre;
  __syncthreads();
  int before = 0;  // entries before the chunk + this chunk's earlier warps
#pragma unroll
  for (int wq = 0; wq < 32; ++wq) before += warp_pre[wq] + (wq < warp ? warp_tot[wq] : 0);
  if (idx0 < vocab_pad) {
    int4 o;
    o.x = before + inc - tsum;
    o.y = o.x + v.x;
    o.z = o.y + v.y;
    o.w = o.z + v.z;
    *reinterpret_cast<int4*>(offset + idx0) = o;
    *reinterpret_cast<int4*>(cursor + idx0) = o;
  }
}

__global__ void __launch_bounds__(256)
place_kernel(const int* __restrict__ ids, int* __restrict__ cursor, int* __restrict__ slot, int n, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  if (id < 0 || id >= vocab) return;
  slot[atomicAdd(&cursor[id], 1)] = i;
}

// perm = slot with every id's segment put into increasing position order; active = the ids that
// occur, each with its first position.  One thread per slot
// counts the smaller positions of its segment (a warp mostly reads the same segment: broadcast).
__global__ void __launch_bounds__(128)
order_kernel(const int* __restrict__ ids, const int* __restrict__ slot, const int* __restrict__ offset,
             const int* __restrict__ count, int* __restrict__ perm, int2* __restrict__ active,
             int* __restrict__ n_active, int n_valid_max, int vocab) {
  const int sidx = blockIdx.x * blockDim.x + threadIdx.x;
  if (sidx >= n_valid_max) return;
  // slots past the number of valid ids were never written; offset[vocab-1] + count[vocab-1] bounds them
  if (sidx >= offset[vocab - 1] + count[vocab - 1]) return;
  const int pos = slot[sidx];
  const int id = ids[pos];
  const int off = offset[id], cnt = count[id];
  int r = 0;
  if (cnt > 1) {
    for (int k = 0; k < cnt; ++k) r += (slot[off + k] < pos);
  }
  perm[off + r] = pos;
  // the first position of every id also enters the list of rows that receive a gradient (in any
  // order: rows are independent of each other)
  if (r == 0) active[atomicAdd(n_active, 1)] = make_int2(id, pos);
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

// the same for rows of whole 16-byte vectors.  A warp's work item is one row of the active list
// times one part of 32*SW vectors of its columns (parts of a row go to neighbouring warps); a lane
// owns SW vectors, whose first gradient reads and dW reads are all issued before the first use,
// and the next item's list entry is read ahead.
template <typename TG, int SW>
__global__ void __launch_bounds__(256, SW == 1 ? 6 : 4)
scatter_rows_vec_kernel(const TG* __restrict__ g, const int* __restrict__ perm, const int* __restrict__ offset,
                        const int* __restrict__ count, const int2* __restrict__ active,
                        const int* __restrict__ n_active, float* __restrict__ dw, int dim, int parts) {
  constexpr int V = VecOf<TG>::N;
  const int lane = threadIdx.x & 31;
  const int warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int wstride = gridDim.x * (blockDim.x >> 5);
  const long long items = (long long)(*n_active) * parts;
  if (warp0 >= items) return;
  int2 ent = active[warp0 / parts];
  for (long long it = warp0; it < items; it += wstride) {
    const int v = ent.x, pos0 = ent.y;
    const int c0 = (int)(it % parts) * (32 * SW * V);
    if (it + wstride < items) ent = active[(it + wstride) / parts];
    const int cnt = count[v];
    float* drow = dw + (long long)v * dim;
    float a[SW][V], old[SW][V];
    {
      const TG* grow = g + (long long)pos0 * dim;
#pragma unroll
      for (int j = 0; j < SW; ++j) {
        const int c = c0 + (j * 32 + lane) * V;
        if (c < dim) {
          ld16(grow + c, a[j]);
#pragma unroll
          for (int e = 0; e < V; e += 4) {
            const float4 o = *reinterpret_cast<const float4*>(drow + c + e);
            old[j][e] = o.x; old[j][e + 1] = o.y; old[j][e + 2] = o.z; old[j][e + 3] = o.w;
          }
        }
      }
    }
    if (cnt > 1) {
      const int off = offset[v];
      for (int k = 1; k < cnt; ++k) {
        const TG* grow = g + (long long)perm[off + k] * dim;
#pragma unroll
        for (int j = 0; j < SW; ++j) {
          const int c = c0 + (j * 32 + lane) * V;
          if (c < dim) {
            float t[V];
            ld16(grow + c, t);
#pragma unroll
            for (int e = 0; e < V; ++e) a[j][e] += t[e];
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < SW; ++j) {
      const int c = c0 + (j * 32 + lane) * V;
      if (c < dim) {
#pragma unroll
        for (int e = 0; e < V; e += 4)
          *reinterpret_cast<float4*>(drow + c + e) =
              make_float4(old[j][e] + a[j][e], old[j][e + 1] + a[j][e + 1], old[j][e + 2] + a[j][e + 2],
                          old[j][e + 3] + a[j][e + 3]);
      }
    }
  }
}

struct EmbScratch {
  int *count, *n_active, *offset, *cursor, *slot, *perm;
  int2* active;
  long long vocab_pad;
};
inline EmbScratch emb_scratch(void* workspace, long long n_ids, long long vocab) {
  EmbScratch e;
  e.vocab_pad = (vocab + 3) / 4 * 4;
  e.count = (int*)workspace;
  e.n_active = e.count + e.vocab_pad;  // cleared together with count
  e.offset = e.n_active + 4;
  e.cursor = e.offset + e.vocab_pad;
  e.slot = e.cursor + e.vocab_pad;
  e.perm = e.slot + n_ids;
  // int offset 3 * vocab_pad + 4 + 2 * n_ids is even for every n_ids: int2 stores stay 8-byte aligned
  e.active = reinterpret_cast<int2*>(e.perm + n_ids);
  return e;
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

// scratch (int32): count, offset, cursor (vocab rounded up to a multiple of 4 each), the number of
// active rows, slot[n_ids], perm[n_ids], active[n_ids] (id, first position); the workspace must be
// 16-byte aligned
long long eisen_embedding_bwd_workspace_bytes(long long n_ids, long long vocab) {
  return (3 * ((vocab + 3) / 4 * 4) + 4 + 4 * n_ids + 1) * 4 + 64;
}

static int embedding_check(const char* who, const void* workspace, long long n_ids, long long vocab) {
  (void)who;
  if (n_ids > 0x7fffffffLL || vocab > 0x7fffffffLL / 4) return fail(EISEN_ERR_LIMIT, "embedding_bwd: more than 2^31 ids or 2^29 rows");
  if (vocab <= 0) return fail(EISEN_ERR_INVALID, "embedding_bwd: empty table");
  if (!workspace) return fail(EISEN_ERR_INVALID, "embedding_bwd: workspace is null");
  if (!aligned16(workspace)) return fail(EISEN_ERR_INVALID, "embedding_bwd: workspace is not 16-byte aligned");
  return 0;
}

// The integer bookkeeping of the scatter (depends on the ids only): groups the positions by id.
int eisen_embedding_bwd_plan(void* stream, const int* ids, void* workspace, long long n_ids, long long vocab) {
  if (n_ids <= 0) return 0;
  if (int rc = embedding_check("plan", workspace, n_ids, vocab)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const EmbScratch e = emb_scratch(workspace, n_ids, vocab);
  if (cudaMemsetAsync(e.count, 0, (size_t)(e.vocab_pad + 4) * 4, s) != cudaSuccess) return fail(EISEN_ERR_CUDA, "embedding_bwd: memset failed");
  const int n = (int)n_ids;
  count_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, e.count, n, (int)vocab);
  scan_kernel<<<(unsigned)((e.vocab_pad + SCAN_CHUNK - 1) / SCAN_CHUNK), 1024, 0, s>>>(e.count, e.offset, e.cursor, (int)e.vocab_pad);
  place_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, e.cursor, e.slot, n, (int)vocab);
  order_kernel<<<(n + 127) / 128, 128, 0, s>>>(ids, e.slot, e.offset, e.count, e.perm, e.active, e.n_active, n, (int)vocab);
  return check_launch("embedding_bwd_plan");
}

// dW[ids[i],:] += g[i,:] with the grouping that eisen_embedding_bwd_plan left in the workspace.
int eisen_embedding_bwd_apply(void* stream, const void* g, int g_dt, float* dw, const void* workspace,
                              long long n_ids, long long dim, long long vocab) {
  if (n_ids <= 0) return 0;
  if (int rc = embedding_check("apply", workspace, n_ids, vocab)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const EmbScratch e = emb_scratch(const_cast<void*>(workspace), n_ids, vocab);
  const bool vec = aligned16(g) && aligned16(dw) && dim % 8 == 0;
  if (g_dt == DT_F32) {
    if (vec) {
      const int parts = (int)((dim + 32 * 4 - 1) / (32 * 4));
      scatter_rows_vec_kernel<float, 1><<<grid_for(std::min(n_ids, vocab) * parts, 8, 6), 256, 0, s>>>((const float*)g, e.perm, e.offset, e.count, e.active, e.n_active, dw, (int)dim, parts);
    } else {
      scatter_rows_kernel<float><<<grid_for(vocab, 8, 8), 256, 0, s>>>((const float*)g, e.perm, e.offset, e.count, dw, (int)vocab, (int)dim);
    }
  } else {
    if (vec) {
      const int parts = (int)((dim + 32 * 8 - 1) / (32 * 8));
      scatter_rows_vec_kernel<__nv_bfloat16, 1><<<grid_for(std::min(n_ids, vocab) * parts, 8, 6), 256, 0, s>>>((const __nv_bfloat16*)g, e.perm, e.offset, e.count, e.active, e.n_active, dw, (int)dim, parts);
    } else {
      scatter_rows_kernel<__nv_bfloat16><<<grid_for(vocab, 8, 8), 256, 0, s>>>((const __nv_bfloat16*)g, e.perm, e.offset, e.count, dw, (int)vocab, (int)dim);
    }
  }
  return check_launch("embedding_bwd_apply");
}

// dW[ids[i],:] += g[i,:] for all i, deterministically: plan + apply.
int eisen_embedding_bwd(void* stream, const void* g, int g_dt, const int* ids, float* dw, void* workspace,
                        long long n_ids, long long dim, long long vocab) {
  if (int rc = eisen_embedding_bwd_plan(stream, ids, workspace, n_ids, vocab)) return rc;
  return eisen_embedding_bwd_apply(stream, g, g_dt, dw, workspace, n_ids, dim, vocab);
}

// copies the grouping computed by the last eisen_embedding_bwd on this workspace:
// perm[n_ids] (positions grouped by id), offset[vocab], count[vocab]
int eisen_embedding_bwd_bookkeeping(void* stream, const void* workspace, long long n_ids, long long vocab,
                                    int* count_out, int* offset_out, int* perm_out) {
  cudaStream_t s = (cudaStream_t)stream;
  const EmbScratch e = emb_scratch(const_cast<void*>(workspace), n_ids, vocab);
  const int *count = e.count, *offset = e.offset, *perm = e.perm;
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
// device.  For them the integer bookkeeping of the scatter (count, offset, cursor, slot, perm, active) lives in
// a fixed array inside the library image instead of a caller-provided workspace.
//
// The array is part of the module: every GPU that loads the library holds
// (3 * 131072 + 4 * 65536 + 8) * 4 bytes = 2.5 MB of it until the process exits.
// ---------------------------------------------------------------------------------------
namespace {
constexpr long long kStaticMaxIds = 65536;     // token positions per call
constexpr long long kStaticMaxVocab = 131072;  // rows of the embedding table
static __device__ __align__(256) int g_embedding_static_scratch[3 * kStaticMaxVocab + 4 * kStaticMaxIds + 8];

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
  // the scratch that has to start at zero (offset, cursor, slot and perm are rewritten where read)
  return eisen_embedding_bwd(stream, g, g_dt, ids, dw, scratch, n_ids, dim, vocab);
}
