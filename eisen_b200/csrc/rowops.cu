// Row-wise kernels: RMSNorm forward / backward, softmax forward / backward, fused
// softmax-cross-entropy forward (loss + log-sum-exp) and backward (dlogits in one pass).
// One warp (RMSNorm) or one CTA (softmax, cross-entropy) per row, 16-byte accesses, shuffle
// reductions; the reference runs one THREAD per row (kernels/ops_f32.cu:539-578 rmsnorm,
// 580-646 cross-entropy and softmax, 5-64 masked cross-entropy).
#include "common.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

// ---------------------------------------------------------------------------------------
// RMSNorm.  y = x * rrms * w,  rrms = 1/sqrt(mean(x^2) + eps)   (src/graph/ops/normalization.rs:141-152)
// ---------------------------------------------------------------------------------------
constexpr int RN_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(RN_WARPS * 32)
rmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                   float* __restrict__ rrms_out, long long rows, int dim, float eps) {
  constexpr int V = VecOf<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5);
  const long long wstride = (long long)gridDim.x * RN_WARPS;
  const bool vec = (dim % V) == 0;
  for (long long row = warp0; row < rows; row += wstride) {
    const T* xr = x + row * dim;
    T* yr = y + row * dim;
    float ss = 0.0f;
    if (vec) {
      for (int c = lane * V; c < dim; c += 32 * V) {
        float v[V];
        ld16(xr + c, v);
#pragma unroll
        for (int k = 0; k < V; ++k) ss += v[k] * v[k];
      }
    } else {
      for (int c = lane; c < dim; c += 32) { float v = to_f32(xr[c]); ss += v * v; }
    }
    ss = warp_sum(ss);
    const float rrms = 1.0f / sqrtf(ss / (float)dim + eps);
    if (rrms_out && lane == 0) rrms_out[row] = rrms;
    if (vec) {
      for (int c = lane * V; c < dim; c += 32 * V) {
        float v[V], wv[V];
        ld16(xr + c, v);
#pragma unroll
        for (int k = 0; k < V; k += 4) {
          const float4 t = *reinterpret_cast<const float4*>(w + c + k);
          wv[k] = t.x; wv[k + 1] = t.y; wv[k + 2] = t.z; wv[k + 3] = t.w;
        }
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] = v[k] * rrms * wv[k];
        st16(yr + c, v);
      }
    } else {
      for (int c = lane; c < dim; c += 32) yr[c] = from_f32<T>(to_f32(xr[c]) * rrms * w[c]);
    }
  }
}

// Backward (src/graph/ops/normalization.rs:155-173):
//   gdxw = sum_d dy*x*w ; dx (+)= rrms*dy*w - x*rrms^3/dim*gdxw ; dw[d] += dy*x*rrms
// Each warp walks rows; every lane keeps the dw partial of the columns it owns in registers
// (NCH chunks of V columns), the CTA folds its warps through shared memory and writes one row of
// `dw_partial` [gridDim.x, dim]; a second kernel sums the partials in a fixed order (no atomics,
// run-to-run deterministic).
template <typename T, int NCH>
__global__ void __launch_bounds__(RN_WARPS * 32)
rmsnorm_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const T* __restrict__ dy,
                   T* __restrict__ dx, float* __restrict__ dw_partial, long long rows, int dim, float eps,
                   int acc_dx) {
  constexpr int V = VecOf<T>::N;
  extern __shared__ float sh_dw[];  // [RN_WARPS][dim]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * RN_WARPS + warp;
  const long long wstride = (long long)gridDim.x * RN_WARPS;
  float dwp[NCH][V], wv[NCH][V];  // a lane owns the same columns for every row: weights stay in registers
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (j * 32 + lane) * V;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      dwp[j][k] = 0.0f;
      wv[j][k] = (c < dim) ? w[c + k] : 0.0f;
    }
  }

  for (long long row = warp0; row < rows; row += wstride) {
    const T* xr = x + row * dim;
    const T* gr = dy + row * dim;
    T* dr = dx + row * dim;
    float xv[NCH][V], gv[NCH][V];
    float ss = 0.0f, gdxw = 0.0f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = (j * 32 + lane) * V;
      if (c < dim) {
        ld16(xr + c, xv[j]);
        ld16(gr + c, gv[j]);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          ss += xv[j][k] * xv[j][k];
          gdxw += gv[j][k] * xv[j][k] * wv[j][k];
        }
      }
    }
    ss = warp_sum(ss);
    gdxw = warp_sum(gdxw);
    const float rrms = 1.0f / sqrtf(ss / (float)dim + eps);
    const float rrc_d = (rrms * rrms * rrms) / (float)dim;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = (j * 32 + lane) * V;
      if (c < dim) {
        float o[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
          o[k] = rrms * (gv[j][k] * wv[j][k]) - xv[j][k] * rrc_d * gdxw;
          dwp[j][k] += gv[j][k] * xv[j][k] * rrms;
        }
        if (acc_dx) {
          float old[V];
          ld16(dr + c, old);
#pragma unroll
          for (int k = 0; k < V; ++k) o[k] += old[k];
        }
        st16(dr + c, o);
      }
    }
  }
  // fold the warps of this CTA
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (j * 32 + lane) * V;
    if (c < dim) {
#pragma unroll
      for (int k = 0; k < V; ++k) sh_dw[warp * dim + c + k] = dwp[j][k];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < dim; c += blockDim.x) {
    float s = 0.0f;
#pragma unroll
    for (int wq = 0; wq < RN_WARPS; ++wq) s += sh_dw[wq * dim + c];
    dw_partial[(long long)blockIdx.x * dim + c] = s;
  }
}

// generic fallback for dims that are not a multiple of the vector width or exceed the register
// budget: one warp per row, dw through f32 atomics
template <typename T>
__global__ void rmsnorm_bwd_generic_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                           const T* __restrict__ dy, T* __restrict__ dx,
                                           float* __restrict__ dw, long long rows, int dim, float eps,
                                           int acc_dx) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long wstride = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long row = warp0; row < rows; row += wstride) {
    const T* xr = x + row * dim;
    const T* gr = dy + row * dim;
    T* dr = dx + row * dim;
    float ss = 0.0f, gdxw = 0.0f;
    for (int c = lane; c < dim; c += 32) {
      float xv = to_f32(xr[c]), gv = to_f32(gr[c]);
      ss += xv * xv;
      gdxw += gv * xv * w[c];
    }
    ss = warp_sum(ss);
    gdxw = warp_sum(gdxw);
    const float rrms = 1.0f / sqrtf(ss / (float)dim + eps);
    const float rrc_d = (rrms * rrms * rrms) / (float)dim;
    for (int c = lane; c < dim; c += 32) {
      float xv = to_f32(xr[c]), gv = to_f32(gr[c]);
      float o = rrms * (gv * w[c]) - xv * rrc_d * gdxw;
      if (acc_dx) o += to_f32(dr[c]);
      dr[c] = from_f32<T>(o);
      atomicAdd(dw + c, gv * xv * rrms);
    }
  }
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                       int nparts, int dim) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= dim) return;
  float s = 0.0f;
  for (int p = 0; p < nparts; ++p) s += partial[(long long)p * dim + c];
  out[c] += s;
}

// ---------------------------------------------------------------------------------------
// softmax over the last dim (src/graph/ops/reduction.rs:476-524): one CTA per row
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int n) {
  __shared__ float sh[32];
  const T* xr = x + (long long)blockIdx.x * n;
  T* yr = y + (long long)blockIdx.x * n;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < n; c += blockDim.x) mx = fmaxf(mx, to_f32(xr[c]));
  mx = block_max(mx, sh);
  float s = 0.0f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) s += expf(to_f32(xr[c]) - mx);
  s = block_sum(s, sh);
  for (int c = threadIdx.x; c < n; c += blockDim.x) yr[c] = from_f32<T>(expf(to_f32(xr[c]) - mx) / s);
}
// dx (+)= y * (dy - sum(dy*y))
template <typename T>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                                          T* __restrict__ dx, int n, int acc) {
  __shared__ float sh[32];
  const long long off = (long long)blockIdx.x * n;
  float dot = 0.0f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) dot += to_f32(dy[off + c]) * to_f32(y[off + c]);
  dot = block_sum(dot, sh);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float v = to_f32(y[off + c]) * (to_f32(dy[off + c]) - dot);
    if (acc) v += to_f32(dx[off + c]);
    dx[off + c] = from_f32<T>(v);
  }
}

// ---------------------------------------------------------------------------------------
// fused softmax-cross-entropy (src/graph/ops/reduction.rs:668-717, masked 888-942)
//   row loss = -ln(softmax(x)[t] + 1e-8) * normaliser      (the 1e-8 is not differentiated)
//   dlogits  = (softmax(x) - onehot(t)) * scale            (rows with t == ignore_index: 0)
// Forward: one CTA per row, one pass with an online max / sum, writes the row loss and the
// log-sum-exp.  A second single-CTA kernel adds the row losses in a fixed order.
// ---------------------------------------------------------------------------------------
constexpr int CE_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const T* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ row_loss,
              float* __restrict__ lse, int V_, int ignore_index, float normalizer) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int t = targets[row];
  if (t == ignore_index) {
    if (threadIdx.x == 0) { row_loss[row] = 0.0f; lse[row] = 0.0f; }
    return;
  }
  const T* xr = logits + row * V_;
  float m = -INFINITY, s = 0.0f;
  if ((V_ % V) == 0 && aligned_row(xr)) {
    for (int c = threadIdx.x * V; c < V_; c += CE_THREADS * V) {
      float v[V];
      ld16(xr + c, v);
      float cm = v[0];
#pragma unroll
      for (int k = 1; k < V; ++k) cm = fmaxf(cm, v[k]);
      if (cm > m) { s *= expf(m - cm); m = cm; }
#pragma unroll
      for (int k = 0; k < V; ++k) s += expf(v[k] - m);
    }
  } else {
    for (int c = threadIdx.x; c < V_; c += CE_THREADS) {
      float v = to_f32(xr[c]);
      if (v > m) { s *= expf(m - v); m = v; }
      s += expf(v - m);
    }
  }
  const float gm = block_max(m, sh);
  s = (m == -INFINITY) ? 0.0f : s * expf(m - gm);
  s = block_sum(s, sh);
  if (threadIdx.x == 0) {
    const float p = expf(to_f32(xr[t]) - gm) / s;
    row_loss[row] = -logf(p + 1e-8f) * normalizer;
    lse[row] = gm + logf(s);
  }
}

__global__ void __launch_bounds__(1024) ce_loss_reduce_kernel(const float* __restrict__ row_loss,
                                                              float* __restrict__ loss, long long rows) {
  __shared__ float sh[32];
  float s = 0.0f;
  for (long long r = threadIdx.x; r < rows; r += blockDim.x) s += row_loss[r];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) *loss = s;
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(const T* __restrict__ logits, const int* __restrict__ targets, const float* __restrict__ lse,
              T* __restrict__ dlogits, const float* __restrict__ grad_out, int V_, int ignore_index,
              float normalizer, int acc) {
  constexpr int V = VecOf<T>::N;
  const long long row = blockIdx.x;
  const int t = targets[row];
  const T* xr = logits + row * V_;
  T* dr = dlogits + row * V_;
  const bool vec = (V_ % V) == 0 && aligned_row(xr) && aligned_row(dr);
  if (t == ignore_index) {
    if (acc) return;
    if (vec) {
      float z[V];
#pragma unroll
      for (int k = 0; k < V; ++k) z[k] = 0.0f;
      for (int c = threadIdx.x * V; c < V_; c += CE_THREADS * V) st16(dr + c, z);
    } else {
      for (int c = threadIdx.x; c < V_; c += CE_THREADS) dr[c] = from_f32<T>(0.0f);
    }
    return;
  }
  const float l = lse[row];
  const float scale = normalizer * (grad_out ? *grad_out : 1.0f);
  if (vec) {
    for (int c = threadIdx.x * V; c < V_; c += CE_THREADS * V) {
      float v[V];
      ld16(xr + c, v);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float g = expf(v[k] - l);
        if (c + k == t) g -= 1.0f;
        v[k] = g * scale;
      }
      if (acc) {
        float o[V];
        ld16(dr + c, o);
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] += o[k];
      }
      st16(dr + c, v);
    }
  } else {
    for (int c = threadIdx.x; c < V_; c += CE_THREADS) {
      float g = expf(to_f32(xr[c]) - l);
      if (c == t) g -= 1.0f;
      g *= scale;
      if (acc) g += to_f32(dr[c]);
      dr[c] = from_f32<T>(g);
    }
  }
}

template <typename T, int NCH>
int launch_rmsnorm_bwd(cudaStream_t s, const T* x, const float* w, const T* dy, T* dx, float* dw,
                       float* ws, long long rows, int dim, float eps, int acc_dx) {
  int grid = grid_for(rows, RN_WARPS, 2);
  const size_t smem = (size_t)RN_WARPS * dim * 4;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_bwd_kernel<T, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(EISEN_ERR_CUDA, cudaGetErrorString(e));
  }
  rmsnorm_bwd_kernel<T, NCH><<<grid, RN_WARPS * 32, smem, s>>>(x, w, dy, dx, ws, rows, dim, eps, acc_dx);
  int rc = check_launch("rmsnorm_bwd");
  if (rc) return rc;
  reduce_partials_kernel<<<(dim + 255) / 256, 256, 0, s>>>(ws, dw, grid, dim);
  return check_launch("rmsnorm_bwd_reduce");
}

template <typename T>
int rmsnorm_bwd_dispatch(cudaStream_t s, const T* x, const float* w, const T* dy, T* dx, float* dw, float* ws,
                         long long rows, int dim, float eps, int acc_dx) {
  constexpr int V = VecOf<T>::N;
  const bool fast = (dim % V) == 0 && dim <= 16 * 32 * V && ((long long)RN_WARPS * dim * 4) <= 200 * 1024 &&
                    aligned16(x) && aligned16(dy) && aligned16(dx) && ws != nullptr;
  if (!fast) {
    const int grid = grid_for(rows, 8, 4);
    rmsnorm_bwd_generic_kernel<T><<<grid, 256, 0, s>>>(x, w, dy, dx, dw, rows, dim, eps, acc_dx);
    return check_launch("rmsnorm_bwd_generic");
  }
  const int nch = (dim + 32 * V - 1) / (32 * V);
  if (nch <= 1) return launch_rmsnorm_bwd<T, 1>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
  if (nch <= 2) return launch_rmsnorm_bwd<T, 2>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
  if (nch <= 4) return launch_rmsnorm_bwd<T, 4>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
  if (nch <= 8) return launch_rmsnorm_bwd<T, 8>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
  return launch_rmsnorm_bwd<T, 16>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
}

}  // namespace
}  // namespace eisen

using namespace eisen;

extern "C" {

int eisen_rmsnorm_fwd(void* stream, const void* x, const float* w, void* y, float* rrms_out, long long rows,
                      long long dim, float eps, int dt) {
  if (rows <= 0) return 0;
  if (!aligned16(x) || !aligned16(y)) return fail(EISEN_ERR_INVALID, "rmsnorm_fwd: unaligned pointer");
  const int grid = grid_for(rows, RN_WARPS, 8);
  EISEN_DISPATCH_DTYPE(dt, T, {
    rmsnorm_fwd_kernel<T><<<grid, RN_WARPS * 32, 0, (cudaStream_t)stream>>>((const T*)x, w, (T*)y, rrms_out,
                                                                          rows, (int)dim, eps);
    return check_launch("rmsnorm_fwd");
  });
}

long long eisen_rmsnorm_bwd_workspace_bytes(long long rows, long long dim) {
  (void)rows;
  return (long long)sm_count() * 2 * dim * 4;
}


// dw (f32, [dim]) is accumulated into; dx is written or accumulated into (acc_dx).
// `workspace` holds eisen_rmsnorm_bwd_workspace_bytes(rows, dim) bytes of scratch.
int eisen_rmsnorm_bwd(void* stream, const void* x, const float* w, const void* dy, void* dx, float* dw,
                      void* workspace, long long rows, long long dim, float eps, int dt, int acc_dx) {
  if (rows <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dt == DT_F32)
    return rmsnorm_bwd_dispatch<float>(s, (const float*)x, w, (const float*)dy, (float*)dx, dw, (float*)workspace,
                                       rows, (int)dim, eps, acc_dx);
  return rmsnorm_bwd_dispatch<__nv_bfloat16>(s, (const __nv_bfloat16*)x, w, (const __nv_bfloat16*)dy,
                                             (__nv_bfloat16*)dx, dw, (float*)workspace, rows, (int)dim, eps, acc_dx);
}

int eisen_softmax_fwd(void* stream, const void* x, void* y, long long rows, long long n, int dt) {
  if (rows <= 0) return 0;
  EISEN_DISPATCH_DTYPE(dt, T, {
    softmax_fwd_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>((const T*)x, (T*)y, (int)n);
    return check_launch("softmax_fwd");
  });
}
int eisen_softmax_bwd(void* stream, const void* y, const void* dy, void* dx, long long rows, long long n, int dt,
                      int accumulate) {
  if (rows <= 0) return 0;
  EISEN_DISPATCH_DTYPE(dt, T, {
    softmax_bwd_kernel<T><<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>((const T*)y, (const T*)dy, (T*)dx, (int)n, accumulate);
    return check_launch("softmax_bwd");
  });
}

// row_loss [rows] and lse [rows] are outputs kept for the backward pass; *loss = sum(row_loss).
int eisen_ce_fwd(void* stream, const void* logits, const int* targets, float* loss, float* row_loss, float* lse,
                 long long rows, long long vocab, int ignore_index, float normalizer, int dt) {
  if (rows <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  EISEN_DISPATCH_DTYPE(dt, T, {
    ce_fwd_kernel<T><<<(unsigned)rows, CE_THREADS, 0, s>>>((const T*)logits, targets, row_loss, lse, (int)vocab,
                                                          ignore_index, normalizer);
    int rc = check_launch("ce_fwd");
    if (rc) return rc;
    ce_loss_reduce_kernel<<<1, 1024, 0, s>>>(row_loss, loss, rows);
    return check_launch("ce_loss_reduce");
  });
}

// dlogits may alias logits (in place).  grad_out: device scalar (the loss gradient) or null for 1.
int eisen_ce_bwd(void* stream, const void* logits, const int* targets, const float* lse, void* dlogits,
                 const float* grad_out, long long rows, long long vocab, int ignore_index, float normalizer,
                 int dt, int accumulate) {
  if (rows <= 0) return 0;
  EISEN_DISPATCH_DTYPE(dt, T, {
    ce_bwd_kernel<T><<<(unsigned)rows, CE_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)logits, targets, lse, (T*)dlogits, grad_out, (int)vocab, ignore_index, normalizer, accumulate);
    return check_launch("ce_bwd");
  });
}

}  // extern "C"
