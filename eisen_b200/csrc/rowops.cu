// Row-wise kernels: RMSNorm forward / backward, softmax forward / backward, fused
// softmax-cross-entropy forward (loss + log-sum-exp) and backward (dlogits in one pass).
// One warp (RMSNorm) or one CTA (softmax, cross-entropy) per row, 16-byte accesses, shuffle
// reductions; the reference runs one THREAD per row (kernels/ops_f32.cu:539-578 rmsnorm,
// 580-646 cross-entropy and softmax, 5-64 masked cross-entropy).
#include <algorithm>

#include "common.cuh"
#include "ptx.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

// ---------------------------------------------------------------------------------------
// RMSNorm.  y = x * rrms * w,  rrms = 1/sqrt(mean(x^2) + eps)   (src/graph/ops/normalization.rs:141-152)
// ---------------------------------------------------------------------------------------
constexpr int RN_WARPS = 8;

__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[4]) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}
__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[8]) {
  const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(u[i] << 16);          // low half = even element
    v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack16(const float (&v)[4]) {
  return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
__device__ __forceinline__ uint4 pack16(const float (&v)[8]) {
  uint32_t u[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);  // .x = low half = even element
    u[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(u[0], u[1], u[2], u[3]);
}

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

// Forward for rows that fit in registers: a warp owns a row, each lane keeps its NCH 16-byte
// vectors packed, so x is read from memory once.
template <typename T, int NCH>
__global__ void __launch_bounds__(RN_WARPS * 32)
rmsnorm_fwd_reg_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                       float* __restrict__ rrms_out, long long rows, int dim, float eps) {
  constexpr int V = VecOf<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5);
  const long long wstride = (long long)gridDim.x * RN_WARPS;
  // the next row of this warp is requested before the current one is reduced and written
  uint4 raw[NCH], nxt[NCH];
  auto load_row = [&](long long row, uint4 (&dst)[NCH]) {
    const T* xr = x + row * dim;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = (j * 32 + lane) * V;
      dst[j] = (row < rows && c < dim) ? *reinterpret_cast<const uint4*>(xr + c) : make_uint4(0, 0, 0, 0);
    }
  };
  load_row(warp0, nxt);
  for (long long row = warp0; row < rows; row += wstride) {
    T* yr = y + row * dim;
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) raw[j] = nxt[j];
    load_row(row + wstride, nxt);
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float v[V];
      unpack16(raw[j], v);
#pragma unroll
      for (int k = 0; k < V; ++k) ss += v[k] * v[k];
    }
    ss = warp_sum(ss);
    const float rrms = 1.0f / sqrtf(ss / (float)dim + eps);
    if (rrms_out && lane == 0) rrms_out[row] = rrms;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = (j * 32 + lane) * V;
      if (c < dim) {
        float v[V], wv[V];
        unpack16(raw[j], v);
#pragma unroll
        for (int k = 0; k < V; k += 4) {
          const float4 t = *reinterpret_cast<const float4*>(w + c + k);
          wv[k] = t.x; wv[k + 1] = t.y; wv[k + 2] = t.z; wv[k + 3] = t.w;
        }
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] = v[k] * rrms * wv[k];
        st16(yr + c, v);
      }
    }
  }
}

template <typename T>
static void rmsnorm_fwd_dispatch(const T* x, const float* w, T* y, float* rrms_out, long long rows, int dim, float eps,
                                 int grid, cudaStream_t s) {
  constexpr int V = VecOf<T>::N;
  const int nch = (dim + 32 * V - 1) / (32 * V);
  if (dim % V == 0 && nch <= 16 && aligned16(w) && aligned16(x) && aligned16(y)) {
    if (nch <= 1) rmsnorm_fwd_reg_kernel<T, 1><<<grid, RN_WARPS * 32, 0, s>>>(x, w, y, rrms_out, rows, dim, eps);
    else if (nch <= 2) rmsnorm_fwd_reg_kernel<T, 2><<<grid, RN_WARPS * 32, 0, s>>>(x, w, y, rrms_out, rows, dim, eps);
    else if (nch <= 4) rmsnorm_fwd_reg_kernel<T, 4><<<grid, RN_WARPS * 32, 0, s>>>(x, w, y, rrms_out, rows, dim, eps);
    else if (nch <= 8) rmsnorm_fwd_reg_kernel<T, 8><<<grid, RN_WARPS * 32, 0, s>>>(x, w, y, rrms_out, rows, dim, eps);
    else rmsnorm_fwd_reg_kernel<T, 16><<<grid, RN_WARPS * 32, 0, s>>>(x, w, y, rrms_out, rows, dim, eps);
  } else {
    rmsnorm_fwd_kernel<T><<<grid, RN_WARPS * 32, 0, s>>>(x, w, y, rrms_out, rows, dim, eps);
  }
}

// Backward (src/graph/ops/normalization.rs:155-173):
//   gdxw = sum_d dy*x*w ; dx (+)= rrms*dy*w - x*rrms^3/dim*gdxw ; dw[d] += dy*x*rrms
// A CTA of 256 threads works on ROWS rows at a time; thread t owns the columns of vector
// t + 256*j (j < NCH) for every row, so its weights and its share of dw stay in registers for the
// whole kernel and dw needs no reduction inside the CTA.  The two row sums go through one
// shuffle + shared-memory exchange per group of ROWS rows.  Each CTA writes one row of
// `dw_partial` [gridDim.x, dim]; a second kernel adds the partials in a fixed order (no atomics,
// run-to-run deterministic).
// 16-byte read of data that is used once: no allocation in L1
template <typename T>
__device__ __forceinline__ uint4 ld_stream16(const T* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

#ifndef EISEN_RMS_BWD_PACKED
#define EISEN_RMS_BWD_PACKED 1
#endif
constexpr bool RMS_BWD_PACKED = EISEN_RMS_BWD_PACKED != 0;
constexpr int RB_THREADS = 256;
constexpr int RB_ROWS = 4;

// FULL: rows is a multiple of RB_ROWS and dim == NCH * RB_THREADS * V, so no element is masked.
template <typename T, int NCH, bool FULL>
__global__ void __launch_bounds__(RB_THREADS, (NCH * VecOf<T>::N <= 8) ? 2 : 1)
rmsnorm_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const T* __restrict__ dy,
                   T* __restrict__ dx, float* __restrict__ dw_partial, long long rows, int dim, float eps,
                   int acc_dx) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[2][RB_THREADS / 32][2 * RB_ROWS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wv[NCH][V], dwp[NCH][V];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * RB_THREADS) * V;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      dwp[j][k] = 0.0f;
      wv[j][k] = (FULL || c < dim) ? w[c + k] : 0.0f;
    }
  }
  int buf = 0;
  const long long groups = (rows + RB_ROWS - 1) / RB_ROWS;
  // the rows stay packed in registers (16 bytes per vector) and are widened where used; with one
  // vector per thread and row the next group's rows are requested before the current group is reduced,
  // so that the barrier below does not drain the memory pipeline
  constexpr bool PREFETCH = NCH == 1;
  uint4 xr[RB_ROWS][NCH], gr[RB_ROWS][NCH], xn[RB_ROWS][NCH], gn[RB_ROWS][NCH];
  auto load_group = [&](long long gi, uint4 (&xd)[RB_ROWS][NCH], uint4 (&gd)[RB_ROWS][NCH]) {
    const long long r0 = gi * RB_ROWS;
#pragma unroll
    for (int r = 0; r < RB_ROWS; ++r) {
      const bool ok = gi < groups && (FULL || r0 + r < rows);
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int c = (threadIdx.x + j * RB_THREADS) * V;
        if (ok && (FULL || c < dim)) {
          xd[r][j] = ld_stream16(x + (r0 + r) * dim + c);
          gd[r][j] = ld_stream16(dy + (r0 + r) * dim + c);
        } else {
          xd[r][j] = make_uint4(0, 0, 0, 0);
          gd[r][j] = make_uint4(0, 0, 0, 0);
        }
      }
    }
  };
  if (PREFETCH) load_group(blockIdx.x, xn, gn);
  for (long long gi = blockIdx.x; gi < groups; gi += gridDim.x) {
    const long long r0 = gi * RB_ROWS;
    float part[2 * RB_ROWS];
    if (PREFETCH) {
#pragma unroll
      for (int r = 0; r < RB_ROWS; ++r)
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          xr[r][j] = xn[r][j];
          gr[r][j] = gn[r][j];
        }
      load_group(gi + gridDim.x, xn, gn);
    } else {
      load_group(gi, xr, gr);
    }
#pragma unroll
    for (int r = 0; r < RB_ROWS; ++r) {
      float ss = 0.0f, gd = 0.0f, ss1 = 0.0f, gd1 = 0.0f;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        float xv[V], gv[V];
        unpack16(xr[r][j], xv);
        unpack16(gr[r][j], gv);
        if (RMS_BWD_PACKED) {
          // packed f32x2 arithmetic
#pragma unroll
          for (int k = 0; k < V; k += 2) {
            float t0, t1;
            ffma2(ss, ss1, xv[k], xv[k + 1], xv[k], xv[k + 1], ss, ss1);
            fmul2(t0, t1, gv[k], gv[k + 1], xv[k], xv[k + 1]);
            ffma2(gd, gd1, t0, t1, wv[j][k], wv[j][k + 1], gd, gd1);
          }
        } else {
#pragma unroll
          for (int k = 0; k < V; k += 2) {
            ss = fmaf(xv[k], xv[k], ss);
            ss1 = fmaf(xv[k + 1], xv[k + 1], ss1);
            gd = fmaf(gv[k] * wv[j][k], xv[k], gd);
            gd1 = fmaf(gv[k + 1] * wv[j][k + 1], xv[k + 1], gd1);
          }
        }
      }
      part[2 * r] = ss + ss1;
      part[2 * r + 1] = gd + gd1;
    }
    // eight sums over the warp in nine shuffles: each round halves the number of values a lane
    // carries; afterwards lane l holds the warp total of value ((l>>4)&1)*4 + ((l>>3)&1)*2 + ((l>>2)&1)
    static_assert(RB_ROWS == 4, "the reduction below is written for 8 values");
    float w4[4], w2[2], w1;
    {
      const bool hi = lane & 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float keep = hi ? part[i + 4] : part[i];
        const float give = hi ? part[i] : part[i + 4];
        w4[i] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
      }
      const bool h8 = lane & 8;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float keep = h8 ? w4[i + 2] : w4[i];
        const float give = h8 ? w4[i] : w4[i + 2];
        w2[i] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
      }
      const bool h4 = lane & 4;
      const float keep = h4 ? w2[1] : w2[0];
      const float give = h4 ? w2[0] : w2[1];
      w1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
    }
    const int vidx = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if ((lane & 3) == 0) sh[buf][warp][vidx] = w1;
    __syncthreads();
    {
      // lane l adds value (l & 7) over the warps of the CTA: even values are sums of squares, odd
      // ones the dy*x*w sums.  The lane pair of a row turns them into that row's two coefficients
      // (one square root per lane instead of one per row and thread); they go round by shuffle.
      float t = 0.0f;
#pragma unroll
      for (int wq = 0; wq < RB_THREADS / 32; ++wq) t += sh[buf][wq][lane & 7];
      const float other = __shfl_xor_sync(0xffffffffu, t, 1);
      const float ssv = (lane & 1) ? other : t;
      const float gdv = (lane & 1) ? t : other;
      const float rr = 1.0f / sqrtf(ssv / (float)dim + eps);
      const float coef = (rr * rr * rr) / (float)dim * gdv;
      const float mine = (lane & 1) ? coef : rr;
#pragma unroll
      for (int i = 0; i < 2 * RB_ROWS; ++i) part[i] = __shfl_sync(0xffffffffu, mine, i);
    }
    buf ^= 1;  // the other buffer is free: everyone passed the barrier of the group before
#pragma unroll
    for (int r = 0; r < RB_ROWS; ++r) {
      if (FULL || r0 + r < rows) {
        const float rrms = part[2 * r];
        const float coef = part[2 * r + 1];
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
          const int c = (threadIdx.x + j * RB_THREADS) * V;
          if (FULL || c < dim) {
            float xv[V], gv[V], o[V];
            unpack16(xr[r][j], xv);
            unpack16(gr[r][j], gv);
            const float ncoef = -coef;
            if (RMS_BWD_PACKED) {
#pragma unroll
              for (int k = 0; k < V; k += 2) {
                float a0, a1, b0, b1, t0, t1;
                fmul2(a0, a1, gv[k], gv[k + 1], wv[j][k], wv[j][k + 1]);
                fmul2(b0, b1, xv[k], xv[k + 1], ncoef, ncoef);
                ffma2(o[k], o[k + 1], a0, a1, rrms, rrms, b0, b1);
                fmul2(t0, t1, gv[k], gv[k + 1], xv[k], xv[k + 1]);
                ffma2(dwp[j][k], dwp[j][k + 1], t0, t1, rrms, rrms, dwp[j][k], dwp[j][k + 1]);
              }
            } else {
#pragma unroll
              for (int k = 0; k < V; ++k) {
                o[k] = fmaf(gv[k] * wv[j][k], rrms, xv[k] * ncoef);
                dwp[j][k] = fmaf(gv[k] * xv[k], rrms, dwp[j][k]);
              }
            }
            T* dr = dx + (r0 + r) * dim + c;
            if (acc_dx) {
              float old[V];
              ld16(dr, old);
#pragma unroll
              for (int k = 0; k < V; ++k) o[k] += old[k];
            }
            st16(dr, o);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (threadIdx.x + j * RB_THREADS) * V;
    if (FULL || c < dim) {
#pragma unroll
      for (int k = 0; k < V; ++k) dw_partial[(long long)blockIdx.x * dim + c + k] = dwp[j][k];
    }
  }
}


// Forward with the rows staged in shared memory by bulk asynchronous copies, the forward twin of
// rmsnorm_bwd_staged_kernel: a CTA of 256 threads takes ROWS rows per stage, thread t owns vector t
// of every row and keeps its weights in registers; the row sums of squares go through one
// shuffle reduction and one barrier per stage.  Needs dim == 256 vectors and rows % ROWS == 0.
template <typename T, int S, int CTAS>
__global__ void __launch_bounds__(RB_THREADS, CTAS)
rmsnorm_fwd_staged_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                          float* __restrict__ rrms_out, long long groups, float eps) {
  constexpr int V = VecOf<T>::N;
  constexpr int DIM = RB_THREADS * V;
  constexpr int ROWS = 4;
  constexpr uint32_t STAGE_BYTES = ROWS * DIM * sizeof(T);
  extern __shared__ __align__(128) uint8_t rs_smem[];
  __shared__ uint64_t full_bar[S];
  __shared__ float sh[2][RB_THREADS / 32][ROWS];
  __shared__ int abort_flag;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) mbar_init(&full_bar[i], 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  float wv[V];
#pragma unroll
  for (int k = 0; k < V; ++k) wv[k] = w[threadIdx.x * V + k];
  const long long g0 = blockIdx.x, gstride = gridDim.x;
  const long long n_mine = g0 < groups ? (groups - g0 + gstride - 1) / gstride : 0;
  auto issue = [&](long long k) {
    if (threadIdx.x == 0 && k < n_mine) {
      const int st = (int)(k % S);
      const long long r0 = (g0 + k * gstride) * ROWS;
      mbar_arrive_expect_tx(&full_bar[st], STAGE_BYTES);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(rs_smem + (size_t)st * STAGE_BYTES)), "l"(x + r0 * DIM), "r"(STAGE_BYTES),
                   "r"(smem_u32(&full_bar[st])) : "memory");
    }
  };
  for (int k = 0; k < S - 1; ++k) issue(k);
  int buf = 0;
  for (long long k = 0; k < n_mine; ++k) {
    const int st = (int)(k % S);
    const uint32_t ph = (uint32_t)((k / S) & 1);
    const long long r0 = (g0 + k * gstride) * ROWS;
    mbar_wait(&full_bar[st], ph, &abort_flag, nullptr, FAULT_WAIT_FULL);
    const T* sx = reinterpret_cast<const T*>(rs_smem + (size_t)st * STAGE_BYTES) + threadIdx.x * V;
    float xv[ROWS][V], part[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      ld16(sx + r * DIM, xv[r]);
      float a = 0.0f, b = 0.0f;
#pragma unroll
      for (int e = 0; e < V; e += 2) { a = fmaf(xv[r][e], xv[r][e], a); b = fmaf(xv[r][e + 1], xv[r][e + 1], b); }
      part[r] = a + b;
    }
    // four sums over the warp by recursive halving: lane l ends with the total of row ((l>>4)&1)*2 + ((l>>3)&1)
    float w2[2];
    const bool hi = lane & 16;
#pragma unroll
    for (int i = 0; i < 2; ++i) w2[i] = (hi ? part[i + 2] : part[i]) + __shfl_xor_sync(0xffffffffu, hi ? part[i] : part[i + 2], 16);
    const bool h8 = lane & 8;
    float w1 = (h8 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, h8 ? w2[0] : w2[1], 8);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 4);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
    if ((lane & 7) == 0) sh[buf][warp][((lane >> 4) & 1) * 2 + ((lane >> 3) & 1)] = w1;
    __syncthreads();
    issue(k + S - 1);  // its stage was last read before this barrier (the rows now sit in registers)
    float t = 0.0f;
#pragma unroll
    for (int wq = 0; wq < RB_THREADS / 32; ++wq) t += sh[buf][wq][lane & 3];
    const float rr = 1.0f / sqrtf(t / (float)DIM + eps);
    buf ^= 1;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float rrms = __shfl_sync(0xffffffffu, rr, r);
      if (rrms_out && threadIdx.x == 0) rrms_out[r0 + r] = rrms;
      float o[V];
#pragma unroll
      for (int e = 0; e < V; ++e) o[e] = xv[r][e] * rrms * wv[e];
      st16(y + (r0 + r) * DIM + threadIdx.x * V, o);
    }
  }
}

// Backward with the rows staged in shared memory by bulk asynchronous copies (one 1-D copy per
// tensor and group of ROWS rows, completion on an mbarrier): S stages per CTA are in flight instead
// of what fits the registers, and without row buffers in registers three or four CTAs fit an SM.
// Column ownership and the reduction of the two row sums are those of rmsnorm_bwd_kernel; the CTA's
// column sums of dw go to dw itself by vector reductions (dw_direct) or, for a fixed order, to
// dw_partial for reduce_partials_kernel.  A stage is refilled right after the barrier of the iteration that follows its
// last use, when every thread is known to be done with it.  Needs dim == 256 vectors and rows % ROWS == 0.
template <typename T, int ROWS, int S, int CTAS, bool PK = false>
__global__ void __launch_bounds__(RB_THREADS, CTAS)
rmsnorm_bwd_staged_kernel(const T* __restrict__ x, const float* __restrict__ w, const T* __restrict__ dy,
                          T* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ dw_direct,
                          long long groups, float eps, int acc_dx) {
  constexpr int V = VecOf<T>::N;
  constexpr int DIM = RB_THREADS * V;
  constexpr int NVAL = 2 * ROWS;
  constexpr uint32_t TENSOR_BYTES = ROWS * DIM * sizeof(T);
  static_assert(ROWS == 2 || ROWS == 4, "two or four rows per group");
  extern __shared__ __align__(128) uint8_t rs_smem[];
  __shared__ uint64_t full_bar[S];
  __shared__ float sh[2][RB_THREADS / 32][NVAL];
  __shared__ int abort_flag;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) mbar_init(&full_bar[i], 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  float wv[V], dwp[V];
#pragma unroll
  for (int k = 0; k < V; ++k) { wv[k] = w[threadIdx.x * V + k]; dwp[k] = 0.0f; }
  const long long g0 = blockIdx.x, gstride = gridDim.x;
  const long long n_mine = g0 < groups ? (groups - g0 + gstride - 1) / gstride : 0;
  auto issue = [&](long long k) {
    if (threadIdx.x == 0 && k < n_mine) {
      const int st = (int)(k % S);
      const long long r0 = (g0 + k * gstride) * ROWS;
      uint8_t* dst = rs_smem + (size_t)st * 2 * TENSOR_BYTES;
      mbar_arrive_expect_tx(&full_bar[st], 2 * TENSOR_BYTES);
      const uint32_t bar = smem_u32(&full_bar[st]);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(dst)), "l"(x + r0 * DIM), "r"(TENSOR_BYTES), "r"(bar) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(dst + TENSOR_BYTES)), "l"(dy + r0 * DIM), "r"(TENSOR_BYTES), "r"(bar) : "memory");
    }
  };
  for (int k = 0; k < S - 1; ++k) issue(k);
  int buf = 0;
  for (long long k = 0; k < n_mine; ++k) {
    const int st = (int)(k % S);
    const uint32_t ph = (uint32_t)((k / S) & 1);
    const long long r0 = (g0 + k * gstride) * ROWS;
    mbar_wait(&full_bar[st], ph, &abort_flag, nullptr, FAULT_WAIT_FULL);
    const T* sx = reinterpret_cast<const T*>(rs_smem + (size_t)st * 2 * TENSOR_BYTES) + threadIdx.x * V;
    const T* sg = sx + ROWS * DIM;
    float part[NVAL];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      float xv[V], gv[V];
      ld16(sx + r * DIM, xv);
      ld16(sg + r * DIM, gv);
      float ss = 0.0f, gd = 0.0f, ss1 = 0.0f, gd1 = 0.0f;
#pragma unroll
      for (int e = 0; e < V; e += 2) {
        if (PK) {  // two columns per instruction (measured slower than one: 0.71 against 0.73 of the HBM copy rate)
          float t0, t1;
          fmul2(t0, t1, gv[e], gv[e + 1], wv[e], wv[e + 1]);
          ffma2(ss, ss1, xv[e], xv[e + 1], xv[e], xv[e + 1], ss, ss1);
          ffma2(gd, gd1, t0, t1, xv[e], xv[e + 1], gd, gd1);
        } else {
          ss = fmaf(xv[e], xv[e], ss);
          ss1 = fmaf(xv[e + 1], xv[e + 1], ss1);
          gd = fmaf(gv[e] * wv[e], xv[e], gd);
          gd1 = fmaf(gv[e + 1] * wv[e + 1], xv[e + 1], gd1);
        }
      }
      part[2 * r] = ss + ss1;
      part[2 * r + 1] = gd + gd1;
    }
    // NVAL sums over the warp by recursive halving; lane l ends with the total of value vidx(l)
    float w1;
    int vidx;
    if constexpr (ROWS == 4) {
      float w4[4], w2[2];
      const bool hi = lane & 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) w4[i] = (hi ? part[i + 4] : part[i]) + __shfl_xor_sync(0xffffffffu, hi ? part[i] : part[i + 4], 16);
      const bool h8 = lane & 8;
#pragma unroll
      for (int i = 0; i < 2; ++i) w2[i] = (h8 ? w4[i + 2] : w4[i]) + __shfl_xor_sync(0xffffffffu, h8 ? w4[i] : w4[i + 2], 8);
      const bool h4 = lane & 4;
      w1 = (h4 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? w2[0] : w2[1], 4);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
      vidx = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    } else {
      float w2[2];
      const bool hi = lane & 16;
#pragma unroll
      for (int i = 0; i < 2; ++i) w2[i] = (hi ? part[i + 2] : part[i]) + __shfl_xor_sync(0xffffffffu, hi ? part[i] : part[i + 2], 16);
      const bool h8 = lane & 8;
      w1 = (h8 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, h8 ? w2[0] : w2[1], 8);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 4);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
      w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
      vidx = ((lane >> 4) & 1) * 2 + ((lane >> 3) & 1);
    }
    if ((lane & (ROWS == 4 ? 3 : 7)) == 0) sh[buf][warp][vidx] = w1;
    __syncthreads();
    issue(k + S - 1);  // its stage was last read in the iteration before this one
    {
      float t = 0.0f;
#pragma unroll
      for (int wq = 0; wq < RB_THREADS / 32; ++wq) t += sh[buf][wq][lane & (NVAL - 1)];
      const float other = __shfl_xor_sync(0xffffffffu, t, 1);
      const float ssv = (lane & 1) ? other : t;
      const float gdv = (lane & 1) ? t : other;
      const float rr = 1.0f / sqrtf(ssv / (float)DIM + eps);
      const float coef = (rr * rr * rr) / (float)DIM * gdv;
      const float mine = (lane & 1) ? coef : rr;
#pragma unroll
      for (int i = 0; i < NVAL; ++i) part[i] = __shfl_sync(0xffffffffu, mine, i);
    }
    buf ^= 1;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float rrms = part[2 * r], ncoef = -part[2 * r + 1];
      float xv[V], gv[V], o[V];
      ld16(sx + r * DIM, xv);
      ld16(sg + r * DIM, gv);
#pragma unroll
      for (int e = 0; e < V; e += 2) {
        if (PK) {
          float t0, t1, u0, u1, v0, v1;
          fmul2(t0, t1, gv[e], gv[e + 1], wv[e], wv[e + 1]);
          fmul2(u0, u1, xv[e], xv[e + 1], ncoef, ncoef);
          ffma2(o[e], o[e + 1], t0, t1, rrms, rrms, u0, u1);
          fmul2(v0, v1, gv[e], gv[e + 1], xv[e], xv[e + 1]);
          ffma2(dwp[e], dwp[e + 1], v0, v1, rrms, rrms, dwp[e], dwp[e + 1]);
        } else {
          o[e] = fmaf(gv[e] * wv[e], rrms, xv[e] * ncoef);
          o[e + 1] = fmaf(gv[e + 1] * wv[e + 1], rrms, xv[e + 1] * ncoef);
          dwp[e] = fmaf(gv[e] * xv[e], rrms, dwp[e]);
          dwp[e + 1] = fmaf(gv[e + 1] * xv[e + 1], rrms, dwp[e + 1]);
        }
      }
      T* dr = dx + (r0 + r) * DIM + threadIdx.x * V;
      if (acc_dx) {
        float old[V];
        ld16(dr, old);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] += old[e];
      }
      st16(dr, o);
    }
  }
  if (dw_direct) {  // the CTA's column sums go straight into dw (16-byte vector reductions, any order)
#pragma unroll
    for (int e = 0; e < V; e += 4)
      asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(dw_direct + threadIdx.x * V + e), "f"(dwp[e]),
                   "f"(dwp[e + 1]), "f"(dwp[e + 2]), "f"(dwp[e + 3]) : "memory");
    return;
  }
#pragma unroll
  for (int e = 0; e < V; ++e) dw_partial[(long long)blockIdx.x * DIM + threadIdx.x * V + e] = dwp[e];
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


// Warp-per-row form of the backward for rows of 32 * NV 16-byte vectors (NV <= 8: 2048 bf16 or 1024
// f32 columns).  A warp owns whole rows, so the two row sums are ten shuffles and the kernel has no
// barrier inside its loop; lane l owns the columns of vectors l + 32 j for every row it sees and
// keeps their dw partial in registers; the weights sit in shared memory.  Rows are requested one
// iteration ahead (two register buffers, the loop is unrolled by two so that no copy is needed).
// At the end the warps of a CTA add their dw partials in a fixed order through shared memory and
// the CTA writes one row of dw_partial, which reduce_partials_kernel adds up (no atomics).
constexpr int RW_WARPS = 8;
int g_rms_bwd_mode = 2;  // eisen_rmsnorm_bwd_set_mode
bool g_rms_fwd_staged = true;  // eisen_rmsnorm_fwd_set_mode

template <typename T, int NV>
__global__ void __launch_bounds__(RW_WARPS * 32, 1)
rmsnorm_bwd_warp_kernel(const T* __restrict__ x, const float* __restrict__ w, const T* __restrict__ dy,
                        T* __restrict__ dx, float* __restrict__ dw_partial, long long rows, int dim, float eps,
                        int acc_dx) {
  constexpr int V = VecOf<T>::N;
  extern __shared__ float rw_smem[];
  float* sw = rw_smem;         // [dim] weights
  float* sacc = rw_smem + dim;  // [dim] dw of this CTA
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int c = threadIdx.x; c < dim; c += RW_WARPS * 32) { sw[c] = w[c]; sacc[c] = 0.0f; }
  __syncthreads();
  float dwp[NV][V];
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int k = 0; k < V; ++k) dwp[j][k] = 0.0f;
  const long long w0 = (long long)blockIdx.x * RW_WARPS + warp;
  const long long nw = (long long)gridDim.x * RW_WARPS;
  const float inv_dim = 1.0f / (float)dim;

  auto load_row = [&](long long row, uint4 (&xd)[NV], uint4 (&gd)[NV]) {
    if (row < rows) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const long long off = row * dim + (lane + 32 * j) * V;
        xd[j] = ld_stream16(x + off);
        gd[j] = ld_stream16(dy + off);
      }
    }
  };
  auto do_row = [&](long long row, const uint4 (&xd)[NV], const uint4 (&gdv)[NV]) {
    float ss = 0.0f, gsum = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float xv[V], gv[V];
      unpack16(xd[j], xv);
      unpack16(gdv[j], gv);
      const float* wp = sw + (lane + 32 * j) * V;
#pragma unroll
      for (int k = 0; k < V; k += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(wp + k);
        ss = fmaf(xv[k], xv[k], ss);             gsum = fmaf(gv[k] * w4.x, xv[k], gsum);
        ss = fmaf(xv[k + 1], xv[k + 1], ss);     gsum = fmaf(gv[k + 1] * w4.y, xv[k + 1], gsum);
        ss = fmaf(xv[k + 2], xv[k + 2], ss);     gsum = fmaf(gv[k + 2] * w4.z, xv[k + 2], gsum);
        ss = fmaf(xv[k + 3], xv[k + 3], ss);     gsum = fmaf(gv[k + 3] * w4.w, xv[k + 3], gsum);
      }
    }
    ss = warp_sum(ss);
    gsum = warp_sum(gsum);
    const float rrms = 1.0f / sqrtf(ss * inv_dim + eps);
    const float ncoef = -(rrms * rrms * rrms) * inv_dim * gsum;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float xv[V], gv[V], o[V];
      unpack16(xd[j], xv);
      unpack16(gdv[j], gv);
      const float* wp = sw + (lane + 32 * j) * V;
#pragma unroll
      for (int k = 0; k < V; k += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(wp + k);
        const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[k + e] = fmaf(gv[k + e] * ww[e], rrms, xv[k + e] * ncoef);
          dwp[j][k + e] = fmaf(gv[k + e] * xv[k + e], rrms, dwp[j][k + e]);
        }
      }
      T* dr = dx + row * dim + (lane + 32 * j) * V;
      if (acc_dx) {
        float old[V];
        ld16(dr, old);
#pragma unroll
        for (int k = 0; k < V; ++k) o[k] += old[k];
      }
      st16(dr, o);
    }
  };

  uint4 xa[NV], ga[NV], xb[NV], gb[NV];
  load_row(w0, xa, ga);
  for (long long row = w0; row < rows; row += 2 * nw) {
    load_row(row + nw, xb, gb);
    do_row(row, xa, ga);
    load_row(row + 2 * nw, xa, ga);
    if (row + nw < rows) do_row(row + nw, xb, gb);
  }
  // dw of this CTA: the warps add their partials one after the other (fixed order)
  for (int wq = 0; wq < RW_WARPS; ++wq) {
    if (warp == wq) {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        float* ap = sacc + (lane + 32 * j) * V;
#pragma unroll
        for (int k = 0; k < V; ++k) ap[k] += dwp[j][k];
      }
    }
    __syncthreads();
  }
  for (int c = threadIdx.x; c < dim; c += RW_WARPS * 32) dw_partial[(long long)blockIdx.x * dim + c] = sacc[c];
}

inline int rmsnorm_bwd_warp_grid(long long rows) {
  const long long need = (rows + RW_WARPS - 1) / RW_WARPS;
  const long long cap = sm_count();
  return (int)(need < cap ? (need < 1 ? 1 : need) : cap);
}

inline int rmsnorm_bwd_grid(long long rows) {
  return grid_for((rows + RB_ROWS - 1) / RB_ROWS, 1, 2);  // persistent: two resident CTAs per SM
}

// out[c] += sum_p partial[p][c]: 32 columns per CTA, 8 warps each summing every 8th partial,
// folded through shared memory in a fixed order
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int nparts, int dim) {
  __shared__ float sh[8][33];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.0f;
  if (c < dim)
    for (int p = g; p < nparts; p += 8) s += partial[(long long)p * dim + c];
  sh[g][lane] = s;
  __syncthreads();
  if (g == 0 && c < dim) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += sh[i][lane];
    out[c] += t;
  }
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

// f32 logits keep the precise expf (parity with the CPU arm); bf16 logits use the fast one
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T>
__device__ __forceinline__ float exp_t(float x) {
  if constexpr (sizeof(T) == 2) return __expf(x);
  else return expf(x);
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const T* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ row_loss,
              float* __restrict__ lse, int V_, int ignore_index, float normalizer, int* __restrict__ bad_target_flag) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int t = targets[row];
  // a target outside [0, V) that is not the ignore index would index past the row: the row is
  // skipped like an ignored one and the caller's flag is raised
  const bool out_of_range = t != ignore_index && (t < 0 || t >= V_);
  if (t == ignore_index || out_of_range) {
    if (threadIdx.x == 0) {
      row_loss[row] = 0.0f;
      if (lse) lse[row] = 0.0f;
      if (out_of_range && bad_target_flag) *bad_target_flag = 1;
    }
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
      if (cm > m) { s *= exp_t<T>(m - cm); m = cm; }
#pragma unroll
      for (int k = 0; k < V; ++k) s += exp_t<T>(v[k] - m);
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
    if (lse) lse[row] = gm + logf(s);
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
  if (t == ignore_index || t < 0 || t >= V_) {  // out-of-range targets: no gradient (the forward raised the flag)
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
        float g = exp_t<T>(v[k] - l);
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

// Cross-entropy forward and backward in one pass over a row: the row is read from global memory
// once into shared memory, the online max / sum runs while it arrives, and dlogits =
// (softmax - onehot) * scale is written back over the logits.  One read and one write of the row
// instead of a forward read plus a backward read and write.  The loss gradient is a launch
// argument (`scale` includes it), so the op that uses this kernel must be the last one before the
// loss.  Rows that do not fit `smem_elems` are read from global memory a second time.
template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_fused_kernel(T* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ row_loss,
                float* __restrict__ lse_out, int V_, int ignore_index, float normalizer, float scale, int smem_elems,
                int* __restrict__ bad_target_flag) {
  constexpr int V = VecOf<T>::N;
  extern __shared__ uint4 ce_row_raw[];
  T* srow = reinterpret_cast<T*>(ce_row_raw);
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int t = targets[row];
  T* xr = logits + row * V_;
  const bool vec = (V_ % V) == 0 && aligned_row(xr);
  const bool out_of_range = t != ignore_index && (t < 0 || t >= V_);
  if (t == ignore_index || out_of_range) {
    if (vec) {
      float z[V];
#pragma unroll
      for (int k = 0; k < V; ++k) z[k] = 0.0f;
      for (int c = threadIdx.x * V; c < V_; c += CE_THREADS * V) st16(xr + c, z);
    } else {
      for (int c = threadIdx.x; c < V_; c += CE_THREADS) xr[c] = from_f32<T>(0.0f);
    }
    if (threadIdx.x == 0) {
      row_loss[row] = 0.0f;
      if (lse_out) lse_out[row] = 0.0f;
      if (out_of_range && bad_target_flag) *bad_target_flag = 1;
    }
    return;
  }
  const bool staged = V_ <= smem_elems;
  float m = -INFINITY, s = 0.0f;
  if (vec) {
    for (int c = threadIdx.x * V; c < V_; c += CE_THREADS * V) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xr + c);
      if (staged) *reinterpret_cast<uint4*>(srow + c) = raw;
      float v[V];
      unpack16(raw, v);
      float cm = v[0];
#pragma unroll
      for (int k = 1; k < V; ++k) cm = fmaxf(cm, v[k]);
      if (cm > m) { s *= exp_t<T>(m - cm); m = cm; }
#pragma unroll
      for (int k = 0; k < V; ++k) s += exp_t<T>(v[k] - m);
    }
  } else {
    for (int c = threadIdx.x; c < V_; c += CE_THREADS) {
      const T raw = xr[c];
      if (staged) srow[c] = raw;
      const float v = to_f32(raw);
      if (v > m) { s *= expf(m - v); m = v; }
      s += expf(v - m);
    }
  }
  const float gm = block_max(m, sh);
  s = (m == -INFINITY) ? 0.0f : s * expf(m - gm);
  s = block_sum(s, sh);  // the barriers inside also publish the staged row to the whole CTA
  const float l = gm + logf(s);
  if (threadIdx.x == 0) {
    const float xt = to_f32(staged ? srow[t] : xr[t]);
    row_loss[row] = -logf(expf(xt - gm) / s + 1e-8f) * normalizer;
    if (lse_out) lse_out[row] = l;
  }
  __syncthreads();  // the target logit is read before anyone overwrites it
  const T* src = staged ? srow : xr;
  if (vec) {
    for (int c = threadIdx.x * V; c < V_; c += CE_THREADS * V) {
      float v[V];
      ld16(src + c, v);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float g = exp_t<T>(v[k] - l);
        if (c + k == t) g -= 1.0f;
        v[k] = g * scale;
      }
      st16(xr + c, v);
    }
  } else {
    for (int c = threadIdx.x; c < V_; c += CE_THREADS) {
      float g = expf(to_f32(src[c]) - l);
      if (c == t) g -= 1.0f;
      xr[c] = from_f32<T>(g * scale);
    }
  }
}

// Register-resident form of ce_fused_kernel for rows of up to 1024 * NV 16-byte vectors: a CTA of
// 1024 threads holds the whole row in registers (NV vectors per thread), so there is no staging
// copy, every load of the row is in flight at once and two CTAs per SM keep 2048 threads busy.
// Each exponential is computed once: after the sum it replaces its logit in the same registers (in
// T, so a bf16 row keeps bf16 exponentials; the row sum and the target's own gradient are formed
// from the f32 values), and the gradient is e * scale / sum.  Keeping the exponentials in f32 beside
// the row needs 64 registers, i.e. one CTA per SM, and measured slower (0.67 against 0.51 ms at
// 16384 x 32000 bf16).
template <typename T, int NV>
__global__ void __launch_bounds__(1024, 2)
ce_fused_reg_kernel(T* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ row_loss,
                    float* __restrict__ lse_out, int V_, int ignore_index, float normalizer, float scale,
                    int* __restrict__ bad_target_flag) {
  constexpr int V = VecOf<T>::N;
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int t = targets[row];
  T* xr = logits + row * V_;
  const int nvec = V_ / V;
  const bool out_of_range = t != ignore_index && (t < 0 || t >= V_);
  if (t == ignore_index || out_of_range) {
    const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = threadIdx.x + j * 1024;
      if (v < nvec) *reinterpret_cast<uint4*>(xr + (long long)v * V) = z;
    }
    if (threadIdx.x == 0) {
      row_loss[row] = 0.0f;
      if (lse_out) lse_out[row] = 0.0f;
      if (out_of_range && bad_target_flag) *bad_target_flag = 1;
    }
    return;
  }
  // vectors past the end of the row read as -inf: they drop out of the maximum and add 0 to the sum
  constexpr uint32_t NEG_INF = sizeof(T) == 2 ? 0xff80ff80u : 0xff800000u;
  uint4 raw[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = threadIdx.x + j * 1024;
    raw[j] = (v < nvec) ? ld_stream16(xr + (long long)v * V) : make_uint4(NEG_INF, NEG_INF, NEG_INF, NEG_INF);
  }
  // the thread that holds the target's vector keeps the target's logit in f32
  const bool holder = (t / V) % 1024 == (int)threadIdx.x;
  float xt = 0.0f;
  if (holder) {
    const int jt = (t / V) / 1024, kt = t % V;
    uint4 r = raw[0];
#pragma unroll
    for (int j = 1; j < NV; ++j)
      if (j == jt) r = raw[j];
    float x[V];
    unpack16(r, x);
#pragma unroll
    for (int k = 0; k < V; ++k)
      if (k == kt) xt = x[k];
  }
  float m;
  if constexpr (sizeof(T) == 2) {  // the maximum on packed pairs
    auto pair = [](uint32_t w) { return *reinterpret_cast<const __nv_bfloat162*>(&w); };
    __nv_bfloat162 m2 = pair(raw[0].x);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      m2 = __hmax2(m2, pair(raw[j].x));
      m2 = __hmax2(m2, pair(raw[j].y));
      m2 = __hmax2(m2, pair(raw[j].z));
      m2 = __hmax2(m2, pair(raw[j].w));
    }
    m = fmaxf(__low2float(m2), __high2float(m2));
  } else {
    m = -INFINITY;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      float x[V];
      unpack16(raw[j], x);
#pragma unroll
      for (int k = 0; k < V; ++k) m = fmaxf(m, x[k]);
    }
  }
  const float gm = block_max(m, sh);
  float s = 0.0f;
  const float ngm2 = -gm * 1.4426950408889634f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    float x[V];
    unpack16(raw[j], x);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      if constexpr (sizeof(T) == 2) x[k] = ex2_approx(fmaf(x[k], 1.4426950408889634f, ngm2));
      else x[k] = expf(x[k] - gm);
      s += x[k];
    }
    raw[j] = pack16(x);  // the exponentials take the place of the logits
  }
  s = block_sum(s, sh);
  const float l = gm + logf(s);
  const float pscale = scale / s;  // softmax = e / s
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = threadIdx.x + j * 1024;
    if (v < nvec) {
      float x[V];
      unpack16(raw[j], x);
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] *= pscale;
      st16(xr + (long long)v * V, x);
    }
  }
  if (holder) {
    const float pt = expf(xt - gm) / s;
    row_loss[row] = -logf(pt + 1e-8f) * normalizer;
    if (lse_out) lse_out[row] = l;
    xr[t] = from_f32<T>((pt - 1.0f) * scale);  // after this thread's own vector store to the same address
  }
}

template <typename T, int NCH>
int launch_rmsnorm_bwd(cudaStream_t s, const T* x, const float* w, const T* dy, T* dx, float* dw,
                       float* ws, long long rows, int dim, float eps, int acc_dx) {
  const int grid = rmsnorm_bwd_grid(rows);
  if (rows % RB_ROWS == 0 && dim == NCH * RB_THREADS * VecOf<T>::N)
    rmsnorm_bwd_kernel<T, NCH, true><<<grid, RB_THREADS, 0, s>>>(x, w, dy, dx, ws, rows, dim, eps, acc_dx);
  else
    rmsnorm_bwd_kernel<T, NCH, false><<<grid, RB_THREADS, 0, s>>>(x, w, dy, dx, ws, rows, dim, eps, acc_dx);
  int rc = check_launch("rmsnorm_bwd");
  if (rc) return rc;
  reduce_partials_kernel<<<(dim + 31) / 32, 256, 0, s>>>(ws, dw, grid, dim);
  return check_launch("rmsnorm_bwd_reduce");
}

template <typename T>
int rmsnorm_bwd_dispatch(cudaStream_t s, const T* x, const float* w, const T* dy, T* dx, float* dw, float* ws,
                         long long rows, int dim, float eps, int acc_dx) {
  constexpr int V = VecOf<T>::N;
  const int nch = (dim + RB_THREADS * V - 1) / (RB_THREADS * V);
  const bool fast = (dim % V) == 0 && nch <= 4 && aligned16(x) && aligned16(dy) && aligned16(dx) && ws != nullptr;
  if (!fast) {
    const int grid = grid_for(rows, 8, 4);
    rmsnorm_bwd_generic_kernel<T><<<grid, 256, 0, s>>>(x, w, dy, dx, dw, rows, dim, eps, acc_dx);
    return check_launch("rmsnorm_bwd_generic");
  }
  if (g_rms_bwd_mode >= 2 && dim == RB_THREADS * V && rows % 4 == 0 && rows >= 4 && aligned16(w)) {
    // staged kernel: mode 2 = 4 rows x 3 stages, 2 CTAs per SM; 3 = 2 rows x 4 stages, 3 CTAs; 4 = 2 rows x 3 stages, 4 CTAs
    const int mode = g_rms_bwd_mode;
    // 6 = mode 2 with two columns per arithmetic instruction (packed f32x2)
    const int rows_per = (mode == 2 || mode == 5 || mode == 6) ? 4 : 2, stages = mode == 3 ? 4 : (mode == 5 ? 2 : 3),
              ctas = (mode == 2 || mode == 6) ? 2 : (mode == 3 || mode == 5 ? 3 : 4);
    const long long groups = rows / rows_per;
    const long long cap = (long long)sm_count() * ctas;
    const int grid = (int)(groups < cap ? groups : cap);
    const size_t smem = (size_t)stages * 2 * rows_per * dim * sizeof(T);
    // Outside the fixed-order mode the CTAs add their column sums into dw themselves: no second launch (7 us of a
    // 42 us call at 16384 x 2048).  In the fixed-order mode a second kernel adds the partials in CTA order.
    const bool direct = !deterministic() && sizeof(T) == 2 && aligned16(dw);  // the f32 path keeps one order always
    static bool attr[5][2][MAX_DEVICE_SLOTS] = {{{false}}};
    auto go = [&](auto kern) -> int {
      bool& done = attr[mode - 2][sizeof(T) == 2][device_slot()];
      if (!done) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 1;
        done = true;
      }
      kern<<<grid, RB_THREADS, smem, s>>>(x, w, dy, dx, ws, direct ? dw : nullptr, groups, eps, acc_dx);
      return 0;
    };
    int bad = mode == 2 ? go(rmsnorm_bwd_staged_kernel<T, 4, 3, 2>)
            : mode == 3 ? go(rmsnorm_bwd_staged_kernel<T, 2, 4, 3>)
            : mode == 4 ? go(rmsnorm_bwd_staged_kernel<T, 2, 3, 4>)
            : mode == 5 ? go(rmsnorm_bwd_staged_kernel<T, 4, 2, 3>) : go(rmsnorm_bwd_staged_kernel<T, 4, 3, 2, true>);
    if (bad) return fail(EISEN_ERR_CUDA, "rmsnorm_bwd: shared-memory attribute");
    int rc = check_launch("rmsnorm_bwd_staged");
    if (rc || direct) return rc;
    reduce_partials_kernel<<<(dim + 31) / 32, 256, 0, s>>>(ws, dw, grid, dim);
    return check_launch("rmsnorm_bwd_reduce");
  }
  if (g_rms_bwd_mode == 1 && dim % (32 * V) == 0 && dim / (32 * V) <= 8 && aligned16(w)) {
    const int nv = dim / (32 * V);
    const int grid = rmsnorm_bwd_warp_grid(rows);
    const size_t smem = (size_t)dim * 8;
    auto go = [&](auto kern) { kern<<<grid, RW_WARPS * 32, smem, s>>>(x, w, dy, dx, ws, rows, dim, eps, acc_dx); };
    switch (nv) {
      case 1: go(rmsnorm_bwd_warp_kernel<T, 1>); break;
      case 2: go(rmsnorm_bwd_warp_kernel<T, 2>); break;
      case 3: go(rmsnorm_bwd_warp_kernel<T, 3>); break;
      case 4: go(rmsnorm_bwd_warp_kernel<T, 4>); break;
      case 5: go(rmsnorm_bwd_warp_kernel<T, 5>); break;
      case 6: go(rmsnorm_bwd_warp_kernel<T, 6>); break;
      case 7: go(rmsnorm_bwd_warp_kernel<T, 7>); break;
      default: go(rmsnorm_bwd_warp_kernel<T, 8>); break;
    }
    int rc = check_launch("rmsnorm_bwd_warp");
    if (rc) return rc;
    reduce_partials_kernel<<<(dim + 31) / 32, 256, 0, s>>>(ws, dw, grid, dim);
    return check_launch("rmsnorm_bwd_reduce");
  }
  if (nch <= 1) return launch_rmsnorm_bwd<T, 1>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
  if (nch <= 2) return launch_rmsnorm_bwd<T, 2>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
  return launch_rmsnorm_bwd<T, 4>(s, x, w, dy, dx, dw, ws, rows, dim, eps, acc_dx);
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
    if (g_rms_fwd_staged && dim == RB_THREADS * VecOf<T>::N && rows % 4 == 0 && rows >= 4 && aligned16(w)) {
      // rows staged in shared memory: 3 stages of 4 rows, four CTAs per SM
      constexpr int ST = 3, CT = 4;
      const long long groups = rows / 4;
      const long long cap = (long long)sm_count() * CT;
      const size_t smem = (size_t)ST * 4 * dim * sizeof(T);
      static bool attr[2][MAX_DEVICE_SLOTS] = {{false}};
      bool& done = attr[sizeof(T) == 2][device_slot()];
      if (!done) {
        if (cudaFuncSetAttribute(rmsnorm_fwd_staged_kernel<T, ST, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
          return fail(EISEN_ERR_CUDA, "rmsnorm_fwd: shared-memory attribute");
        done = true;
      }
      rmsnorm_fwd_staged_kernel<T, ST, CT><<<(int)(groups < cap ? groups : cap), RB_THREADS, smem, (cudaStream_t)stream>>>(
          (const T*)x, w, (T*)y, rrms_out, groups, eps);
      return check_launch("rmsnorm_fwd_staged");
    }
    rmsnorm_fwd_dispatch<T>((const T*)x, w, (T*)y, rrms_out, rows, (int)dim, eps, grid, (cudaStream_t)stream);
    return check_launch("rmsnorm_fwd");
  });
}

int eisen_rmsnorm_fwd_set_mode(int staged) {
  g_rms_fwd_staged = staged != 0;
  return 0;
}

int eisen_rmsnorm_bwd_set_mode(int mode) {
  if (mode < 0 || mode > 6) return fail(EISEN_ERR_INVALID, "rmsnorm_bwd_set_mode: mode must be in [0, 6]");
  g_rms_bwd_mode = mode;
  return 0;
}

long long eisen_rmsnorm_bwd_workspace_bytes(long long rows, long long dim) {
  const long long g = std::max<long long>(std::max<long long>(rmsnorm_bwd_grid(rows), rmsnorm_bwd_warp_grid(rows)), 4LL * sm_count());
  return g * dim * 4 + 256;
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
// bad_target_flag (device int, may be null) is set to 1 when a target is neither ignore_index nor
// inside [0, vocab); such rows are skipped like ignored ones, in the forward and in the backward.
int eisen_ce_fwd(void* stream, const void* logits, const int* targets, float* loss, float* row_loss, float* lse,
                 long long rows, long long vocab, int ignore_index, float normalizer, int dt, int* bad_target_flag) {
  if (rows <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  EISEN_DISPATCH_DTYPE(dt, T, {
    ce_fwd_kernel<T><<<(unsigned)rows, CE_THREADS, 0, s>>>((const T*)logits, targets, row_loss, lse, (int)vocab,
                                                          ignore_index, normalizer, bad_target_flag);
    int rc = check_launch("ce_fwd");
    if (rc || !loss) return rc;
    ce_loss_reduce_kernel<<<1, 1024, 0, s>>>(row_loss, loss, rows);
    return check_launch("ce_loss_reduce");
  });
}

// Forward and backward of the cross-entropy in one launch, in place: on return `logits` holds
// dlogits = (softmax - onehot) * normalizer * grad_scale (zero for ignored rows), *loss the summed
// row losses, row_loss [rows] each row's share and lse (may be null) the log-sum-exp.
int eisen_ce_fused(void* stream, void* logits, const int* targets, float* loss, float* row_loss, float* lse,
                   long long rows, long long vocab, int ignore_index, float normalizer, float grad_scale, int dt,
                   int* bad_target_flag) {
  if (rows <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  static int max_smem[MAX_DEVICE_SLOTS] = {0};
  static bool attr_f32[MAX_DEVICE_SLOTS] = {false}, attr_bf16[MAX_DEVICE_SLOTS] = {false};
  const int slot = device_slot();
  if (!max_smem[slot]) {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || v <= 0) v = 48 * 1024;
    max_smem[slot] = v;
  }
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int VW = VecOf<T>::N;
    const long long nvec = vocab / VW;
    if (vocab % VW == 0 && aligned16(logits) && nvec <= 8 * 1024 && vocab >= 2048) {
      // the row fits the registers of one 1024-thread CTA
      auto go = [&](auto kern) {
        kern<<<(unsigned)rows, 1024, 0, s>>>((T*)logits, targets, row_loss, lse, (int)vocab, ignore_index, normalizer,
                                             normalizer * grad_scale, bad_target_flag);
      };
      if (nvec <= 1024) go(ce_fused_reg_kernel<T, 1>);
      else if (nvec <= 2048) go(ce_fused_reg_kernel<T, 2>);
      else if (nvec <= 4096) go(ce_fused_reg_kernel<T, 4>);
      else go(ce_fused_reg_kernel<T, 8>);
      int rc = check_launch("ce_fused");
      if (rc) return rc;
      if (loss) {
        ce_loss_reduce_kernel<<<1, 1024, 0, s>>>(row_loss, loss, rows);
        return check_launch("ce_loss_reduce");
      }
      return 0;
    }
    // three CTAs per SM when the row allows it (a 32000-entry bf16 row is 62.5 KB)
    size_t row_bytes = ((size_t)vocab * sizeof(T) + 15) & ~size_t(15);
    size_t smem = row_bytes;
    const size_t cap = (size_t)max_smem[slot] - 1024;
    if (smem > cap) smem = 0;  // row too long for shared memory: second pass reads global memory
    bool& attr = sizeof(T) == 2 ? attr_bf16[slot] : attr_f32[slot];
    if (!attr) {
      if (cudaFuncSetAttribute(ce_fused_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap) != cudaSuccess)
        return fail(EISEN_ERR_CUDA, "ce_fused: shared-memory attribute");
      attr = true;
    }
    ce_fused_kernel<T><<<(unsigned)rows, CE_THREADS, smem, s>>>((T*)logits, targets, row_loss, lse, (int)vocab, ignore_index,
                                                                normalizer, normalizer * grad_scale,
                                                                smem ? (int)(smem / sizeof(T)) : 0, bad_target_flag);
    int rc = check_launch("ce_fused");
    if (rc) return rc;
    if (loss) {
      ce_loss_reduce_kernel<<<1, 1024, 0, s>>>(row_loss, loss, rows);
      return check_launch("ce_loss_reduce");
    }
    return 0;
  });
}

int eisen_ce_loss_reduce(void* stream, const float* row_loss, float* loss, long long rows) {
  if (rows <= 0) return 0;
  ce_loss_reduce_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(row_loss, loss, rows);
  return check_launch("ce_loss_reduce");
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
