// Bandwidth-bound elementwise kernels of the training step: residual add, gradient accumulate,
// SiLU / mul / fused SwiGLU forward and backward, RoPE forward and backward (interleaved pairs),
// [B,S,H,D] <-> [B,H,S,D] transposes, GQA head replication, casts, fill, scale.
// Every kernel moves 16 bytes per thread per access (4 f32 or 8 bf16), is grid-strided with the
// grid sized against the SM count, and computes in f32.
// Reference counterparts: kernels/ops_f32.cu:66-156 (add, accumulate, fill, scale, mul, silu),
// 694-760 (transpose_0213, rope), 787-840 (repeat_kv); kernels/ops_bf16.cu:4-24, 406-560.
#include "common.cuh"
#include <initializer_list>
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

namespace {

constexpr int EW_THREADS = 256;

// Generic vector kernel: f(i0, count) handles elements [i0, i0+count), count == VEC except in
// the ragged tail.
template <int VEC, typename F>
__global__ void __launch_bounds__(EW_THREADS) vec_kernel(long long n, F f) {
  const long long nvec = (n + VEC - 1) / VEC;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const long long i0 = v * VEC;
    f(i0, (i0 + VEC <= n) ? VEC : (int)(n - i0));
  }
}

template <int VEC, typename F>
int launch_vec(cudaStream_t s, long long n, F f, const char* what) {
  if (n <= 0) return 0;
  const int grid = grid_for((n + VEC - 1) / VEC, EW_THREADS, 8);
  vec_kernel<VEC, F><<<grid, EW_THREADS, 0, s>>>(n, f);
  return check_launch(what);
}

template <typename T>
__device__ __forceinline__ void load_n(const T* p, float (&v)[VecOf<T>::N], int cnt) {
  if (cnt == VecOf<T>::N) {
    ld16(p, v);
  } else {
#pragma unroll
    for (int i = 0; i < VecOf<T>::N; ++i) v[i] = i < cnt ? to_f32(p[i]) : 0.0f;
  }
}
template <typename T>
__device__ __forceinline__ void store_n(T* p, const float (&v)[VecOf<T>::N], int cnt) {
  if (cnt == VecOf<T>::N) {
    st16(p, v);
  } else {
#pragma unroll
    for (int i = 0; i < VecOf<T>::N; ++i)
      if (i < cnt) p[i] = from_f32<T>(v[i]);
  }
}
template <typename T>
__device__ __forceinline__ void store_acc_n(T* p, float (&v)[VecOf<T>::N], int cnt, bool acc) {
  if (acc) {
    float o[VecOf<T>::N];
    load_n(p, o, cnt);
#pragma unroll
    for (int i = 0; i < VecOf<T>::N; ++i) v[i] += o[i];
  }
  store_n(p, v, cnt);
}

// f32 tensors keep the precise expf (parity with the CPU arms at 1e-5); bf16 tensors use the fast
// exponential and division, whose error is far below bf16 rounding
template <typename T>
__device__ __forceinline__ float sigmoid_t(float x) {
  if constexpr (sizeof(T) == 2) return __fdividef(1.0f, 1.0f + __expf(-x));
  else return 1.0f / (1.0f + expf(-x));
}

template <typename T>
__global__ void reduce_leading_kernel(const T* src, float* dst, long long n, long long m, int acc) {
  const long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (j >= m) return;
  float s = 0.0f;
  for (long long i = j; i < n; i += m) s += to_f32(src[i]);
  dst[j] = acc ? dst[j] + s : s;
}

__global__ void rope_table_kernel(float2* table, int S, int half, float base, float head_dim) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S * half) return;
  const int pos = i / half, pair = i % half;
  const float theta = (float)pos / powf(base, (2.0f * (float)pair) / head_dim);
  float sn, cs;
  sincosf(theta, &sn, &cs);
  table[i] = make_float2(cs, sn);
}

bool all_aligned(std::initializer_list<const void*> ps) {
  for (const void* p : ps)
    if (p && !aligned16(p)) return false;
  return true;
}

}  // namespace
}  // namespace eisen

using namespace eisen;

#define REQUIRE_ALIGNED(...)                                                              \
  if (!all_aligned({__VA_ARGS__})) return fail(EISEN_ERR_INVALID, "pointers must be 16-byte aligned")

extern "C" {

int eisen_fill_f32(void* stream, float* p, float value, long long n) {
  REQUIRE_ALIGNED(p);
  return launch_vec<4>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
    float v[4] = {value, value, value, value};
    store_n(p + i, v, c);
  }, "fill_f32");
}

int eisen_scale_f32(void* stream, float* p, float s, long long n) {
  REQUIRE_ALIGNED(p);
  return launch_vec<4>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
    float v[4];
    load_n(p + i, v, c);
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] *= s;
    store_n(p + i, v, c);
  }, "scale_f32");
}

int eisen_cast(void* stream, const void* src, int src_dt, void* dst, int dst_dt, long long n) {
  REQUIRE_ALIGNED(src, dst);
  cudaStream_t s = (cudaStream_t)stream;
  if (src_dt == dst_dt) {
    const size_t bytes = (size_t)n * (src_dt == DT_F32 ? 4 : 2);
    if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s) != cudaSuccess)
      return fail(EISEN_ERR_CUDA, "cast: copy failed");
    return 0;
  }
  if (src_dt == DT_F32) {
    const float* a = (const float*)src;
    __nv_bfloat16* b = (__nv_bfloat16*)dst;
    return launch_vec<8>(s, n, [=] __device__(long long i, int c) {
      float v[8];
      if (c == 8) {
        float lo[4], hi[4];
        ld16(a + i, lo);
        ld16(a + i + 4, hi);
#pragma unroll
        for (int k = 0; k < 4; ++k) { v[k] = lo[k]; v[4 + k] = hi[k]; }
      } else {
        for (int k = 0; k < 8; ++k) v[k] = k < c ? a[i + k] : 0.0f;
      }
      store_n(b + i, v, c);
    }, "cast_f32_bf16");
  }
  const __nv_bfloat16* a = (const __nv_bfloat16*)src;
  float* b = (float*)dst;
  return launch_vec<8>(s, n, [=] __device__(long long i, int c) {
    float v[8];
    load_n(a + i, v, c);
    if (c == 8) {
      float lo[4] = {v[0], v[1], v[2], v[3]}, hi[4] = {v[4], v[5], v[6], v[7]};
      st16(b + i, lo);
      st16(b + i + 4, hi);
    } else {
      for (int k = 0; k < c; ++k) b[i + k] = v[k];
    }
  }, "cast_bf16_f32");
}

// out[i] = a[i] + b[i % b_numel]; b_numel == n for the plain residual add, smaller for a
// trailing-dims broadcast (bias [out], additive mask [1,S,S]).
int eisen_add(void* stream, const void* a, const void* b, void* out, long long n, long long b_numel, int dt) {
  REQUIRE_ALIGNED(a, b, out);
  if (b_numel <= 0 || n % b_numel) return fail(EISEN_ERR_INVALID, "add: b must broadcast over leading dims");
  cudaStream_t s = (cudaStream_t)stream;
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* pa = (const T*)a; const T* pb = (const T*)b; T* po = (T*)out;
    const bool vec_b = (b_numel % V) == 0;
    if (b_numel == n) {  // plain residual add: no broadcast index arithmetic
      return launch_vec<V>(s, n, [=] __device__(long long i, int c) {
        float x[V], y[V];
        load_n(pa + i, x, c);
        load_n(pb + i, y, c);
#pragma unroll
        for (int k = 0; k < V; ++k) x[k] += y[k];
        store_n(po + i, x, c);
      }, "add");
    }
    return launch_vec<V>(s, n, [=] __device__(long long i, int c) {
      float x[V], y[V];
      load_n(pa + i, x, c);
      if (vec_b && c == V) {
        ld16(pb + (i % b_numel), y);
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) y[k] = k < c ? to_f32(pb[(i + k) % b_numel]) : 0.0f;
      }
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] += y[k];
      store_n(po + i, x, c);
    }, "add");
  });
}

// dst[i] (+)= src[i]; dst and src may differ in dtype (f32 parameter gradients fed by bf16
// activation gradients)
int eisen_accumulate(void* stream, void* dst, int dst_dt, const void* src, int src_dt, long long n, int accumulate) {
  REQUIRE_ALIGNED(dst, src);
  cudaStream_t s = (cudaStream_t)stream;
  const bool acc = accumulate != 0;
  if (dst_dt == src_dt) {
    EISEN_DISPATCH_DTYPE(dst_dt, T, {
      constexpr int V = VecOf<T>::N;
      T* pd = (T*)dst; const T* ps = (const T*)src;
      return launch_vec<V>(s, n, [=] __device__(long long i, int c) {
        float x[V];
        load_n(ps + i, x, c);
        store_acc_n(pd + i, x, c, acc);
      }, "accumulate");
    });
  }
  if (dst_dt == DT_F32) {
    float* pd = (float*)dst; const __nv_bfloat16* ps = (const __nv_bfloat16*)src;
    return launch_vec<8>(s, n, [=] __device__(long long i, int c) {
      float x[8];
      load_n(ps + i, x, c);
      for (int k = 0; k < c; ++k) pd[i + k] = acc ? pd[i + k] + x[k] : x[k];
    }, "accumulate_bf16_to_f32");
  }
  __nv_bfloat16* pd = (__nv_bfloat16*)dst; const float* ps = (const float*)src;
  return launch_vec<8>(s, n, [=] __device__(long long i, int c) {
    float x[8];
    for (int k = 0; k < 8; ++k) x[k] = k < c ? ps[i + k] : 0.0f;
    store_acc_n(pd + i, x, c, acc);
  }, "accumulate_f32_to_bf16");
}

// dst[j] (+)= sum over i with i % m == j of src[i]  (gradient of a broadcast operand)
int eisen_reduce_leading(void* stream, const void* src, int src_dt, float* dst, long long n, long long m, int accumulate) {
  if (m <= 0 || n % m) return fail(EISEN_ERR_INVALID, "reduce_leading: n must be a multiple of m");
  const int grid = (int)((m + 255) / 256);
  if (src_dt == DT_F32)
    reduce_leading_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)src, dst, n, m, accumulate);
  else
    reduce_leading_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, dst, n, m, accumulate);
  return check_launch("reduce_leading");
}

int eisen_mul_fwd(void* stream, const void* a, const void* b, void* out, long long n, int dt) {
  REQUIRE_ALIGNED(a, b, out);
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* pa = (const T*)a; const T* pb = (const T*)b; T* po = (T*)out;
    return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      float x[V], y[V];
      load_n(pa + i, x, c);
      load_n(pb + i, y, c);
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] *= y[k];
      store_n(po + i, x, c);
    }, "mul_fwd");
  });
}

// da (+)= dout*b ; db (+)= dout*a ; either output may be null
int eisen_mul_bwd(void* stream, const void* a, const void* b, const void* dout, void* da, void* db,
                  long long n, int dt, int acc_a, int acc_b) {
  REQUIRE_ALIGNED(a, b, dout, da, db);
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* pa = (const T*)a; const T* pb = (const T*)b; const T* pg = (const T*)dout;
    T* pda = (T*)da; T* pdb = (T*)db;
    const bool aa = acc_a != 0, ab = acc_b != 0;
    return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      float x[V], y[V], g[V], r[V];
      load_n(pa + i, x, c);
      load_n(pb + i, y, c);
      load_n(pg + i, g, c);
      if (pda) {
#pragma unroll
        for (int k = 0; k < V; ++k) r[k] = g[k] * y[k];
        store_acc_n(pda + i, r, c, aa);
      }
      if (pdb) {
#pragma unroll
        for (int k = 0; k < V; ++k) r[k] = g[k] * x[k];
        store_acc_n(pdb + i, r, c, ab);
      }
    }, "mul_bwd");
  });
}

int eisen_silu_fwd(void* stream, const void* x, void* y, long long n, int dt) {
  REQUIRE_ALIGNED(x, y);
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* px = (const T*)x; T* py = (T*)y;
    return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      float v[V];
      load_n(px + i, v, c);
#pragma unroll
      for (int k = 0; k < V; ++k) v[k] = v[k] * sigmoid_t<T>(v[k]);
      store_n(py + i, v, c);
    }, "silu_fwd");
  });
}

// dx (+)= dy * (silu + sig*(1-silu))   (src/graph/ops/elementwise.rs:451-457)
int eisen_silu_bwd(void* stream, const void* x, const void* dy, void* dx, long long n, int dt, int accumulate) {
  REQUIRE_ALIGNED(x, dy, dx);
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* px = (const T*)x; const T* pg = (const T*)dy; T* pd = (T*)dx;
    const bool acc = accumulate != 0;
    return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      float v[V], g[V];
      load_n(px + i, v, c);
      load_n(pg + i, g, c);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float sig = sigmoid_t<T>(v[k]);
        float silu = v[k] * sig;
        g[k] = g[k] * (silu + sig * (1.0f - silu));
      }
      store_acc_n(pd + i, g, c, acc);
    }, "silu_bwd");
  });
}

// out = silu(gate) * up   (replaces silu + mul, src/nn/transformer.rs:41-44)
int eisen_swiglu_fwd(void* stream, const void* gate, const void* up, void* out, long long n, int dt) {
  REQUIRE_ALIGNED(gate, up, out);
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* pg = (const T*)gate; const T* pu = (const T*)up; T* po = (T*)out;
    return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      float g[V], u[V];
      load_n(pg + i, g, c);
      load_n(pu + i, u, c);
#pragma unroll
      for (int k = 0; k < V; ++k) g[k] = (g[k] * sigmoid_t<T>(g[k])) * u[k];
      store_n(po + i, g, c);
    }, "swiglu_fwd");
  });
}

}  // extern "C"

namespace eisen {
namespace {
// Five streams (three read, two written).  With one 16-byte vector per thread and iteration the
// kernel waits on memory most of the time (long-scoreboard stalls, 36 % issue utilisation): here a
// thread requests two vectors of each input before it touches the first.
template <typename T, bool ACC>
__global__ void __launch_bounds__(EW_THREADS)
swiglu_bwd_kernel(const T* __restrict__ pg, const T* __restrict__ pu, const T* __restrict__ ph, T* __restrict__ pdg,
                  T* __restrict__ pdu, long long nvec) {
  constexpr int V = VecOf<T>::N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; v0 < nvec; v0 += 2 * stride) {
    const long long v1 = v0 + stride;
    const bool two = v1 < nvec;
    const long long i0 = v0 * V, i1 = (two ? v1 : v0) * V;
    float g0[V], u0[V], h0[V], g1[V], u1[V], h1[V];
    ld16(pg + i0, g0); ld16(pu + i0, u0); ld16(ph + i0, h0);
    ld16(pg + i1, g1); ld16(pu + i1, u1); ld16(ph + i1, h1);
    float a0[V], b0[V], a1[V], b1[V];
    if (ACC) { ld16(pdg + i0, a0); ld16(pdu + i0, b0); ld16(pdg + i1, a1); ld16(pdu + i1, b1); }
    float dg[V], du[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float sig = sigmoid_t<T>(g0[k]);
      const float silu = g0[k] * sig;
      du[k] = h0[k] * silu;
      dg[k] = (h0[k] * u0[k]) * (silu + sig * (1.0f - silu));
      if (ACC) { dg[k] += a0[k]; du[k] += b0[k]; }
    }
    st16(pdg + i0, dg);
    st16(pdu + i0, du);
    if (two) {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float sig = sigmoid_t<T>(g1[k]);
        const float silu = g1[k] * sig;
        du[k] = h1[k] * silu;
        dg[k] = (h1[k] * u1[k]) * (silu + sig * (1.0f - silu));
        if (ACC) { dg[k] += a1[k]; du[k] += b1[k]; }
      }
      st16(pdg + i1, dg);
      st16(pdu + i1, du);
    }
  }
}
}  // namespace
}  // namespace eisen

extern "C" {

// dgate (+)= dh*up*silu'(gate) ; dup (+)= dh*silu(gate): one pass instead of mul_bwd + silu_bwd
int eisen_swiglu_bwd(void* stream, const void* gate, const void* up, const void* dh, void* dgate, void* dup,
                     long long n, int dt, int accumulate) {
  REQUIRE_ALIGNED(gate, up, dh, dgate, dup);
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* pg = (const T*)gate; const T* pu = (const T*)up; const T* ph = (const T*)dh;
    T* pdg = (T*)dgate; T* pdu = (T*)dup;
    const bool acc = accumulate != 0;
    if (n % V == 0) {
      const long long nvec = n / V;
      const int grid = grid_for((nvec + 1) / 2, EW_THREADS, 4);
      if (acc) swiglu_bwd_kernel<T, true><<<grid, EW_THREADS, 0, (cudaStream_t)stream>>>(pg, pu, ph, pdg, pdu, nvec);
      else swiglu_bwd_kernel<T, false><<<grid, EW_THREADS, 0, (cudaStream_t)stream>>>(pg, pu, ph, pdg, pdu, nvec);
      return check_launch("swiglu_bwd");
    }
    return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      float g[V], u[V], h[V], dg[V], du[V];
      load_n(pg + i, g, c);
      load_n(pu + i, u, c);
      load_n(ph + i, h, c);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float sig = sigmoid_t<T>(g[k]);
        float silu = g[k] * sig;
        du[k] = h[k] * silu;
        dg[k] = (h[k] * u[k]) * (silu + sig * (1.0f - silu));
      }
      store_acc_n(pdg + i, dg, c, acc);
      store_acc_n(pdu + i, du, c, acc);
    }, "swiglu_bwd");
  });
}

// ---------------------------------------------------------------------------------------
// RoPE (interleaved pairs; src/graph/ops/transform.rs:541-610).  The (cos, sin) of every
// (position, pair) is tabulated once with the reference's f32 formula
// theta = pos / 10000^(2p/D), so the streaming kernels are pure loads and FMAs.
// ---------------------------------------------------------------------------------------
int eisen_rope_table(void* stream, float* table_cos_sin, long long seq_len, long long head_dim, float base) {
  const int half = (int)(head_dim / 2);
  const long long n = seq_len * half;
  if (n <= 0) return 0;
  rope_table_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (float2*)table_cos_sin, (int)seq_len, half, base, (float)head_dim);
  return check_launch("rope_table");
}

// x, y: [B, S, hidden]; pairs (2p, 2p+1) inside each head.  inverse = 1 applies the transposed
// rotation (the backward pass).  y may alias x.
int eisen_rope(void* stream, const void* x, void* y, const float* table_cos_sin, long long B, long long S,
               long long hidden, long long head_dim, int dt, int inverse, int accumulate) {
  REQUIRE_ALIGNED(x, y);
  if (head_dim % 2 || hidden % head_dim) return fail(EISEN_ERR_INVALID, "rope: hidden must be a multiple of an even head_dim");
  const long long n = B * S * hidden;
  const float2* tab = (const float2*)table_cos_sin;
  const int half = (int)(head_dim / 2);
  const bool acc = accumulate != 0;
  const float sgn = inverse ? -1.0f : 1.0f;
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* px = (const T*)x; T* py = (T*)y;
    // a 16-byte vector never straddles a row when hidden % V == 0; otherwise go pair by pair
    if (hidden % V == 0 && head_dim % V == 0 && n < 0x7fffffffLL) {
      // common case: a vector stays inside one head and 32-bit index arithmetic is enough
      const unsigned hid = (unsigned)hidden, hdm = (unsigned)head_dim, sl = (unsigned)S;
      return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
        float v[V], r[V];
        load_n(px + i, v, c);
        const unsigned iu = (unsigned)i;
        const unsigned row = iu / hid;
        const unsigned pos = row % sl;
        const unsigned p0 = ((iu - row * hid) % hdm) >> 1;  // first pair of this vector inside its head
        const float2* trow = tab + pos * half + p0;
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          const float2 cs = trow[k >> 1];
          const float sn = sgn * cs.y;
          r[k] = v[k] * cs.x - v[k + 1] * sn;
          r[k + 1] = v[k] * sn + v[k + 1] * cs.x;
        }
        store_acc_n(py + i, r, c, acc);
      }, "rope");
    }
    if (hidden % V == 0) {
      return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
        float v[V], r[V];
        load_n(px + i, v, c);
        const long long row = i / hidden;
        const int col = (int)(i - row * hidden);
        const int pos = (int)(row % S);
#pragma unroll
        for (int k = 0; k < V; k += 2) {
          const int pair = ((col + k) % (int)head_dim) >> 1;
          const float2 cs = tab[pos * half + pair];
          const float sn = sgn * cs.y;
          r[k] = v[k] * cs.x - v[k + 1] * sn;
          r[k + 1] = v[k] * sn + v[k + 1] * cs.x;
        }
        store_acc_n(py + i, r, c, acc);
      }, "rope");
    }
    return launch_vec<2>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      const long long row = i / hidden;
      const int col = (int)(i - row * hidden);
      const int pos = (int)(row % S);
      const int pair = (col % (int)head_dim) >> 1;
      const float2 cs = tab[pos * half + pair];
      const float sn = sgn * cs.y;
      const float a = to_f32(px[i]), b = to_f32(px[i + 1]);
      float r0 = a * cs.x - b * sn, r1 = a * sn + b * cs.x;
      if (acc) { r0 += to_f32(py[i]); r1 += to_f32(py[i + 1]); }
      py[i] = from_f32<T>(r0);
      py[i + 1] = from_f32<T>(r1);
    }, "rope_scalar");
  });
}

// ---------------------------------------------------------------------------------------
// layout ops
// ---------------------------------------------------------------------------------------
// y[b,h,s,:] (+)= x[b,s,h,:]  with x [B,S,H,D], y [B,H,S,D]
int eisen_transpose_0213(void* stream, const void* x, void* y, long long B, long long S, long long H,
                         long long D, int dt, int accumulate) {
  REQUIRE_ALIGNED(x, y);
  const long long n = B * S * H * D;
  const bool acc = accumulate != 0;
  EISEN_DISPATCH_DTYPE(dt, T, {
    constexpr int V = VecOf<T>::N;
    const T* px = (const T*)x; T* py = (T*)y;
    if (D % V == 0) {
      return launch_vec<V>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
        // i indexes the output [B,H,S,D]
        const long long d = i % D, s = (i / D) % S, h = (i / (D * S)) % H, b = i / (D * S * H);
        float v[V];
        load_n(px + ((b * S + s) * H + h) * D + d, v, c);
        store_acc_n(py + i, v, c, acc);
      }, "transpose_0213");
    }
    return launch_vec<1>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      const long long d = i % D, s = (i / D) % S, h = (i / (D * S)) % H, b = i / (D * S * H);
      float v = to_f32(px[((b * S + s) * H + h) * D + d]);
      if (acc) v += to_f32(py[i]);
      py[i] = from_f32<T>(v);
    }, "transpose_0213_scalar");
  });
}

// y[b, kv*r + j, s, :] = x[b, kv, s, :]   (src/graph/ops/gqa.rs:146-160)
int eisen_repeat_kv_fwd(void* stream, const void* x, void* y, long long B, long long KV, long long S,
                        long long D, long long r, int dt) {
  REQUIRE_ALIGNED(x, y);
  const long long n = B * KV * r * S * D;
  EISEN_DISPATCH_DTYPE(dt, T, {
    const T* px = (const T*)x; T* py = (T*)y;
    const long long SD = S * D;
    return launch_vec<1>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      const long long sd = i % SD, qh = (i / SD) % (KV * r), b = i / (SD * KV * r);
      py[i] = px[(b * KV + qh / r) * SD + sd];
    }, "repeat_kv_fwd");
  });
}
// dx[b, kv, s, :] (+)= sum_j dy[b, kv*r + j, s, :]   (src/graph/ops/gqa.rs:170-181)
int eisen_repeat_kv_bwd(void* stream, const void* dy, void* dx, long long B, long long KV, long long S,
                        long long D, long long r, int dt, int accumulate) {
  REQUIRE_ALIGNED(dy, dx);
  const long long n = B * KV * S * D;
  const bool acc = accumulate != 0;
  EISEN_DISPATCH_DTYPE(dt, T, {
    const T* pg = (const T*)dy; T* pd = (T*)dx;
    const long long SD = S * D;
    return launch_vec<1>((cudaStream_t)stream, n, [=] __device__(long long i, int c) {
      const long long sd = i % SD, kv = (i / SD) % KV, b = i / (SD * KV);
      float s = 0.0f;
      for (long long j = 0; j < r; ++j) s += to_f32(pg[(b * KV * r + kv * r + j) * SD + sd]);
      if (acc) s += to_f32(pd[i]);
      pd[i] = from_f32<T>(s);
    }, "repeat_kv_bwd");
  });
}

}  // extern "C"
