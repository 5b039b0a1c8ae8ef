// Fused AdamW over a flat parameter buffer and the global gradient-norm reduction.
// Reference: adamw_step_f32 (kernels/ops_f32.cu:762-784) launched once per parameter tensor and
// a host-side f64 norm over gradients copied back to the host (src/nn/optim.rs:250-289).  Here:
// one launch over the flat buffer, 16-byte accesses, the clip coefficient and the data-parallel
// 1/world scale folded in, an optional bf16 shadow copy of the weights written in the same pass,
// and the norm reduced on the device in f64.
#include "common.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

constexpr int OPT_THREADS = 256;

// update of src/nn/optim.rs:537-542:
//   w *= 1 - lr*wd ; m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ; w -= lr*(m*bc1)/(sqrt(v*bc2)+eps)
__device__ __forceinline__ void adamw_one(float& w, float g, float& m, float& v, float lr, float b1, float b2,
                                          float eps, float wd, float bc1, float bc2) {
  const float decayed = w * (1.0f - lr * wd);
  m = b1 * m + (1.0f - b1) * g;
  v = b2 * v + (1.0f - b2) * g * g;
  const float mh = m * bc1, vh = v * bc2;
  w = decayed - lr * mh / (sqrtf(vh) + eps);
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ZERO_G: the gradient is cleared as it is read, so that no separate memset stands between this step and
// the next backward pass
template <bool ZERO_G>
__global__ void __launch_bounds__(OPT_THREADS)
adamw_kernel(float* __restrict__ w, __nv_bfloat16* __restrict__ w_bf16, float* __restrict__ g,
             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1, float b2, float eps,
             float wd, float bc1, float bc2, float grad_scale, const double* __restrict__ sumsq,
             float max_norm, const float* __restrict__ hyper) {
  // step-dependent scalars from device memory (a launch recorded once and replayed every step)
  if (hyper != nullptr) { lr = hyper[0]; bc1 = hyper[1]; bc2 = hyper[2]; }
  float gs = grad_scale;
  if (sumsq != nullptr && max_norm > 0.0f) {
    // clip coefficient of src/nn/optim.rs:283-287 applied to the scaled gradient
    const float norm = (float)sqrt(*sumsq) * fabsf(grad_scale);
    if (norm > 0.0f) gs *= fminf(max_norm / (norm + 1e-6f), 1.0f);
  }
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 w4 = reinterpret_cast<float4*>(w)[i];
    const float4 g4 = reinterpret_cast<const float4*>(g)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    adamw_one(w4.x, g4.x * gs, m4.x, v4.x, lr, b1, b2, eps, wd, bc1, bc2);
    adamw_one(w4.y, g4.y * gs, m4.y, v4.y, lr, b1, b2, eps, wd, bc1, bc2);
    adamw_one(w4.z, g4.z * gs, m4.z, v4.z, lr, b1, b2, eps, wd, bc1, bc2);
    adamw_one(w4.w, g4.w * gs, m4.w, v4.w, lr, b1, b2, eps, wd, bc1, bc2);
    reinterpret_cast<float4*>(w)[i] = w4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    if (ZERO_G) reinterpret_cast<float4*>(g)[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (w_bf16) {
      uint2 o;
      o.x = pack2(w4.x, w4.y);
      o.y = pack2(w4.z, w4.w);
      reinterpret_cast<uint2*>(w_bf16)[i] = o;
    }
  }
  // ragged tail (n % 4 elements)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (nvec << 2) + threadIdx.x;
    float ww = w[i], mm = m[i], vv = v[i];
    adamw_one(ww, g[i] * gs, mm, vv, lr, b1, b2, eps, wd, bc1, bc2);
    w[i] = ww; m[i] = mm; v[i] = vv;
    if (ZERO_G) g[i] = 0.0f;
    if (w_bf16) w_bf16[i] = __float2bfloat16(ww);
  }
}

__global__ void __launch_bounds__(OPT_THREADS)
sumsq_partial_kernel(const float* __restrict__ x, long long n, double* __restrict__ partial) {
  __shared__ double sh[OPT_THREADS / 32];
  double acc = 0.0;
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 t = reinterpret_cast<const float4*>(x)[i];
    // squares in f32 are exact enough per element; the running sum is f64
    acc += (double)t.x * (double)t.x + (double)t.y * (double)t.y + (double)t.z * (double)t.z +
           (double)t.w * (double)t.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float t = x[(nvec << 2) + threadIdx.x];
    acc += (double)t * (double)t;
  }
  acc = warp_sum_d(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int i = 0; i < OPT_THREADS / 32; ++i) s += sh[i];
    partial[blockIdx.x] = s;
  }
}

__global__ void sumsq_final_kernel(const double* __restrict__ partial, int nparts, double* __restrict__ out,
                                   int accumulate) {
  // one warp, fixed order
  double s = 0.0;
  for (int i = threadIdx.x; i < nparts; i += 32) s += partial[i];
  s = warp_sum_d(s);
  if (threadIdx.x == 0) *out = accumulate ? *out + s : s;
}

}  // namespace

int sumsq_grid(long long n) { return grid_for(n >> 2, OPT_THREADS * 4, 4); }

}  // namespace eisen

using namespace eisen;

extern "C" {

// One AdamW step over n contiguous f32 elements.  w_bf16 (may be null) receives the updated
// weights rounded to bf16.  The gradient is read as g * grad_scale; when sumsq (device f64,
// the squared L2 norm of the unscaled gradient) is not null and max_norm > 0 the global clip
// coefficient min(1, max_norm / (norm + 1e-6)) is applied as well.
int eisen_adamw_step(void* stream, float* w, void* w_bf16, const float* g, float* m, float* v, long long n,
                     float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                     float grad_scale, const double* sumsq, float max_norm) {
  return eisen_adamw_step_dev(stream, w, w_bf16, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale,
                              sumsq, max_norm, nullptr);
}

// As eisen_adamw_step; when hyper (device float[3]) is not null the kernel takes lr, bc1 and bc2 from
// it instead of from the arguments.
int eisen_adamw_step_dev(void* stream, float* w, void* w_bf16, const float* g, float* m, float* v, long long n,
                         float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                         float grad_scale, const double* sumsq, float max_norm, const float* hyper) {
  return eisen_adamw_step_ex(stream, w, w_bf16, const_cast<float*>(g), m, v, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2,
                             grad_scale, sumsq, max_norm, hyper, 0);
}

// As eisen_adamw_step_dev; zero_grad != 0 clears g while it is read.
int eisen_adamw_step_ex(void* stream, float* w, void* w_bf16, float* g, float* m, float* v, long long n, float lr,
                        float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2, float grad_scale,
                        const double* sumsq, float max_norm, const float* hyper, int zero_grad) {
  if (n <= 0) return 0;
  if (!aligned16(w) || !aligned16(g) || !aligned16(m) || !aligned16(v) || (w_bf16 && (reinterpret_cast<uintptr_t>(w_bf16) & 7)))
    return fail(EISEN_ERR_INVALID, "adamw_step: buffers must be 16-byte aligned");
  const int grid = grid_for(n >> 2, OPT_THREADS, 8);
  if (zero_grad)
    adamw_kernel<true><<<grid, OPT_THREADS, 0, (cudaStream_t)stream>>>(w, (__nv_bfloat16*)w_bf16, g, m, v, n, lr, beta1, beta2, eps,
                                                                      weight_decay, bc1, bc2, grad_scale, sumsq, max_norm, hyper);
  else
    adamw_kernel<false><<<grid, OPT_THREADS, 0, (cudaStream_t)stream>>>(w, (__nv_bfloat16*)w_bf16, g, m, v, n, lr, beta1, beta2, eps,
                                                                       weight_decay, bc1, bc2, grad_scale, sumsq, max_norm, hyper);
  return check_launch("adamw_step");
}

long long eisen_sumsq_workspace_bytes(long long n) { return (long long)sumsq_grid(n) * 8 + 64; }

// *out (device f64) (+)= sum of x[i]^2, reduced in f64 in a fixed order
int eisen_sumsq(void* stream, const float* x, long long n, void* workspace, double* out, int accumulate) {
  if (!aligned16(x)) return fail(EISEN_ERR_INVALID, "sumsq: x must be 16-byte aligned");
  if (!workspace) return fail(EISEN_ERR_INVALID, "sumsq: workspace is null");
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = sumsq_grid(n);
  sumsq_partial_kernel<<<grid, OPT_THREADS, 0, s>>>(x, n, (double*)workspace);
  int rc = check_launch("sumsq_partial");
  if (rc) return rc;
  sumsq_final_kernel<<<1, 32, 0, s>>>((const double*)workspace, grid, out, accumulate);
  return check_launch("sumsq_final");
}

}  // extern "C"
