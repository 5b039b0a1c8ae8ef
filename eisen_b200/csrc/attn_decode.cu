// Attention of ONE new query position against the cached keys and values of the positions before
// it (autoregressive generation with a KV cache; the reference lists KV caching as future work,
// README.md:94, and re-runs the whole context per token, examples/train_llm.rs:560-584).
//
//   o[h, :] = softmax(scale * q[h, :] . K[0..n, h / r, :]^T) V[0..n, h / r, :]
//
// the chain bmm -> mul(scale) -> softmax -> bmm of src/nn/attention.rs:339-375 for a single row
// (the causal mask of that row admits every cached key).  Bandwidth-bound: the cache is read
// once.  One CTA per query head; each warp takes every 4th key, the lanes split head_dim, with an
// online maximum / sum per warp, merged over the warps at the end.
#include "common.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

constexpr int AD_WARPS = 4;
constexpr int AD_MAX_PER_LANE = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(AD_WARPS * 32)
attn_decode_kernel(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc, T* __restrict__ o,
                   int n_keys, int Hq, int Hkv, int D, long long row_stride, float scale) {
  __shared__ float sh_m[AD_WARPS], sh_s[AD_WARPS];
  __shared__ float sh_acc[AD_WARPS][256];
  const int h = blockIdx.x, kvh = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (D + 31) / 32;
  float qv[AD_MAX_PER_LANE], acc[AD_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < AD_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    qv[i] = (i < per && d < D) ? to_f32(q[(long long)h * D + d]) * scale : 0.0f;
    acc[i] = 0.0f;
  }
  float m = -INFINITY, s = 0.0f;
  for (int j = warp; j < n_keys; j += AD_WARPS) {
    const T* kr = kc + (long long)j * row_stride + (long long)kvh * D;
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < AD_MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (i < per && d < D) dot += qv[i] * to_f32(kr[d]);
    }
    dot = warp_sum(dot);
    const float nm = fmaxf(m, dot);
    const float corr = expf(m - nm), p = expf(dot - nm);
    s = s * corr + p;
    const T* vr = vc + (long long)j * row_stride + (long long)kvh * D;
#pragma unroll
    for (int i = 0; i < AD_MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (i < per && d < D) acc[i] = acc[i] * corr + p * to_f32(vr[d]);
    }
    m = nm;
  }
  if (lane == 0) { sh_m[warp] = m; sh_s[warp] = s; }
#pragma unroll
  for (int i = 0; i < AD_MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (i < per && d < D) sh_acc[warp][d] = acc[i];
  }
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int w = 0; w < AD_WARPS; ++w) gm = fmaxf(gm, sh_m[w]);
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < AD_WARPS; ++w) total += (sh_m[w] == -INFINITY) ? 0.0f : sh_s[w] * expf(sh_m[w] - gm);
  for (int d = threadIdx.x; d < D; d += AD_WARPS * 32) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < AD_WARPS; ++w)
      if (sh_m[w] != -INFINITY) v += sh_acc[w][d] * expf(sh_m[w] - gm);
    o[(long long)h * D + d] = from_f32<T>(v / total);
  }
}

}  // namespace
}  // namespace eisen

extern "C" int eisen_attn_decode(void* stream, const void* q, const void* k_cache, const void* v_cache, void* o,
                                 long long n_keys, long long Hq, long long Hkv, long long D, long long cache_row_stride,
                                 float scale, int dtype) {
  using namespace eisen;
  if (n_keys <= 0 || Hq <= 0) return fail(EISEN_ERR_INVALID, "attn_decode: needs at least one cached key and one head");
  if (Hkv <= 0 || Hq % Hkv) return fail(EISEN_ERR_INVALID, "attn_decode: Hq must be a multiple of Hkv");
  if (D <= 0 || D > 256) return fail(EISEN_ERR_INVALID, "attn_decode: head_dim must be in [1, 256]");
  if (cache_row_stride < Hkv * D) return fail(EISEN_ERR_INVALID, "attn_decode: cache rows are shorter than Hkv * head_dim");
  if (n_keys > 0x7fffffffLL) return fail(EISEN_ERR_LIMIT, "attn_decode: more than 2^31-1 keys");
  EISEN_DISPATCH_DTYPE(dtype, T, {
    attn_decode_kernel<T><<<(unsigned)Hq, AD_WARPS * 32, 0, (cudaStream_t)stream>>>(
        (const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)o, (int)n_keys, (int)Hq, (int)Hkv, (int)D, cache_row_stride, scale);
    return check_launch("attn_decode");
  });
}
