// Epilogue store of one 32-column chunk of an accumulator row, shared by the single-CTA and the
// paired-CTA GEMM kernels: bf16 / f32 store, read-modify-write accumulate, or f32 red.global.add.
#pragma once
#include "ptx.cuh"
#include "gemm_tc.h"

namespace eisen {

// v[0..32) = alpha-scaled accumulator values of row `row`, columns [col0, col0 + 32)
// Early load of the bf16 addend of one chunk (32 columns of one row), so that its latency overlaps
// the TMEM load and the stores of the chunk before.  Returns false when the chunk is ragged or
// unaligned; the store then reads the addend itself.
__device__ __forceinline__ bool gemm_prefetch_addend(const void* R, long long ldr, int row, int col0, int N, bool row_ok,
                                                     uint4 (&pre)[4]) {
  if (!row_ok || col0 + 32 > N) return false;
  const __nv_bfloat16* r_row = reinterpret_cast<const __nv_bfloat16*>(R) + (long long)row * ldr + col0;
  if (reinterpret_cast<uintptr_t>(r_row) & 15) return false;
#pragma unroll
  for (int j = 0; j < 4; ++j) pre[j] = reinterpret_cast<const uint4*>(r_row)[j];
  return true;
}

// In GEMM_OUT_BF16_ACC mode the addend is read from R (leading dimension ldr): R == C accumulates
// in place, another R adds a residual tensor while storing.  `pre` holds the addend when
// `have_pre` is set (see gemm_prefetch_addend).
__device__ __forceinline__ void gemm_store_chunk32(void* C, long long ldc, const void* R, long long ldr, int out_mode,
                                                   int row, int col0, int N, float (&v)[32], const uint4 (&pre)[4],
                                                   bool have_pre) {
  const bool full = (col0 + 32 <= N);
  if (out_mode == GEMM_OUT_BF16 || out_mode == GEMM_OUT_BF16_ACC) {
    __nv_bfloat16* c_row = reinterpret_cast<__nv_bfloat16*>(C) + (long long)row * ldc + col0;
    const __nv_bfloat16* r_row = reinterpret_cast<const __nv_bfloat16*>(R) + (long long)row * ldr + col0;
    const bool vec = full && ((reinterpret_cast<uintptr_t>(c_row) & 15) == 0) &&
                     (out_mode != GEMM_OUT_BF16_ACC || (reinterpret_cast<uintptr_t>(r_row) & 15) == 0);
    if (vec) {
      uint4* dst = reinterpret_cast<uint4*>(c_row);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (out_mode == GEMM_OUT_BF16_ACC) {
          uint4 old = have_pre ? pre[j] : reinterpret_cast<const uint4*>(r_row)[j];
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(o2[e]);
            v[j * 8 + 2 * e] += f.x;
            v[j * 8 + 2 * e + 1] += f.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
        o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
        o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
        o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
        dst[j] = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < N; ++i) {
        float x = v[i];
        if (out_mode == GEMM_OUT_BF16_ACC) x += __bfloat162float(r_row[i]);
        c_row[i] = __float2bfloat16(x);
      }
    }
  } else {
    float* c_row = reinterpret_cast<float*>(C) + (long long)row * ldc + col0;
    const bool vec = full && ((reinterpret_cast<uintptr_t>(c_row) & 15) == 0);
    if (out_mode == GEMM_OUT_F32_ATOMIC) {
      if (vec) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(c_row + 4 * j),
                       "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                       : "memory");
      } else {
        for (int i = 0; i < 32 && col0 + i < N; ++i) atomicAdd(c_row + i, v[i]);
      }
    } else if (vec) {
      float4* dst = reinterpret_cast<float4*>(c_row);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (out_mode == GEMM_OUT_F32_ACC) {
          float4 old = dst[j];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        dst[j] = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < N; ++i) {
        float x = v[i];
        if (out_mode == GEMM_OUT_F32_ACC) x += c_row[i];
        c_row[i] = x;
      }
    }
  }
}

}  // namespace eisen
