// C entry points of the tcgen05 GEMMs (eisen_gemm_bf16 and its fused-epilogue variants) and the
// choice between the single-CTA (gemm_tc.cu) and the paired-CTA (gemm_tc2.cu) kernel.
#include "errors.h"
#include "gemm_tc.h"
#include "../../include/eisen_b200.h"

#include <atomic>

namespace eisen {
static std::atomic<int> g_gemm_mode{0};  // 0 = choose per shape, 1 = single-CTA tiles only, 2 = paired-CTA tiles only
}

extern "C" {

int eisen_gemm_set_mode(int mode) {
  if (mode < 0 || mode > 2) return eisen::fail(EISEN_ERR_INVALID, "gemm_set_mode: mode must be 0, 1 or 2");
  eisen::g_gemm_mode.store(mode);
  return 0;
}

int eisen_gemm_set_band(int band) {
  if (band < 0) return eisen::fail(EISEN_ERR_INVALID, "gemm_set_band: band must be >= 0");
  eisen::gemm_pair_set_band(band);
  return 0;
}

int eisen_gemm_reserve_sms(int n) {
  if (n < 0 || n > 64) return eisen::fail(EISEN_ERR_INVALID, "gemm_reserve_sms: n must be in [0, 64]");
  eisen::gemm_set_reserved_sms(n);
  return 0;
}

static int gemm_dispatch(void* stream, int a_mn, int b_mn, long long M, long long N, long long K, const void* A,
                         long long lda, const void* B, long long ldb, void* C, long long ldc, const void* R, long long ldr,
                         int out_mode, int split_k, float alpha, int* status) {
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL)
    return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16: a dimension exceeds 2^31-1");
  if (out_mode < 0 || out_mode > 4) return eisen::fail(EISEN_ERR_INVALID, "gemm_bf16: bad out_mode");  // mode 5 has its own entry point
  // tile shape: the paired-CTA kernel (256 x 256 per cluster) when the problem has at least one
  // full pair tile in each dimension, else the single-CTA kernel (128 x 256)
  const int mode = eisen::g_gemm_mode.load();
  const bool pair = mode == 2 || (mode == 0 && M >= 256 && N >= 128);
  if (split_k == 0) {
    if (out_mode != eisen::GEMM_OUT_F32_ATOMIC || eisen::deterministic()) split_k = 1;  // one writer per element
    else split_k = pair ? eisen::gemm_pair_auto_split_k((int)M, (int)N, (int)K) : eisen::gemm_tc_auto_split_k((int)M, (int)N, (int)K);
  }
  const char* err = nullptr;
  int rc = pair ? eisen::gemm_bf16_tc_pair((cudaStream_t)stream, a_mn, b_mn, (int)M, (int)N, (int)K, A, lda, B, ldb, C, ldc,
                                           R, ldr, out_mode, split_k, alpha, status, &err)
                : eisen::gemm_bf16_tc((cudaStream_t)stream, a_mn, b_mn, (int)M, (int)N, (int)K, A, lda, B, ldb, C, ldc,
                                      R, ldr, out_mode, split_k, alpha, status, &err);
  if (rc) return eisen::fail(rc == 1 ? EISEN_ERR_INVALID : EISEN_ERR_CUDA, err ? err : "gemm_bf16 failed");
  if (M > 0 && N > 0 && K > 0) eisen::count_launch();
  return 0;
}

int eisen_gemm_bf16(void* stream, int a_mn, int b_mn, long long M, long long N, long long K, const void* A,
                    long long lda, const void* B, long long ldb, void* C, long long ldc, int out_mode,
                    int split_k, float alpha, int* status) {
  return gemm_dispatch(stream, a_mn, b_mn, M, N, K, A, lda, B, ldb, C, ldc, nullptr, 0, out_mode, split_k, alpha, status);
}

int eisen_gemm_bf16_residual(void* stream, int a_mn, int b_mn, long long M, long long N, long long K, const void* A,
                             long long lda, const void* B, long long ldb, const void* R, long long ldr, void* C,
                             long long ldc, float alpha, int* status) {
  if (!R) return eisen::fail(EISEN_ERR_INVALID, "gemm_bf16_residual: R is null");
  return gemm_dispatch(stream, a_mn, b_mn, M, N, K, A, lda, B, ldb, C, ldc, R, ldr, eisen::GEMM_OUT_BF16_ACC, 1, alpha, status);
}

int eisen_gemm_bf16_rope(void* stream, long long M, long long N, long long K, const void* A, long long lda, const void* B,
                         long long ldb, void* C, long long ldc, const float* table_cos_sin, long long seq_len,
                         long long head_dim, int* status) {
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL || seq_len > 0x7fffffffLL || head_dim > 0x7fffffffLL)
    return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16_rope: a dimension exceeds 2^31-1");
  const char* err = nullptr;
  int rc = eisen::gemm_bf16_pair_rope((cudaStream_t)stream, (int)M, (int)N, (int)K, A, lda, B, ldb, C, ldc, table_cos_sin,
                                      (int)seq_len, (int)head_dim, status, &err);
  if (rc) return eisen::fail(rc == 1 ? EISEN_ERR_INVALID : EISEN_ERR_CUDA, err ? err : "gemm_bf16_rope failed");
  if (M > 0 && N > 0 && K > 0) eisen::count_launch();
  return 0;
}

int eisen_gemm_bf16_swiglu(void* stream, long long M, long long N, long long K, const void* A, long long lda,
                           const void* Bg, const void* Bu, long long ldb, void* G, void* U, void* H, long long ldo,
                           int* status) {
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL)
    return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16_swiglu: a dimension exceeds 2^31-1");
  const char* err = nullptr;
  int rc = eisen::gemm_bf16_pair_swiglu((cudaStream_t)stream, (int)M, (int)N, (int)K, A, lda, Bg, Bu, ldb, G, U, H, ldo,
                                        status, &err);
  if (rc) return eisen::fail(rc == 1 ? EISEN_ERR_INVALID : EISEN_ERR_CUDA, err ? err : "gemm_bf16_swiglu failed");
  if (M > 0 && N > 0 && K > 0) eisen::count_launch();
  return 0;
}

int eisen_gemm_bf16_concat_k(void* stream, int a_mn, int b_mn, long long M, long long N, int n_seg, const void* const* A,
                             const long long* lda, const void* const* B, const long long* ldb, const long long* K,
                             void* C, long long ldc, int out_mode, int split_k, float alpha, int* status) {
  if (n_seg < 1 || n_seg > 3 || !A || !B || !lda || !ldb || !K)
    return eisen::fail(EISEN_ERR_INVALID, "gemm_bf16_concat_k: 1 to 3 segments, no null arrays");
  if (out_mode < 0 || out_mode > 4) return eisen::fail(EISEN_ERR_INVALID, "gemm_bf16_concat_k: bad out_mode");
  int k32[3];
  long long ktotal = 0;
  for (int i = 0; i < n_seg; ++i) {
    if (K[i] > 0x7fffffffLL) return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16_concat_k: a dimension exceeds 2^31-1");
    k32[i] = (int)K[i];
    ktotal += K[i];
  }
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || ktotal > 0x7fffffffLL)
    return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16_concat_k: a dimension exceeds 2^31-1");
  if (split_k == 0)
    split_k = (out_mode == eisen::GEMM_OUT_F32_ATOMIC && !eisen::deterministic())
                  ? eisen::gemm_pair_auto_split_k((int)M, (int)N, (int)ktotal) : 1;
  const char* err = nullptr;
  int rc = eisen::gemm_bf16_pair_concat_k((cudaStream_t)stream, a_mn, b_mn, (int)M, (int)N, n_seg, A, lda, B, ldb, k32, C, ldc,
                                          nullptr, 0, out_mode, split_k, alpha, status, &err);
  if (rc) return eisen::fail(rc == 1 ? EISEN_ERR_INVALID : EISEN_ERR_CUDA, err ? err : "gemm_bf16_concat_k failed");
  if (M > 0 && N > 0) eisen::count_launch();
  return 0;
}

int eisen_gemm_bf16_multi_n(void* stream, int a_mn, int b_mn, long long M, long long K, const void* A, long long lda,
                            int n_seg, const void* const* B, const long long* ldb, const long long* N, void* const* C,
                            const long long* ldc, const int* out_mode, int split_k, float alpha,
                            const float* table_cos_sin, long long seq_len, long long head_dim, int* status) {
  if (n_seg < 1 || n_seg > 3 || !B || !ldb || !N || !C || !ldc || !out_mode)
    return eisen::fail(EISEN_ERR_INVALID, "gemm_bf16_multi_n: 1 to 3 segments, no null arrays");
  int n32[3];
  long long ntotal = 0;
  for (int i = 0; i < n_seg; ++i) {
    if (N[i] > 0x7fffffffLL) return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16_multi_n: a dimension exceeds 2^31-1");
    if (out_mode[i] < 0 || out_mode[i] > 5 || out_mode[i] == eisen::GEMM_OUT_BF16_ACC)
      return eisen::fail(EISEN_ERR_INVALID, "gemm_bf16_multi_n: output modes 0 (bf16), 2 (f32), 4 (f32 add) and 5 (bf16 + RoPE)");
    n32[i] = (int)N[i];
    ntotal += N[i];
  }
  if (M > 0x7fffffffLL || K > 0x7fffffffLL || ntotal > 0x7fffffffLL || seq_len > 0x7fffffffLL || head_dim > 0x7fffffffLL)
    return eisen::fail(EISEN_ERR_LIMIT, "gemm_bf16_multi_n: a dimension exceeds 2^31-1");
  const char* err = nullptr;
  int rc = eisen::gemm_bf16_pair_multi_n((cudaStream_t)stream, a_mn, b_mn, (int)M, (int)K, A, lda, n_seg, B, ldb, n32, C, ldc,
                                         out_mode, split_k, alpha, table_cos_sin, (int)seq_len, (int)head_dim, status, &err);
  if (rc) return eisen::fail(rc == 1 ? EISEN_ERR_INVALID : EISEN_ERR_CUDA, err ? err : "gemm_bf16_multi_n failed");
  if (M > 0 && K > 0) eisen::count_launch();
  return 0;
}

}  // extern "C"
