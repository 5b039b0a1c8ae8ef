// Internal interface of the tcgen05 GEMM (see gemm_tc.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace eisen {

enum GemmOutMode : int {
  GEMM_OUT_BF16 = 0,        // C(bf16)  = alpha * acc
  GEMM_OUT_BF16_ACC = 1,    // C(bf16) += alpha * acc
  GEMM_OUT_F32 = 2,         // C(f32)   = alpha * acc
  GEMM_OUT_F32_ACC = 3,     // C(f32)  += alpha * acc   (read-modify-write, one writer per element)
  GEMM_OUT_F32_ATOMIC = 4,  // C(f32)  += alpha * acc   (red.global.add, any number of writers)
  GEMM_OUT_BF16_ROPE = 5,   // C(bf16)  = rope(bf16(alpha * acc))   (paired kernel, complete tiles only)
};

// a_mn / b_mn: 0 = K-major operand ([rows][K]), 1 = MN-major operand ([K][rows]).
// Returns 0 on success; *err points at a static message otherwise.  Asynchronous on `stream`.
int gemm_bf16_tc(cudaStream_t stream, int a_mn, int b_mn, int M, int N, int K, const void* A,
                 long long lda, const void* B, long long ldb, void* C, long long ldc, const void* R, long long ldr,
                 int out_mode, int split_k, float alpha, int* status, const char** err);

// paired-CTA (cta_group::2) variant: 256 x 256 tile per cluster of two CTAs (gemm_tc2.cu)
int gemm_bf16_tc_pair(cudaStream_t stream, int a_mn, int b_mn, int M, int N, int K, const void* A, long long lda,
                      const void* B, long long ldb, void* C, long long ldc, const void* R, long long ldr, int out_mode,
                      int split_k, float alpha, int* status, const char** err);
// gate / up projections with the SwiGLU product in the epilogue (dual mode of the paired kernel)
int gemm_bf16_pair_swiglu(cudaStream_t stream, int M, int N, int K, const void* A, long long lda, const void* Bg,
                          const void* Bu, long long ldb, void* G, void* U, void* H, long long ldo, int* status,
                          const char** err);
// projection followed by interleaved-pair RoPE in the epilogue: rows are tokens of sequences of
// seq_len positions, columns are heads of head_dim; table is [seq_len][head_dim / 2] (cos, sin)
int gemm_bf16_pair_rope(cudaStream_t stream, int M, int N, int K, const void* A, long long lda, const void* B,
                        long long ldb, void* C, long long ldc, const float* table, int seq_len, int head_dim,
                        int* status, const char** err);
// C (op)= A1 B1^T + A2 B2^T + A3 B3^T in one pass over up to three operand pairs (K segments)
int gemm_bf16_pair_concat_k(cudaStream_t stream, int a_mn, int b_mn, int M, int N, int n_seg, const void* const* A,
                            const long long* lda, const void* const* B, const long long* ldb, const int* K, void* C,
                            long long ldc, const void* R, long long ldr, int out_mode, int split_k, float alpha,
                            int* status, const char** err);
// C_i (op)= A B_i^T for up to three B operands that share A, each with its own output (N segments)
int gemm_bf16_pair_multi_n(cudaStream_t stream, int a_mn, int b_mn, int M, int K, const void* A, long long lda, int n_seg,
                           const void* const* B, const long long* ldb, const int* N, void* const* C, const long long* ldc,
                           const int* out_mode, int split_k, float alpha, const float* rope_table, int seq_len,
                           int head_dim, int* status, const char** err);
int gemm_pair_auto_split_k(int M, int N, int K);
// m-tiles per band of the paired kernel's tile order; 0 = chosen by the DRAM-traffic model
void gemm_pair_set_band(int band);
int gemm_num_sms();
// SMs the persistent GEMM grids leave free (for a communication kernel that runs beside them)
int gemm_reserved_sms();
void gemm_set_reserved_sms(int n);

// split factor that fills the machine when M*N alone gives fewer tiles than SMs
int gemm_tc_auto_split_k(int M, int N, int K);

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer);
int make_tmap_bf16_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_elems, const uint32_t* box);
int make_tmap_f32_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_elems, const uint32_t* box);

}  // namespace eisen
