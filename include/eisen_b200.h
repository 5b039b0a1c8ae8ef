/*
 * eisen_b200 — C ABI of the B200-native (sm_100a) training-step hot path of philsupertramp/eisen.
 *
 * Two layers are exported from libeisen_b200.so:
 *
 *  (1) Kernel level (this first half): one entry point per device operation.  These replace the
 *      `stream.launch_builder(&f).arg(..).launch(cfg)` calls in the `Device::Gpu` arms of the
 *      reference's `impl Graph` ops (src/graph/ops/*.rs) and of `AdamW` (src/nn/optim.rs).
 *      Plain pointers and sizes only; every call is asynchronous on the given CUDA stream
 *      (`void* stream` is a `cudaStream_t`), performs no allocation and no synchronisation, and
 *      keeps no pointer after it returns.  Scratch memory is passed in by the caller and sized by
 *      the matching `*_workspace_bytes` query.
 *
 *  (2) Graph level (second half): the host-side mirror of the reference's `Graph` / tape / nn
 *      modules / AdamW, driven through opaque handles, for callers that want the whole engine
 *      behaviour (tensor ids, Wengert-list backward, pooled activations, save points).
 *
 * Conventions
 *   - return value: 0 = success, otherwise an `EISEN_ERR_*` code; eisen_last_error() gives the
 *     message of the last failure on the calling thread.  Nothing aborts.
 *   - dtype arguments: EISEN_F32 or EISEN_BF16.  Gradient ("d*") outputs take an `accumulate`
 *     flag: 0 writes, 1 adds to what is there (the reference's kernels always add,
 *     kernels/ops_f32.cu, except bmm_backward_* which overwrite).
 *   - all tensors are row-major and contiguous unless strides are passed.
 */
#ifndef EISEN_B200_H
#define EISEN_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#define EISEN_F32 0
#define EISEN_BF16 1
#define EISEN_F64 3 /* eisen_dp_* only: the squared gradient norm */
#define EISEN_I64 4 /* eisen_dp_* only: counters of a host-side handshake */

#define EISEN_OK 0
#define EISEN_ERR_INVALID 1
#define EISEN_ERR_CUDA 2
#define EISEN_ERR_KERNEL 3
#define EISEN_ERR_OOM 4
#define EISEN_ERR_LIMIT 5
#define EISEN_ERR_COMM 6    /* NCCL missing, reported an error, or the communicator was aborted */
#define EISEN_ERR_TIMEOUT 7 /* eisen_dp_wait ran past its deadline (the communicator is aborted) */

/* message of the last failed call on this thread ("" if none) */
const char* eisen_last_error(void);
/* version string of the library */
const char* eisen_version(void);
/* number of kernels this library has launched in the process so far */
long long eisen_launch_count(void);
/* Fixed-order arithmetic (process-wide, default off).  Three kernels of the Bf16Mixed path add f32 values in
 * an order that varies from run to run: weight-gradient GEMMs that split the token dimension over several
 * SM clusters (red.global.add), the attention backward, whose key-tile CTAs add their dQ tiles to one
 * buffer, and the staged RMSNorm backward on bf16 rows, whose CTAs add their column sums of dw to one vector.  With the
 * switch on, a weight-gradient GEMM whose split is left to the library uses one slice per tile, the
 * attention backward writes every key tile's dQ to its own slice of the workspace
 * (eisen_attn_bwd_workspace_bytes grows by the number of key tiles) and sums the slices in key order, and
 * the RMSNorm backward writes per-CTA partials that a second launch adds in CTA order: gradients are then
 * bit-identical from run to run, at a few percent of step time.  The reference's
 * kernels have no atomics on this path (one thread per output element), so they are run-to-run exact too. */
int eisen_set_deterministic(int on);
int eisen_get_deterministic(void);

/* Self-test of the bounded waits inside the pipelined kernels (no counterpart in the reference,
 * whose kernels do not wait on one another): one warp waits budget_cycles on a barrier nobody
 * signals, gives up, and writes fault code 99 into *status (device int) the way a stuck kernel
 * would.  report5 (device int[5], may be null): first wait succeeded, second wait succeeded, abort
 * flag, first wait used its budget, second wait returned at once. */
int eisen_selftest_bounded_wait(void* stream, int* status, long long budget_cycles, int* report5);

/* ------------------------------------------------------------------------------------------
 * Dense contractions
 * ------------------------------------------------------------------------------------------ */

/* bf16 x bf16 -> f32-accumulated GEMM on tcgen05 tensor cores (TMA-fed, TMEM accumulators).
 *   C[M,N] (op)= alpha * sum_k A(m,k) * B(n,k)
 * a_mn / b_mn = 0: operand stored [rows][K] (K contiguous); 1: stored [K][rows].
 * out_mode: 0 bf16 store, 1 bf16 accumulate, 2 f32 store, 3 f32 accumulate, 4 f32 atomic
 * accumulate (required for split_k > 1; split_k = 0 lets the library choose).
 * status (device int, may be null) receives a non-zero code if a bounded wait inside the kernel
 * ran out.  Leading dimensions of A and B must be multiples of 8 elements, bases 16-byte aligned.
 * Replaces matmul_f32 / matmul_backward_a_f32 / matmul_backward_b_f32 (kernels/ops_f32.cu:158-259),
 * matmul_trans_b_f32 / matmul_trans_a_f32 (842-882) and the bf16-operand variants
 * (kernels/ops_bf16.cu:26-223) launched from src/graph/ops/linear.rs:136-213, 402-481, 615-730. */
int eisen_gemm_bf16(void* stream, int a_mn, int b_mn, long long M, long long N, long long K, const void* A,
                    long long lda, const void* B, long long ldb, void* C, long long ldc, int out_mode,
                    int split_k, float alpha, int* status);

/* C(bf16)[M,N] = alpha * sum_k A(m,k) B(n,k) + R(bf16)[M,N]: the residual add of
 * src/nn/transformer.rs:36 and :47 (`g.add(x, attn_out)`, `g.add(res1, ffn2_out)`) done in the
 * epilogue of the projection that produces the second addend.  R may not alias C. */
int eisen_gemm_bf16_residual(void* stream, int a_mn, int b_mn, long long M, long long N, long long K, const void* A,
                             long long lda, const void* B, long long ldb, const void* R, long long ldr, void* C,
                             long long ldc, float alpha, int* status);
/* A projection followed by RoPE (src/nn/attention.rs:320-333: Linear, then rope on q and k), with
 * the rotation in the GEMM epilogue: C = bf16(rope(A B)), rotated in f32 and rounded once.  A is [M,K] row-major with M = batch *
 * seq_len token rows, B the [K,N] weight, table_cos_sin the table of eisen_rope_table for
 * (seq_len, head_dim).  M and N must be multiples of 256, head_dim a multiple of 8 dividing N. */
int eisen_gemm_bf16_rope(void* stream, long long M, long long N, long long K, const void* A, long long lda, const void* B,
                         long long ldb, void* C, long long ldc, const float* table_cos_sin, long long seq_len,
                         long long head_dim, int* status);
/* Backward of the three projections of GroupedQueryAttention::forward_with_mask
 * (src/nn/attention.rs:316-318: q_proj, k_proj, v_proj on the same input) as two launches instead
 * of six.  The reference runs matmul's backward closure three times (src/graph/ops/linear.rs:
 * 615-730), each adding its `dC W^T` into the input's gradient and writing its own dW.
 *
 * eisen_gemm_bf16_concat_k: C[M,N] (op)= alpha * sum_i sum_k A_i(m,k) B_i(n,k) over n_seg <= 3 operand
 * pairs with their own K_i (every K_i but the last a multiple of 64): the three `dC W^T` products
 * summed in the f32 accumulator in one pass, no bf16 rounding or read-modify-write in between.
 * Operand conventions, out_mode and split_k as in eisen_gemm_bf16; all pairs share a_mn / b_mn.
 *
 * eisen_gemm_bf16_multi_n: C_i[M,N_i] (op)= alpha * sum_k A(m,k) B_i(n,k) for n_seg <= 3 B operands that
 * share A, each with its own output matrix, leading dimension and out_mode (0, 2, 4 or 5; every N_i but
 * the last a multiple of 256): the three `A^T dC` weight gradients in one launch (out_mode 4, split_k 0
 * = chosen for the whole tile set), or the three forward projections with RoPE on some of them
 * (out_mode 5 uses table_cos_sin / seq_len / head_dim as eisen_gemm_bf16_rope does). */
int eisen_gemm_bf16_concat_k(void* stream, int a_mn, int b_mn, long long M, long long N, int n_seg, const void* const* A,
                             const long long* lda, const void* const* B, const long long* ldb, const long long* K,
                             void* C, long long ldc, int out_mode, int split_k, float alpha, int* status);
int eisen_gemm_bf16_multi_n(void* stream, int a_mn, int b_mn, long long M, long long K, const void* A, long long lda,
                            int n_seg, const void* const* B, const long long* ldb, const long long* N, void* const* C,
                            const long long* ldc, const int* out_mode, int split_k, float alpha,
                            const float* table_cos_sin, long long seq_len, long long head_dim, int* status);
/* Gate and up projections of the SiLU-gated MLP with the product in the GEMM epilogue
 * (src/nn/transformer.rs:41-44: Linear, Linear, silu, mul):
 *   G = bf16(A Bg), U = bf16(A Bu), H = bf16(silu(G) * U)
 * A is [M,K] row-major, Bg / Bu are the [K,N] weights (leading dimension ldb), G / U / H are
 * [M,N] bf16 with leading dimension ldo.  G and U may be null (a forward pass that keeps nothing
 * for a backward pass).  M must be a multiple of 256 and N of 128. */
int eisen_gemm_bf16_swiglu(void* stream, long long M, long long N, long long K, const void* A, long long lda,
                           const void* Bg, const void* Bu, long long ldb, void* G, void* U, void* H, long long ldo,
                           int* status);

/* Tile shape of eisen_gemm_bf16: 0 = chosen per problem shape, 1 = single-CTA 128x256 tiles,
 * 2 = paired-CTA 256x256 tiles (tcgen05 cta_group::2, one cluster of two CTAs per tile).
 * Process-wide; meant for tests and measurements. */
int eisen_gemm_set_mode(int mode);
/* Tile order of the paired-CTA kernel: the 256-row tiles are walked in bands of `band` tiles (all
 * column tiles of a band before the next band).  0 = chosen per problem from a DRAM-traffic model,
 * which only leaves the plain column-major order for operands beyond the L2 size.  Process-wide;
 * meant for tests and measurements. */
int eisen_gemm_set_band(int band);
/* The tensor-core GEMMs are persistent kernels, one CTA per SM.  A collective that should run
 * beside them (the gradient all-reduce of a data-parallel step, on its own stream) finds no SM
 * until they exit; n > 0 makes every later GEMM launch leave n SMs free.  No counterpart in the
 * reference (single GPU).  Default 0. */
int eisen_gemm_reserve_sms(int n);

/* f32 SIMT GEMM with element strides and a batch dimension (f32 parity path):
 *   C[b,m,n] (+)= sum_k A[b*a_bs + m*a_ms + k*a_ks] * B[b*b_bs + k*b_ks + n*b_ns]
 * Replaces the same reference kernels for f32 tensors plus bmm_f32 and bmm_backward_*
 * (kernels/ops_f32.cu:342-511; src/graph/ops/linear.rs:1302-1386). */
int eisen_gemm_f32_strided(void* stream, const float* A, const float* B, float* C, long long batch, long long M,
                           long long N, long long K, long long a_bs, long long a_ms, long long a_ks,
                           long long b_bs, long long b_ks, long long b_ns, long long c_bs, long long ldc,
                           int accumulate);

/* ------------------------------------------------------------------------------------------
 * Flash attention with grouped-query heads (bf16, tcgen05).  Layout of all tensors: [B, S, H, D]
 * with explicit element strides for batch, sequence and head (D contiguous), so the projections'
 * [B,S,hidden] outputs are consumed in place: no reshape / transpose_0213 / repeat_kv copies
 * (src/nn/attention.rs:305-331, 379-384).  Query head h reads KV head h / (Hq/Hkv).
 * Forward replaces flash_attention_f32 (kernels/ops_f32.cu:648-692, inference only in the
 * reference, src/graph/ops/attention.rs:15-18) and the training chain bmm -> mul -> add(mask)
 * -> softmax -> bmm (src/nn/attention.rs:339-375); backward replaces that chain's gradient
 * kernels (bmm_backward_*, softmax_backward_f32, mul/add backward, repeat_kv_backward).
 * lse: [B, Hq, S] f32 log-sum-exp of the scaled, masked scores (natural log).
 * ------------------------------------------------------------------------------------------ */
int eisen_attn_fwd(void* stream, const void* q, const void* k, const void* v, void* o, float* lse, long long B,
                   long long S, long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss,
                   long long q_hs, long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs,
                   long long o_ss, long long o_hs, float scale, int causal, int* status);
/* The extended pair, for the accuracy of dq and dk in deep models.  dS = P * (dP - delta) subtracts two
 * numbers that both carry the common component of the value vectors (dP = dO . V_j, delta = dO . O); rounding
 * errors of O (bf16) and of P (bf16 inside P V) scale with that component while the difference does not, and
 * the value vectors of a deep model share a large mean: against the f32 path the gradients of the q and k
 * weights were off by 3e-2 (relative L2) at 16 blocks where all other gradients were within 1.6e-2.
 *   eisen_attn_center_values: mean[B, Hkv, D] (f32) = mean of v over the sequence, v_centered (bf16,
 *     contiguous [B, S, Hkv, D]) = v - mean.  v may be f32 (v_dtype = EISEN_F32; strides in elements): a value
 *     projection that writes f32 and is rounded only after the subtraction keeps the token-specific part of v
 *     to bf16 precision, where rounding v itself loses it to the common component.
 *   eisen_attn_fwd_ex with v = v_centered and v_mean = mean: o = bf16(P V_c + mean) (the same output) and
 *     o_aux (bf16, O's strides, may be null) = bf16(P V_c), the centred output.
 *   eisen_attn_bwd_ex with v = v_centered, o = that centred output: delta = dO . O_c and dP = dO . V_c differ
 *     by the same constant from the uncentred ones, so dS, dq, dk are the same numbers computed without the
 *     cancellation, and dv = P^T dO does not see the shift at all.
 * Without v_mean (null) the forward is eisen_attn_fwd and o_aux, if given, receives what the rounding of O
 * drops (o_f32 - float(bf16(o_f32))); eisen_attn_bwd_ex then takes it as o_lo and forms delta from O + O_lo,
 * which removes the rounding error of O but not that of P.  table_cos_sin as in eisen_attn_bwd_unrope. */
int eisen_attn_center_values(void* stream, const void* v, int v_dtype, void* v_centered, float* mean, long long B,
                             long long S, long long Hkv, long long D, long long kv_bs, long long kv_ss, long long kv_hs);
int eisen_attn_fwd_ex(void* stream, const void* q, const void* k, const void* v, void* o, void* o_aux, const float* v_mean,
                      float* lse, long long B, long long S, long long Hq, long long Hkv, long long D, long long q_bs,
                      long long q_ss, long long q_hs, long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs,
                      long long o_ss, long long o_hs, float scale, int causal, int* status);
int eisen_attn_bwd_ex(void* stream, const void* q, const void* k, const void* v, const void* o, const void* o_lo,
                      const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B,
                      long long S, long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                      long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss, long long o_hs,
                      float scale, int causal, const float* table_cos_sin, int* status);
/* eisen_attn_bwd for q and k that were rotated by RoPE right before the attention
 * (src/nn/attention.rs:320-333): dq and dk come out rotated back by the angles of their positions
 * (table_cos_sin of eisen_rope_table for (S, D)), i.e. as the gradients of the un-rotated projections,
 * so the backward closure of `rope` has nothing left to launch.  The rotation is applied in f32
 * before the one rounding to bf16. */
int eisen_attn_bwd_unrope(void* stream, const void* q, const void* k, const void* v, const void* o, const float* lse,
                          const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B, long long S,
                          long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                          long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss,
                          long long o_hs, float scale, int causal, const float* table_cos_sin, int* status);
/* Variant of the head_dim-64 forward: 3 (default) = one 128-row query tile per CTA, two CTAs resident
 * per SM whose phases the hardware interleaves, the probabilities handed to the P V product through
 * tensor memory (tcgen05.st; the product reads its A operand from TMEM); 1 = the same with P staged in
 * shared memory; 2 = two tiles per CTA sharing every K / V tile and taking turns with the
 * exponentials.  Process-wide; meant for tests and measurements. */
int eisen_attn_set_fwd_tiles(int tiles);
/* Variant of the head_dim-64 backward: 1 = the score tiles are formed transposed (S^T = K Q^T,
 * dP^T = V dO^T: TMEM lane = key), so P^T goes back to TMEM and the dV product reads it from there,
 * and one shared-memory tile (dS^T) serves both dK and dQ; 0 = P and dS through shared memory.
 * Process-wide; meant for tests and measurements. */
int eisen_attn_set_bwd_mode(int transposed);
long long eisen_attn_bwd_workspace_bytes(long long B, long long S, long long Hq, long long Hkv, long long D);
/* dq, dk, dv are written (not accumulated); they use the strides of q and k/v respectively. */
int eisen_attn_bwd(void* stream, const void* q, const void* k, const void* v, const void* o, const float* lse,
                   const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B, long long S,
                   long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                   long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss,
                   long long o_hs, float scale, int causal, int* status);

/* One new query position against a KV cache (generation; no counterpart in the reference, which
 * re-runs the whole context per token): o[h,:] = softmax(scale * q[h,:] K[0..n_keys, h/(Hq/Hkv), :]^T) V[...].
 * q, o: [Hq, D]; k_cache, v_cache: rows of cache_row_stride elements holding [Hkv, D]; D <= 256. */
int eisen_attn_decode(void* stream, const void* q, const void* k_cache, const void* v_cache, void* o, long long n_keys,
                      long long Hq, long long Hkv, long long D, long long cache_row_stride, float scale, int dtype);

/* ------------------------------------------------------------------------------------------
 * Row-wise ops
 * ------------------------------------------------------------------------------------------ */

/* RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w; w is f32 [dim]; rrms_out (f32 [rows]) may be null.
 * Replaces rmsnorm_f32 / rmsnorm_bf16 (kernels/ops_f32.cu:539-551, ops_bf16.cu:660-681;
 * src/graph/ops/normalization.rs:88). */
int eisen_rmsnorm_fwd(void* stream, const void* x, const float* w, void* y, float* rrms_out, long long rows,
                      long long dim, float eps, int dtype);
/* 1 (default): rows of exactly 256 16-byte vectors are staged in shared memory by bulk asynchronous
 * copies; 0: always the warp-per-row kernel.  Process-wide; meant for tests and measurements. */
int eisen_rmsnorm_fwd_set_mode(int staged);
long long eisen_rmsnorm_bwd_workspace_bytes(long long rows, long long dim);
/* Kernel of eisen_rmsnorm_bwd where several apply: 0 = CTA-wide kernel with the rows in registers,
 * 1 = warp per row, 2 (default) / 3 / 4 / 5 = rows staged in shared memory by bulk asynchronous copies
 * (4 rows x 3 stages, 2 x 4, 2 x 3, 4 x 2 per CTA; rows of exactly 256 16-byte vectors), 6 = as 2 with
 * two columns per arithmetic instruction (packed f32x2; measured slower).  Process-wide; meant for tests and measurements. */
int eisen_rmsnorm_bwd_set_mode(int mode);
/* dx (op)= ..., dw (f32) += ...  Replaces rmsnorm_backward_f32 and its bf16 variants
 * (kernels/ops_f32.cu:553-578; src/graph/ops/normalization.rs:122). */
int eisen_rmsnorm_bwd(void* stream, const void* x, const float* w, const void* dy, void* dx, float* dw,
                      void* workspace, long long rows, long long dim, float eps, int dtype, int accumulate_dx);

/* softmax over the last dimension and its backward (kernels/ops_f32.cu:625-646). */
int eisen_softmax_fwd(void* stream, const void* x, void* y, long long rows, long long n, int dtype);
int eisen_softmax_bwd(void* stream, const void* y, const void* dy, void* dx, long long rows, long long n,
                      int dtype, int accumulate);

/* Fused softmax-cross-entropy.  Row loss = -ln(softmax(x)[t] + 1e-8) * normalizer; rows whose
 * target equals ignore_index contribute nothing.  Outputs: *loss (device f32), row_loss [rows],
 * lse [rows].  Replaces cross_entropy_f32 / cross_entropy_masked_f32 (kernels/ops_f32.cu:580-598,
 * 5-30; src/graph/ops/reduction.rs:610, 823).  Targets are int32 (the reference passes f32).
 * bad_target_flag (device int, may be null) is set when a target is neither ignore_index nor inside
 * [0, vocab); such rows are skipped like ignored ones here and in eisen_ce_bwd (the reference does
 * not check and reads past the row). */
int eisen_ce_fwd(void* stream, const void* logits, const int* targets, float* loss, float* row_loss, float* lse,
                 long long rows, long long vocab, int ignore_index, float normalizer, int dtype,
                 int* bad_target_flag);
/* dlogits (op)= (softmax(x) - onehot) * normalizer * (*grad_out); dlogits may alias logits.
 * Replaces cross_entropy_backward_f32 / cross_entropy_masked_backward_f32 (600-623, 32-64). */
int eisen_ce_bwd(void* stream, const void* logits, const int* targets, const float* lse, void* dlogits,
                 const float* grad_out, long long rows, long long vocab, int ignore_index, float normalizer,
                 int dtype, int accumulate);

/* Cross-entropy forward and backward in one launch, in place: each row is read once (staged in
 * shared memory), its loss is formed, and dlogits = (softmax - onehot) * normalizer * grad_scale
 * is written over the logits (zero for ignored and out-of-range rows).  For an op that ends in
 * the loss, where the loss gradient is known when the logits are: one read and one write of
 * [rows, vocab] instead of the two reads and one write of eisen_ce_fwd + eisen_ce_bwd
 * (cross_entropy_f32 + cross_entropy_backward_f32, kernels/ops_f32.cu:580-623).  loss and lse may
 * be null (a caller that works through the rows in chunks adds row_loss itself). */
int eisen_ce_fused(void* stream, void* logits, const int* targets, float* loss, float* row_loss, float* lse,
                   long long rows, long long vocab, int ignore_index, float normalizer, float grad_scale, int dtype,
                   int* bad_target_flag);
/* *loss = sum(row_loss[0..rows)) in a fixed order (the second half of eisen_ce_fwd) */
int eisen_ce_loss_reduce(void* stream, const float* row_loss, float* loss, long long rows);

/* ------------------------------------------------------------------------------------------
 * Elementwise / layout ops
 * ------------------------------------------------------------------------------------------ */
int eisen_fill_f32(void* stream, float* p, float value, long long n);                  /* fill_f32, ops_f32.cu:101 */
int eisen_scale_f32(void* stream, float* p, float s, long long n);                     /* scale_f32, ops_f32.cu:107 */
int eisen_cast(void* stream, const void* src, int src_dtype, void* dst, int dst_dtype, long long n); /* cast_*, ops_bf16.cu:4-24 */
/* out[i] = a[i] + b[i % b_numel]  (add_f32, ops_f32.cu:66-82) */
int eisen_add(void* stream, const void* a, const void* b, void* out, long long n, long long b_numel, int dtype);
/* dst[i] (op)= src[i], mixed dtypes allowed  (accumulate_f32, ops_f32.cu:84-99) */
int eisen_accumulate(void* stream, void* dst, int dst_dtype, const void* src, int src_dtype, long long n,
                     int accumulate);
/* dst[j] (op)= sum_{i % m == j} src[i]  (broadcast-operand gradient of accumulate_f32) */
int eisen_reduce_leading(void* stream, const void* src, int src_dtype, float* dst, long long n, long long m,
                         int accumulate);
int eisen_mul_fwd(void* stream, const void* a, const void* b, void* out, long long n, int dtype);  /* mul_f32, ops_f32.cu:113 */
int eisen_mul_bwd(void* stream, const void* a, const void* b, const void* dout, void* da, void* db, long long n,
                  int dtype, int accumulate_a, int accumulate_b);                      /* mul_backward_f32, ops_f32.cu:119 */
int eisen_silu_fwd(void* stream, const void* x, void* y, long long n, int dtype);      /* silu_f32, ops_f32.cu:135 */
int eisen_silu_bwd(void* stream, const void* x, const void* dy, void* dx, long long n, int dtype, int accumulate); /* :142 */
/* fused SwiGLU: out = silu(gate) * up and its one-pass backward (replaces silu + mul and their
 * backward kernels on the path src/nn/transformer.rs:41-44) */
int eisen_swiglu_fwd(void* stream, const void* gate, const void* up, void* out, long long n, int dtype);
int eisen_swiglu_bwd(void* stream, const void* gate, const void* up, const void* dh, void* dgate, void* dup,
                     long long n, int dtype, int accumulate);
/* RoPE on interleaved pairs (rope_f32 / rope_backward_f32, ops_f32.cu:724-760;
 * src/graph/ops/transform.rs:517-531).  table_cos_sin: [seq_len, head_dim/2] pairs of f32. */
int eisen_rope_table(void* stream, float* table_cos_sin, long long seq_len, long long head_dim, float base);
int eisen_rope(void* stream, const void* x, void* y, const float* table_cos_sin, long long B, long long S,
               long long hidden, long long head_dim, int dtype, int inverse, int accumulate);
/* y[B,H,S,D] (op)= x[B,S,H,D]  (transpose_0213_f32 and its backward, ops_f32.cu:694-722) */
int eisen_transpose_0213(void* stream, const void* x, void* y, long long B, long long S, long long H, long long D,
                         int dtype, int accumulate);
/* GQA head replication and its backward (repeat_kv_f32 / repeat_kv_backward_f32, ops_f32.cu:787-840) */
int eisen_repeat_kv_fwd(void* stream, const void* x, void* y, long long B, long long KV, long long S, long long D,
                        long long repeats, int dtype);
int eisen_repeat_kv_bwd(void* stream, const void* dy, void* dx, long long B, long long KV, long long S,
                        long long D, long long repeats, int dtype, int accumulate);

/* ------------------------------------------------------------------------------------------
 * Embedding
 * ------------------------------------------------------------------------------------------ */
/* out[i,:] = W[ids[i],:]  (gather_f32 / gather_bf16_*, ops_f32.cu:513-524, ops_bf16.cu:225, 716;
 * src/graph/ops/transform.rs:203-227).  ids are int32.  bad_id_flag (device int, may be null) is
 * set when an id is outside [0, vocab); such rows read row 0 (the reference does not check). */
int eisen_embedding_fwd(void* stream, const void* w, int w_dtype, const int* ids, void* out, int out_dtype,
                        long long n_ids, long long dim, long long vocab, int* bad_id_flag);
long long eisen_embedding_bwd_workspace_bytes(long long n_ids, long long vocab);
/* dW[ids[i],:] += g[i,:], deterministic, no floating-point atomics
 * (gather_backward_f32, ops_f32.cu:526-537; src/graph/ops/transform.rs:259). */
int eisen_embedding_bwd(void* stream, const void* g, int g_dtype, const int* ids, float* dw, void* workspace,
                        long long n_ids, long long dim, long long vocab);
/* The two halves of eisen_embedding_bwd: _plan groups the positions by id (integer work that
 * depends on the ids only and may run as soon as they are known); _apply adds the gradient rows
 * with the grouping a _plan call left in `workspace` (16-byte aligned). */
int eisen_embedding_bwd_plan(void* stream, const int* ids, void* workspace, long long n_ids, long long vocab);
int eisen_embedding_bwd_apply(void* stream, const void* g, int g_dtype, float* dw, const void* workspace,
                              long long n_ids, long long dim, long long vocab);
/* integer bookkeeping of the last eisen_embedding_bwd on `workspace` (device int32 outputs, any
 * may be null): count[vocab], offset[vocab] (exclusive prefix), perm[n_ids] (positions grouped
 * by id in position order) */
int eisen_embedding_bwd_bookkeeping(void* stream, const void* workspace, long long n_ids, long long vocab,
                                    int* count_out, int* offset_out, int* perm_out);

/* Embedding backward for callers that cannot allocate device memory (no counterpart in the
 * reference).  Same result as eisen_embedding_bwd, but the integer scratch (count, offset, cursor, slot, active,
 * perm) is a fixed 2.5 MB array inside the library instead of a caller-provided workspace: meant
 * for hosts that own all device memory under a fixed budget, or that must not call cudaMalloc
 * inside a training step.  Limits: n_ids <= 65536 and vocab <= 131072, larger sizes return
 * EISEN_ERR_LIMIT.  The call allocates nothing.  The first call on each device looks up the
 * array's device address (cudaGetSymbolAddress, with that device current); make that first call
 * before any stream capture.  All calls on a device share the one array and it keeps the last
 * call's contents (each call clears the part that must start at zero), so two calls that overlap
 * on the GPU, e.g. on different streams, race: keep them on one stream or otherwise ordered. */
int eisen_embedding_bwd_static(void* stream, const void* g, int g_dtype, const int* ids, float* dw,
                               long long n_ids, long long dim, long long vocab);

/* ------------------------------------------------------------------------------------------
 * Optimizer
 * ------------------------------------------------------------------------------------------ */
/* Fused AdamW over a flat f32 buffer (adamw_step_f32, ops_f32.cu:762-784; src/nn/optim.rs:415-481,
 * one launch per tensor there).  See optim.cu for the exact update. */
int eisen_adamw_step(void* stream, float* w, void* w_bf16, const float* g, float* m, float* v, long long n,
                     float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                     float grad_scale, const double* sumsq, float max_norm);
/* The same update with the step-dependent scalars (lr, bc1, bc2) read from device memory when
 * hyper is not null: for a launch that is recorded once in a CUDA graph and replayed every step. */
int eisen_adamw_step_dev(void* stream, float* w, void* w_bf16, const float* g, float* m, float* v, long long n,
                         float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                         float grad_scale, const double* sumsq, float max_norm, const float* hyper);
/* eisen_adamw_step_dev that also clears the gradient as it reads it (zero_grad != 0), which stands for the
 * `zero_grad` memset of the next step (src/nn/optim.rs zero_grad) at no extra pass over memory. */
int eisen_adamw_step_ex(void* stream, float* w, void* w_bf16, float* g, float* m, float* v, long long n, float lr,
                        float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2, float grad_scale,
                        const double* sumsq, float max_norm, const float* hyper, int zero_grad);
long long eisen_sumsq_workspace_bytes(long long n);
/* *out (device f64) (op)= sum x^2 — the device-side half of AdamW::clip_grad_norm
 * (src/nn/optim.rs:250-281 copies every gradient to the host instead). */
int eisen_sumsq(void* stream, const float* x, long long n, void* workspace, double* out, int accumulate);

/* ==========================================================================================
 * Graph level: host-side mirror of the reference's Graph / tape / modules / AdamW.
 *
 * A graph owns its tensors; ids are indices into its tensor list and stay valid until
 * eisen_graph_restore_save_point / eisen_graph_clear_activations pops them (src/graph/mod.rs:
 * 336-365, 432-435).  Each op runs its forward at once on the graph's stream and, unless no_grad
 * is set, pushes a tape node; eisen_graph_backward seeds the loss gradient with ones and walks
 * the tape in reverse (src/graph/mod.rs:670-796).  precision: 0 = Fp32, 1 = Bf16Mixed (bf16
 * activations and activation gradients, f32 master parameters with a bf16 shadow, f32 parameter
 * gradients).  Leaves allocated before eisen_graph_mark_params are parameters.
 * All handles are `void*`; out-parameters are written only on success.
 * ========================================================================================== */
typedef void (*eisen_block_cb)(long long layer, void* user);

int eisen_graph_create(int precision, void* stream, void** out);                       /* Graph::new, src/graph/mod.rs:152-307 */
int eisen_graph_destroy(void* g);
/* VRAM budget and parameter streaming (src/graph/mod.rs:283-288, src/graph/memory.rs:64-266).
 * A graph created while EISEN_VRAM_BUDGET_MB is set (or given a budget here before the model is
 * built) counts every device byte it allocates against the budget: an activation allocation that
 * would exceed it first drops the cached pool buffers and then fails with EISEN_ERR_OOM (the
 * reference panics).  A TransformerLM built under a budget homes its 2-D block weights in
 * page-locked host memory (src/nn/transformer.rs:92-101).
 * eisen_graph_plan_streaming is Graph::plan_streaming: parameters cost 16 bytes per element
 * (weight, gradient, two moments); pinned ones stay on the device, the others are taken in id order
 * while they fit budget - reserve - pinned, then the largest resident ones give way until the
 * largest streamed tensor has room to pass through.  apply = 0 only reports; apply = 1 also moves
 * resident parameters to device memory and streamed ones to host memory.  Streamed weights are GEMM
 * operands through a ring of device staging buffers filled on a copy stream (started a block ahead
 * by the model) instead of the reference's blocking upload inside every matmul
 * (src/graph/ops/linear.rs:804-807); their gradients and AdamW moments stay in host memory.
 * Outputs (any may be null): resident ids (pinned first), streamed ids, bytes4 = resident bytes,
 * resident headroom, streamed f32 bytes, streaming headroom (the largest streamed tensor). */
int eisen_graph_set_vram_budget(void* g, long long budget_bytes, long long activation_reserve_bytes);
int eisen_graph_vram_usage(void* g, long long* used_bytes, long long* budget_bytes);
int eisen_graph_plan_streaming(void* g, long long budget_bytes, long long activation_reserve_bytes, const long long* pinned,
                               int n_pinned, int apply, long long* resident_ids, int* n_resident, long long* streamed_ids,
                               int* n_streamed, long long* bytes4);
int eisen_graph_alloc(void* g, const long long* shape, int ndim, const float* host_data, long long* id_out); /* Graph::alloc */
int eisen_graph_alloc_ids(void* g, const long long* shape, int ndim, const int* host_ids, long long* id_out); /* int32 token ids */
int eisen_graph_alloc_pooled(void* g, const long long* shape, int ndim, long long* id_out);  /* Graph::alloc_pooled, :437-556 */
int eisen_graph_load_tensor_data(void* g, long long id, const float* host, long long n);     /* :368-430 */
int eisen_graph_sync_to_cpu(void* g, long long id, float* out);                        /* Tensor::sync_to_cpu */
int eisen_graph_sync_grad_to_cpu(void* g, long long id, float* out);                   /* Graph::sync_grad_to_cpu */
int eisen_graph_shape(void* g, long long id, long long* shape_out, int* ndim_out);
int eisen_graph_tensor_ptrs(void* g, long long id, void** data, void** grad, int* dtype, int* grad_dtype);
int eisen_graph_set_no_grad(void* g, int flag);                                        /* Graph.no_grad */
/* The graph's mode flags (no_grad: ops record no tape entry; skip_forward: ops allocate their output but
 * launch no forward kernel, used while a checkpointed block is re-recorded).  Both are set for a scope
 * by the model code and restored when the scope ends, also when an op inside it fails. */
int eisen_graph_get_flags(void* g, int* no_grad, int* skip_forward);
int eisen_graph_mark_params(void* g);                                                  /* :328-330 */
int eisen_graph_mark_save_point(void* g, long long* out);                              /* :332-334 */
int eisen_graph_restore_save_point(void* g, long long save_point);                     /* :336-365 */
int eisen_graph_clear_activations(void* g);                                            /* :432-435 */
int eisen_graph_tape_clear(void* g);                                                   /* g.tape.nodes.clear() */
int eisen_graph_reinterpret_shape(void* g, long long id, const long long* shape, int ndim); /* ops/transform.rs:413-426 */
int eisen_graph_zero_grad(void* g, long long id);
int eisen_graph_backward(void* g, long long loss_id);                                  /* :670-796 */
int eisen_graph_synchronize(void* g);   /* waits for the stream and raises recorded kernel faults */
/* CUDA-graph capture of a whole step (no counterpart in the reference, which synchronises after almost
 * every launch): everything the graph-level calls enqueue between capture_begin and capture_end is
 * recorded instead of run, and eisen_graph_replay launches it as one executable graph.  For steps
 * that are launch-bound (a 14M-parameter model: about 1500 launches of a few microseconds).  Rules:
 * run the identical step eagerly first (the capture may not allocate: a pool miss fails with
 * EISEN_ERR_INVALID), feed token ids through tensors that live below the parameter watermark and
 * refresh their contents between replays, read the loss from the device pointer the loss tensor had
 * during capture.  capture_abort ends a capture after a failed call. */
int eisen_graph_capture_begin(void* g);
int eisen_graph_capture_end(void* g, void** exec_out);
int eisen_graph_capture_abort(void* g);
int eisen_graph_replay(void* exec, void* stream);
int eisen_graph_exec_destroy(void* exec);
/* runs eisen_selftest_bounded_wait on the graph's stream against the graph's own fault word: the
 * next eisen_graph_synchronize must return EISEN_ERR_KERNEL and clear the word */
int eisen_graph_selftest_bounded_wait(void* g, long long budget_cycles);
int eisen_graph_counts(void* g, long long* num_tensors, long long* tape_len, long long* num_params);
/* out5: pool bytes in use, pool bytes cached, device bytes allocated, pool hits, pool misses */
int eisen_graph_pool_stats(void* g, long long* out5);
/* flat parameter buffers (f32 weights, bf16 shadow or null, f32 gradients) and their length */
int eisen_graph_param_arena(void* g, void** weights, void** shadow, void** grads, long long* elems);

/* ops: src/graph/ops/elementwise.rs (add 7, mul 188, silu 337), linear.rs (matmul 35/526,
 * matmul_trans_b 301, bmm 1198), reduction.rs (softmax 397, cross_entropy 529, masked 724),
 * normalization.rs (rms_norm 8), transform.rs (transpose_0213 7, gather 132, reshape 329,
 * rope 467), gqa.rs (repeat_kv 13), attention.rs (flash_attention 7).  Targets < 0 stand for
 * IGNORE_INDEX (usize::MAX, src/data/fim.rs:173). */
int eisen_graph_add(void* g, long long a, long long b, long long* out);
int eisen_graph_mul(void* g, long long a, long long b, long long* out);
int eisen_graph_silu(void* g, long long a, long long* out);
int eisen_graph_swiglu(void* g, long long gate, long long up, long long* out);          /* fused silu(gate)*up */
int eisen_graph_matmul(void* g, long long a, long long b, long long* out);
int eisen_graph_matmul_trans_b(void* g, long long a, long long b, long long* out);
int eisen_graph_matmul_add(void* g, long long a, long long b, long long r, long long* out); /* r + a b, fused epilogue (Bf16Mixed) */
int eisen_graph_bmm(void* g, long long a, long long b, int trans_b, long long* out);
int eisen_graph_softmax(void* g, long long a, long long* out);
int eisen_graph_cross_entropy(void* g, long long logits, const long long* targets, long long n, long long* out);
int eisen_graph_cross_entropy_masked(void* g, long long logits, const long long* targets, long long n, long long* out);
/* LM head and cross-entropy as one op (src/nn/transformer.rs:189-195 followed by
 * src/graph/ops/reduction.rs:529-944): loss = mean over the n_valid rows whose target is >= 0 of
 * -ln(softmax(h W)[t] + 1e-8).  h [rows, k]; w [k, vocab], or with trans_b the tied table
 * [vocab, k]; target_ids an id tensor of eisen_graph_alloc_ids (-1 = ignored).  The rows are worked
 * through in chunks of chunk_rows (0 = all at once), so only a [chunk_rows, vocab] slab of logits
 * exists at any time and each slab is read once and overwritten with its gradient.  The gradients
 * of h and w are formed during this call with a loss gradient of 1: the result must be the tensor
 * eisen_graph_backward is called on (checked there).  With no_grad set only the loss is computed. */
int eisen_graph_lm_head_cross_entropy(void* g, long long h, long long w, long long target_ids, long long n_valid,
                                      int trans_b, long long chunk_rows, long long* out);
int eisen_graph_rms_norm(void* g, long long x, long long w, float eps, long long* out);
int eisen_graph_rope(void* g, long long a, long long head_dim, long long* out);
int eisen_graph_gather(void* g, long long weights, long long indices, long long* out);
int eisen_graph_reshape(void* g, long long a, const long long* shape, int ndim, long long* out);
int eisen_graph_transpose_0213(void* g, long long a, long long* out);
int eisen_graph_repeat_kv(void* g, long long a, long long repeats, long long* out);
int eisen_graph_flash_attention(void* g, long long q, long long k, long long v, float scale, int causal, long long* out);
/* fused causal GQA attention with backward on [B,S,heads*head_dim] projections (Bf16Mixed) */
int eisen_graph_attention(void* g, long long q, long long k, long long v, long long num_heads,
                          long long num_kv_heads, int causal, long long* out);

/* TransformerLM (src/nn/transformer.rs:69-211) */
int eisen_lm_create(void* g, long long vocab, long long hidden, long long heads, long long kv_heads, long long ffn,
                    long long layers, int tie_weights, void** out);
int eisen_lm_destroy(void* lm);
int eisen_lm_set_fused(void* lm, int fused);   /* 0: the reference's op-by-op attention / MLP chain */
/* before_block(l, user) is called inside eisen_lm_train_micro_step[_dev] just before the forward
 * pass first reads the parameters of block l (l == -1: embedding, l == layers: final norm and
 * head); it may make the graph's stream wait for work on other streams (a sharded data-parallel
 * step waits here for the all-gather of those weights).  Null removes the hook. */
int eisen_lm_set_forward_hook(void* lm, eisen_block_cb before_block, void* user);
/* eisen_lm_train_micro_step[_dev] with checkpoint != 0: keep != 0 keeps every block's attention
 * output and log-sum-exp from the first forward pass (2 bytes per activation element plus 4 bytes
 * per head and token) and leaves the attention forward out of the block's re-run; everything else
 * of the block is recomputed.  Default 0: the whole block is recomputed, as the reference's
 * mark_save_point / restore_save_point loop does. */
int eisen_lm_set_keep_attention(void* lm, int keep);
/* eisen_lm_train_micro_step[_dev]: fused != 0 (default) runs head projection and cross-entropy as
 * eisen_graph_lm_head_cross_entropy in chunks of chunk_rows token rows (0 = all rows at once);
 * fused == 0 runs matmul + cross_entropy_masked as the reference does. */
int eisen_lm_set_head_fusion(void* lm, int fused, long long chunk_rows);
int eisen_lm_forward(void* lm, void* g, long long x_ids, long long* logits_out);       /* Module::forward, :184-196 */
int eisen_lm_params(void* lm, long long* ids_out, int* n_out);                         /* Module::params, :198-210 */
/* Greedy generation, the loop of examples/train_llm.rs:560-584: max_new_tokens times the argmax of
 * the last position's logits (the last of equal maxima, as Rust's max_by), context window
 * max_context.  kv_cache = 0 runs it as the reference does, the whole context through the forward
 * pass for every token.  kv_cache = 1 keeps every layer's rotated keys and its values on the device:
 * the prompt runs once, every further token is one row through the projections plus
 * eisen_attn_decode over the cache (the reference lists KV caching as future work, README.md:94);
 * it needs n_prompt + max_new_tokens <= max_context (EISEN_ERR_LIMIT otherwise), because a sliding
 * window re-positions every cached key.  last_logits (host f32 [vocab], may be null) receives the
 * logits behind the last token.  Synchronises the graph's stream once per token (the argmax is
 * taken on the host, as in the reference). */
int eisen_lm_generate(void* lm, void* g, const int* prompt, long long n_prompt, long long max_new_tokens, long long max_context,
                      int kv_cache, int* out_tokens, float* last_logits);
/* Weights-only checkpoint (save_weights, examples/train_llm.rs:92-105): every parameter tensor in id
 * order as f32 little-endian, the `eisen_model.bin` the reference's converter reads.  load_weights is
 * its inverse for an identically built model (the reference has no loader). */
int eisen_graph_save_weights(void* g, const char* path);
int eisen_graph_load_weights(void* g, const char* path);
/* Hugging Face export (examples/export_hf_pipeline.rs:200-300, src/tools/huggingface.rs:88-146): writes the
 * f32 master weights as LlamaForCausalLM tensors (Linear weights transposed to [out, in], q / k rows
 * permuted from interleaved-pair to rotate-half RoPE order) and, if config_path is not null, config.json. */
int eisen_lm_export_hf(void* lm, void* g, const char* safetensors_path, const char* config_path,
                       long long max_position_embeddings);
/* one micro-step: forward, masked cross-entropy over n_targets rows, backward; with checkpoint
 * != 0 each block is re-run under a save point during the backward (src/graph/mod.rs:332-365).
 * after_block(l, user) fires when the gradients of block l are final (l == layers: final norm
 * and head, l == -1: embedding); it may enqueue work on other streams. */
int eisen_lm_train_micro_step(void* lm, void* g, long long x_ids, const long long* targets, long long n_targets,
                              int checkpoint, eisen_block_cb after_block, void* user, long long* loss_id);

/* same, with the targets already on the device (an id tensor from eisen_graph_alloc_ids holding
 * -1 for ignored rows) and their number of valid rows */
int eisen_lm_train_micro_step_dev(void* lm, void* g, long long x_ids, long long target_ids, long long n_valid,
                                  int checkpoint, eisen_block_cb after_block, void* user, long long* loss_id);

/* Per-class device timing of the tensor-core kernels of a graph, taken with CUDA events on the
 * graph's stream around each launch while enabled.  eisen_graph_prof_read synchronises the
 * stream, sums the intervals and resets them.  out[class][0..2] = milliseconds, algorithmic
 * FLOPs, launches for class 0 = GEMM, 1 = attention forward, 2 = attention backward. */
int eisen_graph_prof_enable(void* g, int on);
int eisen_graph_prof_read(void* g, double* out9);

/* AdamW (src/nn/optim.rs): zero_grad 207, clip_grad_norm 250, step 334 */
int eisen_optim_create(void* g, const long long* params, int n, float lr, void** out);
int eisen_optim_destroy(void* opt);
int eisen_optim_config(void* opt, float lr, float beta1, float beta2, float eps, float weight_decay);
int eisen_optim_zero_grad(void* opt);
int eisen_optim_clip_grad_norm(void* opt, float max_norm, float* norm_out, float* coef_out);
int eisen_optim_step(void* opt);
/* clip (max_norm > 0) and step without a host round trip; the gradient is read as g * grad_scale */
int eisen_optim_step_fused(void* opt, float max_norm, float grad_scale);
int eisen_optim_is_flat(void* opt, int* flat);
/* For a step replayed from a CUDA graph (eisen_graph_capture_*): an optimizer step enqueued during
 * capture takes lr and the bias corrections from device memory, refreshed by a copy node from a
 * page-locked host record; eisen_optim_advance (t += 1, new bias corrections, current lr into that
 * record) must be called before every replay, and once before the capture itself. */
int eisen_optim_advance(void* opt);
/* Optimizer state of a checkpoint: step count, hyper-parameters and the AdamW moments (of this
 * rank's ranges for a sharded optimizer), so that weights file + state file resume a run bit for
 * bit.  The reference saves weights only (examples/train_llm.rs:93-105) and lists optimizer state
 * as future work (README.md:88).  load_state rejects a file written for another model or sharding. */
int eisen_optim_save_state(void* opt, const char* path);
int eisen_optim_load_state(void* opt, const char* path);
/* Sharded optimizer state (ZeRO-1; no counterpart in the reference): this rank keeps AdamW moments
 * only for n_pieces element ranges [piece_lo[i], piece_hi[i]) of the flat parameter arena and
 * updates only those (master weights and their bf16 copies); the exchange layer brings in the
 * other ranks' updated ranges.  One optimizer step is: eisen_optim_begin_step (t += 1), for the
 * clip eisen_optim_sumsq_piece over all pieces (accumulating into the 8-byte device value at
 * eisen_optim_sumsq_ptr, which the caller sums across ranks), then eisen_optim_step_piece for
 * every piece (the update of src/nn/optim.rs:334-481 on that range, clip coefficient
 * min(1, max_norm / (sqrt(sumsq) * grad_scale + 1e-6)) when max_norm > 0). */
int eisen_optim_create_sharded(void* g, const long long* params, int n, float lr, const long long* piece_lo,
                               const long long* piece_hi, int n_pieces, void** out);
int eisen_optim_begin_step(void* opt);
int eisen_optim_sumsq_piece(void* opt, int piece, int accumulate, void* stream); /* stream null: the graph's */
int eisen_optim_step_piece(void* opt, int piece, float max_norm, float grad_scale);
/* eisen_optim_step_piece on a stream of the caller's choice (null: the graph's), optionally clearing the
 * piece's gradients as they are read.  With the pieces cut at block boundaries and launched in forward order
 * on a side stream, the update of step t runs beside the forward pass of step t + 1, which waits (an event
 * per piece, from the model's forward hook) only for the block it is about to read. */
int eisen_optim_step_piece_on(void* opt, int piece, float max_norm, float grad_scale, void* stream, int zero_grads);
int eisen_optim_sumsq_ptr(void* opt, void** out);

/* ------------------------------------------------------------------------------------------
 * Data-parallel exchange (no counterpart in the reference, which is single-GPU): one process per
 * GPU, every rank runs the whole step on its own micro-batch, the flat f32 gradient buffer
 * (eisen_graph_param_arena) is summed across ranks bucket by bucket while the backward pass is
 * still running (eisen_lm_train_micro_step's after_block callback says when a bucket is final).
 * Thin checked layer over NCCL, bound at run time (dlopen of libnccl.so.2).  All collectives are
 * in place or caller-buffered, asynchronous on the given stream, and allocate nothing.
 *   unique id: rank 0 calls eisen_dp_unique_id and hands the 128 bytes to every rank by its own
 *   means (a file, a socket, an environment variable); every rank then calls eisen_dp_init with
 *   its CUDA device current.
 * Failure handling: no call waits without a limit.  eisen_dp_poll_error reads the communicator's
 * asynchronous error state (ncclCommGetAsyncError); eisen_dp_wait polls the stream and that state
 * until the stream is idle or deadline_ms have passed, and on an error or a missed deadline aborts
 * the communicator (ncclCommAbort) and returns EISEN_ERR_COMM / EISEN_ERR_TIMEOUT; afterwards
 * every call on the handle fails with EISEN_ERR_COMM until it is destroyed and a new one made.
 * ------------------------------------------------------------------------------------------ */
int eisen_dp_available(void);                      /* 1 if NCCL could be bound in this process */
int eisen_dp_unique_id(void* out128);
int eisen_dp_init(int rank, int world, const void* unique_id128, void** comm_out);
int eisen_dp_destroy(void* comm);
/* rank, world and the number of collectives enqueued on this handle so far (each may be null) */
int eisen_dp_rank_world(void* comm, int* rank, int* world, long long* launched);
/* ptr[0..n) = sum over ranks, in place */
int eisen_dp_allreduce_bucket(void* comm, void* ptr, long long n, int dtype, void* stream);
/* recv[0..recv_n) = sum over ranks of their send[rank * recv_n ..]; recv may be send + rank * recv_n */
int eisen_dp_reduce_scatter(void* comm, const void* send, void* recv, long long recv_n, int dtype, void* stream);
/* recv[r * send_n ..] = rank r's send[0..send_n); send may be recv + rank * send_n */
int eisen_dp_all_gather(void* comm, const void* send, void* recv, long long send_n, int dtype, void* stream);
int eisen_dp_broadcast(void* comm, void* ptr, long long n, int dtype, int root, void* stream);
int eisen_dp_group_begin(void);                    /* ncclGroupStart: the calls up to group_end become one launch */
int eisen_dp_group_end(void);
int eisen_dp_poll_error(void* comm);
int eisen_dp_wait(void* comm, void* stream, long long deadline_ms);
int eisen_dp_abort(void* comm);

/* ------------------------------------------------------------------------------------------
 * Input side: pre-tokenised u16 token files (BinaryDataLoader, src/data/dataloader.rs:89-214, with
 * the fill-in-the-middle transform of src/data/fim.rs:96-180).  Host only: batches are written to
 * caller-provided buffers (pinned ones for asynchronous copies); ids and targets are int32, the
 * ignore index is -1.  A batch takes batch * (seq_len + 1) consecutive tokens of the file.
 * ------------------------------------------------------------------------------------------ */
int eisen_loader_open(const char* path, long long seq_len, long long batch, void** handle_out);
int eisen_loader_close(void* loader);
long long eisen_loader_total_batches(void* loader);
/* FIM on: control tokens base_vocab .. base_vocab + 3 (prefix, suffix, middle, pad); `rate` of the
 * sequences are transformed, `spm_rate` of those in suffix-prefix-middle order. */
int eisen_loader_set_fim(void* loader, long long base_vocab, float rate, float spm_rate);
int eisen_loader_seed(void* loader, unsigned long long seed);   /* xorshift64 state, default 1337 */
int eisen_loader_reset(void* loader);                           /* back to the start of the file */
/* x, targets: [batch * seq_len].  Returns 0, or 1 when no complete batch is left. */
int eisen_loader_next(void* loader, int* x, int* targets, int* has_masked);

#ifdef __cplusplus
}
#endif
#endif /* EISEN_B200_H */
