// bf16 x bf16 -> f32 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// TMEM, operands staged in shared memory by TMA with 128-byte swizzle).
//
//   C[M,N] (op)= sum_k A(m,k) * B(n,k)
//
// Each operand is either K-major (memory [rows=M or N][K], K contiguous) or MN-major
// (memory [K][M or N], M/N contiguous); the three Linear products of a training step map to
//   forward  Y  = X  W      : A = X  K-major,  B = W  MN-major   (W stored [in,out])
//   dX          = dY W^T    : A = dY K-major,  B = W  K-major
//   dW         += X^T dY    : A = X  MN-major, B = dY MN-major   (K = tokens)
// which replaces the reference's matmul_f32 / matmul_backward_a_f32 / matmul_backward_b_f32
// (kernels/ops_f32.cu:158-259) and their bf16-operand variants (kernels/ops_bf16.cu:26-176).
//
// Persistent kernel, one CTA per SM, 128x256 output tile, BK = 64, 4-stage TMA ring.
// Warp 0 produces (TMA), warp 1 issues MMAs, warps 2-5 drain TMEM (two 256-column
// accumulators, so the epilogue of tile i overlaps the main loop of tile i+1).
#include "ptx.cuh"
#include "gemm_tc.h"
#include "gemm_epilogue.cuh"
#include "errors.h"

#include <cuda.h>
#include <cstdio>
#include <mutex>
#include <unordered_map>

namespace eisen {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int ACC_COLS = BN;  // TMEM columns of one accumulator
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct GemmKParams {
  int M, N, K;
  int a_mn, b_mn;
  void* C;
  long long ldc;
  const void* R;  // addend of the bf16 accumulate mode (C itself, or a residual tensor)
  long long ldr;
  int out_mode;
  int split_k;
  int kblocks_per_split;
  int kblocks_total;
  int m_tiles, n_tiles;
  int total_tiles;
  float alpha;
  int* status;
};

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmKParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles want a 1024-byte aligned base
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full_bar = bars + 2 * STAGES;  // [2]
  uint64_t* tmem_empty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * ACC_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = p.m_tiles * p.n_tiles;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
        const int ks = t / tiles_mn;
        const int mn = t - ks * tiles_mn;
        const int mt = mn % p.m_tiles;
        const int nt = mn / p.m_tiles;
        const int m0 = mt * BM, n0 = nt * BN;
        const int kb0 = ks * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FAULT_WAIT_EMPTY);
          mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
          uint8_t* sa = smem_a + stage * A_STAGE_BYTES;
          uint8_t* sb = smem_b + stage * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), &tmA, &full_bar[stage], m0 + 64 * j, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tmB, &full_bar[stage], n0 + 64 * j, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      // K-major: 8-row groups 1024 B apart.  MN-major: 64-wide slabs 8192 B apart (one TMA box
      // of 64 k-rows x 128 B), 8-row K groups 1024 B apart.
      const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 16, a_sbo = 1024;
      const uint32_t b_lbo = p.b_mn ? 64 * BK * 2 : 16, b_sbo = 1024;
      // advance of the start address per UMMA_K = 16 elements of K
      const uint32_t a_kstep = p.a_mn ? 16 * 128 : 32;
      const uint32_t b_kstep = p.b_mn ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
        const int ks = t / tiles_mn;
        const int kb0 = ks * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, FAULT_WAIT_TMEM_EMPTY);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, FAULT_WAIT_FULL);
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem_a + stage * A_STAGE_BYTES);
          const uint32_t sb = smem_u32(smem_b + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_kstep, a_lbo, a_sbo);
            const uint64_t db = make_smem_desc(sb + k * b_kstep, b_lbo, b_sbo);
            umma_bf16_ss(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs are done
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full_bar[acc]);  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue: TMEM -> registers -> global ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < p.total_tiles; t += gridDim.x) {
      const int ks = t / tiles_mn;
      const int mn = t - ks * tiles_mn;
      const int mt = mn % p.m_tiles;
      const int nt = mn / p.m_tiles;
      const int row = mt * BM + q * 32 + lane;
      const int n0 = nt * BN;
      const int kb0 = ks * p.kblocks_per_split;
      const bool has_k = kb0 < p.kblocks_total;  // an empty K range contributes nothing
      mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.status, FAULT_WAIT_TMEM_FULL);
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * ACC_COLS + (uint32_t(q * 32) << 16);
      const bool row_ok = row < p.M;
      const bool acc_bf16 = p.out_mode == GEMM_OUT_BF16_ACC && has_k;
      uint4 pre_cur[4], pre_next[4];
      bool have_cur = acc_bf16 && gemm_prefetch_addend(p.R, p.ldr, row, n0, p.N, row_ok, pre_cur);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        // the addend of the next chunk is requested before this chunk's TMEM load and stores
        const bool have_next = acc_bf16 && c + 1 < BN / 32 &&
                               gemm_prefetch_addend(p.R, p.ldr, row, col0 + 32, p.N, row_ok, pre_next);
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row_ok && col0 < p.N && has_k) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          gemm_store_chunk32(p.C, p.ldc, p.R, p.ldr, p.out_mode, row, col0, p.N, v, pre_cur, have_cur);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) pre_cur[j] = pre_next[j];
        have_cur = have_next;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let copies that may still be in flight land before the CTA goes away
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * ACC_COLS);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

}  // namespace

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t row_stride_elems, uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return 1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

int make_tmap_bf16_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_elems /*rank-1, of dims 1..*/, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return 1;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5];
  cuuint32_t e[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_elems[i] * 2;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

// f32 tensor, 128-byte swizzle (box rows of 32 floats)
int make_tmap_f32_nd(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides_elems /*rank-1, of dims 1..*/, const uint32_t* box) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return 1;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5];
  cuuint32_t e[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_elems[i] * 4;
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, rank, const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

static int g_reserved_sms = 0;
static int g_num_sms = 0;
static int num_sms() {
  if (!g_num_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

int gemm_bf16_tc(cudaStream_t stream, int a_mn, int b_mn, int M, int N, int K, const void* A,
                 long long lda, const void* B, long long ldb, void* C, long long ldc, const void* R, long long ldr,
                 int out_mode, int split_k, float alpha, int* status, const char** err) {
  static bool attr_set[MAX_DEVICE_SLOTS] = {false};
  const int slot = device_slot();
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) {
    if (err) *err = "gemm_bf16_tc: operand rows must be 16-byte aligned (leading dimension % 8 == 0)";
    return 1;
  }
  if (split_k < 1) split_k = 1;
  if (split_k > 1 && out_mode != GEMM_OUT_F32_ATOMIC) {
    if (err) *err = "gemm_bf16_tc: split_k > 1 needs the f32 atomic output mode";
    return 1;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, 64, BM);
  else       rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
  if (rc) { if (err) *err = "gemm_bf16_tc: cuTensorMapEncodeTiled failed for A"; return 2; }
  if (!b_mn) rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, 64, BN);
  else       rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
  if (rc) { if (err) *err = "gemm_bf16_tc: cuTensorMapEncodeTiled failed for B"; return 2; }

  GemmKParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.out_mode = out_mode;
  p.R = R ? R : C; p.ldr = R ? ldr : ldc;
  p.m_tiles = (M + BM - 1) / BM;
  p.n_tiles = (N + BN - 1) / BN;
  p.kblocks_total = (K + BK - 1) / BK;
  if (split_k > p.kblocks_total) split_k = p.kblocks_total;
  p.kblocks_per_split = (p.kblocks_total + split_k - 1) / split_k;
  split_k = (p.kblocks_total + p.kblocks_per_split - 1) / p.kblocks_per_split;
  p.split_k = split_k;
  p.total_tiles = p.m_tiles * p.n_tiles * split_k;
  p.alpha = alpha;
  p.status = status;
  if (!attr_set[slot]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) { if (err) *err = cudaGetErrorString(e); return 3; }
    attr_set[slot] = true;
  }
  int avail = num_sms() - g_reserved_sms;
  if (avail < 1) avail = 1;
  int grid = p.total_tiles < avail ? p.total_tiles : avail;
  gemm_bf16_tc_kernel<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { if (err) *err = cudaGetErrorString(e); return 3; }
  return 0;
}

int gemm_num_sms() { return num_sms(); }
int gemm_reserved_sms() { return g_reserved_sms; }
void gemm_set_reserved_sms(int n) { g_reserved_sms = n < 0 ? 0 : n; }

int gemm_tc_auto_split_k(int M, int N, int K) {
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int kblocks = (K + BK - 1) / BK;
  const int sms = num_sms();
  if (tiles >= sms) return 1;
  int s = (2 * sms + tiles - 1) / tiles;  // aim for about two waves
  int max_s = kblocks / 8;                // keep at least 8 k-blocks per split
  if (max_s < 1) max_s = 1;
  if (s > max_s) s = max_s;
  return s < 1 ? 1 : s;
}

}  // namespace eisen
