// Flash attention forward and backward with grouped-query heads on tcgen05 tensor cores.
//
// Tensors are [B, S, H, D] views with element strides (D contiguous), D in {64, 128}, bf16.
// Query head h uses KV head h / (Hq / Hkv); nothing is replicated or transposed in memory.
// All tiles are 128 x 128 (queries x keys); operands reach shared memory by TMA with 128-byte
// swizzle and are consumed by tcgen05.mma either K-major or MN-major, so one resident tile serves
// both A*B^T and A^T*B style products; accumulators live in TMEM.
//
// Forward: softmax warps read S = Q K^T from TMEM and hand P (bf16) to the P V product.  At D = 64
// (attn_fwd64_kernel) a CTA owns one 128-query tile (two CTAs per SM), P goes back to TMEM and is
// read from there as the product's A operand, O stays in TMEM and is rescaled lazily; variants with
// P staged in shared memory and with two query tiles per CTA stay selectable.  At D = 128
// (attn_fwd_kernel) two query tiles per CTA share the K / V tiles, P goes through shared memory and
// each P V product is a fresh TMEM accumulator folded into f32 registers with the online-softmax rescale.
// Backward: one 128-key tile of one KV head per CTA, looping over the query heads of its group and
// over query tiles; dV and dK stay in TMEM for the whole loop (the GQA reduce), dQ tiles are added
// to an f32 workspace.  Details sit above each kernel.
// It replaces the reference's materialised chain bmm -> mul(scale) -> add(mask) -> softmax -> bmm
// and its gradient kernels (src/nn/attention.rs:339-375; kernels/ops_f32.cu:342-511, 625-646,
// 787-840); the reference has no fused backward (src/graph/ops/attention.rs:15-18).
#include <atomic>

#include "ptx.cuh"
#include "common.cuh"
#include "errors.h"
#include "gemm_tc.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

constexpr float LOG2E = 1.4426950408889634f;

// variant of the head_dim-64 forward: 3 = one query tile per CTA with P through TMEM, 1 = the same
// with P through shared memory, 2 = two query tiles per CTA (one CTA per SM)
std::atomic<int> g_attn_fwd_tiles{3};
// head_dim-64 backward: 1 = transposed score tiles with P^T handed to the dV product through TMEM
std::atomic<int> g_attn_bwd_transposed{1};

struct AttnParams {
  int B, S, Hq, Hkv, D;
  int causal;
  float scale;
  // outputs / side inputs (element strides)
  void* o; long long o_bs, o_ss, o_hs;
  // forward, may be null: bf16 tensor with O's strides that receives the part of the f32 output that the
  // rounding of O drops (o_lo = bf16(o_f32 - float(bf16(o_f32)))); the backward forms delta = dO . (O + O_lo)
  void* o_lo;
  // forward, may be null: f32 [B, Hkv, D] vector that was subtracted from every value row before the call
  // (eisen_attn_center_values).  The output gets it added back, and o_lo then receives the output
  // before the addition, bf16(sum_j P_ij (V_j - mean)), the tensor the backward pass forms delta from.
  const float* v_mean;
  float* lse;        // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  float* dq_acc;     // [B, S, Hq, D] f32
  void* dk; void* dv; long long kv_bs, kv_ss, kv_hs;
  // backward only, may be null: (cos, sin) table [S][D / 2]; dK (and dQ, in the conversion kernel) are
  // then written rotated back by the RoPE angles of their positions
  const float2* unrope_tab;
  // backward, fixed-order mode: key tile jt writes its dQ tiles to slice jt of dq_acc (dq_slice elements
  // apart) instead of adding them to one buffer; the conversion kernel sums the slices in key order
  int det;
  long long dq_slice;
  int* status;
};

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// the bf16 pair that the rounding of (a, b) to bf16 drops
__device__ __forceinline__ uint32_t pack_bf16x2_lo(float a, float b) {
  const float ha = __bfloat162float(__float2bfloat16_rn(a)), hb = __bfloat162float(__float2bfloat16_rn(b));
  return pack_bf16x2(a - ha, b - hb);
}

// Eight output columns of one row.  Plain: out = bf16(x).  With `aux`: the part the rounding drops goes
// there as well.  With `mean` (the vector the values were centred by): out = bf16(x + mean) and aux, if
// given, receives bf16(x), the centred output.
__device__ __forceinline__ void store_out8(__nv_bfloat16* out, __nv_bfloat16* aux, const float* mean, const float (&x)[8]) {
  float y[8];
  if (mean) {
    const float4 m0 = *reinterpret_cast<const float4*>(mean), m1 = *reinterpret_cast<const float4*>(mean + 4);
    const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = x[e] + mm[e];
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = x[e];
  }
  uint4 o;
  o.x = pack_bf16x2(y[0], y[1]); o.y = pack_bf16x2(y[2], y[3]); o.z = pack_bf16x2(y[4], y[5]); o.w = pack_bf16x2(y[6], y[7]);
  *reinterpret_cast<uint4*>(out) = o;
  if (aux) {
    uint4 a;
    if (mean) {
      a.x = pack_bf16x2(x[0], x[1]); a.y = pack_bf16x2(x[2], x[3]); a.z = pack_bf16x2(x[4], x[5]); a.w = pack_bf16x2(x[6], x[7]);
    } else {
      a.x = pack_bf16x2_lo(x[0], x[1]); a.y = pack_bf16x2_lo(x[2], x[3]); a.z = pack_bf16x2_lo(x[4], x[5]); a.w = pack_bf16x2_lo(x[6], x[7]);
    }
    *reinterpret_cast<uint4*>(aux) = a;
  }
}

// writes 32 consecutive bf16 of row `row` starting at column `col0` (multiple of 32) into a
// [128 x 128] bf16 tile stored as two 128B-swizzled [128 x 64] halves, 16 KB apart
__device__ __forceinline__ void store_row_chunk32(uint32_t tile_base, int row, int col0, const uint32_t (&pk)[16]) {
  const uint32_t half = tile_base + (col0 >> 6) * 16384u;
  const int chunk0 = (col0 & 63) >> 3;  // first 16-byte chunk inside the 128-byte row
#pragma unroll
  for (int j = 0; j < 4; ++j)
    st_shared_v4(half + swz128(row, chunk0 + j), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
}

// =====================================================================================
// forward (used at D = 128; D = 64 has attn_fwd64_kernel below): two 128-query tiles of one head
// per CTA.  Warps 0-3 run the softmax of tile A, warps 4-7 that of tile B (thread = query row), the
// next two warps issue TMA and MMAs.  K and V tiles are loaded once and used by both query tiles;
// while one tile's softmax runs on the SIMT side the tensor core works on the other tile's
// S = Q K^T and PV products.
// =====================================================================================
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct FwdCfg {
  static constexpr int TILE = 128 * D * 2;  // bytes of a [128 x D] bf16 tile
  static constexpr int P_TILE = 128 * 128 * 2;
  static constexpr int NSV = (D == 64) ? 2 : 1;  // V stages (shared memory is the limit at D = 128)
  static constexpr int OFF_Q = 0;                 // 2 tiles
  static constexpr int OFF_K = 2 * TILE;          // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * TILE;  // NSV stages
  static constexpr int OFF_P = OFF_V + NSV * TILE;  // 2 tiles
  static constexpr int OFF_BAR = OFF_P + 2 * P_TILE;
  // SPLIT threads share a query row (each takes 128 / SPLIT score columns and D / SPLIT output
  // columns); the row maximum is exchanged through shared memory.  Shared memory leaves room for
  // the exchange buffer only at D = 64.
  static constexpr int SPLIT = (D == 64) ? 2 : 1;
  static constexpr int OFF_XMAX = OFF_BAR + 256;             // float [2 tiles][SPLIT][128]
  static constexpr int SMEM = OFF_XMAX + (SPLIT > 1 ? 2 * SPLIT * 128 * 4 : 0) + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SWARPS = 8 * SPLIT;                   // softmax warps
  static constexpr int THREADS = (SWARPS + 2) * 32;
};

template <int D>
__global__ void __launch_bounds__(FwdCfg<D>::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using Cfg = FwdCfg<D>;
  constexpr int ATOMS = D / 64;
  constexpr int NSV = Cfg::NSV;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // per query tile
  uint64_t* p_ready = bars + 11;    // per query tile (one arrival per warp)
  uint64_t* o_full = bars + 13;     // per query tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* exp_done = bars + 16;   // per query tile: its exponentials of a key tile are issued

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + 127) / 128;
  // blocks are handed out x-fastest, so with the tile index in z every head's heavy (late) causal
  // tiles start before anybody's light ones
  const int pair = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int qtA = 2 * pair, qtB = 2 * pair + 1;
  const bool b_valid = qtB < n_qt;
  const int h = blockIdx.x, b = blockIdx.y;
  const int kvh = h / (p.Hq / p.Hkv);
  const int nA = p.causal ? min(qtA + 1, n_qt) : n_qt;                 // key tiles of query tile A
  const int nB = b_valid ? (p.causal ? min(qtB + 1, n_qt) : n_qt) : 0;  // key tiles of query tile B
  const int n_kv = max(nA, nB);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4 * Cfg::SPLIT);  // one arrival per warp
      mbar_init(&o_full[i], 1);
      mbar_init(&exp_done[i], 4 * Cfg::SPLIT);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == Cfg::SWARPS + 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;        // S of tile A at +0, of tile B at +128
  const uint32_t tm_O = tmem_base + 256;  // PV of tile A at +0, of tile B at +D

  if (warp == Cfg::SWARPS) {
    // ---------------- TMA ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, (b_valid ? 2 : 1) * Cfg::TILE);
#pragma unroll
      for (int a = 0; a < ATOMS; ++a) {
        tma_load_4d(smem + Cfg::OFF_Q + a * 16384, &tmQ, q_full, a * 64, h, qtA * 128, b);
        if (b_valid) tma_load_4d(smem + Cfg::OFF_Q + Cfg::TILE + a * 16384, &tmQ, q_full, a * 64, h, qtB * 128, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        mbar_arrive_expect_tx(&k_full[st], Cfg::TILE);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_4d(smem + Cfg::OFF_K + st * Cfg::TILE + a * 16384, &tmK, &k_full[st], a * 64, kvh, j * 128, b);
        const int sv = j % NSV;
        const uint32_t phv = (j / NSV) & 1;
        mbar_wait(&v_empty[sv], phv ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        mbar_arrive_expect_tx(&v_full[sv], Cfg::TILE);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
          tma_load_4d(smem + Cfg::OFF_V + sv * Cfg::TILE + a * 16384, &tmV, &v_full[sv], a * 64, kvh, j * 128, b);
      }
    }
  } else if (warp == Cfg::SWARPS + 1) {
    // ---------------- MMA ----------------
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q);
      auto issue_s = [&](int t, int j) {  // S_t = Q_t K_j^T
        const uint32_t sK = smem_u32(smem + Cfg::OFF_K + (j & 1) * Cfg::TILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384u + (k & 3) * 32u;
          umma_bf16_ss(tm_S + t * 128, make_smem_desc(sQ + t * Cfg::TILE + off, 16, 1024),
                       make_smem_desc(sK + off, 16, 1024), idesc_s, k > 0);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int j) {  // O_t = P_t V_j (fresh accumulator, folded by the softmax warps)
        const uint32_t sP = smem_u32(smem + Cfg::OFF_P + t * Cfg::P_TILE);
        const uint32_t sV = smem_u32(smem + Cfg::OFF_V + (j % NSV) * Cfg::TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 128 keys in steps of 16
          const uint64_t da = make_smem_desc(sP + (k >> 2) * 16384u + (k & 3) * 32u, 16, 1024);
          const uint64_t db = make_smem_desc(sV + k * 2048u, 16384, 1024);  // V is MN-major: [key][d]
          umma_bf16_ss(tm_O + t * D, da, db, idesc_pv, k > 0);
        }
        umma_commit(&o_full[t]);
      };
      mbar_wait(q_full, 0, abort_flag, p.status, FAULT_WAIT_ATTN);
      mbar_wait(&k_full[0], 0, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      issue_s(0, 0);
      if (b_valid) issue_s(1, 0);
      umma_commit(&k_empty[0]);
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t jph = j & 1;
        const uint32_t phv = (j / NSV) & 1;
        const bool more = j + 1 < n_kv;
        const uint32_t kph1 = ((j + 1) >> 1) & 1;
        if (j < nA) {
          mbar_wait(&p_ready[0], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
          mbar_wait(&v_full[j % NSV], phv, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_pv(0, j);
          if (j + 1 < nA) {
            mbar_wait(&k_full[(j + 1) & 1], kph1, abort_flag, p.status, FAULT_WAIT_ATTN);
            tc_fence_after_sync();
            issue_s(0, j + 1);
          }
        }
        if (j < nB) {
          mbar_wait(&p_ready[1], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
          mbar_wait(&v_full[j % NSV], phv, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_pv(1, j);
          if (j + 1 < nB) {
            mbar_wait(&k_full[(j + 1) & 1], kph1, abort_flag, p.status, FAULT_WAIT_ATTN);
            tc_fence_after_sync();
            issue_s(1, j + 1);
          }
        }
        umma_commit(&v_empty[j % NSV]);
        if (more) umma_commit(&k_empty[(j + 1) & 1]);
      }
    }
  } else {
    // ---------------- softmax + output ----------------
    // warp w: query tile (w >> 2) & 1, TMEM lane quarter w & 3, column part w >> 3 (of SPLIT).
    // A thread owns one query row, CW = 128 / SPLIT of its score columns and DW = D / SPLIT of its
    // output columns; with SPLIT = 2 the two threads of a row agree on the row maximum through
    // shared memory and add their partial row sums at the end.
    constexpr int SPLIT = Cfg::SPLIT;
    constexpr int CW = 128 / SPLIT;
    constexpr int DW = D / SPLIT;
    const int t = (warp >> 2) & 1;
    const int part = warp >> 3;
    const int n_mine = t ? nB : nA;
    const int qt = t ? qtB : qtA;
    const int row = (warp & 3) * 32 + lane;
    const int qrow = qt * 128 + row;
    const uint32_t lane_off = uint32_t((warp & 3) * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    const uint32_t tS = tm_S + t * 128 + part * CW + lane_off;
    const uint32_t tO = tm_O + t * D + part * DW + lane_off;
    const uint32_t sP = smem_u32(smem + Cfg::OFF_P + t * Cfg::P_TILE);
    float* xmax = reinterpret_cast<float*>(smem + Cfg::OFF_XMAX) + t * SPLIT * 128;  // [SPLIT][128]
    float m = -INFINITY, l = 0.0f, alpha_prev = 1.0f;
    float acc[DW];
#pragma unroll
    for (int i = 0; i < DW; ++i) acc[i] = 0.0f;

    auto fold = [&](uint32_t ph, float alpha) {  // acc = acc * alpha + (P V of the finished tile)
      mbar_wait(&o_full[t], ph, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < DW / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tO + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          ffma2(acc[c * 32 + i], acc[c * 32 + i + 1], acc[c * 32 + i], acc[c * 32 + i + 1], alpha, alpha,
                __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      }
      tc_fence_before_sync();
    };

    for (int j = 0; j < n_mine; ++j) {
      const uint32_t jph = j & 1;
      const bool need_mask = (p.causal && j == qt) || ((j + 1) * 128 > p.S);
      mbar_wait(&s_full[t], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      // pass 1: maximum over this thread's columns
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < CW / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tS + c * 32, r);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kc = j * 128 + part * CW + c * 32 + i;
            if (!(kc >= p.S || (p.causal && kc > qrow))) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        } else {
          float m0 = __uint_as_float(r[0]), m1 = __uint_as_float(r[1]), m2 = __uint_as_float(r[2]), m3 = __uint_as_float(r[3]);
#pragma unroll
          for (int i = 4; i < 28; i += 8) {
            m0 = fmax3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
            m1 = fmax3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
            m2 = fmax3(m2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
            m3 = fmax3(m3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
          }
          m0 = fmax3(m0, __uint_as_float(r[28]), __uint_as_float(r[29]));
          m1 = fmax3(m1, __uint_as_float(r[30]), __uint_as_float(r[31]));
          mx = fmax3(mx, fmaxf(m0, m1), fmaxf(m2, m3));
        }
      }
      if constexpr (SPLIT > 1) {
        // exchange with the thread that owns the other columns of this row (named barrier per
        // query tile: 256 threads; two buffers alternate so that one barrier per key tile suffices)
        float* xb = xmax;  // one buffer, protected by the two barriers of this iteration
        xb[part * 128 + row] = mx;
        asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(128 * SPLIT) : "memory");
        mx = fmaxf(mx, xb[(part ^ 1) * 128 + row]);
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;  // a fully masked row keeps p = 0
      const float alpha = ex2_approx((m - m_use) * sl2);
      const float msl2 = m_use * sl2;
      // the previous tile's P V is complete by now (the tensor core ran it before this S)
      if (j > 0) fold(jph ^ 1, alpha_prev);
      // The two query tiles take turns with the exponentials (A0, B0, A1, B1, ...): the special
      // function unit is the busiest unit of this kernel, and while one tile keeps it busy the
      // other tile's barrier round trips, tensor-core products, maxima and folds run beside it
      // instead of all warps competing for it at once and then all leaving it idle.
      if (t == 0) {
        if (j > 0 && b_valid) mbar_wait(&exp_done[1], jph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
      } else {
        if (j < nA) mbar_wait(&exp_done[0], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
      }
      // pass 2: probabilities -> shared memory (bf16), partial row sum
      float rs0 = 0.0f, rs1 = 0.0f, rs2 = 0.0f, rs3 = 0.0f;
      const float nmsl2 = -msl2;
#pragma unroll 1
      for (int c = 0; c < CW / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tS + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float x0, x1, x2, x3;
            ffma2(x0, x1, __uint_as_float(r[i]), __uint_as_float(r[i + 1]), sl2, sl2, nmsl2, nmsl2);
            ffma2(x2, x3, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]), sl2, sl2, nmsl2, nmsl2);
            x0 = ex2_approx(x0); x1 = ex2_approx(x1); x2 = ex2_approx(x2); x3 = ex2_approx(x3);
            fadd2(rs0, rs1, rs0, rs1, x0, x1);
            fadd2(rs2, rs3, rs2, rs3, x2, x3);
            pk[i >> 1] = pack_bf16x2(x0, x1);
            pk[(i >> 1) + 1] = pack_bf16x2(x2, x3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(r[i]), sl2, nmsl2));
            float p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), sl2, nmsl2));
            const int kc = j * 128 + part * CW + c * 32 + i;
            if (kc >= p.S || (p.causal && kc > qrow)) p0 = 0.0f;
            if (kc + 1 >= p.S || (p.causal && kc + 1 > qrow)) p1 = 0.0f;
            rs0 += p0;
            rs1 += p1;
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
        }
        store_row_chunk32(sP, row, part * CW + c * 32, pk);
      }
      rs0 += rs2;
      rs1 += rs3;
      mbar_arrive_warp(&exp_done[t]);
      l = fmaf(l, alpha, rs0 + rs1);
      m = m_new;
      alpha_prev = alpha;
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive_warp(&p_ready[t]);
      if constexpr (SPLIT > 1) {
        // the exchange buffer may be rewritten only after both threads of every row have read it
        asm volatile("bar.sync %0, %1;" ::"r"(3 + t), "r"(128 * SPLIT) : "memory");
      }
    }
    if (n_mine > 0) {
      fold((n_mine - 1) & 1, alpha_prev);
      if constexpr (SPLIT > 1) {
        // total row sum = sum of the two partial sums (both were rescaled with the same maxima)
        xmax[part * 128 + row] = l;
        asm volatile("bar.sync %0, %1;" ::"r"(1 + t), "r"(128 * SPLIT) : "memory");
        l += xmax[(part ^ 1) * 128 + row];
      }
      if (qrow < p.S) {
        const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + (long long)b * p.o_bs + (long long)qrow * p.o_ss +
                              (long long)h * p.o_hs + part * DW;
        __nv_bfloat16* lrow = p.o_lo ? reinterpret_cast<__nv_bfloat16*>(p.o_lo) + (orow - reinterpret_cast<__nv_bfloat16*>(p.o)) : nullptr;
        const float* mrow = (p.v_mean && l > 0.0f) ? p.v_mean + ((long long)b * p.Hkv + kvh) * D + part * DW : nullptr;
#pragma unroll
        for (int c = 0; c < DW / 8; ++c) {
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = acc[c * 8 + e] * inv;
          store_out8(orow + c * 8, lrow ? lrow + c * 8 : nullptr, mrow ? mrow + c * 8 : nullptr, x);
        }
        if (p.lse && part == 0) p.lse[((long long)b * p.Hq + h) * p.S + qrow] = (l > 0.0f) ? m * p.scale + logf(l) : -INFINITY;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == Cfg::SWARPS + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}
// =====================================================================================
// forward at head_dim 64.  Same roles as attn_fwd_kernel (two 128-query tiles per CTA, two threads
// per query row, one TMA and one MMA warp), with a shorter dependency chain per key tile:
//   * a thread reads its 64 scores from TMEM once and keeps them in registers; as soon as all
//     threads of a query tile have done so, the tensor core may start the tile's next S = Q K^T,
//     which then runs beside the exponentials instead of after them;
//   * O stays in TMEM and P V accumulates into it.  The running maximum used for the exponentials
//     is only replaced when the true maximum has grown by more than 2^8 (in the exp2 domain); then,
//     and only then, O is read, scaled and written back.  P <= 2^8 keeps bf16 P and the f32 row sum
//     exact enough, and the final O / l does not depend on which maximum was used.
// =====================================================================================
// NT = query tiles per CTA.  NT = 2: the two tiles share every K / V tile and take turns with the
// exponentials (one CTA per SM).  NT = 1: half the shared memory, tensor memory and threads, so
// that two CTAs are resident per SM and the hardware interleaves their phases; K and V are then
// fetched once per query tile (from L2), and V has a single stage.
template <int NT, bool PTM = false>
struct Fwd64Cfg {
  static_assert(!PTM || NT == 1, "P through TMEM is built for one query tile per CTA");
  static constexpr int TILE = 128 * 64 * 2;
  static constexpr int P_TILE = PTM ? 0 : 128 * 128 * 2;  // PTM: P goes to TMEM, no shared-memory tile
  static constexpr int NSV = (NT == 2 || PTM) ? 2 : 1;  // V stages
  static constexpr int OFF_Q = 0;                 // NT tiles
  static constexpr int OFF_K = NT * TILE;         // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * TILE;  // NSV stages
  static constexpr int OFF_P = OFF_V + NSV * TILE;  // NT tiles
  static constexpr int OFF_BAR = OFF_P + NT * P_TILE;
  static constexpr int OFF_XMAX = OFF_BAR + 256;  // float [NT tiles][2 buffers][2 parts][128]
  static constexpr int SMEM = OFF_XMAX + NT * 2 * 2 * 128 * 4 + 1024;
  static constexpr int TMEM_COLS = NT == 2 ? 512 : 256;
  static constexpr int SWARPS = 8 * NT;
  static constexpr int THREADS = (SWARPS + 2) * 32;
  static constexpr int CTAS_PER_SM = NT == 2 ? 1 : 2;
};

template <int NT, bool PTM = false>
__global__ void __launch_bounds__(Fwd64Cfg<NT, PTM>::THREADS, Fwd64Cfg<NT, PTM>::CTAS_PER_SM)
attn_fwd64_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using Cfg = Fwd64Cfg<NT, PTM>;
  constexpr int NSV = Cfg::NSV;
  constexpr int D = 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // per query tile: S is in TMEM
  uint64_t* s_free = bars + 11;     // per query tile (8 arrivals, one per warp): S has been read into registers
  uint64_t* p_ready = bars + 13;    // per query tile (8 arrivals, one per warp): P is in shared memory
  uint64_t* o_full = bars + 15;     // per query tile: the P V product issued last is complete
  uint64_t* exp_done = bars + 17;   // per query tile (8 arrivals): its exponentials of a key tile are issued
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + 127) / 128;
  // blocks are handed out x-fastest, so with the tile index in z every head's heavy (late) causal
  // tiles start before anybody's light ones
  const int pair = (int)gridDim.z - 1 - (int)blockIdx.z;
  const int qtA = NT * pair, qtB = NT * pair + 1;
  const bool b_valid = NT == 2 && qtB < n_qt;
  const int h = blockIdx.x, b = blockIdx.y;
  const int kvh = h / (p.Hq / p.Hkv);
  const int nA = p.causal ? min(qtA + 1, n_qt) : n_qt;
  const int nB = b_valid ? (p.causal ? min(qtB + 1, n_qt) : n_qt) : 0;
  const int n_kv = max(nA, nB);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 8);   // one arrival per warp (eight warps per query tile)
      mbar_init(&p_ready[i], 8);
      mbar_init(&o_full[i], 1);
      mbar_init(&exp_done[i], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == Cfg::SWARPS + 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_S = tmem_base;        // S of tile A at +0, of tile B at +128
  const uint32_t tm_O = tmem_base + NT * 128;  // O of tile A at +0, of tile B at +64
  const uint32_t tm_P = tmem_base + 192;       // PTM: P as bf16 pairs, 64 columns (A operand of P V)

  if (warp == Cfg::SWARPS) {
    // ---------------- TMA ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, (b_valid ? 2 : 1) * Cfg::TILE);
      tma_load_4d(smem + Cfg::OFF_Q, &tmQ, q_full, 0, h, qtA * 128, b);
      if (b_valid) tma_load_4d(smem + Cfg::OFF_Q + Cfg::TILE, &tmQ, q_full, 0, h, qtB * 128, b);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        mbar_arrive_expect_tx(&k_full[st], Cfg::TILE);
        tma_load_4d(smem + Cfg::OFF_K + st * Cfg::TILE, &tmK, &k_full[st], 0, kvh, j * 128, b);
        const int sv = j % NSV;
        const uint32_t phv = (j / NSV) & 1;
        mbar_wait(&v_empty[sv], phv ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        mbar_arrive_expect_tx(&v_full[sv], Cfg::TILE);
        tma_load_4d(smem + Cfg::OFF_V + sv * Cfg::TILE, &tmV, &v_full[sv], 0, kvh, j * 128, b);
      }
    }
  } else if (warp == Cfg::SWARPS + 1) {
    // ---------------- MMA ----------------
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(128, D, 0, 1);
      const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q);
      auto issue_s = [&](int t, int j) {  // S_t = Q_t K_j^T
        const uint32_t sK = smem_u32(smem + Cfg::OFF_K + (j & 1) * Cfg::TILE);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tm_S + t * 128, make_smem_desc(sQ + t * Cfg::TILE + k * 32u, 16, 1024),
                       make_smem_desc(sK + k * 32u, 16, 1024), idesc_s, k > 0);
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int j) {  // O_t (+)= P_t V_j
        const uint32_t sP = smem_u32(smem + Cfg::OFF_P + t * Cfg::P_TILE);
        const uint32_t sV = smem_u32(smem + Cfg::OFF_V + (j % NSV) * Cfg::TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 128 keys in steps of 16
          const uint64_t db = make_smem_desc(sV + k * 2048u, 16384, 1024);  // V is MN-major: [key][d]
          if (PTM) {
            // A from TMEM: lane = query row, 16 keys of a step = 8 columns of bf16 pairs
            umma_bf16_ts(tm_O + t * D, tm_P + k * 8u, db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          } else {
            const uint64_t da = make_smem_desc(sP + (k >> 2) * 16384u + (k & 3) * 32u, 16, 1024);
            umma_bf16_ss(tm_O + t * D, da, db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(&o_full[t]);
      };
      mbar_wait(q_full, 0, abort_flag, p.status, FAULT_WAIT_ATTN);
      mbar_wait(&k_full[0], 0, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      issue_s(0, 0);
      if (b_valid) issue_s(1, 0);
      umma_commit(&k_empty[0]);
      for (int j = 0; j < n_kv; ++j) {
        const uint32_t jph = j & 1;
        const uint32_t phv = (j / NSV) & 1;
        const uint32_t kph1 = ((j + 1) >> 1) & 1;
        // the next S of a tile may start once the tile's threads hold the current S in registers
        if (j + 1 < nA) {
          mbar_wait(&s_free[0], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
          mbar_wait(&k_full[(j + 1) & 1], kph1, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_s(0, j + 1);
        }
        if (j + 1 < nB) {
          mbar_wait(&s_free[1], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
          mbar_wait(&k_full[(j + 1) & 1], kph1, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_s(1, j + 1);
        }
        if (j + 1 < n_kv) umma_commit(&k_empty[(j + 1) & 1]);
        if (j < nA) {
          mbar_wait(&p_ready[0], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
          mbar_wait(&v_full[j % NSV], phv, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_pv(0, j);
        }
        if (j < nB) {
          mbar_wait(&p_ready[1], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
          mbar_wait(&v_full[j % NSV], phv, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_pv(1, j);
        }
        umma_commit(&v_empty[j % NSV]);
      }
    }
  } else {
    // ---------------- softmax + output ----------------
    // warp w: query tile (w >> 2) & 1, TMEM lane quarter w & 3, column half w >> 3.  A thread owns
    // one query row, 64 of its score columns and 32 of its output columns.
    const int t = NT == 2 ? (warp >> 2) & 1 : 0;
    const int part = NT == 2 ? warp >> 3 : warp >> 2;
    const int n_mine = t ? nB : nA;
    const int qt = t ? qtB : qtA;
    const int row = (warp & 3) * 32 + lane;
    const int qrow = qt * 128 + row;
    const uint32_t lane_off = uint32_t((warp & 3) * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    const uint32_t tS = tm_S + t * 128 + part * 64 + lane_off;
    const uint32_t tO = tm_O + t * D + part * 32 + lane_off;
    const uint32_t sP = smem_u32(smem + Cfg::OFF_P + t * Cfg::P_TILE);
    const uint32_t tP = tm_P + part * 32 + lane_off;  // PTM: this thread's 64 probabilities = 32 columns of its lane
    float* xbase = reinterpret_cast<float*>(smem + Cfg::OFF_XMAX) + t * 512;  // [2 buffers][2 parts][128]
    const int bar_id = 1 + t;
    float m_used = -INFINITY, l = 0.0f;

    for (int j = 0; j < n_mine; ++j) {
      const uint32_t jph = j & 1;
      const bool need_mask = (p.causal && j == qt) || ((j + 1) * 128 > p.S);
      mbar_wait(&s_full[t], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      uint32_t ra[32], rb[32];
      tmem_ld_32x32b_x32(tS, ra);
      tmem_ld_32x32b_x32(tS + 32, rb);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(&s_free[t]);
      if (need_mask) {
        const int kc0 = j * 128 + part * 64;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (kc0 + i >= p.S || (p.causal && kc0 + i > qrow)) ra[i] = 0xff800000u;
          if (kc0 + 32 + i >= p.S || (p.causal && kc0 + 32 + i > qrow)) rb[i] = 0xff800000u;
        }
      }
      float mx;
      {
        float m0 = __uint_as_float(ra[0]), m1 = __uint_as_float(ra[1]), m2 = __uint_as_float(rb[0]), m3 = __uint_as_float(rb[1]);
#pragma unroll
        for (int i = 2; i < 30; i += 4) {
          m0 = fmax3(m0, __uint_as_float(ra[i]), __uint_as_float(ra[i + 1]));
          m1 = fmax3(m1, __uint_as_float(ra[i + 2]), __uint_as_float(ra[i + 3]));
          m2 = fmax3(m2, __uint_as_float(rb[i]), __uint_as_float(rb[i + 1]));
          m3 = fmax3(m3, __uint_as_float(rb[i + 2]), __uint_as_float(rb[i + 3]));
        }
        m0 = fmax3(m0, __uint_as_float(ra[30]), __uint_as_float(ra[31]));
        m2 = fmax3(m2, __uint_as_float(rb[30]), __uint_as_float(rb[31]));
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      {
        // the two threads of a row exchange their maxima; the buffers alternate, so the one
        // barrier of the next key tile also orders this tile's reads before the next reuse
        float* xb = xbase + (j & 1) * 256;
        xb[part * 128 + row] = mx;
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(256) : "memory");
        mx = fmaxf(mx, xb[(part ^ 1) * 128 + row]);
      }
      const float m_new = fmaxf(m_used, mx);
      float alpha = 1.0f;
      bool resc = false;
      if (m_used == -INFINITY) {
        m_used = m_new;  // nothing accumulated under the old value (l == 0, O == 0)
      } else if ((m_new - m_used) * sl2 > 8.0f) {
        alpha = ex2_approx((m_used - m_new) * sl2);
        resc = true;
        m_used = m_new;
      }
      const float nmsl2 = (m_used == -INFINITY) ? 0.0f : -m_used * sl2;  // a fully masked row keeps p = 0
      if (j > 0) {
        // the previous P V has read P from shared memory and has been added to O (it was issued
        // when this tile's last P was ready, a whole softmax ago: the wait is normally over)
        mbar_wait(&o_full[t], jph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, resc)) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t q8[8];
            tmem_ld_32x32b_x8(tO + c * 8, q8);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) q8[i] = __float_as_uint(__uint_as_float(q8[i]) * alpha);
            tmem_st_32x32b_x8(tO + c * 8, q8);
          }
          tmem_st_wait();
        }
      }
      // the two query tiles take turns with the exponentials (A0, B0, A1, B1, ...)
      if (NT == 2) {
        if (t == 0) {
          if (j > 0 && b_valid) mbar_wait(&exp_done[1], jph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        } else {
          if (j < nA) mbar_wait(&exp_done[0], jph, abort_flag, p.status, FAULT_WAIT_ATTN);
        }
      }
      // probabilities: bf16, stored to the P tile eight at a time as they are produced (the stores
      // run in the shadow of the exponentials), and their row sum
      float rs0 = 0.0f, rs1 = 0.0f, rs2 = 0.0f, rs3 = 0.0f;
      const uint32_t p_half = sP + part * 16384u;  // this thread's 64 columns are one 128-byte row of a half tile
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int u = 0; u < 8; u += 4) {
          float x0, x1, x2, x3;
          ffma2(x0, x1, __uint_as_float(ra[i + u]), __uint_as_float(ra[i + u + 1]), sl2, sl2, nmsl2, nmsl2);
          ffma2(x2, x3, __uint_as_float(ra[i + u + 2]), __uint_as_float(ra[i + u + 3]), sl2, sl2, nmsl2, nmsl2);
          x0 = ex2_approx(x0); x1 = ex2_approx(x1); x2 = ex2_approx(x2); x3 = ex2_approx(x3);
          fadd2(rs0, rs1, rs0, rs1, x0, x1);
          fadd2(rs2, rs3, rs2, rs3, x2, x3);
          pk[u >> 1] = pack_bf16x2(x0, x1);
          pk[(u >> 1) + 1] = pack_bf16x2(x2, x3);
        }
        if (PTM) tmem_st_32x32b_x4(tP + (i >> 1), pk);
        else st_shared_v4(p_half + swz128(row, i >> 3), pk[0], pk[1], pk[2], pk[3]);
      }
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int u = 0; u < 8; u += 4) {
          float x0, x1, x2, x3;
          ffma2(x0, x1, __uint_as_float(rb[i + u]), __uint_as_float(rb[i + u + 1]), sl2, sl2, nmsl2, nmsl2);
          ffma2(x2, x3, __uint_as_float(rb[i + u + 2]), __uint_as_float(rb[i + u + 3]), sl2, sl2, nmsl2, nmsl2);
          x0 = ex2_approx(x0); x1 = ex2_approx(x1); x2 = ex2_approx(x2); x3 = ex2_approx(x3);
          fadd2(rs0, rs1, rs0, rs1, x0, x1);
          fadd2(rs2, rs3, rs2, rs3, x2, x3);
          pk[u >> 1] = pack_bf16x2(x0, x1);
          pk[(u >> 1) + 1] = pack_bf16x2(x2, x3);
        }
        if (PTM) tmem_st_32x32b_x4(tP + 16 + (i >> 1), pk);
        else st_shared_v4(p_half + swz128(row, 4 + (i >> 3)), pk[0], pk[1], pk[2], pk[3]);
        // the turn is handed over with 24 of the 64 exponentials still to go: the other tile needs
        // a few hundred clocks from the barrier to its first exponential (measured: better than
        // handing over at the end, at 16 or at 32 to go)
        if (NT == 2 && i == 0) mbar_arrive_warp(&exp_done[t]);
      }
      l = fmaf(l, alpha, (rs0 + rs1) + (rs2 + rs3));
      if (PTM) {
        tmem_st_wait();
        tc_fence_before_sync();
      } else {
        tc_fence_before_sync();
        fence_proxy_async_smem();
      }
      mbar_arrive_warp(&p_ready[t]);
    }
    if (n_mine > 0) {
      mbar_wait(&o_full[t], (n_mine - 1) & 1, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      uint32_t ro[32];
      tmem_ld_32x32b_x32(tO, ro);
      tmem_ld_wait();
      // total row sum = sum of the two partial sums (both used the same maxima)
      float* xb = xbase + (n_mine & 1) * 256;
      xb[part * 128 + row] = l;
      asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(256) : "memory");
      l += xb[(part ^ 1) * 128 + row];
      if (qrow < p.S) {
        const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + (long long)b * p.o_bs + (long long)qrow * p.o_ss +
                              (long long)h * p.o_hs + part * 32;
        __nv_bfloat16* lrow = p.o_lo ? reinterpret_cast<__nv_bfloat16*>(p.o_lo) + (orow - reinterpret_cast<__nv_bfloat16*>(p.o)) : nullptr;
        const float* mrow = (p.v_mean && l > 0.0f) ? p.v_mean + ((long long)b * p.Hkv + kvh) * D + part * 32 : nullptr;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float x[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) x[e] = __uint_as_float(ro[c * 8 + e]) * inv;
          store_out8(orow + c * 8, lrow ? lrow + c * 8 : nullptr, mrow ? mrow + c * 8 : nullptr, x);
        }
        if (p.lse && part == 0)
          p.lse[((long long)b * p.Hq + h) * p.S + qrow] = (l > 0.0f) ? m_used * p.scale + logf(l) : -INFINITY;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == Cfg::SWARPS + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// =====================================================================================
// backward: one 128-key tile of one KV head per CTA, looping over the query heads of its group
// and over query tiles.  Warps 0-15 compute (warp w touches TMEM lanes (w%4)*32.. and the column
// quarter w/4), warp 16 issues TMA, warp 17 issues MMAs.
//   S = Q K^T, dP = dO V^T                  -> TMEM
//   P = exp2(S*c - lse), dS = P*(dP - delta) -> shared memory (bf16); the softmax scale is applied
//                                              once to dQ (in the conversion kernel) and to dK
//   dV += P^T dO, dK += dS^T Q              -> TMEM, kept across the whole loop (the GQA reduce)
//   dQ  = dS K                              -> TMEM -> f32 red.global.add into a workspace
// Transposed form (TS, D = 64, the default there): the score tiles are formed as S^T = K Q^T and
// dP^T = V dO^T, so a compute thread owns a key and 32 queries; P^T goes back to TMEM as bf16 pairs and
// the dV product reads its A operand from there; dS^T goes to one shared-memory tile that serves dK
// (K-major A) and dQ (MN-major A).  lse and delta now belong to the columns: -lse*log2(e) and -delta
// of the query tile sit in shared memory (two buffers) and every thread reads its 32 of each.
// With D = 64 the dQ tile has TMEM columns of its own.  The S / dP products of the next query tile
// are then issued as soon as the compute warps have read the current S / dP into registers, ahead
// of the current dV, dK, dQ: the tensor core works on them while the exponentials run, and the
// compute warps go from one query tile to the next without waiting for a product (only their
// stores of P / dS wait for the products that still read the tile before).  With D = 128 dQ reuses
// the S columns (512 columns in total): its read-out comes first and S / dP follow it.
// =====================================================================================
template <int D, bool TS = false>
struct BwdCfg {
  static_assert(!TS || D == 64, "the transposed form is built for head_dim 64");
  static constexpr int TILE = 128 * D * 2;
  static constexpr int P_TILE = 128 * 128 * 2;
  static constexpr int NS = (D == 64) ? 3 : 1;  // Q / dO stages
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;               // NS stages
  static constexpr int OFF_DO = OFF_Q + NS * TILE;     // NS stages
  static constexpr int OFF_P = OFF_DO + NS * TILE;     // TS: no P tile; [3 buffers][-lse2, -delta][128] floats instead
  static constexpr int OFF_DS = OFF_P + (TS ? 3072 : P_TILE);
  static constexpr bool DQ_OWN = (D == 64);  // dQ has its own TMEM columns
  // with D = 64 a [128 x 64] f32 tile (two 128-byte-swizzled halves of 32 columns) stages dQ for
  // the TMA unit, which adds it to the f32 accumulation buffer
  static constexpr int OFF_DQS = OFF_DS + P_TILE;
  static constexpr int OFF_BAR = OFF_DQS + (DQ_OWN ? 128 * 64 * 4 : 0);
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + D;
  static constexpr int COL_DQ = DQ_OWN ? 256 + 2 * D : 0;
  static constexpr int COL_PT = 448;                // TS: P^T as bf16 pairs (64 columns), A operand of dV
  static constexpr int CWARPS = 16;                 // compute warps
  static constexpr int THREADS = (CWARPS + 2) * 32;
};

template <int D, bool TS = false>
__global__ void __launch_bounds__(BwdCfg<D, TS>::THREADS, 1)  // 18 warps: five on one scheduler, hence 96 registers
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const __grid_constant__ CUtensorMap tmDQ, const AttnParams p) {
  using Cfg = BwdCfg<D, TS>;
  constexpr int ATOMS = D / 64;
  constexpr int NS = Cfg::NS;
  constexpr int NCT = Cfg::CWARPS * 32;  // compute threads
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;        // 1
  uint64_t* qdo_full = bars + 1;   // NS (<= 3)
  uint64_t* qdo_empty = bars + 4;  // NS
  uint64_t* sdp_full = bars + 7;   // 1
  uint64_t* pds_ready = bars + 8;  // 1 (one arrival per compute warp)
  uint64_t* dq_full = bars + 9;    // 1
  uint64_t* dq_read = bars + 10;   // 1 (one arrival per compute warp)
  uint64_t* sdp_free = bars + 11;  // 1 (one arrival per compute warp): S / dP are in registers
  uint64_t* stage_free = bars + 12;  // 1 (one arrival, thread 0): the TMA unit has read the dQ staging tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // key tile; tile 0 has the most work under the causal mask.  It is the slowest grid index, so
  // the longest blocks of all heads start first.
  const int jt = blockIdx.z;
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int rep = p.Hq / p.Hkv;
  const int n_qt = (p.S + 127) / 128;
  const int i0 = p.causal ? jt : 0;
  const int per_head = n_qt - i0;
  const int iters = per_head * rep;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < NS; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, Cfg::CWARPS);  // one arrival per warp
    mbar_init(dq_full, 1);
    mbar_init(dq_read, Cfg::CWARPS);
    mbar_init(sdp_free, Cfg::CWARPS);
    mbar_init(stage_free, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
    prefetch_tmap(&tmDQ);
  }
  if (warp == Cfg::CWARPS + 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == Cfg::CWARPS) {
    // ---------------- TMA ----------------
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * Cfg::TILE);
#pragma unroll
      for (int a = 0; a < ATOMS; ++a) {
        tma_load_4d(smem + Cfg::OFF_K + a * 16384, &tmK, kv_full, a * 64, kvh, jt * 128, b);
        tma_load_4d(smem + Cfg::OFF_V + a * 16384, &tmV, kv_full, a * 64, kvh, jt * 128, b);
      }
      for (int it = 0; it < iters; ++it) {
        const int st = it % NS;
        const uint32_t ph = (it / NS) & 1;
        const int h = kvh * rep + it / per_head;
        const int qi = i0 + it % per_head;
        mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        mbar_arrive_expect_tx(&qdo_full[st], 2 * Cfg::TILE);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a) {
          tma_load_4d(smem + Cfg::OFF_Q + st * Cfg::TILE + a * 16384, &tmQ, &qdo_full[st], a * 64, h, qi * 128, b);
          tma_load_4d(smem + Cfg::OFF_DO + st * Cfg::TILE + a * 16384, &tmdO, &qdo_full[st], a * 64, h, qi * 128, b);
        }
      }
    }
  } else if (warp == Cfg::CWARPS + 1) {
    // ---------------- MMA ----------------
    if (lane == 0 && iters > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // Q K^T, dO V^T
      const uint32_t idesc_t = make_idesc_bf16(128, D, 1, 1);     // P^T dO, dS^T Q
      const uint32_t idesc_q = make_idesc_bf16(128, D, 0, 1);     // dS K
      const uint32_t sK = smem_u32(smem + Cfg::OFF_K), sV = smem_u32(smem + Cfg::OFF_V);
      const uint32_t sP = smem_u32(smem + Cfg::OFF_P), sDS = smem_u32(smem + Cfg::OFF_DS);
      auto issue_sdp = [&](int it) {
        const int st = it % NS;
        const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q + st * Cfg::TILE);
        const uint32_t sDO = smem_u32(smem + Cfg::OFF_DO + st * Cfg::TILE);
        mbar_wait(&qdo_full[st], (it / NS) & 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        tc_fence_after_sync();
        // TS: the transposed products S^T = K Q^T and dP^T = V dO^T (TMEM lane = key, column = query)
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384u + (k & 3) * 32u;
          const uint64_t dq_ = make_smem_desc(sQ + off, 16, 1024), dk_ = make_smem_desc(sK + off, 16, 1024);
          umma_bf16_ss(tmem_base + Cfg::COL_S, TS ? dk_ : dq_, TS ? dq_ : dk_, idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384u + (k & 3) * 32u;
          const uint64_t do_ = make_smem_desc(sDO + off, 16, 1024), dv_ = make_smem_desc(sV + off, 16, 1024);
          umma_bf16_ss(tmem_base + Cfg::COL_DP, TS ? dv_ : do_, TS ? do_ : dv_, idesc_s, k > 0);
        }
        umma_commit(sdp_full);
      };
      mbar_wait(kv_full, 0, abort_flag, p.status, FAULT_WAIT_ATTN);
      issue_sdp(0);
      for (int it = 0; it < iters; ++it) {
        const int st = it % NS;
        const uint32_t iph = it & 1;
        const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q + st * Cfg::TILE);
        const uint32_t sDO = smem_u32(smem + Cfg::OFF_DO + st * Cfg::TILE);
        if (Cfg::DQ_OWN && it + 1 < iters) {
          // the next S / dP start as soon as the compute warps hold the current ones in registers:
          // they run beside the exponentials, and the compute warps find them ready afterwards
          mbar_wait(sdp_free, iph, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_sdp(it + 1);
        }
        mbar_wait(pds_ready, iph, abort_flag, p.status, FAULT_WAIT_ATTN);
        tc_fence_after_sync();
        // K dimension of the next three products = the 128 query rows (dV, dK) or 128 keys (dQ)
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dV += P^T dO
          if (TS)  // A = P^T from TMEM: lane = key, 16 queries of a step = 8 columns of bf16 pairs
            umma_bf16_ts(tmem_base + Cfg::COL_DV, tmem_base + Cfg::COL_PT + k * 8u,
                         make_smem_desc(sDO + k * 2048u, 16384, 1024), idesc_q, (it > 0 || k > 0));
          else
            umma_bf16_ss(tmem_base + Cfg::COL_DV, make_smem_desc(sP + k * 2048u, 16384, 1024),
                         make_smem_desc(sDO + k * 2048u, 16384, 1024), idesc_t, (it > 0 || k > 0));
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dK += dS^T Q  (TS: the dS tile holds dS^T, rows = keys: K-major A)
          if (TS)
            umma_bf16_ss(tmem_base + Cfg::COL_DK, make_smem_desc(sDS + (k >> 2) * 16384u + (k & 3) * 32u, 16, 1024),
                         make_smem_desc(sQ + k * 2048u, 16384, 1024), idesc_q, (it > 0 || k > 0));
          else
            umma_bf16_ss(tmem_base + Cfg::COL_DK, make_smem_desc(sDS + k * 2048u, 16384, 1024),
                         make_smem_desc(sQ + k * 2048u, 16384, 1024), idesc_t, (it > 0 || k > 0));
        }
        if (Cfg::DQ_OWN && it > 0) {  // the dQ tile of the query tile before has been read out
          mbar_wait(dq_read, iph ^ 1, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dQ = dS K  (TS: dS^T read MN-major, its rows are the keys of the contraction)
          if (TS)
            umma_bf16_ss(tmem_base + Cfg::COL_DQ, make_smem_desc(sDS + k * 2048u, 16384, 1024),
                         make_smem_desc(sK + k * 2048u, 16384, 1024), idesc_t, k > 0);
          else
            umma_bf16_ss(tmem_base + Cfg::COL_DQ, make_smem_desc(sDS + (k >> 2) * 16384u + (k & 3) * 32u, 16, 1024),
                         make_smem_desc(sK + k * 2048u, 16384, 1024), idesc_q, k > 0);
        }
        umma_commit(dq_full);
        umma_commit(&qdo_empty[st]);
        if (!Cfg::DQ_OWN && it + 1 < iters) {  // dQ sits in the S columns: wait until it has been read out
          mbar_wait(dq_read, iph, abort_flag, p.status, FAULT_WAIT_ATTN);
          tc_fence_after_sync();
          issue_sdp(it + 1);
        }
      }
    }
  } else {
    // ---------------- compute warps ----------------
    const int q4 = warp & 3;        // TMEM lane quarter
    const int cq = warp >> 2;       // column quarter
    const int row = q4 * 32 + lane;
    const uint32_t lane_off = uint32_t(q4 * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    const uint32_t sP = smem_u32(smem + Cfg::OFF_P), sDS = smem_u32(smem + Cfg::OFF_DS);
    constexpr int DQC = D / 4;  // dQ / dK / dV columns per thread

    // adds this thread's part of the dQ tile of iteration `it` to the f32 accumulation buffer
    auto drain_dq = [&](int it) {
      const int h = kvh * rep + it / per_head;
      const int qrow = (i0 + it % per_head) * 128 + row;
      mbar_wait(dq_full, it & 1, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      float* dq_row = p.dq_acc + (p.det ? (long long)jt * p.dq_slice : 0LL) + (((long long)b * p.S + qrow) * p.Hq + h) * D + cq * DQC;
      if constexpr (DQC == 16) {
        // TMEM -> registers -> swizzled shared-memory tile -> one TMA reduce-add per half tile.
        // Adding 16-byte pieces of 32 different rows with one red.global per warp instruction was
        // the slowest part of this kernel; the TMA unit adds whole 128-byte rows, and rows past
        // the end of the sequence are clipped by the tensor map.
        uint32_t r[16];
        tmem_ld_32x32b_x16(tmem_base + Cfg::COL_DQ + cq * DQC + lane_off, r);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(dq_read);
        if (it > 0) {
          // the reduce of the query tile before has read the staging tile: thread 0 asks the TMA unit
          // (it issued that reduce a whole tile ago) and tells the others through a barrier word, which
          // costs them a wait only if they are ahead of thread 0's warp.  (A bar.sync of all 512 compute
          // threads stood here before: 510 -> 531 TFLOP/s.  Moving the reduce to the MMA thread, so that
          // the compute warps need no barrier at all, measured 450.)
          if (threadIdx.x == 0) {
            tma_store_wait_read<0>();
            mbar_arrive(stage_free);
          }
          mbar_wait(stage_free, (it - 1) & 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        }
        const uint32_t half = smem_u32(smem + Cfg::OFF_DQS) + (cq >> 1) * 16384u;
#pragma unroll
        for (int jv = 0; jv < 4; ++jv)
          st_shared_v4(half + swz128(row, (cq & 1) * 4 + jv), r[4 * jv], r[4 * jv + 1], r[4 * jv + 2], r[4 * jv + 3]);
        // the caller fences these stores together with its own and then calls issue_dq_reduce
        return;
      } else {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + Cfg::COL_DQ + cq * DQC + lane_off, r);
        tmem_ld_wait();
        // dQ shares the S columns: they are free for the next S / dP from here on
        tc_fence_before_sync();
        mbar_arrive_warp(dq_read);
        if (p.det) {
          if (qrow < p.S) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<uint4*>(dq_row + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
          }
          return;
        }
        // The [128 x 128] f32 tile is staged where P and dS lie (64 KB in a row; the products that read
        // them are complete, dq_full says so, and the next probabilities are a whole S / dP product and
        // their exponentials away) as four 128-byte-swizzled quarters of 32 columns, and the TMA unit adds
        // the quarters to the f32 buffer: whole 128-byte rows, clipped at the end of the sequence.  One
        // red.global of 16-byte pieces of 32 different rows per warp instruction stood here before.
        const uint32_t quarter = smem_u32(smem + Cfg::OFF_P) + cq * 16384u;
#pragma unroll
        for (int jv = 0; jv < 8; ++jv)
          st_shared_v4(quarter + swz128(row, jv), r[4 * jv], r[4 * jv + 1], r[4 * jv + 2], r[4 * jv + 3]);
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, %0;" ::"r"(NCT) : "memory");
        if (threadIdx.x == 0) {
          const int qi = i0 + it % per_head;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            tma_reduce_add_4d(&tmDQ, smem_u32(smem + Cfg::OFF_P) + c * 16384u, c * 32, h, qi * 128, b);
          tma_store_commit();
        }
        return;
      }
    };


    // after the staging tile of iteration `it` is complete and fenced in every compute warp: one
    // thread hands it to the TMA unit (two halves of 32 columns)
    auto issue_dq_reduce = [&](int it) {
      asm volatile("bar.sync 1, %0;" ::"r"(NCT) : "memory");
      if (threadIdx.x == 0) {
        const int h = kvh * rep + it / per_head;
        const int qi = i0 + it % per_head;
        if (p.det) {  // the map's last dimension runs over (key tile, batch element)
          tma_store_4d(&tmDQ, smem_u32(smem + Cfg::OFF_DQS), 0, h, qi * 128, jt * p.B + b);
          tma_store_4d(&tmDQ, smem_u32(smem + Cfg::OFF_DQS) + 16384u, 32, h, qi * 128, jt * p.B + b);
        } else {
          tma_reduce_add_4d(&tmDQ, smem_u32(smem + Cfg::OFF_DQS), 0, h, qi * 128, b);
          tma_reduce_add_4d(&tmDQ, smem_u32(smem + Cfg::OFF_DQS) + 16384u, 32, h, qi * 128, b);
        }
        tma_store_commit();
      }
    };

    // TS: the statistics belong to the columns (queries) of the transposed tiles, so every thread needs
    // all 128 of them: -lse * log2(e) and -delta of a query tile sit in shared memory, three buffers in
    // turn.  Threads 0..255 fetch one value each; the value for iteration it + 1 is requested at the top
    // of iteration it >= 1 and stored before that iteration's barrier (in issue_dq_reduce), which its
    // readers follow; the buffer's previous readers (iteration it - 2) are behind the barrier of it - 1.
    float* stat = reinterpret_cast<float*>(smem + Cfg::OFF_P);
    auto stat_load = [&](int it) -> float {
      if (threadIdx.x >= 256 || it >= iters) return 0.0f;
      const int sh = kvh * rep + it / per_head;
      const int sq = (i0 + it % per_head) * 128 + (int)(threadIdx.x & 127);
      if (sq >= p.S) return threadIdx.x < 128 ? -INFINITY : 0.0f;  // -inf -> p = 0
      const long long idx = ((long long)b * p.Hq + sh) * p.S + sq;
      return threadIdx.x < 128 ? -p.lse[idx] * LOG2E : -p.delta[idx];
    };
    auto stat_store = [&](int it, float v) {
      if (threadIdx.x < 256 && it < iters) stat[(it % 3) * 256 + threadIdx.x] = v;
    };
    if (TS) {
      stat_store(0, stat_load(0));
      stat_store(1, stat_load(1));
      asm volatile("bar.sync 1, %0;" ::"r"(NCT) : "memory");
    }

    for (int it = 0; it < iters; ++it) {
      const uint32_t iph = it & 1;
      const int h = kvh * rep + it / per_head;
      const int qi = i0 + it % per_head;
      const int qrow = qi * 128 + row;
      const bool row_ok = qrow < p.S;
      const long long stat_idx = ((long long)b * p.Hq + h) * p.S + qrow;
      float lse2 = 0.0f, dlt = 0.0f, stat_next = 0.0f;
      if (TS) {
        if (it >= 1) stat_next = stat_load(it + 1);
      } else {
        lse2 = row_ok ? p.lse[stat_idx] * LOG2E : INFINITY;  // +inf -> p = 0
        dlt = row_ok ? p.delta[stat_idx] : 0.0f;
      }
      const bool need_mask = (p.causal && qi == jt) || ((jt + 1) * 128 > p.S);
      mbar_wait(sdp_full, iph, abort_flag, p.status, FAULT_WAIT_ATTN);
      tc_fence_after_sync();
      if (TS) {
        // lane = key row of this CTA's key tile, columns = the 32 queries of this thread's quarter
        const int col0 = cq * 32;
        const int krow = jt * 128 + row;
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tmem_base + Cfg::COL_S + col0 + lane_off, rs);
        tmem_ld_32x32b_x32(tmem_base + Cfg::COL_DP + col0 + lane_off, rd);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive_warp(sdp_free);
        uint32_t pk[16], dk[16];
        const float* sb = stat + (it % 3) * 256 + col0;
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 nl = *reinterpret_cast<const float4*>(sb + i);
            const float4 nd = *reinterpret_cast<const float4*>(sb + 128 + i);
            float p0, p1, p2, p3, d0, d1, d2, d3;
            ffma2(p0, p1, __uint_as_float(rs[i]), __uint_as_float(rs[i + 1]), sl2, sl2, nl.x, nl.y);
            ffma2(p2, p3, __uint_as_float(rs[i + 2]), __uint_as_float(rs[i + 3]), sl2, sl2, nl.z, nl.w);
            fadd2(d0, d1, __uint_as_float(rd[i]), __uint_as_float(rd[i + 1]), nd.x, nd.y);
            fadd2(d2, d3, __uint_as_float(rd[i + 2]), __uint_as_float(rd[i + 3]), nd.z, nd.w);
            p0 = ex2_approx(p0); p1 = ex2_approx(p1); p2 = ex2_approx(p2); p3 = ex2_approx(p3);
            fmul2(d0, d1, d0, d1, p0, p1);
            fmul2(d2, d3, d2, d3, p2, p3);
            pk[i >> 1] = pack_bf16x2(p0, p1);
            pk[(i >> 1) + 1] = pack_bf16x2(p2, p3);
            dk[i >> 1] = pack_bf16x2(d0, d1);
            dk[(i >> 1) + 1] = pack_bf16x2(d2, d3);
          }
        } else {
          const bool key_ok = krow < p.S;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(rs[i]), sl2, sb[i]));
            float p1 = ex2_approx(fmaf(__uint_as_float(rs[i + 1]), sl2, sb[i + 1]));
            const int qr = qi * 128 + col0 + i;
            if (!key_ok || (p.causal && krow > qr)) p0 = 0.0f;
            if (!key_ok || (p.causal && krow > qr + 1)) p1 = 0.0f;
            const float d0 = p0 * (__uint_as_float(rd[i]) + sb[128 + i]);
            const float d1 = p1 * (__uint_as_float(rd[i + 1]) + sb[128 + i + 1]);
            pk[i >> 1] = pack_bf16x2(p0, p1);
            dk[i >> 1] = pack_bf16x2(d0, d1);
          }
        }
        // the products of the query tile before read P^T from TMEM and dS^T from shared memory:
        // dq_full, which the read-out of that tile's dQ waits for, also says that they are done
        if (it > 0) {
          drain_dq(it - 1);
          stat_store(it + 1, stat_next);
        }
        tmem_st_32x32b_x16(tmem_base + Cfg::COL_PT + cq * 16 + lane_off, pk);
        store_row_chunk32(sDS, row, col0, dk);
        tmem_st_wait();
      } else {
        const int col0 = cq * 32;
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tmem_base + Cfg::COL_S + col0 + lane_off, rs);
        tmem_ld_32x32b_x32(tmem_base + Cfg::COL_DP + col0 + lane_off, rd);
        tmem_ld_wait();
        if (Cfg::DQ_OWN) {
          tc_fence_before_sync();
          mbar_arrive_warp(sdp_free);
        }
        uint32_t pk[16], dk[16];
        const float nlse2 = -lse2, ndlt = -dlt;
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0, p1, d0, d1;
            ffma2(p0, p1, __uint_as_float(rs[i]), __uint_as_float(rs[i + 1]), sl2, sl2, nlse2, nlse2);
            fadd2(d0, d1, __uint_as_float(rd[i]), __uint_as_float(rd[i + 1]), ndlt, ndlt);
            p0 = ex2_approx(p0);
            p1 = ex2_approx(p1);
            fmul2(d0, d1, d0, d1, p0, p1);
            pk[i >> 1] = pack_bf16x2(p0, p1);
            dk[i >> 1] = pack_bf16x2(d0, d1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = ex2_approx(fmaf(__uint_as_float(rs[i]), sl2, nlse2));
            float p1 = ex2_approx(fmaf(__uint_as_float(rs[i + 1]), sl2, nlse2));
            const int kc = jt * 128 + col0 + i;
            if (kc >= p.S || (p.causal && kc > qrow)) p0 = 0.0f;
            if (kc + 1 >= p.S || (p.causal && kc + 1 > qrow)) p1 = 0.0f;
            const float d0 = p0 * (__uint_as_float(rd[i]) + ndlt);
            const float d1 = p1 * (__uint_as_float(rd[i + 1]) + ndlt);
            pk[i >> 1] = pack_bf16x2(p0, p1);
            dk[i >> 1] = pack_bf16x2(d0, d1);
          }
        }
        // the products of the query tile before read P / dS from shared memory: dq_full, which
        // the read-out of that tile's dQ waits for, also says that they are done
        if (Cfg::DQ_OWN && it > 0) drain_dq(it - 1);
        if (!Cfg::DQ_OWN && it > 0 && !p.det) {
          // D = 128: the TMA unit still may be reading the dQ tile staged over P and dS a query tile ago
          if (threadIdx.x == 0) {
            tma_store_wait_read<0>();
            mbar_arrive(stage_free);
          }
          mbar_wait(stage_free, (it - 1) & 1, abort_flag, p.status, FAULT_WAIT_ATTN);
        }
        store_row_chunk32(sP, row, col0, pk);
        store_row_chunk32(sDS, row, col0, dk);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();  // covers the P / dS stores and, with D = 64, the dQ staging stores
      mbar_arrive_warp(pds_ready);
      if (Cfg::DQ_OWN) {
        if (it > 0) issue_dq_reduce(it - 1);  // off the path to the next products
      } else {
        drain_dq(it);
      }
    }
    if (Cfg::DQ_OWN && iters > 0) {
      drain_dq(iters - 1);
      fence_proxy_async_smem();
      issue_dq_reduce(iters - 1);
      if (threadIdx.x == 0) tma_store_wait<0>();  // the staging tile and the adds outlive nothing
    }
    if (!Cfg::DQ_OWN && iters > 0 && !p.det && threadIdx.x == 0) tma_store_wait<0>();  // the staged tile outlives nothing
    // dK / dV of this key tile: TMEM -> bf16 -> global (the last dq_full wait covers them)
    if (iters > 0) {
      tc_fence_after_sync();
      const int krow = jt * 128 + row;
      const long long base = (long long)b * p.kv_bs + (long long)krow * p.kv_ss + (long long)kvh * p.kv_hs + cq * DQC;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(which ? p.dk : p.dv) + base;
        const int colbase = (which ? Cfg::COL_DK : Cfg::COL_DV) + cq * DQC;
        const float mul = which ? p.scale : 1.0f;  // dS was kept unscaled
        // dK of a rotated k: the pairs (2i, 2i + 1) of this thread's columns turn back by the angles of the key's position
        const bool unrope = which && p.unrope_tab != nullptr && krow < p.S;
        auto rotate_back = [&](auto& r) {
          constexpr int n = (int)(sizeof(r) / sizeof(uint32_t));
          const float4* tp = reinterpret_cast<const float4*>(p.unrope_tab + (long long)krow * (D / 2) + (cq * DQC) / 2);
#pragma unroll
          for (int i = 0; i < n; i += 4) {
            const float4 t = __ldg(tp + (i >> 2));  // (cos, sin) of two pairs
            const float x0 = __uint_as_float(r[i]), y0 = __uint_as_float(r[i + 1]);
            const float x1 = __uint_as_float(r[i + 2]), y1 = __uint_as_float(r[i + 3]);
            r[i] = __float_as_uint(x0 * t.x + y0 * t.y);
            r[i + 1] = __float_as_uint(y0 * t.x - x0 * t.y);
            r[i + 2] = __float_as_uint(x1 * t.z + y1 * t.w);
            r[i + 3] = __float_as_uint(y1 * t.z - x1 * t.w);
          }
        };
        if constexpr (DQC == 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_base + colbase + lane_off, r);
          tmem_ld_wait();
          if (unrope) rotate_back(r);
          if (krow < p.S) {
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
              o.y = pack_bf16x2(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
              o.z = pack_bf16x2(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
              o.w = pack_bf16x2(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + i) = o;
            }
          }
        } else {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + colbase + lane_off, r);
          tmem_ld_wait();
          if (unrope) rotate_back(r);
          if (krow < p.S) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
              o.y = pack_bf16x2(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
              o.z = pack_bf16x2(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
              o.w = pack_bf16x2(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + i) = o;
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == Cfg::CWARPS + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// delta[b,h,s] = sum_d o[b,s,h,d] * do[b,s,h,d]; D/8 lanes per (b,s,h) row, 16 bytes per lane
template <int D>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ o_lo,
                  const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                  int B, int S, int H, long long bs, long long ss, long long hs) {
  constexpr int LPR = D / 8;  // lanes per row (8 or 16)
  const long long total = (long long)B * S * H;
  const int lane = threadIdx.x & 31;
  // the loop runs on warp bases so that every lane of a warp takes part in each shuffle
  for (long long tb = blockIdx.x * (long long)blockDim.x + (threadIdx.x - lane); tb < total * LPR;
       tb += (long long)gridDim.x * blockDim.x) {
    const long long t = tb + lane;
    const bool valid = t < total * LPR;
    const long long w = valid ? t / LPR : 0;
    const int c = (int)(t % LPR) * 8;
    const int h = (int)(w % H);
    const int s = (int)((w / H) % S);
    const int b = (int)(w / ((long long)H * S));
    const long long off = (long long)b * bs + (long long)s * ss + (long long)h * hs + c;
    float acc = 0.0f;
    if (valid) {
      float x[8], y[8];
      ld16(o + off, x);
      ld16(d_o + off, y);
      if (o_lo) {
        float xl[8];
        ld16(o_lo + off, xl);
#pragma unroll
        for (int k = 0; k < 8; ++k) x[k] += xl[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) acc += x[k] * y[k];
    }
#pragma unroll
    for (int m = LPR / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
    if (valid && (t % LPR) == 0) delta[((long long)b * H + h) * S + s] = acc;
  }
}

// The two preparations of the backward in one pass: delta[b,h,s] = sum_d o*do (as attn_delta_kernel)
// and dq_acc = 0 (the f32 buffer the key-tile CTAs add their dQ tiles to; contiguous [B,S,H,D], so the
// thread that reads vector i of O / dO clears the 32 bytes of vector i).  32-bit index arithmetic
// (the caller checks B*S*H*D < 2^31), two vectors per thread requested before the first use.  A row's
// LPR lanes always sit in one warp and are valid together (LPR divides 32 and the row count is whole).
template <int D>
__global__ void __launch_bounds__(256)
attn_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ o_lo,
                 const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                 float* __restrict__ dq_acc, unsigned nvec, unsigned S, unsigned H, long long bs, long long ss, long long hs) {
  constexpr unsigned LPR = D / 8;  // lanes per (b,s,h) row
  const unsigned stride = gridDim.x * blockDim.x;
  const unsigned lane = threadIdx.x & 31;
  const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  // the loop runs on warp bases so that every lane of a warp takes part in each shuffle
  for (unsigned base = blockIdx.x * blockDim.x + (threadIdx.x - lane); base < nvec; base += 2 * stride) {
    const bool warp_two = base + stride < nvec;  // uniform over the warp
    const unsigned tt[2] = {base + lane, base + stride + lane};
    const bool valid[2] = {tt[0] < nvec, warp_two && tt[1] < nvec};
    long long off[2];
    unsigned bq[2], hq[2], sq[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const unsigned t = valid[u] ? tt[u] : 0u;
      const unsigned w = t / LPR, c = (t % LPR) * 8;
      hq[u] = w % H;
      const unsigned ws = w / H;
      sq[u] = ws % S;
      bq[u] = ws / S;
      off[u] = (long long)bq[u] * bs + (long long)sq[u] * ss + (long long)hq[u] * hs + c;
    }
    float x0[8], y0[8], x1[8], y1[8];
    ld16(o + off[0], x0); ld16(d_o + off[0], y0);
    ld16(o + off[1], x1); ld16(d_o + off[1], y1);
    if (o_lo) {  // the part of the forward's f32 output that its rounding to bf16 dropped
      float l0[8], l1[8];
      ld16(o_lo + off[0], l0);
      ld16(o_lo + off[1], l1);
#pragma unroll
      for (int k = 0; k < 8; ++k) { x0[k] += l0[k]; x1[k] += l1[k]; }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (valid[u]) {
        float4* zp = reinterpret_cast<float4*>(dq_acc + (size_t)tt[u] * 8);
        zp[0] = z;
        zp[1] = z;
      }
    }
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { a0 = fmaf(x0[k], y0[k], a0); a1 = fmaf(x1[k], y1[k], a1); }
#pragma unroll
    for (unsigned m = LPR / 2; m > 0; m >>= 1) {
      a0 += __shfl_xor_sync(0xffffffffu, a0, m);
      a1 += __shfl_xor_sync(0xffffffffu, a1, m);
    }
    if (valid[0] && (tt[0] % LPR) == 0) delta[((size_t)bq[0] * H + hq[0]) * S + sq[0]] = a0;
    if (valid[1] && (tt[1] % LPR) == 0) delta[((size_t)bq[1] * H + hq[1]) * S + sq[1]] = a1;
  }
}

// dq (bf16, strided [B,S,H,D]) = dq_acc (f32, contiguous [B,S,H,D]); UNROPE: rotated back by the RoPE
// angles of the row's position (table [S][D / 2] of (cos, sin)) before the rounding
// n_slices > 1 (fixed-order mode): acc holds one [B,S,H,D] slice per key tile, `slice` elements apart; row s
// sums slices 0 .. s / 128 under the causal mask (later key tiles wrote nothing there), all of them otherwise
template <bool UNROPE>
__global__ void __launch_bounds__(256)
attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows /*B*S*H*/,
                       int S, int H, int D, long long bs, long long ss, long long hs, float scale,
                       const float2* __restrict__ unrope_tab, int n_slices, long long slice, int causal) {
  const int per_row = D / 8;
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const int h = (int)(r % H);
    const int s = (int)((r / H) % S);
    const long long b = r / ((long long)H * S);
    float lo[4], hi[4];
    float4 t0 = make_float4(1.0f, 0.0f, 1.0f, 0.0f), t1 = t0;
    if (UNROPE) {  // requested together with the accumulator's two vectors
      const float4* tp = reinterpret_cast<const float4*>(unrope_tab + (long long)s * (D / 2) + (c >> 1));
      t0 = __ldg(tp);
      t1 = __ldg(tp + 1);
    }
    ld16(acc + r * D + c, lo);
    ld16(acc + r * D + c + 4, hi);
    if (n_slices > 1) {
      const int last = causal ? min(s >> 7, n_slices - 1) : n_slices - 1;
      for (int j = 1; j <= last; ++j) {
        float lo2[4], hi2[4];
        ld16(acc + j * slice + r * D + c, lo2);
        ld16(acc + j * slice + r * D + c + 4, hi2);
#pragma unroll
        for (int e = 0; e < 4; ++e) { lo[e] += lo2[e]; hi[e] += hi2[e]; }
      }
    }
    // the backward kernel accumulates dS K with dS unscaled: the softmax scale is applied here
    float v[8] = {lo[0] * scale, lo[1] * scale, lo[2] * scale, lo[3] * scale,
                  hi[0] * scale, hi[1] * scale, hi[2] * scale, hi[3] * scale};
    if (UNROPE) {
      // dQ of a rotated q: the four (even, odd) pairs turn back by the angles of the query's position
      const float cs[4] = {t0.x, t0.z, t1.x, t1.z}, sn[4] = {t0.y, t0.w, t1.y, t1.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float x = v[2 * e], y = v[2 * e + 1];
        v[2 * e] = x * cs[e] + y * sn[e];
        v[2 * e + 1] = y * cs[e] - x * sn[e];
      }
    }
    st16(dq + b * bs + (long long)s * ss + (long long)h * hs + c, v);
  }
}

// mean[b, h, :] = mean over s of v[b, s, h, :]; one CTA per (b, h), f32 sums in a fixed order
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&x)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) { ld16(p, x); }
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

template <typename T>
__global__ void __launch_bounds__(256)
attn_value_mean_kernel(const T* __restrict__ v, float* __restrict__ mean, int S, int H, int D, long long bs,
                       long long ss, long long hs) {
  __shared__ float sh[8][128];
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const int per_row = D / 8;                 // 16-byte vectors per row: 8 or 16
  const int rows_per_pass = 256 / per_row;   // 32 or 16 rows at a time
  const int c = (threadIdx.x % per_row) * 8, r0 = threadIdx.x / per_row;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const T* base = v + (long long)b * bs + (long long)h * hs + c;
  for (int s = r0; s < S; s += rows_per_pass) {
    float x[8];
    load8<T>(base + (long long)s * ss, x);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += x[e];
  }
  // threads with the same column chunk sit per_row apart: reduce them through shared memory in a fixed order
  float* slot = &sh[0][0];
  for (int e = 0; e < 8; ++e) {
    __syncthreads();
    slot[threadIdx.x] = acc[e];
    __syncthreads();
    if (threadIdx.x < per_row) {
      float t = 0.0f;
      for (int r = 0; r < rows_per_pass; ++r) t += slot[r * per_row + threadIdx.x];
      mean[((long long)b * H + h) * D + threadIdx.x * 8 + e] = t / (float)S;
    }
  }
}

// vc[b, s, h, :] = bf16(v[b, s, h, :] - mean[b, h, :]) (vc contiguous [B, S, H, D])
template <typename T>
__global__ void __launch_bounds__(256)
attn_value_center_kernel(const T* __restrict__ v, const float* __restrict__ mean, __nv_bfloat16* __restrict__ vc,
                         long long rows /*B*S*H*/, int S, int H, int D, long long bs, long long ss, long long hs) {
  const int per_row = D / 8;
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c = (int)(i % per_row) * 8;
    const int h = (int)(r % H);
    const int s = (int)((r / H) % S);
    const long long b = r / ((long long)H * S);
    float x[8];
    load8<T>(v + b * bs + (long long)s * ss + (long long)h * hs + c, x);
    const float* m = mean + (b * H + h) * D + c;
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] -= m[e];
    st16(vc + r * D + c, x);
  }
}

int make_qkv_tmap(CUtensorMap* tm, const void* base, int B, int S, int H, int D, long long bs, long long ss,
                  long long hs) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t strides[3] = {(uint64_t)hs, (uint64_t)ss, (uint64_t)bs};
  const uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_bf16_nd(tm, base, 4, dims, strides, box);
}

int check_args(long long B, long long S, long long Hq, long long Hkv, long long D, const long long* strides, int n) {
  if (D != 64 && D != 128) return fail(EISEN_ERR_INVALID, "attention: head_dim must be 64 or 128");
  if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return fail(EISEN_ERR_INVALID, "attention: bad B/S/H (Hq % Hkv must be 0)");
  if (B > 65535 || Hq > 65535) return fail(EISEN_ERR_LIMIT, "attention: B and Hq must be <= 65535");
  for (int i = 0; i < n; ++i)
    if (strides[i] % 8) return fail(EISEN_ERR_INVALID, "attention: strides must be multiples of 8 elements");
  return 0;
}

}  // namespace
}  // namespace eisen

using namespace eisen;

extern "C" {

int eisen_attn_set_bwd_mode(int transposed) {
  if (transposed != 0 && transposed != 1) return fail(EISEN_ERR_INVALID, "attn_set_bwd_mode: 0 or 1");
  g_attn_bwd_transposed.store(transposed);
  return 0;
}

int eisen_attn_set_fwd_tiles(int tiles) {
  if (tiles < 1 || tiles > 3)
    return fail(EISEN_ERR_INVALID, "attn_set_fwd_tiles: 1 or 2 query tiles per CTA, or 3 = one tile with P through TMEM");
  g_attn_fwd_tiles.store(tiles);
  return 0;
}

static int attn_fwd_impl(void* stream, const void* q, const void* k, const void* v, void* o, void* o_lo,
                         const float* v_mean, float* lse, long long B, long long S, long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss,
                         long long q_hs, long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs,
                         long long o_ss, long long o_hs, float scale, int causal, int* status) {
  const long long st[9] = {q_bs, q_ss, q_hs, kv_bs, kv_ss, kv_hs, o_bs, o_ss, o_hs};
  int rc = check_args(B, S, Hq, Hkv, D, st, 9);
  if (rc) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(o_lo))
    return fail(EISEN_ERR_INVALID, "attn_fwd: unaligned pointer");
  CUtensorMap tq, tk, tv;
  if (make_qkv_tmap(&tq, q, (int)B, (int)S, (int)Hq, (int)D, q_bs, q_ss, q_hs) ||
      make_qkv_tmap(&tk, k, (int)B, (int)S, (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs) ||
      make_qkv_tmap(&tv, v, (int)B, (int)S, (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs))
    return fail(EISEN_ERR_CUDA, "attn_fwd: cuTensorMapEncodeTiled failed");
  AttnParams p{};
  p.B = (int)B; p.S = (int)S; p.Hq = (int)Hq; p.Hkv = (int)Hkv; p.D = (int)D;
  p.causal = causal; p.scale = scale;
  p.o = o; p.o_bs = o_bs; p.o_ss = o_ss; p.o_hs = o_hs;
  p.o_lo = o_lo;
  p.v_mean = v_mean;
  p.lse = lse; p.status = status;
  dim3 grid((unsigned)Hq, (unsigned)B, (unsigned)(((S + 127) / 128 + 1) / 2));  // two query tiles per CTA
  cudaStream_t s = (cudaStream_t)stream;
  if (D == 64) {
    // one query tile per CTA and two CTAs per SM, or two query tiles per CTA (see Fwd64Cfg)
    static bool set64[2][MAX_DEVICE_SLOTS] = {{false}};
    const int slot = device_slot();
    const int nt = g_attn_fwd_tiles.load();
    if (nt == 3) {
      static bool set3[MAX_DEVICE_SLOTS] = {false};
      if (!set3[slot]) {
        if (cudaFuncSetAttribute(attn_fwd64_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Fwd64Cfg<1, true>::SMEM) != cudaSuccess)
          return fail(EISEN_ERR_CUDA, "attn_fwd: smem attribute");
        set3[slot] = true;
      }
      dim3 grid1((unsigned)Hq, (unsigned)B, (unsigned)((S + 127) / 128));
      attn_fwd64_kernel<1, true><<<grid1, Fwd64Cfg<1, true>::THREADS, Fwd64Cfg<1, true>::SMEM, s>>>(tq, tk, tv, p);
    } else if (nt == 2) {
      if (!set64[1][slot]) {
        if (cudaFuncSetAttribute(attn_fwd64_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd64Cfg<2>::SMEM) != cudaSuccess)
          return fail(EISEN_ERR_CUDA, "attn_fwd: smem attribute");
        set64[1][slot] = true;
      }
      attn_fwd64_kernel<2><<<grid, Fwd64Cfg<2>::THREADS, Fwd64Cfg<2>::SMEM, s>>>(tq, tk, tv, p);
    } else {
      if (!set64[0][slot]) {
        if (cudaFuncSetAttribute(attn_fwd64_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, Fwd64Cfg<1>::SMEM) != cudaSuccess)
          return fail(EISEN_ERR_CUDA, "attn_fwd: smem attribute");
        set64[0][slot] = true;
      }
      dim3 grid1((unsigned)Hq, (unsigned)B, (unsigned)((S + 127) / 128));
      attn_fwd64_kernel<1><<<grid1, Fwd64Cfg<1>::THREADS, Fwd64Cfg<1>::SMEM, s>>>(tq, tk, tv, p);
    }
  } else {
    static bool set128[MAX_DEVICE_SLOTS] = {false};
    if (!set128[device_slot()]) { if (cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<128>::SMEM) != cudaSuccess) return fail(EISEN_ERR_CUDA, "attn_fwd: smem attribute"); set128[device_slot()] = true; }
    attn_fwd_kernel<128><<<grid, FwdCfg<128>::THREADS, FwdCfg<128>::SMEM, s>>>(tq, tk, tv, p);
  }
  return check_launch("attn_fwd");
}

int eisen_attn_fwd(void* stream, const void* q, const void* k, const void* v, void* o, float* lse, long long B,
                   long long S, long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss,
                   long long q_hs, long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs,
                   long long o_ss, long long o_hs, float scale, int causal, int* status) {
  return attn_fwd_impl(stream, q, k, v, o, nullptr, nullptr, lse, B, S, Hq, Hkv, D, q_bs, q_ss, q_hs, kv_bs, kv_ss, kv_hs, o_bs,
                       o_ss, o_hs, scale, causal, status);
}

int eisen_attn_fwd_ex(void* stream, const void* q, const void* k, const void* v, void* o, void* o_aux, const float* v_mean,
                      float* lse, long long B, long long S, long long Hq, long long Hkv, long long D, long long q_bs,
                      long long q_ss, long long q_hs, long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs,
                      long long o_ss, long long o_hs, float scale, int causal, int* status) {
  if (v_mean && (reinterpret_cast<uintptr_t>(v_mean) & 15)) return fail(EISEN_ERR_INVALID, "attn_fwd: unaligned pointer");
  return attn_fwd_impl(stream, q, k, v, o, o_aux, v_mean, lse, B, S, Hq, Hkv, D, q_bs, q_ss, q_hs, kv_bs, kv_ss, kv_hs, o_bs,
                       o_ss, o_hs, scale, causal, status);
}

int eisen_attn_center_values(void* stream, const void* v, int v_dtype, void* v_centered, float* mean, long long B,
                             long long S, long long Hkv, long long D, long long kv_bs, long long kv_ss, long long kv_hs) {
  if (D != 64 && D != 128) return fail(EISEN_ERR_INVALID, "attention: head_dim must be 64 or 128");
  if (v_dtype != EISEN_F32 && v_dtype != EISEN_BF16) return fail(EISEN_ERR_INVALID, "attn_center_values: v must be f32 or bf16");
  if (B <= 0 || S <= 0 || Hkv <= 0 || B * Hkv > 0x7fffffffLL || S > 0x7fffffffLL)
    return fail(EISEN_ERR_INVALID, "attn_center_values: bad B/S/H");
  if (!v || !v_centered || !mean || !aligned16(v) || !aligned16(v_centered) || !aligned16(mean) || (kv_bs % 8) || (kv_ss % 8) || (kv_hs % 8))
    return fail(EISEN_ERR_INVALID, "attn_center_values: null or unaligned pointer, or strides that are not multiples of 8");
  cudaStream_t s = (cudaStream_t)stream;
  const int grid2 = grid_for(B * S * Hkv * D / 8, 256, 8);
  if (v_dtype == EISEN_F32) {
    attn_value_mean_kernel<float><<<(unsigned)(B * Hkv), 256, 0, s>>>((const float*)v, mean, (int)S, (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs);
    int rc = check_launch("attn_value_mean");
    if (rc) return rc;
    attn_value_center_kernel<float><<<grid2, 256, 0, s>>>((const float*)v, mean, (__nv_bfloat16*)v_centered, B * S * Hkv, (int)S,
                                                          (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs);
  } else {
    attn_value_mean_kernel<__nv_bfloat16><<<(unsigned)(B * Hkv), 256, 0, s>>>((const __nv_bfloat16*)v, mean, (int)S, (int)Hkv, (int)D,
                                                                             kv_bs, kv_ss, kv_hs);
    int rc = check_launch("attn_value_mean");
    if (rc) return rc;
    attn_value_center_kernel<__nv_bfloat16><<<grid2, 256, 0, s>>>((const __nv_bfloat16*)v, mean, (__nv_bfloat16*)v_centered,
                                                                  B * S * Hkv, (int)S, (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs);
  }
  return check_launch("attn_value_center");
}

// workspace layout: dq_acc f32 [B,S,Hq,D] (in the fixed-order mode one such slice per 128-key tile) | delta f32 [B,Hq,S]
long long eisen_attn_bwd_workspace_bytes(long long B, long long S, long long Hq, long long Hkv, long long D) {
  (void)Hkv;
  const long long slices = deterministic() ? (S + 127) / 128 : 1;
  return slices * B * S * Hq * D * 4 + B * Hq * S * 4 + 256;
}

static int attn_bwd_impl(void* stream, const void* q, const void* k, const void* v, const void* o, const void* o_lo,
                         const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B, long long S,
                         long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                         long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss,
                         long long o_hs, float scale, int causal, const float* unrope_table, int* status) {
  const long long st[9] = {q_bs, q_ss, q_hs, kv_bs, kv_ss, kv_hs, o_bs, o_ss, o_hs};
  if (unrope_table && (reinterpret_cast<uintptr_t>(unrope_table) & 15))
    return fail(EISEN_ERR_INVALID, "attn_bwd: the rotation table must be 16-byte aligned");
  int rc = check_args(B, S, Hq, Hkv, D, st, 9);
  if (rc) return rc;
  if (!workspace) return fail(EISEN_ERR_INVALID, "attn_bwd: workspace is null");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(o_lo) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv) || !aligned16(workspace))
    return fail(EISEN_ERR_INVALID, "attn_bwd: unaligned pointer");
  cudaStream_t s = (cudaStream_t)stream;
  float* dq_acc = (float*)workspace;
  const long long n_elems = B * S * Hq * D;
  const bool det = deterministic();
  const long long n_kt = (S + 127) / 128;
  if (det && n_kt * B > 0x7fffffffLL) return fail(EISEN_ERR_LIMIT, "attn_bwd: too many (key tile, batch) slices");
  float* delta = dq_acc + (det ? n_kt : 1) * n_elems;
  if (n_elems < 0x7fffffffLL && !det) {
    // delta and the clearing of the dQ accumulation buffer in one pass
    const unsigned nvec = (unsigned)(n_elems / 8);
    const int grid = grid_for((nvec + 1) / 2, 256, 8);
    if (D == 64)
      attn_prep_kernel<64><<<grid, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)o_lo, (const __nv_bfloat16*)d_o,
                                                delta, dq_acc, nvec, (unsigned)S, (unsigned)Hq, o_bs, o_ss, o_hs);
    else
      attn_prep_kernel<128><<<grid, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)o_lo, (const __nv_bfloat16*)d_o,
                                                 delta, dq_acc, nvec, (unsigned)S, (unsigned)Hq, o_bs, o_ss, o_hs);
  } else {
    // fixed-order mode: every slice element that the conversion reads is written by its key tile, nothing to clear
    if (!det && cudaMemsetAsync(dq_acc, 0, (size_t)n_elems * 4, s) != cudaSuccess)
      return fail(EISEN_ERR_CUDA, "attn_bwd: memset failed");
    // total threads is a multiple of 32 (S*H*D/8 with D/8 in {8,16}), so every shuffle group is complete
    if (D == 64)
      attn_delta_kernel<64><<<grid_for(B * S * Hq * 8, 256, 8), 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)o_lo,
                                                                            (const __nv_bfloat16*)d_o, delta, (int)B, (int)S,
                                                                            (int)Hq, o_bs, o_ss, o_hs);
    else
      attn_delta_kernel<128><<<grid_for(B * S * Hq * 16, 256, 8), 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)o_lo,
                                                                              (const __nv_bfloat16*)d_o, delta, (int)B, (int)S,
                                                                              (int)Hq, o_bs, o_ss, o_hs);
  }
  rc = check_launch("attn_delta");
  if (rc) return rc;
  CUtensorMap tq, tk, tv, tdo;
  // dO uses the strides of O
  if (make_qkv_tmap(&tq, q, (int)B, (int)S, (int)Hq, (int)D, q_bs, q_ss, q_hs) ||
      make_qkv_tmap(&tk, k, (int)B, (int)S, (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs) ||
      make_qkv_tmap(&tv, v, (int)B, (int)S, (int)Hkv, (int)D, kv_bs, kv_ss, kv_hs) ||
      make_qkv_tmap(&tdo, d_o, (int)B, (int)S, (int)Hq, (int)D, o_bs, o_ss, o_hs))
    return fail(EISEN_ERR_CUDA, "attn_bwd: cuTensorMapEncodeTiled failed");
  CUtensorMap tdq;
  {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hq, (uint64_t)S, (uint64_t)(det ? n_kt * B : B)};  // slices are contiguous
    const uint64_t strides[3] = {(uint64_t)D, (uint64_t)(Hq * D), (uint64_t)(S * Hq * D)};
    const uint32_t box[4] = {32, 1, 128, 1};
    if (make_tmap_f32_nd(&tdq, dq_acc, 4, dims, strides, box)) return fail(EISEN_ERR_CUDA, "attn_bwd: cuTensorMapEncodeTiled failed for dQ");
  }
  AttnParams p{};
  p.B = (int)B; p.S = (int)S; p.Hq = (int)Hq; p.Hkv = (int)Hkv; p.D = (int)D;
  p.causal = causal; p.scale = scale;
  p.lse = const_cast<float*>(lse); p.delta = delta; p.dq_acc = dq_acc;
  p.dk = dk; p.dv = dv; p.kv_bs = kv_bs; p.kv_ss = kv_ss; p.kv_hs = kv_hs;
  p.unrope_tab = reinterpret_cast<const float2*>(unrope_table);
  p.det = det ? 1 : 0;
  p.dq_slice = n_elems;
  p.status = status;
  dim3 grid((unsigned)Hkv, (unsigned)B, (unsigned)((S + 127) / 128));
  if (D == 64 && g_attn_bwd_transposed.load()) {
    static bool set64t[MAX_DEVICE_SLOTS] = {false};
    if (!set64t[device_slot()]) {
      if (cudaFuncSetAttribute(attn_bwd_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<64, true>::SMEM) !=
          cudaSuccess)
        return fail(EISEN_ERR_CUDA, "attn_bwd: smem attribute");
      set64t[device_slot()] = true;
    }
    attn_bwd_kernel<64, true><<<grid, BwdCfg<64, true>::THREADS, BwdCfg<64, true>::SMEM, s>>>(tq, tk, tv, tdo, tdq, p);
  } else if (D == 64) {
    static bool set64[MAX_DEVICE_SLOTS] = {false};
    if (!set64[device_slot()]) { if (cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<64>::SMEM) != cudaSuccess) return fail(EISEN_ERR_CUDA, "attn_bwd: smem attribute"); set64[device_slot()] = true; }
    attn_bwd_kernel<64><<<grid, BwdCfg<64>::THREADS, BwdCfg<64>::SMEM, s>>>(tq, tk, tv, tdo, tdq, p);
  } else {
    static bool set128[MAX_DEVICE_SLOTS] = {false};
    if (!set128[device_slot()]) { if (cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<128>::SMEM) != cudaSuccess) return fail(EISEN_ERR_CUDA, "attn_bwd: smem attribute"); set128[device_slot()] = true; }
    attn_bwd_kernel<128><<<grid, BwdCfg<128>::THREADS, BwdCfg<128>::SMEM, s>>>(tq, tk, tv, tdo, tdq, p);
  }
  rc = check_launch("attn_bwd");
  if (rc) return rc;
  if (unrope_table)
    attn_dq_convert_kernel<true><<<grid_for(B * S * Hq * D / 8, 256, 8), 256, 0, s>>>(
        dq_acc, (__nv_bfloat16*)dq, B * S * Hq, (int)S, (int)Hq, (int)D, q_bs, q_ss, q_hs, scale,
        reinterpret_cast<const float2*>(unrope_table), det ? (int)n_kt : 1, n_elems, causal);
  else
    attn_dq_convert_kernel<false><<<grid_for(B * S * Hq * D / 8, 256, 8), 256, 0, s>>>(
        dq_acc, (__nv_bfloat16*)dq, B * S * Hq, (int)S, (int)Hq, (int)D, q_bs, q_ss, q_hs, scale, nullptr,
        det ? (int)n_kt : 1, n_elems, causal);
  return check_launch("attn_dq_convert");
}

int eisen_attn_bwd(void* stream, const void* q, const void* k, const void* v, const void* o, const float* lse,
                   const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B, long long S,
                   long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                   long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss,
                   long long o_hs, float scale, int causal, int* status) {
  return attn_bwd_impl(stream, q, k, v, o, nullptr, lse, d_o, dq, dk, dv, workspace, B, S, Hq, Hkv, D, q_bs, q_ss, q_hs, kv_bs,
                       kv_ss, kv_hs, o_bs, o_ss, o_hs, scale, causal, nullptr, status);
}

int eisen_attn_bwd_unrope(void* stream, const void* q, const void* k, const void* v, const void* o, const float* lse,
                          const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B, long long S,
                          long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                          long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss,
                          long long o_hs, float scale, int causal, const float* table_cos_sin, int* status) {
  if (!table_cos_sin) return fail(EISEN_ERR_INVALID, "attn_bwd_unrope: the rotation table is null");
  return attn_bwd_impl(stream, q, k, v, o, nullptr, lse, d_o, dq, dk, dv, workspace, B, S, Hq, Hkv, D, q_bs, q_ss, q_hs, kv_bs,
                       kv_ss, kv_hs, o_bs, o_ss, o_hs, scale, causal, table_cos_sin, status);
}

int eisen_attn_bwd_ex(void* stream, const void* q, const void* k, const void* v, const void* o, const void* o_lo,
                      const float* lse, const void* d_o, void* dq, void* dk, void* dv, void* workspace, long long B,
                      long long S, long long Hq, long long Hkv, long long D, long long q_bs, long long q_ss, long long q_hs,
                      long long kv_bs, long long kv_ss, long long kv_hs, long long o_bs, long long o_ss, long long o_hs,
                      float scale, int causal, const float* table_cos_sin, int* status) {
  return attn_bwd_impl(stream, q, k, v, o, o_lo, lse, d_o, dq, dk, dv, workspace, B, S, Hq, Hkv, D, q_bs, q_ss, q_hs, kv_bs,
                       kv_ss, kv_hs, o_bs, o_ss, o_hs, scale, causal, table_cos_sin, status);
}

}  // extern "C"
