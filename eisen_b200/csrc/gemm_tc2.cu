// Paired-CTA variant of the bf16 tcgen05 GEMM (see gemm_tc.cu for the operand conventions).
//
// Two CTAs of a cluster work on one 256 x 256 output tile: each CTA stages its own 128 rows of A
// and its own 128 columns of B (32 KB per k-block instead of 48 KB for a 128 x 256 tile), the
// leader CTA issues tcgen05.mma.cta_group::2 with M = 256, and each CTA's TMEM receives its
// 128 x 256 half of the accumulator.  The 128 x 256 single-CTA tile is limited by the ~64 B/clk
// at which an SM can take in operands (48 KB per 512 tensor-core clocks); the pair needs 32 KB
// per 512 clocks.  No load is broadcast between the CTAs: each issues its own TMA loads, which
// report their bytes to the leader's barrier.
#include "ptx.cuh"
#include "gemm_tc.h"
#include "gemm_epilogue.cuh"
#include "errors.h"

#include <cuda.h>

#include <climits>

namespace eisen {
namespace {

constexpr int PM = 128;   // rows per CTA (256 per pair)
constexpr int PN = 256;   // columns per pair (128 staged per CTA)
constexpr int BK = 64;
constexpr int PSTAGES = 6;
constexpr int PA_BYTES = PM * BK * 2;        // 16 KB
constexpr int PB_BYTES = (PN / 2) * BK * 2;  // 16 KB
constexpr int PSTAGE_BYTES = PA_BYTES + PB_BYTES;
constexpr int P_THREADS = 192;
constexpr int P_ACC_COLS = PN;
constexpr int P_EPI_BYTES = 4 * 32 * 128;  // per epilogue warp: 32 rows x 64 bf16 columns
constexpr int P_SMEM = PSTAGES * PSTAGE_BYTES + 1024 + 256 + P_EPI_BYTES;

struct PairParams {
  int M, N, K;
  int a_mn, b_mn;
  void* C;
  long long ldc;
  const void* R;  // addend of the bf16 accumulate mode (C itself, or a residual tensor)
  long long ldr;
  int out_mode;
  int split_k, kblocks_per_split, kblocks_total;
  int m_tiles, n_tiles, total_tiles;  // m_tiles counts 256-row pair tiles
  int band;  // m-tiles per band of the tile order (see pair_tile_coords)
  // dual mode (gate / up projections + SwiGLU): CTA 0 of the pair stages 128 columns of B, CTA 1 the
  // same 128 columns of B2, so the 256-column accumulator holds [x B | x B2]; the epilogue stores
  // C = bf16(x B), C2 = bf16(x B2) (both optional) and H = silu(C) * C2.  N counts H's columns.
  int dual;
  void* C2;
  void* H;
  // GEMM_OUT_BF16_ROPE: rotation table [rope_s][rope_hd / 2] of (cos, sin), row -> position row % rope_s
  const float2* rope_tab;
  int rope_s, rope_hd;
  float alpha;
  int* status;
  // segmented launches (the SEG instantiation of the kernel only).
  // K segments: the k-blocks from kseg[1] on come from the operand pair (A2, B2), those from kseg[2]
  // on from (A3, B3): C = A1 B1^T + A2 B2^T + A3 B3^T without intermediate roundings.
  // N segments: the n-tiles from nseg[1] / nseg[2] on read the B operand B2 / B3 and write their own
  // output matrix: three products that share A in one launch.  A launch uses one kind or the other.
  int kseg[3], nseg[3];
  void* Cs[3];
  long long ldcs[3];
  int Ns[3];
  int out_modes[3];
};

// Tile order: the m-tiles are cut into bands of `band` tiles; a band is finished (all its n-tiles,
// m fastest inside the band) before the next one starts.  With band == m_tiles this is plain
// column-major order.  A small band keeps its rows of A in L2 while the n-tiles sweep over B.
__device__ __forceinline__ void pair_tile_coords(const PairParams& p, int mn, int& mt, int& nt) {
  const int per_band = p.band * p.n_tiles;
  const int b = mn / per_band;
  const int in = mn - b * per_band;
  const int m_first = b * p.band;
  const int rows = min(p.band, p.m_tiles - m_first);
  nt = in / rows;
  mt = m_first + (in - nt * rows);
}

struct SegMaps {
  CUtensorMap a[2];  // A2, A3 (K segments)
  CUtensorMap b;     // B3 (B2 travels in the dual mode's slot)
};

template <bool SEG>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_bf16_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ SegMaps seg_maps,
                     const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + PSTAGES * PA_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PSTAGES * PSTAGE_BYTES);
  uint64_t* full_bar = bars;                       // [PSTAGES]  used in the leader (2 arrivals + bytes of both CTAs)
  uint64_t* empty_bar = bars + PSTAGES;            // [PSTAGES]  one per CTA, signalled by the leader's commits
  uint64_t* tmem_full_bar = bars + 2 * PSTAGES;    // [2]        one per CTA, signalled by the leader's commits
  uint64_t* tmem_empty_bar = bars + 2 * PSTAGES + 2;  // [2]     used in the leader (8 arrivals: 4 warps per CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * PSTAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_stage = smem + PSTAGES * PSTAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const uint32_t peer = rank ^ 1u;
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(&full_bar[s], 2);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.dual) prefetch_tmap(&tmB2);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 2 * P_ACC_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above ran beside the tail of the kernel before (programmatic dependent launch);
  // operands, addends and outputs are touched only from here on
  grid_launch_dependents();
  grid_dependency_wait();

  const int tiles_mn = p.m_tiles * p.n_tiles;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ---------------- TMA producer (each CTA loads its own slices) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cluster_id; t < p.total_tiles; t += n_clusters) {
        const int ks = t / tiles_mn;
        const int mn = t - ks * tiles_mn;
        int mt, nt;
        pair_tile_coords(p, mn, mt, nt);
        const int m0 = mt * (2 * PM) + (int)rank * PM;
        int n0 = p.dual ? nt * (PN / 2) : nt * PN + (int)rank * (PN / 2);
        const CUtensorMap* tb = (p.dual && rank == 1) ? &tmB2 : &tmB;
        if (SEG) {
          if (nt >= p.nseg[2]) { tb = &seg_maps.b; n0 -= p.nseg[2] * PN; }
          else if (nt >= p.nseg[1]) { tb = &tmB2; n0 -= p.nseg[1] * PN; }
        }
        const int kb0 = ks * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, FAULT_WAIT_EMPTY);
          const uint32_t full_leader = mapa_cluster(smem_u32(&full_bar[stage]), 0);
          mbar_arrive_expect_tx_cluster(full_leader, PSTAGE_BYTES);
          uint8_t* sa = smem_a + stage * PA_BYTES;
          uint8_t* sb = smem_b + stage * PB_BYTES;
          int k0 = kb * BK;
          const CUtensorMap* ta = &tmA;
          if (SEG) {
            if (kb >= p.kseg[2]) { ta = &seg_maps.a[1]; tb = &seg_maps.b; k0 -= p.kseg[2] * BK; }
            else if (kb >= p.kseg[1]) { ta = &seg_maps.a[0]; tb = &tmB2; k0 -= p.kseg[1] * BK; }
          }
          if (!p.a_mn) {
            tma_load_2d_pair(sa, ta, full_leader, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < PM / 64; ++j) tma_load_2d_pair(sa + j * (64 * BK * 2), ta, full_leader, m0 + 64 * j, k0);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, tb, full_leader, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < (PN / 2) / 64; ++j)
              tma_load_2d_pair(sb + j * (64 * BK * 2), tb, full_leader, n0 + 64 * j, k0);
          }
          if (++stage == PSTAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc_bf16(2 * PM, PN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 16, a_sbo = 1024;
      const uint32_t b_lbo = p.b_mn ? 64 * BK * 2 : 16, b_sbo = 1024;
      const uint32_t a_kstep = p.a_mn ? 16 * 128 : 32;
      const uint32_t b_kstep = p.b_mn ? 16 * 128 : 32;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = cluster_id; t < p.total_tiles; t += n_clusters) {
        const int ks = t / tiles_mn;
        const int kb0 = ks * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, FAULT_WAIT_TMEM_EMPTY);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * P_ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, FAULT_WAIT_FULL);
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem_a + stage * PA_BYTES);
          const uint32_t sb = smem_u32(smem_b + stage * PB_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_kstep, a_lbo, a_sbo);
            const uint64_t db = make_smem_desc(sb + k * b_kstep, b_lbo, b_sbo);
            umma_bf16_ss_pair(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // release the stage in both CTAs once these MMAs have read it
          const uint32_t e_local = smem_u32(&empty_bar[stage]);
          umma_commit_pair(mapa_cluster(e_local, 0));
          umma_commit_pair(mapa_cluster(e_local, 1));
          if (++stage == PSTAGES) { stage = 0; phase ^= 1; }
        }
        const uint32_t f_local = smem_u32(&tmem_full_bar[acc]);
        umma_commit_pair(mapa_cluster(f_local, 0));
        umma_commit_pair(mapa_cluster(f_local, 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 128 x 256 half, TMEM -> registers -> global ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = cluster_id; t < p.total_tiles; t += n_clusters) {
      const int ks = t / tiles_mn;
      const int mn = t - ks * tiles_mn;
      int mt, nt;
      pair_tile_coords(p, mn, mt, nt);
      const int row = mt * (2 * PM) + (int)rank * PM + q * 32 + lane;
      int n0 = p.dual ? nt * (PN / 2) : nt * PN;
      // output matrix of this tile (one per N segment)
      void* Cp = p.C;
      long long ldc = p.ldc;
      const void* Rp = p.R;
      long long ldr = p.ldr;
      int Nn = p.N, out_mode = p.out_mode;
      if (SEG) {
        const int sg = nt >= p.nseg[2] ? 2 : (nt >= p.nseg[1] ? 1 : 0);
        n0 -= p.nseg[sg] * PN;
        Cp = p.Cs[sg]; ldc = p.ldcs[sg]; Nn = p.Ns[sg]; out_mode = p.out_modes[sg];
        if (sg > 0) { Rp = Cp; ldr = ldc; }
      }
      const int kb0 = ks * p.kblocks_per_split;
      const bool has_k = kb0 < p.kblocks_total;
      mbar_wait(&tmem_full_bar[acc], acc_phase, abort_flag, p.status, FAULT_WAIT_TMEM_FULL);
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * P_ACC_COLS + (uint32_t(q * 32) << 16);
      const bool row_ok = row < p.M;
      const bool acc_bf16 = out_mode == GEMM_OUT_BF16_ACC && has_k;
      const int row0 = row - lane;  // first row of this warp
      // bf16 outputs of complete 32 x 256 slabs go through shared memory, so that a store (and an
      // addend load) covers 128 contiguous bytes of four rows instead of 16 bytes of 32 rows
      const bool rope = out_mode == GEMM_OUT_BF16_ROPE;  // the host admits complete tiles only
      const bool staged = has_k && (out_mode == GEMM_OUT_BF16 || out_mode == GEMM_OUT_BF16_ACC || rope) &&
                          row0 + 32 <= p.M && n0 + PN <= Nn && (ldc % 8) == 0 &&
                          (reinterpret_cast<uintptr_t>(Cp) & 15) == 0 &&
                          (!acc_bf16 || ((ldr % 8) == 0 && (reinterpret_cast<uintptr_t>(Rp) & 15) == 0));
      if (p.dual) {
        // complete slabs only (the host checks M % 256 == 0 and N % 128 == 0).  Per 64 columns:
        // gate and up are rounded to bf16 first, H is computed from the rounded values (what the
        // separate SwiGLU kernel reads), then the three 32 x 64 slabs go through the staging tile
        // one after the other and are stored as 128 contiguous bytes of four rows per instruction.
        uint8_t* st = epi_stage + q * (32 * 128);
        const int rr = lane >> 3, seg = lane & 7;
        const long long out_off = (long long)(row0 + rr) * p.ldc + n0 + seg * 8;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t gq[32], uq[32], hq[32];
          {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(taddr + c * 64, r0);
            tmem_ld_32x32b_x32(taddr + c * 64 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              gq[i] = pack_bf16x2(__uint_as_float(r0[2 * i]) * p.alpha, __uint_as_float(r0[2 * i + 1]) * p.alpha);
              gq[16 + i] = pack_bf16x2(__uint_as_float(r1[2 * i]) * p.alpha, __uint_as_float(r1[2 * i + 1]) * p.alpha);
            }
            tmem_ld_32x32b_x32(taddr + PN / 2 + c * 64, r0);
            tmem_ld_32x32b_x32(taddr + PN / 2 + c * 64 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              uq[i] = pack_bf16x2(__uint_as_float(r0[2 * i]) * p.alpha, __uint_as_float(r0[2 * i + 1]) * p.alpha);
              uq[16 + i] = pack_bf16x2(__uint_as_float(r1[2 * i]) * p.alpha, __uint_as_float(r1[2 * i + 1]) * p.alpha);
            }
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gq[i]));
            const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uq[i]));
            const float h0 = (g.x * __fdividef(1.0f, 1.0f + __expf(-g.x))) * u.x;
            const float h1 = (g.y * __fdividef(1.0f, 1.0f + __expf(-g.y))) * u.y;
            hq[i] = pack_bf16x2(h0, h1);
          }
          auto store_slab = [&](const uint32_t (&src)[32], void* out) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_uint4(src[4 * j], src[4 * j + 1], src[4 * j + 2], src[4 * j + 3]);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rw = 4 * i + rr;
              const uint4 o = *reinterpret_cast<const uint4*>(st + rw * 128 + ((seg ^ (rw & 7)) << 4));
              *reinterpret_cast<uint4*>(dst + out_off + (long long)(4 * i) * p.ldc + c * 64) = o;
            }
            __syncwarp();
          };
          if (p.C) store_slab(gq, p.C);
          if (p.C2) store_slab(uq, p.C2);
          store_slab(hq, p.H);
        }
      } else if (staged) {
        uint8_t* st = epi_stage + q * (32 * 128);
        const int rr = lane >> 3, seg = lane & 7;
        __nv_bfloat16* c_base = reinterpret_cast<__nv_bfloat16*>(Cp) + (long long)(row0 + rr) * ldc + n0 + seg * 8;
        const __nv_bfloat16* r_base =
            reinterpret_cast<const __nv_bfloat16*>(Rp) + (long long)(row0 + rr) * ldr + n0 + seg * 8;
#pragma unroll 1
        for (int c = 0; c < PN / 64; ++c) {
          // addend rows: requested before the TMEM load so that their latency runs beside it
          uint4 pre[8];  // the addend's eight rows
          if (acc_bf16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) pre[i] = *reinterpret_cast<const uint4*>(r_base + (long long)(4 * i) * ldr + c * 64);
          }
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(taddr + c * 64, r0);
          tmem_ld_32x32b_x32(taddr + c * 64 + 32, r1);
          tmem_ld_wait();
          if (rope) {
            // RoPE on the f32 accumulators, one rounding to bf16 afterwards (a projection followed by a separate
            // RoPE kernel rounds twice).  The chunk goes through the staging tile in two halves of 32 f32 columns
            // (the same 32 x 128 bytes); a thread then holds four columns (two pairs) of eight rows.
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t* rr32 = h ? r1 : r0;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                    make_uint4(rr32[4 * j], rr32[4 * j + 1], rr32[4 * j + 2], rr32[4 * j + 3]);
              __syncwarp();
              const int col = n0 + c * 64 + h * 32 + seg * 4;
              const int pair0 = (col % p.rope_hd) >> 1;
              uint4 ang[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int pos = (row0 + 4 * i + rr) % p.rope_s;
                ang[i] = __ldg(reinterpret_cast<const uint4*>(p.rope_tab + (long long)pos * (p.rope_hd >> 1) + pair0));
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int rw = 4 * i + rr;
                const uint4 x = *reinterpret_cast<const uint4*>(st + rw * 128 + ((seg ^ (rw & 7)) << 4));
                const float x0 = __uint_as_float(x.x) * p.alpha, y0 = __uint_as_float(x.y) * p.alpha;
                const float x1 = __uint_as_float(x.z) * p.alpha, y1 = __uint_as_float(x.w) * p.alpha;
                const float c0 = __uint_as_float(ang[i].x), s0 = __uint_as_float(ang[i].y);
                const float c1 = __uint_as_float(ang[i].z), s1 = __uint_as_float(ang[i].w);
                uint2 o;
                o.x = pack_bf16x2(x0 * c0 - y0 * s0, x0 * s0 + y0 * c0);
                o.y = pack_bf16x2(x1 * c1 - y1 * s1, x1 * s1 + y1 * c1);
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(Cp) + (long long)(row0 + rw) * ldc + col) = o;
              }
              __syncwarp();
            }
            continue;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]) * p.alpha, __uint_as_float(r0[8 * j + 1]) * p.alpha);
            o.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]) * p.alpha, __uint_as_float(r0[8 * j + 3]) * p.alpha);
            o.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]) * p.alpha, __uint_as_float(r0[8 * j + 5]) * p.alpha);
            o.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]) * p.alpha, __uint_as_float(r0[8 * j + 7]) * p.alpha);
            *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
            o.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]) * p.alpha, __uint_as_float(r1[8 * j + 1]) * p.alpha);
            o.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]) * p.alpha, __uint_as_float(r1[8 * j + 3]) * p.alpha);
            o.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]) * p.alpha, __uint_as_float(r1[8 * j + 5]) * p.alpha);
            o.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]) * p.alpha, __uint_as_float(r1[8 * j + 7]) * p.alpha);
            *reinterpret_cast<uint4*>(st + lane * 128 + (((j + 4) ^ (lane & 7)) << 4)) = o;
          }
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
              const int i = 4 * h + ii;
              const int rw = 4 * i + rr;
              uint4 o = *reinterpret_cast<const uint4*>(st + rw * 128 + ((seg ^ (rw & 7)) << 4));
              if (acc_bf16) {
                // the product is rounded to bf16 before the addend is added, as a separate matmul
                // followed by an add would do
                const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&o);
                const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&pre[i]);
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 fa = __bfloat1622float2(a2[e]), fb = __bfloat1622float2(b2[e]);
                  w[e] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
                }
                o = make_uint4(w[0], w[1], w[2], w[3]);
              }
              *reinterpret_cast<uint4*>(c_base + (long long)(4 * i) * ldc + c * 64) = o;
            }
          }
          __syncwarp();
        }
      } else {
      uint4 pre_cur[4], pre_next[4];
      bool have_cur = acc_bf16 && gemm_prefetch_addend(Rp, ldr, row, n0, Nn, row_ok, pre_cur);
#pragma unroll 1
      for (int c = 0; c < PN / 32; ++c) {
        const int col0 = n0 + c * 32;
        // the addend of the next chunk is requested before this chunk's TMEM load and stores
        const bool have_next = acc_bf16 && c + 1 < PN / 32 &&
                               gemm_prefetch_addend(Rp, ldr, row, col0 + 32, Nn, row_ok, pre_next);
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row_ok && col0 < Nn && has_k) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          gemm_store_chunk32(Cp, ldc, Rp, ldr, out_mode, row, col0, Nn, v, pre_cur, have_cur);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) pre_cur[j] = pre_next[j];
        have_cur = have_next;
      }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_cluster(smem_u32(&tmem_empty_bar[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves while the other may still signal it or read its operands
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 2 * P_ACC_COLS);
  }
  (void)peer;
}

}  // namespace

// DRAM traffic model of the tile order: A's rows of a band are read once if the band fits in L2
// (else once per n-tile); B is read once per band unless all of it fits in L2.  Returns the band
// height (in m-tiles) with the least modelled traffic.
static int g_band_override = 0;
void gemm_pair_set_band(int band) { g_band_override = band < 0 ? 0 : band; }

static int pair_band(int M, int N, int K, int m_tiles, int n_tiles) {
  if (g_band_override > 0) return g_band_override < m_tiles ? g_band_override : m_tiles;
  const double l2_fit = 75e6;  // bytes of one operand that stay resident next to the streams
  const double a_total = 2.0 * M * K, b_total = 2.0 * N * K;
  double best = -1.0;
  int best_band = m_tiles;
  for (int band = m_tiles;; band = (band + 1) / 2) {
    const int n_bands = (m_tiles + band - 1) / band;
    const double a_band = 2.0 * band * (2 * PM) * K;
    const double a_tr = a_total * (a_band <= l2_fit ? 1.0 : (double)n_tiles);
    const double b_tr = b_total * (b_total <= l2_fit ? 1.0 : (double)n_bands);
    const double tr = a_tr + b_tr;
    if (best < 0.0 || tr < best * 0.95) { best = tr; best_band = band; }
    if (band <= 4) break;
  }
  return best_band;
}

static int pair_launch(cudaStream_t stream, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmB2,
                       const PairParams& p, const char** err, const SegMaps* seg = nullptr) {
  static bool attr_set[MAX_DEVICE_SLOTS] = {false};
  static const SegMaps no_seg = {};
  const int slot = device_slot();
  if (!attr_set[slot]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tc2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_bf16_tc2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
    if (e != cudaSuccess) { if (err) *err = cudaGetErrorString(e); return 3; }
    attr_set[slot] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (gemm_num_sms() / 2), 1, 1);
  cfg.blockDim = dim3(P_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  // persistent grid: as many clusters as can be resident at once (SM pairs must share a TPC)
  static int max_clusters[MAX_DEVICE_SLOTS] = {0};
  if (!max_clusters[slot]) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_tc2_kernel<false>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = gemm_num_sms() / 2;
    }
    max_clusters[slot] = n;
  }
  int avail = max_clusters[slot] - (gemm_reserved_sms() + 1) / 2;
  if (avail < 1) avail = 1;
  const int clusters = p.total_tiles < avail ? p.total_tiles : avail;
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cudaError_t e = seg ? cudaLaunchKernelEx(&cfg, gemm_bf16_tc2_kernel<true>, tmA, tmB, tmB2, *seg, p)
                      : cudaLaunchKernelEx(&cfg, gemm_bf16_tc2_kernel<false>, tmA, tmB, tmB2, no_seg, p);
  if (e != cudaSuccess) { if (err) *err = cudaGetErrorString(e); return 3; }
  return 0;
}

static void pair_no_segments(PairParams& p) {
  for (int i = 0; i < 3; ++i) {
    p.kseg[i] = p.nseg[i] = i == 0 ? 0 : INT_MAX;
    p.Cs[i] = p.C; p.ldcs[i] = p.ldc; p.Ns[i] = p.N; p.out_modes[i] = p.out_mode;
  }
}

static void pair_set_split(PairParams& p, int split_k) {
  if (split_k < 1) split_k = 1;
  if (split_k > p.kblocks_total) split_k = p.kblocks_total;
  p.kblocks_per_split = (p.kblocks_total + split_k - 1) / split_k;
  p.split_k = (p.kblocks_total + p.kblocks_per_split - 1) / p.kblocks_per_split;
  p.total_tiles = p.m_tiles * p.n_tiles * p.split_k;
}

static int pair_auto_split(int tiles, int kblocks) {
  const int clusters = gemm_num_sms() / 2;
  int max_s = kblocks / 8;  // at least 8 k-blocks (512 of k) per split
  if (max_s < 1) max_s = 1;
  if (max_s > 32) max_s = 32;
  int best_s = 1;
  double best = -1.0;
  for (int s = 1; s <= max_s; ++s) {
    const long long t = (long long)tiles * s;
    const long long waves = (t + clusters - 1) / clusters;
    const double score = (double)t / (double)(waves * clusters) - 0.015 * (s - 1);
    if (score > best + 1e-9) { best = score; best_s = s; }
  }
  return best_s;
}

// C (op)= sum over up to three operand pairs of A_i B_i^T, accumulated in one pass (K segments).
// All pairs share the majors; every K_i but the last must be a multiple of 64.
int gemm_bf16_pair_concat_k(cudaStream_t stream, int a_mn, int b_mn, int M, int N, int n_seg, const void* const* A,
                            const long long* lda, const void* const* B, const long long* ldb, const int* K, void* C,
                            long long ldc, const void* R, long long ldr, int out_mode, int split_k, float alpha,
                            int* status, const char** err) {
  if (M <= 0 || N <= 0) return 0;
  if (n_seg < 1 || n_seg > 3) { if (err) *err = "gemm_bf16_concat_k: 1 to 3 segments"; return 1; }
  CUtensorMap ma[3], mb[3];
  int kb_start[3] = {0, INT_MAX, INT_MAX}, kblocks = 0, ktotal = 0;
  for (int i = 0; i < n_seg; ++i) {
    if (K[i] <= 0 || (i + 1 < n_seg && K[i] % BK)) {
      if (err) *err = "gemm_bf16_concat_k: every K but the last must be a positive multiple of 64";
      return 1;
    }
    if ((lda[i] % 8) || (ldb[i] % 8) || (reinterpret_cast<uintptr_t>(A[i]) & 15) || (reinterpret_cast<uintptr_t>(B[i]) & 15)) {
      if (err) *err = "gemm_bf16_concat_k: operand rows must be 16-byte aligned (leading dimension % 8 == 0)";
      return 1;
    }
    int rc = a_mn ? make_tmap_bf16_2d(&ma[i], A[i], M, K[i], lda[i], 64, BK) : make_tmap_bf16_2d(&ma[i], A[i], K[i], M, lda[i], 64, PM);
    if (!rc) rc = b_mn ? make_tmap_bf16_2d(&mb[i], B[i], N, K[i], ldb[i], 64, BK) : make_tmap_bf16_2d(&mb[i], B[i], K[i], N, ldb[i], 64, PN / 2);
    if (rc) { if (err) *err = "gemm_bf16_concat_k: cuTensorMapEncodeTiled failed"; return 2; }
    kb_start[i] = kblocks;
    kblocks += (K[i] + BK - 1) / BK;
    ktotal += K[i];
  }
  if (split_k > 1 && out_mode != GEMM_OUT_F32_ATOMIC) {
    if (err) *err = "gemm_bf16_concat_k: split_k > 1 needs the f32 atomic output mode";
    return 1;
  }
  PairParams p;
  p.M = M; p.N = N; p.K = ktotal;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.out_mode = out_mode;
  p.R = R ? R : C; p.ldr = R ? ldr : ldc;
  p.m_tiles = (M + 2 * PM - 1) / (2 * PM);
  p.n_tiles = (N + PN - 1) / PN;
  p.kblocks_total = kblocks;
  pair_set_split(p, split_k);
  p.band = pair_band(M, N, ktotal, p.m_tiles, p.n_tiles);
  p.alpha = alpha;
  p.status = status;
  p.dual = 0; p.C2 = nullptr; p.H = nullptr;
  p.rope_tab = nullptr; p.rope_s = 1; p.rope_hd = 2;
  pair_no_segments(p);
  for (int i = 1; i < n_seg; ++i) p.kseg[i] = kb_start[i];
  SegMaps sm;
  sm.a[0] = ma[n_seg > 1 ? 1 : 0];
  sm.a[1] = ma[n_seg > 2 ? 2 : 0];
  sm.b = mb[n_seg > 2 ? 2 : 0];
  return pair_launch(stream, ma[0], mb[0], mb[n_seg > 1 ? 1 : 0], p, err, &sm);
}

// Up to three products that share A in one launch (N segments): C_i (op)= A B_i^T, each with its own
// output matrix and output mode.  Every N_i but the last must be a multiple of 256.  The RoPE output
// mode (complete tiles only: M % 256 == 0, N_i % 256 == 0) uses one table for all segments that ask for it.
int gemm_bf16_pair_multi_n(cudaStream_t stream, int a_mn, int b_mn, int M, int K, const void* A, long long lda, int n_seg,
                           const void* const* B, const long long* ldb, const int* N, void* const* C, const long long* ldc,
                           const int* out_mode, int split_k, float alpha, const float* rope_table, int seq_len,
                           int head_dim, int* status, const char** err) {
  if (M <= 0 || K <= 0) return 0;
  if (n_seg < 1 || n_seg > 3) { if (err) *err = "gemm_bf16_multi_n: 1 to 3 segments"; return 1; }
  if ((lda % 8) || (reinterpret_cast<uintptr_t>(A) & 15)) {
    if (err) *err = "gemm_bf16_multi_n: operand rows must be 16-byte aligned (leading dimension % 8 == 0)";
    return 1;
  }
  CUtensorMap ma, mb[3];
  if (a_mn ? make_tmap_bf16_2d(&ma, A, M, K, lda, 64, BK) : make_tmap_bf16_2d(&ma, A, K, M, lda, 64, PM)) {
    if (err) *err = "gemm_bf16_multi_n: cuTensorMapEncodeTiled failed for A";
    return 2;
  }
  PairParams p;
  int nt_start[3] = {0, INT_MAX, INT_MAX}, n_tiles = 0, n_total = 0;
  bool all_atomic = true;
  for (int i = 0; i < n_seg; ++i) {
    if (N[i] <= 0 || (i + 1 < n_seg && N[i] % PN)) {
      if (err) *err = "gemm_bf16_multi_n: every N but the last must be a positive multiple of 256";
      return 1;
    }
    if ((ldb[i] % 8) || (reinterpret_cast<uintptr_t>(B[i]) & 15) || !C[i]) {
      if (err) *err = "gemm_bf16_multi_n: operand rows must be 16-byte aligned, outputs must not be null";
      return 1;
    }
    if (out_mode[i] == GEMM_OUT_BF16_ROPE &&
        ((M % (2 * PM)) || (N[i] % PN) || head_dim < 8 || (head_dim % 8) || (N[i] % head_dim) || seq_len <= 0 || !rope_table ||
         (reinterpret_cast<uintptr_t>(rope_table) & 15) || (ldc[i] % 8) || (reinterpret_cast<uintptr_t>(C[i]) & 15))) {
      if (err) *err = "gemm_bf16_multi_n: the RoPE output mode needs complete 256 x 256 tiles, a table and 16-byte aligned rows";
      return 1;
    }
    if (b_mn ? make_tmap_bf16_2d(&mb[i], B[i], N[i], K, ldb[i], 64, BK) : make_tmap_bf16_2d(&mb[i], B[i], K, N[i], ldb[i], 64, PN / 2)) {
      if (err) *err = "gemm_bf16_multi_n: cuTensorMapEncodeTiled failed for B";
      return 2;
    }
    all_atomic = all_atomic && out_mode[i] == GEMM_OUT_F32_ATOMIC;
    nt_start[i] = n_tiles;
    n_tiles += (N[i] + PN - 1) / PN;
    n_total += N[i];
  }
  p.M = M; p.N = n_total; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C[0]; p.ldc = ldc[0]; p.out_mode = out_mode[0];
  p.R = C[0]; p.ldr = ldc[0];
  p.m_tiles = (M + 2 * PM - 1) / (2 * PM);
  p.n_tiles = n_tiles;
  p.kblocks_total = (K + BK - 1) / BK;
  if (split_k == 0) split_k = (all_atomic && !deterministic()) ? pair_auto_split(p.m_tiles * n_tiles, p.kblocks_total) : 1;
  if (split_k > 1 && !all_atomic) {
    if (err) *err = "gemm_bf16_multi_n: split_k > 1 needs the f32 atomic output mode in every segment";
    return 1;
  }
  pair_set_split(p, split_k);
  p.band = pair_band(M, n_total, K, p.m_tiles, p.n_tiles);
  p.alpha = alpha;
  p.status = status;
  p.dual = 0; p.C2 = nullptr; p.H = nullptr;
  p.rope_tab = reinterpret_cast<const float2*>(rope_table);
  p.rope_s = seq_len > 0 ? seq_len : 1;
  p.rope_hd = head_dim >= 2 ? head_dim : 2;
  pair_no_segments(p);
  for (int i = 0; i < n_seg; ++i) {
    p.nseg[i] = nt_start[i];
    p.Cs[i] = C[i]; p.ldcs[i] = ldc[i]; p.Ns[i] = N[i]; p.out_modes[i] = out_mode[i];
  }
  SegMaps sm;
  sm.a[0] = ma; sm.a[1] = ma;
  sm.b = mb[n_seg > 2 ? 2 : 0];
  return pair_launch(stream, ma, mb[0], mb[n_seg > 1 ? 1 : 0], p, err, &sm);
}

int gemm_bf16_tc_pair(cudaStream_t stream, int a_mn, int b_mn, int M, int N, int K, const void* A, long long lda,
                      const void* B, long long ldb, void* C, long long ldc, const void* R, long long ldr, int out_mode, int split_k,
                      float alpha, int* status, const char** err) {
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
  if (!a_mn) rc = make_tmap_bf16_2d(&tmA, A, K, M, lda, 64, PM);
  else       rc = make_tmap_bf16_2d(&tmA, A, M, K, lda, 64, BK);
  if (rc) { if (err) *err = "gemm_bf16_tc: cuTensorMapEncodeTiled failed for A"; return 2; }
  if (!b_mn) rc = make_tmap_bf16_2d(&tmB, B, K, N, ldb, 64, PN / 2);
  else       rc = make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK);
  if (rc) { if (err) *err = "gemm_bf16_tc: cuTensorMapEncodeTiled failed for B"; return 2; }

  PairParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.out_mode = out_mode;
  p.R = R ? R : C; p.ldr = R ? ldr : ldc;
  p.m_tiles = (M + 2 * PM - 1) / (2 * PM);
  p.n_tiles = (N + PN - 1) / PN;
  p.kblocks_total = (K + BK - 1) / BK;
  if (split_k > p.kblocks_total) split_k = p.kblocks_total;
  p.kblocks_per_split = (p.kblocks_total + split_k - 1) / split_k;
  split_k = (p.kblocks_total + p.kblocks_per_split - 1) / p.kblocks_per_split;
  p.split_k = split_k;
  p.total_tiles = p.m_tiles * p.n_tiles * split_k;
  p.band = pair_band(M, N, K, p.m_tiles, p.n_tiles);
  p.alpha = alpha;
  p.status = status;
  p.dual = 0; p.C2 = nullptr; p.H = nullptr;
  p.rope_tab = nullptr; p.rope_s = 1; p.rope_hd = 2;
  return pair_launch(stream, tmA, tmB, tmB, p, err);
}

// Gate / up projections with the SwiGLU product in the epilogue (dual mode of the kernel):
// G = bf16(A Bg), U = bf16(A Bu) (each may be null), H = silu(G) * U.  A is [M,K] K-major, Bg / Bu are
// [K,N] (MN-major), outputs are [M,N] bf16 with leading dimension ldo.  M % 256 == 0, N % 128 == 0.
int gemm_bf16_pair_swiglu(cudaStream_t stream, int M, int N, int K, const void* A, long long lda, const void* Bg,
                          const void* Bu, long long ldb, void* G, void* U, void* H, long long ldo, int* status,
                          const char** err) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((M % (2 * PM)) || (N % (PN / 2))) {
    if (err) *err = "gemm_bf16_swiglu: M must be a multiple of 256 and N a multiple of 128";
    return 1;
  }
  if ((lda % 8) || (ldb % 8) || (ldo % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(Bg) & 15) ||
      (reinterpret_cast<uintptr_t>(Bu) & 15) || (reinterpret_cast<uintptr_t>(H) & 15) || (reinterpret_cast<uintptr_t>(G) & 15) ||
      (reinterpret_cast<uintptr_t>(U) & 15) || !H) {
    if (err) *err = "gemm_bf16_swiglu: pointers and rows must be 16-byte aligned, H must not be null";
    return 1;
  }
  CUtensorMap tmA, tmB, tmB2;
  if (make_tmap_bf16_2d(&tmA, A, K, M, lda, 64, PM) || make_tmap_bf16_2d(&tmB, Bg, N, K, ldb, 64, BK) ||
      make_tmap_bf16_2d(&tmB2, Bu, N, K, ldb, 64, BK)) {
    if (err) *err = "gemm_bf16_swiglu: cuTensorMapEncodeTiled failed";
    return 2;
  }
  PairParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = 0; p.b_mn = 1;
  p.C = G; p.ldc = ldo; p.out_mode = GEMM_OUT_BF16;
  p.R = G; p.ldr = ldo;
  p.dual = 1; p.C2 = U; p.H = H;
  p.rope_tab = nullptr; p.rope_s = 1; p.rope_hd = 2;
  p.m_tiles = M / (2 * PM);
  p.n_tiles = N / (PN / 2);
  p.kblocks_total = (K + BK - 1) / BK;
  p.kblocks_per_split = p.kblocks_total;
  p.split_k = 1;
  p.total_tiles = p.m_tiles * p.n_tiles;
  p.band = pair_band(M, 2 * N, K, p.m_tiles, p.n_tiles);
  p.alpha = 1.0f;
  p.status = status;
  return pair_launch(stream, tmA, tmB, tmB2, p, err);
}

int gemm_bf16_pair_rope(cudaStream_t stream, int M, int N, int K, const void* A, long long lda, const void* B,
                        long long ldb, void* C, long long ldc, const float* table, int seq_len, int head_dim,
                        int* status, const char** err) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((M % (2 * PM)) || (N % PN) || head_dim < 8 || (head_dim % 8) || (N % head_dim) || seq_len <= 0 || !table ||
      (reinterpret_cast<uintptr_t>(table) & 15)) {
    if (err) *err = "gemm_bf16_rope: M and N must be multiples of 256, head_dim a multiple of 8 that divides N";
    return 1;
  }
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15)) {
    if (err) *err = "gemm_bf16_rope: pointers and rows must be 16-byte aligned";
    return 1;
  }
  CUtensorMap tmA, tmB;
  if (make_tmap_bf16_2d(&tmA, A, K, M, lda, 64, PM) || make_tmap_bf16_2d(&tmB, B, N, K, ldb, 64, BK)) {
    if (err) *err = "gemm_bf16_rope: cuTensorMapEncodeTiled failed";
    return 2;
  }
  PairParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = 0; p.b_mn = 1;
  p.C = C; p.ldc = ldc; p.out_mode = GEMM_OUT_BF16_ROPE;
  p.R = C; p.ldr = ldc;
  p.dual = 0; p.C2 = nullptr; p.H = nullptr;
  p.rope_tab = reinterpret_cast<const float2*>(table); p.rope_s = seq_len; p.rope_hd = head_dim;
  p.m_tiles = M / (2 * PM);
  p.n_tiles = N / PN;
  p.kblocks_total = (K + BK - 1) / BK;
  p.kblocks_per_split = p.kblocks_total;
  p.split_k = 1;
  p.total_tiles = p.m_tiles * p.n_tiles;
  p.band = pair_band(M, N, K, p.m_tiles, p.n_tiles);
  p.alpha = 1.0f;
  p.status = status;
  return pair_launch(stream, tmA, tmB, tmB, p, err);
}

int gemm_pair_clusters_hint() { return gemm_num_sms() / 2; }

// Split of the k range for the f32 atomic output mode: the persistent grid works in waves of one
// tile per cluster, so the split is chosen to fill the last wave (176 tiles on 74 clusters are
// 2.4 waves = 79 % busy; split in two they are 4.8 waves = 95 %).  Every extra split costs one
// more pass of f32 atomics over C, charged as 1.5 % each.
int gemm_pair_auto_split_k(int M, int N, int K) {
  const int tiles = ((M + 2 * PM - 1) / (2 * PM)) * ((N + PN - 1) / PN);
  return pair_auto_split(tiles, (K + BK - 1) / BK);
}

}  // namespace eisen
