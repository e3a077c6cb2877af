// Causal attention (bf16, head_dim 128 or 64) on the 5th-generation tensor cores: tcgen05.mma with the score /
// gradient tiles and the output accumulators in tensor memory, operand tiles brought in by TMA.
//
// One CTA owns 128 "row-side" positions of one (batch, head) and streams 64-position "column-side" sub-tiles:
//   forward   rows = queries; per sub-tile of keys:  S = Q K^T  ->  P  ->  O += P V
//             (a first sweep over the keys computes the row max and row sum, so P is normalised BEFORE it is
//              rounded to bf16, exactly as the exported graph does)
//   dQ        rows = queries; per sub-tile of keys:  S = Q K^T, dP = dO V^T  ->  dS  ->  dQ += dS K
//   dK, dV    rows = keys;    per sub-tile of queries: S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T
//                                                       -> dV += P^T dO, dK += dS^T Q
// Warp roles: warp 0 TMA producer (ring of sub-tile pairs), warp 1 MMA issuer and owner of the tensor-memory
// allocation, then the element-wise warps: each thread owns one row and 16-column passes of the 64 score columns, reads
// them with tcgen05.ld, does the softmax / softmax-backward arithmetic and writes the bf16 result over the score buffer
// it came from (tcgen05.st), where the next MMA finds it as its A operand (TS form).  Score tiles are double-buffered
// in tensor memory and two groups of element-wise warps take the sub-tiles in turn, so the MMAs of sub-tile i+1
// overlap the arithmetic of sub-tile i.  The backward kernels use 16 element-wise warps and the whole SM (512
// tensor-memory columns); the forward kernel uses 8, half of the tensor memory and 100 KB of shared memory, and runs
// two CTAs per SM (four sub-tiles in flight per SM).  All three are persistent: a CTA walks its work items (row tile
// x batch x head, long row tiles first) and keeps rings, score buffers and barrier phases running across them, so
// the resident-tile load and the first score products of the next item overlap the last output products and the
// epilogue of the current one.  What limits these kernels is the latency of the hand-offs MMA -> element-wise -> MMA
// (commit, wake-up, tcgen05.ld / st) and the fill / drain of that chain, not the tensor pipe, hence the concurrency.
// The element-wise arithmetic works on bf16 pairs: one cvt.rn.bf16x2 and one mul.bf16x2 reproduce the two roundings
// of a score, one more pair of them the rounding of dS.
//
// Tiles are stored as HD / 64 halves of 64 columns (one 128-byte swizzle atom per row), so the 64-wide heads of the
// nanoGPT configurations are the one-half case of the same code: HD / 16 k-steps per score product, N = HD output
// columns.  A streamed [64 x HD] sub-tile serves two roles with the same bytes: "K-major" B operand of the score product
// (contraction over head_dim) and "MN-major" B operand of the output product (contraction over its 64 rows).
//
// Numerics are those of attn_flash.cu / the generic kernels (scores rounded twice to bf16, guard terms 1e-4 / 2e-4,
// reduce-max term); D = rowsum(dO*O) (l+1e-4)/(l+2e-4) comes from k_attn_tc_prep.
// Every mbarrier wait is bounded; on expiry an error word is set and the CTA drains and frees its tensor memory.
#define PCPB_ADJ_TU
#include "attn_tc.h"
#include "common.cuh"
#include "tc_common.cuh"

namespace pcpb {

namespace {

#ifndef PCPB_ATC_NST_FWD
#define PCPB_ATC_NST_FWD 2
#endif
#ifndef PCPB_ATC_NST_DQ
#define PCPB_ATC_NST_DQ 4
#endif
constexpr float LOG2E = 1.4426950408889634f;
// Element-wise warps per CTA: 16 (two groups of 8) in the backward kernels, which fill the SM alone; 8 (two groups of 4)
// in the forward kernel, which needs half of the tensor memory and half of the shared memory and runs two CTAs per SM
// so that four sub-tiles are in flight per SM and one CTA's prologue / epilogue overlaps the other's main loop.

enum { MODE_FWD = 0, MODE_DQ = 1, MODE_DKV = 2 };

struct AtcParams {
  int B, T, H, Hkv;
  float scale;
  float fwd_guard;                             // added to the softmax denominator in the forward (1e-4, or 0)
  int d, dkv;                                  // model width, kv width
  const bf16* qkn; const bf16* dout;           // row-side tiles that the element-wise warps load themselves
  bf16* o; float* mrow; float* lrow; const float* drow;
  bf16* dqkn; bf16* dqkv;
  int* err;
  int n_items, bh_count;                       // backward kernels: work items (row tile x batch-head), batch-heads
};

template <int MODE, int HD> struct AtcCfg {
  static constexpr int SUB_BYTES = 64 * HD * 2;                // one streamed sub-tile: 16 KB at HD = 128
  static constexpr int STAGE_BYTES = 2 * SUB_BYTES;            // (C1, C2)
  static constexpr int TILE_BYTES = 128 * HD * 2;              // one resident tile: 32 KB at HD = 128
  static constexpr int N_EW = (MODE == MODE_FWD) ? 8 : 16;
  // score buffers in tensor memory = sub-tiles in flight = element-wise groups (one group per buffer)
  static constexpr int NBUF = 2;
  static constexpr int THREADS = 64 + 32 * N_EW;
  static constexpr int CTAS_PER_SM = (MODE == MODE_FWD) ? 2 : 1;
  static constexpr int NCG = N_EW / 4;                       // warps per tensor-memory lane quarter
  static constexpr int PASSES = (NCG == 4) ? 2 : 4;          // 16-column passes of a thread over its share of a sub-tile
  // passes whose score columns are fetched from tensor memory with one wait (0: one wait per pass)
  // The kernels are persistent: a CTA takes work items L = blockIdx.x + k * gridDim.x (row tiles sorted from
  // long to short), and keeps its rings and score buffers running across items, so the prologue and the first score
  // products of the next item overlap the last output products and the epilogue of the current one.
  static constexpr bool PERSIST = true;
  static constexpr int LPR = (MODE == MODE_FWD) ? 4 : (MODE == MODE_DQ) ? 2 : 0;
  static constexpr uint32_t TMEM_COLS = (MODE == MODE_FWD) ? 256u : 512u;
  static constexpr int NST = (MODE == MODE_FWD) ? PCPB_ATC_NST_FWD : (MODE == MODE_DQ) ? PCPB_ATC_NST_DQ : 3;   // ring stages
  // resident row-side tiles in shared memory: K and V (dK/dV kernel), Q and dO (dQ kernel), Q (forward kernel)
  static constexpr int N_RES = (MODE == MODE_FWD) ? 1 : 2;
  // DKV: per warp, double-buffered, six statistics of 32 columns; FWD: exchange of the four partial (max, sum) of a row
  static constexpr int STAT_BYTES = (MODE == MODE_DKV) ? N_EW * 2 * 192 * 4 : (MODE == MODE_FWD) ? 2 * NCG * 128 * 2 * 4 : 16;
  static constexpr int OFF_RING = N_RES * TILE_BYTES;
  static constexpr int OFF_STAT = OFF_RING + NST * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_STAT + STAT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static_assert(SMEM_BYTES <= 232448 / CTAS_PER_SM - 1024 * (CTAS_PER_SM - 1), "more shared memory than the CTAs of one SM can have");
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Optional instrumentation (-DPCPB_ATC_TIMING): cycles spent in each bounded wait (and in the two MMA issue loops),
// accumulated in registers and added to global counters once per warp when the CTA ends.
#ifdef PCPB_ATC_TIMING
__device__ unsigned long long g_atc_t[96];            // 32 counters per kernel mode
#define ATC_T0() const long long t_sec0 = clock64()
#define ATC_T1(slot) tacc[slot] += clock64() - t_sec0
#else
#define ATC_T0()
#define ATC_T1(slot)
#endif
__device__ __forceinline__ bool twait(int code, uint32_t bar, uint32_t parity, int* err, long long& acc) {
#ifdef PCPB_ATC_TIMING
  const long long t0 = clock64();
  const bool r = mbar_wait(bar, parity, err, code);
  acc += clock64() - t0;
  return r;
#else
  return mbar_wait(bar, parity, err, code);
#endif
}

// Store 32 consecutive output columns of one row (f32 accumulators in tensor memory at taddr) as bf16 to dst.
// ADJ: the values are gradients (dQ, dK, dV: outputs of the dot_general VJP), passed through the adjoint-edge step of
// the reference's engine (non-finite -> 0, clamp to +-100).
template <bool ADJ>
__device__ __forceinline__ void store_out_cols(uint32_t taddr, bf16* dst) {
  uint32_t r[32];
  tmem_ld32(taddr, r);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 v;
    v.x = pack2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
    v.y = pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
    v.z = pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
    v.w = pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
    if (ADJ) {
      uint32_t mx2 = 0u;
      adj_track2(mx2, v.x); adj_track2(mx2, v.y); adj_track2(mx2, v.z); adj_track2(mx2, v.w);
      if (adj_over2(mx2)) { v.x = adj_edge2(v.x); v.y = adj_edge2(v.y); v.z = adj_edge2(v.z); v.w = adj_edge2(v.w); }
    }
    *reinterpret_cast<uint4*>(dst + 8 * j) = v;
  }
}

// 16 columns (64-wide heads, four warps per lane quarter)
template <bool ADJ>
__device__ __forceinline__ void store_out_cols16(uint32_t taddr, bf16* dst) {
  uint32_t r[16];
  tmem_ld16_issue(taddr, r);
  tmem_ld_wait16(r);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint4 v;
    v.x = pack2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
    v.y = pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
    v.z = pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
    v.w = pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
    if (ADJ) {
      uint32_t mx2 = 0u;
      adj_track2(mx2, v.x); adj_track2(mx2, v.y); adj_track2(mx2, v.z); adj_track2(mx2, v.w);
      if (adj_over2(mx2)) { v.x = adj_edge2(v.x); v.y = adj_edge2(v.y); v.z = adj_edge2(v.z); v.w = adj_edge2(v.w); }
    }
    *reinterpret_cast<uint4*>(dst + 8 * j) = v;
  }
}

template <int MODE, int HD>
__global__ void __launch_bounds__(AtcCfg<MODE, HD>::THREADS, AtcCfg<MODE, HD>::CTAS_PER_SM)
k_attn_tc(const __grid_constant__ CUtensorMap tm_qkn, const __grid_constant__ CUtensorMap tm_qkv,
          const __grid_constant__ CUtensorMap tm_do, const AtcParams p) {
  using Cfg = AtcCfg<MODE, HD>;
  constexpr int SUB_BYTES = Cfg::SUB_BYTES, STAGE_BYTES = Cfg::STAGE_BYTES, TILE_BYTES = Cfg::TILE_BYTES;
  constexpr bool TWO_HALVES = (HD == 128);                     // a tile row is one or two 64-column halves
  constexpr int NST = Cfg::NST, N_EW = Cfg::N_EW, NCG = Cfg::NCG, PASSES = Cfg::PASSES, NBUF = Cfg::NBUF, LPR = Cfg::LPR;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sRes = base, sRing = base + Cfg::OFF_RING, sBar = base + Cfg::OFF_BAR;
  float* const stat_base = reinterpret_cast<float*>(gen + Cfg::OFF_STAT);
  float* stat = stat_base;
  auto full_bar = [&](int s) { return sBar + 8u * s; };
  auto empty_bar = [&](int s) { return sBar + 8u * (NST + s); };
  auto tfull_bar = [&](int b) { return sBar + 8u * (2 * NST + b); };
  auto tempty_bar = [&](int b) { return sBar + 8u * (2 * NST + 3 + b); };
  auto efull_bar = [&](int e) { return sBar + 8u * (2 * NST + 6 + e); };
  const uint32_t out_bar = sBar + 8u * (2 * NST + 9), res_bar = out_bar + 8, comb_bar = out_bar + 16, tmem_slot = out_bar + 24;
  // forward kernel: the K half of a ring stage is free once the score product has read it and the V half once the
  // output product has, so the two halves have their own full / empty barriers (full_bar / empty_bar serve K)
  auto vfull_bar = [&](int s) { return out_bar + 32u + 8u * s; };
  auto vempty_bar = [&](int s) { return out_bar + 32u + 8u * (NST + s); };
  // persistent kernels: resident tiles free for the next item / output accumulators drained by the epilogue
  const uint32_t res_free_bar = out_bar + 32u + 8u * (2 * NST), out_free_bar = res_free_bar + 8u;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + Cfg::OFF_BAR + 8 * (2 * NST + 9) + 24);

  const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
  const int grp = p.H / p.Hkv;
  long long tacc[16] = {};
#ifdef PCPB_ATC_TIMING
  __shared__ long long ts_tcommit[2], ts_efull[2];           // clock at: T commit issued (per buffer), E published (per group)
#endif                                   // wait cycles by role (instrumented builds only)
#ifdef PCPB_ATC_TIMING
  const long long t_cta0 = clock64();
#endif
  // first backward kernel after the prepare kernel of this layer: evaluate (and clear) the bound on the adjoints that
  // stay on the chip
  if (MODE == MODE_DKV && blockIdx.x == 0 && threadIdx.x == 0) attn_bound_check_and_clear();
  // work items of this CTA
  constexpr bool PERSIST = Cfg::PERSIST;
  const int nt = p.T / 128;
  const int item0 = PERSIST ? (int)blockIdx.x : 0, item_step = PERSIST ? (int)gridDim.x : 1;
  const int n_items = PERSIST ? p.n_items : 1;
  int b, h, hk, r0, n_it, n_q = 0, total_g, row_base, xq, xk, xv;
  auto decode = [&](int L) {
    if (MODE == MODE_DKV) {
      const int x = L / p.bh_count, bhk = L % p.bh_count;    // x ascending = more queries = longer
      b = bhk / p.Hkv; hk = bhk % p.Hkv; h = hk * grp;
      r0 = x * 128;                                          // first key of this item
      n_q = (p.T - r0) / 64;
      n_it = n_q * grp;
    } else if (PERSIST) {
      const int x = L / p.bh_count, bh = L % p.bh_count;
      b = bh / p.H; h = bh % p.H; hk = h / grp;
      r0 = (nt - 1 - x) * 128;                               // first query of this item, long rows first
      n_it = (r0 + 128) / 64;
    } else {
      const int bh = blockIdx.y;
      b = bh / p.H; h = bh % p.H; hk = h / grp;
      r0 = (gridDim.x - 1 - blockIdx.x) * 128;               // first query of this CTA, long rows first
      n_it = (r0 + 128) / 64;
    }
    total_g = (MODE == MODE_FWD) ? 2 * n_it : n_it;
    row_base = b * p.T;                                      // first row of this batch element in [B*T, width]
    xq = h * HD; xk = p.d + hk * HD; xv = p.d + p.dkv + hk * HD;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int t = 0; t < NBUF; ++t) { mbar_init(tfull_bar(t), 1); mbar_init(tempty_bar(t), N_EW / NBUF); mbar_init(efull_bar(t), N_EW / NBUF); }
    if (MODE == MODE_FWD)
      for (int s = 0; s < NST; ++s) { mbar_init(vfull_bar(s), 1); mbar_init(vempty_bar(s), 1); }
    // the row-side tiles arrive by TMA (dK/dV) or are written to tensor memory by the element-wise warps
    mbar_init(out_bar, 1); mbar_init(res_bar, 1); mbar_init(comb_bar, N_EW);
    mbar_init(res_free_bar, 1); mbar_init(out_free_bar, N_EW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(Cfg::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_gen;
  // Tensor-memory columns:
  //   forward   (256 per CTA) score buffers at 0 / 64, output at 128; P overwrites the score buffer it was computed from
  //   dQ        (512) two score buffers at 0 / 128 (T1 at +0, T2 at +64), output at 384; dS overwrites the T1 buffer it
  //             was computed from
  //   dK, dV    (512) two score buffers at 0 / 128, outputs at 256 and 384; P^T and dS^T overwrite the T1 / T2 buffers
  // A 16-bit tile written over a score buffer goes where its writer read: warp group cg owns columns 16cg .. 16cg+15
  // of the buffer and puts its 16 k-values (8 columns) at 16cg, which is also where the MMA of k-step cg looks for them.
  auto t1_col = [&](int buf) { return tmem + (uint32_t)(buf * (MODE == MODE_FWD ? 64 : 128)); };
  auto t2_col = [&](int buf) { return tmem + (uint32_t)(buf * 128 + 64); };
  const uint32_t out1 = tmem + (MODE == MODE_FWD ? 128u : MODE == MODE_DQ ? 384u : 256u), out2 = tmem + 384u;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    // All 32 lanes run the loop (warp-uniform control flow and addresses); one elected lane issues.
    auto load_tile128 = [&](uint32_t dst, const CUtensorMap* m, int x, int y) {
      tma_load_2d_elect(dst, m, res_bar, x, y);              tma_load_2d_elect(dst + 8192, m, res_bar, x, y + 64);
      if (TWO_HALVES) { tma_load_2d_elect(dst + 16384, m, res_bar, x + 64, y); tma_load_2d_elect(dst + 24576, m, res_bar, x + 64, y + 64); }
    };
    bool ok = true;
    int gb = 0, ge = 0, g = 0, k = 0;                        // ring positions run on gb + g (forward V ring: ge + it) across items
    for (int L = item0; L < n_items; ++k, L += item_step) {
      decode(L);
      if (PERSIST && k > 0) {
        // the last score product of the previous item has read the resident tiles
        ok = __all_sync(0xffffffffu, twait(11, res_free_bar, (uint32_t)(k - 1) & 1u, p.err, tacc[0]));
        if (!ok) break;
      }
      mbar_expect_tx_elect(res_bar, Cfg::N_RES * TILE_BYTES);
      if (MODE == MODE_DKV) {
        load_tile128(sRes, &tm_qkn, xk, row_base + r0);
        load_tile128(sRes + TILE_BYTES, &tm_qkv, xv, row_base + r0);
      }
      if (MODE == MODE_FWD) load_tile128(sRes, &tm_qkn, xq, row_base + r0);
      if (MODE == MODE_DQ) {
        load_tile128(sRes, &tm_qkn, xq, row_base + r0);
        load_tile128(sRes + TILE_BYTES, &tm_do, xq, row_base + r0);
      }
      for (g = 0; g < total_g; ++g) {
        const int G = gb + g, s = G % NST;
        ok = __all_sync(0xffffffffu, twait(11, empty_bar(s), (((uint32_t)G / NST) & 1u) ^ 1u, p.err, tacc[0]));
        if (!ok) break;
        const uint32_t c1 = sRing + s * STAGE_BYTES, c2 = c1 + SUB_BYTES;
        if (MODE == MODE_FWD) {
          // K of key sub-tile g % n_it (both sweeps); V of sub-tile it = g - n_it (second sweep) through its own barriers
          const int y = row_base + (g % n_it) * 64;
          mbar_expect_tx_elect(full_bar(s), SUB_BYTES);
          tma_load_2d_elect(c1, &tm_qkn, full_bar(s), xk, y);
          if (TWO_HALVES) tma_load_2d_elect(c1 + 8192, &tm_qkn, full_bar(s), xk + 64, y);
          if (g >= n_it) {
            const int it = g - n_it, sv = (ge + it) % NST;
            ok = __all_sync(0xffffffffu, twait(11, vempty_bar(sv), (((uint32_t)(ge + it) / NST) & 1u) ^ 1u, p.err, tacc[0]));
            if (!ok) { ++g; break; }
            const uint32_t cv = sRing + sv * STAGE_BYTES + SUB_BYTES;
            mbar_expect_tx_elect(vfull_bar(sv), SUB_BYTES);
            tma_load_2d_elect(cv, &tm_qkv, vfull_bar(sv), xv, y);
            if (TWO_HALVES) tma_load_2d_elect(cv + 8192, &tm_qkv, vfull_bar(sv), xv + 64, y);
          }
        } else if (MODE == MODE_DKV) {
          mbar_expect_tx_elect(full_bar(s), STAGE_BYTES);
          const int hh = h + g / n_q, y = row_base + r0 + (g % n_q) * 64;
          tma_load_2d_elect(c1, &tm_qkn, full_bar(s), hh * HD, y);
          tma_load_2d_elect(c2, &tm_do, full_bar(s), hh * HD, y);
          if (TWO_HALVES) {
            tma_load_2d_elect(c1 + 8192, &tm_qkn, full_bar(s), hh * HD + 64, y);
            tma_load_2d_elect(c2 + 8192, &tm_do, full_bar(s), hh * HD + 64, y);
          }
        } else {
          mbar_expect_tx_elect(full_bar(s), STAGE_BYTES);
          const int y = row_base + g * 64;
          tma_load_2d_elect(c1, &tm_qkn, full_bar(s), xk, y);
          tma_load_2d_elect(c2, &tm_qkv, full_bar(s), xv, y);
          if (TWO_HALVES) {
            tma_load_2d_elect(c1 + 8192, &tm_qkn, full_bar(s), xk + 64, y);
            tma_load_2d_elect(c2 + 8192, &tm_qkv, full_bar(s), xv + 64, y);
          }
        }
      }
      if (!ok) break;
      gb += total_g; ge += n_it;
      g = 0;
    }
    if (!ok) {
      // gave up after gb + g ring loads were armed: wait (bounded) for the copies still in flight before the CTA may exit
      const int tot = gb + g;
      for (int j = (tot > NST ? tot - NST : 0); j < tot; ++j) {
        const uint32_t ph = ((uint32_t)j / NST) & 1u;
        for (uint32_t w = 0; w < (1u << 20); ++w) if (mbar_try(full_bar(j % NST), ph)) break;
      }
      if (MODE == MODE_FWD) {
        const int nv = ge + (g > n_it ? g - n_it : 0);           // V loads armed so far (at most; the last may not be)
        for (int j = (nv > NST ? nv - NST : 0); j < nv; ++j) {
          const uint32_t ph = ((uint32_t)j / NST) & 1u;
          for (uint32_t w = 0; w < (1u << 16); ++w) if (mbar_try(vfull_bar(j % NST), ph)) break;
        }
      }
      for (uint32_t w = 0; w < (1u << 20); ++w) if (mbar_try(res_bar, (uint32_t)k & 1u)) break;
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    // All 32 lanes run the loops and the waits; one elected lane issues the MMAs and the commits.
    // score products: M=128, N=64, A and B K-major; output products: M=128, N=HD, A K-major, B MN-major
    constexpr uint32_t ID_T = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    constexpr uint32_t ID_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    bool ok = true;
    int gb = 0, ge = 0;                                      // score products / result tiles of the items done so far (even)
    // g: position in the item (selects nothing here but the last-tile test); gb + g: ring / buffer position
    auto issue_T = [&](int g, bool release_stage) -> bool {
      const int G = gb + g, s = G % NST, buf = G % NBUF;
      if (!__all_sync(0xffffffffu, twait(13, full_bar(s), ((uint32_t)G / NST) & 1u, p.err, tacc[2]))) return false;
      if (!__all_sync(0xffffffffu, twait(14, tempty_bar(buf), (((uint32_t)G / NBUF) & 1u) ^ 1u, p.err, tacc[3]))) return false;
      tc_fence_after();
      ATC_T0();
      const uint32_t c1 = sRing + s * STAGE_BYTES, c2 = c1 + SUB_BYTES;
      // The two independent products of the backward kernels are issued alternately.
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint32_t ao = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
        const uint32_t bo = (uint32_t)(ks >> 2) * 8192u + (uint32_t)(ks & 3) * 32u;
        // first resident tile (Q or K) against the first streamed one; second (dO or V) against the second
        mma_bf16_elect(t1_col(buf), make_desc(sRes + ao, 16, 1024), make_desc(c1 + bo, 16, 1024), ID_T, ks > 0);
        if (MODE != MODE_FWD)
          mma_bf16_elect(t2_col(buf), make_desc(sRes + TILE_BYTES + ao, 16, 1024), make_desc(c2 + bo, 16, 1024), ID_T, ks > 0);
      }
      if (release_stage || MODE == MODE_FWD) mma_commit_elect(empty_bar(s));   // forward: the K half is free after the score product
      mma_commit_elect(tfull_bar(buf));
      // persistent kernels: after the last score product of an item the resident tiles may be replaced
      if (PERSIST && g == total_g - 1) mma_commit_elect(res_free_bar);
#ifdef PCPB_ATC_TIMING
      if (lane == 0) ts_tcommit[buf] = clock64();
#endif
      ATC_T1(10);
      return true;
    };
    int k = 0;
    for (int L = item0; L < n_items && ok; ++k, L += item_step) {
      decode(L);
      if (!(ok = __all_sync(0xffffffffu, twait(12, res_bar, (uint32_t)k & 1u, p.err, tacc[1])))) break;
      int g = 0;
      if (MODE == MODE_FWD)
        for (; g < n_it && ok; ++g) ok = issue_T(g, true);
      const int g0 = g;
      // score products run NBUF - 1 sub-tiles ahead of the output products
      for (int a = 0; a < NBUF - 1 && a < n_it && ok; ++a) ok = issue_T(g0 + a, false);
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + NBUF - 1 < n_it && !(ok = issue_T(g0 + it + NBUF - 1, false))) break;
        // sub-tile `it` belongs to the element-wise group of its score buffer; the result tile lives in that buffer
        // G: ring / score-buffer position (counts the first sweep of the forward kernel too); result tiles are only
        // published in the main sweep, so their barrier (and the forward kernel's V ring) counts ge + it
        const int G = gb + g0 + it, eb = G % NBUF;
        const uint32_t eph = ((uint32_t)(ge + it) / NBUF) & 1u;
        if (!(ok = __all_sync(0xffffffffu, twait(15, efull_bar(eb), eph, p.err, tacc[4])))) break;
#ifdef PCPB_ATC_TIMING
        tacc[14] += clock64() - *(volatile long long*)&ts_efull[eb];     // E published -> MMA warp awake
#endif
        if (PERSIST && it == 0 && k > 0) {
          // the epilogue of the previous item must have read the output accumulators
          if (!(ok = __all_sync(0xffffffffu, twait(15, out_free_bar, (uint32_t)(k - 1) & 1u, p.err, tacc[4])))) break;
        }
        tc_fence_after();
        ATC_T0();
        const int s = (MODE == MODE_FWD) ? ((ge + it) % NST) : (G % NST), buf = eb;
        const uint32_t c1 = sRing + s * STAGE_BYTES, c2 = c1 + SUB_BYTES;
        if (MODE == MODE_FWD) {
          if (!(ok = __all_sync(0xffffffffu, twait(13, vfull_bar(s), ((uint32_t)(ge + it) / NST) & 1u, p.err, tacc[2])))) break;
          tc_fence_after();
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint32_t acc = (it > 0 || ks > 0) ? 1u : 0u;
          if (MODE == MODE_FWD) mma_bf16_ts_elect(out1, t1_col(buf) + 16u * ks, make_desc(c2 + ks * 2048u, 8192, 1024), ID_O, acc);
          if (MODE == MODE_DQ) mma_bf16_ts_elect(out1, t1_col(buf) + 16u * ks, make_desc(c1 + ks * 2048u, 8192, 1024), ID_O, acc);
          if (MODE == MODE_DKV) {
            mma_bf16_ts_elect(out1, t1_col(buf) + 16u * ks, make_desc(c2 + ks * 2048u, 8192, 1024), ID_O, acc);
            mma_bf16_ts_elect(out2, t2_col(buf) + 16u * ks, make_desc(c1 + ks * 2048u, 8192, 1024), ID_O, acc);
          }
        }
        mma_commit_elect(MODE == MODE_FWD ? vempty_bar(s) : empty_bar(s));
        ATC_T1(11);
      }
      if (ok) mma_commit_elect(out_bar);
      gb += total_g; ge += n_it;
    }
  } else {
    // =========================== element-wise warps ===========================
    // NCG warps per tensor-memory lane quarter (4 in the backward kernels, 2 in the forward kernel).  cg numbers the
    // warps of a quarter: it picks the head dimensions / output columns a thread moves, and splits into the sub-tile
    // group (two groups) and, with 4 warps per quarter, the half of the 64 score columns a thread owns.
    const int q = warp & 3, row = q * 32 + lane, cg = (warp - 2) >> 2;
    const int grp2 = (NCG == 4) ? (cg >> 1) : cg, half = (NCG == 4) ? (cg & 1) : 0;   // NBUF groups
    constexpr int SHARE = 16 * PASSES;                       // score columns of a sub-tile a thread owns
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t scale2 = pack2(p.scale, p.scale);
    bool ok = true;
    int gb = 0, k = 0;                                       // sub-tiles of the items done so far (even), item count
    for (int L = item0; L < n_items && ok; ++k, L += item_step) {
    decode(L);
    const int my = r0 + row;                                 // my query (FWD, DQ) or my key (DKV)
    float m_run = -INFINITY, l_run = 0.f, inv1 = 0.f, inv2 = 0.f, Dr = 0.f, mterm = 0.f;
    if (MODE == MODE_DQ) {
      const long long idx = ((long long)b * p.H + h) * p.T + my;
      m_run = p.mrow[idx]; l_run = p.lrow[idx]; Dr = p.drow[idx];
      inv2 = 1.f / (l_run + 2.f * PCPB_GUARD);
      mterm = Dr * (2.f * PCPB_GUARD) * inv2;
    }
    // NBUF groups of warps take the sub-tiles in turn (group = sub-tile index mod NBUF = its score buffer), so the
    // tensor-memory and barrier latencies of one group are spent under the arithmetic of the other.  Within a group a
    // thread owns one row and SHARE (32 or 64) of the 64 columns, in passes of 16.
    int g = grp2;
    if (MODE == MODE_FWD) {
      // ---- sweep 1: row max and row sum of exp over this thread's share of the keys ----
      for (; g < n_it; g += NBUF) {
        const int buf = g % NBUF;
        ok = __all_sync(0xffffffffu, twait(16, tfull_bar(buf), ((uint32_t)(gb + g) / NBUF) & 1u, p.err, tacc[5]));
        if (!ok) break;
        tc_fence_after();
        // both passes' score columns are fetched at once (one exposed tensor-memory latency per sub-tile)
        uint32_t rr[PASSES][16];
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) tmem_ld16_issue(t1_col(buf) + lane_off + (uint32_t)(half * SHARE + pass * 16), rr[pass]);
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) tmem_ld_wait16(rr[pass]);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));          // the values are in registers: release the buffer early
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {
          const int ch = half * SHARE + pass * 16, k0 = g * 64 + ch;
          const bool diag = (k0 + 15 > r0);
          const uint32_t (&r)[16] = rr[pass];
          float sv[16], cm = -INFINITY;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            // bf16(bf16(acc) * scale), two at a time
            const uint32_t s2 = bmul2(pack2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), scale2);
            float s0 = bf_lo(s2), s1 = bf_hi(s2);
            if (diag) {
              if (k0 + 2 * j > my) s0 = -INFINITY;
              if (k0 + 2 * j + 1 > my) s1 = -INFINITY;
            }
            sv[2 * j] = s0; sv[2 * j + 1] = s1;
            cm = fmaxf(cm, fmaxf(s0, s1));
          }
          if (cm > m_run) { l_run *= ex2((m_run - cm) * LOG2E); m_run = cm; }
          if (m_run > -INFINITY) {
            const float mL = m_run * LOG2E;
#pragma unroll
            for (int i = 0; i < 16; ++i) l_run += ex2(fmaf(sv[i], LOG2E, -mL));
          }
        }
      }
      // combine the partial results of each row through shared memory (every warp sums them in the same order)
      if (ok) {
        stat = stat_base + (k & 1) * (NCG * 128 * 2);              // per-item buffer: a fast warp may be one item ahead
        stat[(cg * 128 + row) * 2] = m_run; stat[(cg * 128 + row) * 2 + 1] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(comb_bar);
        ok = __all_sync(0xffffffffu, twait(20, comb_bar, (uint32_t)k & 1u, p.err, tacc[9]));
      }
      if (ok) {
        float mn = -INFINITY;
#pragma unroll
        for (int c = 0; c < NCG; ++c) mn = fmaxf(mn, stat[(c * 128 + row) * 2]);
        float l = 0.f;
#pragma unroll
        for (int c = 0; c < NCG; ++c) l += stat[(c * 128 + row) * 2 + 1] * ex2((stat[(c * 128 + row) * 2] - mn) * LOG2E);
        m_run = mn; l_run = l;
        inv1 = 1.f / (l_run + p.fwd_guard);
      }
    }
    const int g0 = (MODE == MODE_FWD) ? n_it : 0;            // a multiple of NBUF: the buffer of sub-tile `it` is it % NBUF
    const float mL_row = m_run * LOG2E;
    for (int it = grp2; it < n_it && ok; it += NBUF) {
      const int gg = g0 + it, buf = it % NBUF;
      int cbase = 0;                                         // first column-side position of this thread's 32 columns
      // per-warp copy of the column statistics (no cross-warp barrier: a warp that gave up cannot block the others)
      float* st = stat + ((warp - 2) * 2 + ((it / NBUF) & 1)) * 192;
      if (MODE == MODE_DKV) {
        const int hh = h + it / n_q;
        cbase = r0 + (it % n_q) * 64 + half * SHARE;
        const long long idx = ((long long)b * p.H + hh) * p.T + cbase + lane;
        const float mm = p.mrow[idx], ll = p.lrow[idx], dd = p.drow[idx];
        const float i2 = 1.f / (ll + 2.f * PCPB_GUARD);
        st[lane] = mm; st[32 + lane] = 1.f / (ll + PCPB_GUARD); st[64 + lane] = i2; st[96 + lane] = dd;
        st[128 + lane] = dd * (2.f * PCPB_GUARD) * i2; st[160 + lane] = mm * LOG2E;
        __syncwarp();
      } else {
        cbase = it * 64 + half * SHARE;
      }
      ok = __all_sync(0xffffffffu, twait(17, tfull_bar(buf), ((uint32_t)(gb + gg) / NBUF) & 1u, p.err, tacc[6]));
      if (!ok) break;
#ifdef PCPB_ATC_TIMING
      tacc[15] += clock64() - *(volatile long long*)&ts_tcommit[buf];  // T commit issued -> element-wise warp awake
#endif
      tc_fence_after();
      ATC_T0();
      // Fetch the score (and dP) columns of both passes at once where the registers allow it (forward, dQ): one
      // exposed tensor-memory latency per sub-tile instead of one per load.
      // Forward and dQ fetch the score (and dP) columns of LPR passes with one tensor-memory wait (one exposed
      // latency per round instead of one per load); the dK/dV kernel has no registers to spare and waits once per pass.
      constexpr bool BATCH = (LPR > 0);
      constexpr int NQ = BATCH ? LPR : 1;
      uint32_t q1[NQ][16], q2[NQ][16];
#pragma unroll
      for (int pass = 0; pass < PASSES; ++pass) {
        if (BATCH && pass % NQ == 0) {
#pragma unroll
          for (int k = 0; k < NQ; ++k) {
            tmem_ld16_issue(t1_col(buf) + lane_off + (uint32_t)(half * SHARE + (pass + k) * 16), q1[k]);
            if (MODE == MODE_DQ) tmem_ld16_issue(t2_col(buf) + lane_off + (uint32_t)(half * SHARE + (pass + k) * 16), q2[k]);
          }
#pragma unroll
          for (int k = 0; k < NQ; ++k) { tmem_ld_wait16(q1[k]); if (MODE == MODE_DQ) tmem_ld_wait16(q2[k]); }
          if (pass + NQ == PASSES) {                          // everything this thread needs is in registers
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
          }
        }
        const int ch = half * SHARE + pass * 16, c0 = cbase + pass * 16;
        // does the causal boundary cross this block of 32 rows x 16 columns?
        const bool diag = (MODE == MODE_DKV) ? (c0 < r0 + 128) : (c0 + 15 > r0);
        uint32_t (&r1)[16] = q1[pass % NQ];
        if (!BATCH) tmem_ld16_issue(t1_col(buf) + lane_off + (uint32_t)ch, r1);     // waited for together with T2 below
        uint32_t ew[8], pw[8];
        if (MODE == MODE_FWD) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t s2 = bmul2(pack2(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1])), scale2);
            float e0 = ex2(fmaf(bf_lo(s2), LOG2E, -mL_row)) * inv1, e1 = ex2(fmaf(bf_hi(s2), LOG2E, -mL_row)) * inv1;
            if (diag) {
              if (c0 + 2 * j > my) e0 = 0.f;
              if (c0 + 2 * j + 1 > my) e1 = 0.f;
            }
            ew[j] = pack2(e0, e1);
          }
        } else {
          uint32_t (&r2)[16] = q2[pass % NQ];
          if (!BATCH) {
            tmem_ld16_issue(t2_col(buf) + lane_off + (uint32_t)ch, r2);
            tmem_ld_wait16(r1); tmem_ld_wait16(r2);
            if (pass == PASSES - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(tempty_bar(buf));
            }
          }
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            // statistics of the four columns of this group: broadcast row values (dQ) or per-column values (dK, dV)
            float mm[4], i1[4], i2[4], dd[4], mt[4], mL[4];
            if (MODE == MODE_DQ) {
#pragma unroll
              for (int e = 0; e < 4; ++e) { mm[e] = m_run; i1[e] = 0.f; i2[e] = inv2; dd[e] = Dr; mt[e] = mterm; mL[e] = mL_row; }
            } else {
              const float4* s4 = reinterpret_cast<const float4*>(st) + pass * 4 + j4;
              const float4 a = s4[0], bq = s4[8], c = s4[16], d4 = s4[24], e4 = s4[32], f = s4[40];
              mm[0] = a.x; mm[1] = a.y; mm[2] = a.z; mm[3] = a.w;
              i1[0] = bq.x; i1[1] = bq.y; i1[2] = bq.z; i1[3] = bq.w;
              i2[0] = c.x; i2[1] = c.y; i2[2] = c.z; i2[3] = c.w;
              dd[0] = d4.x; dd[1] = d4.y; dd[2] = d4.z; dd[3] = d4.w;
              mt[0] = e4.x; mt[1] = e4.y; mt[2] = e4.z; mt[3] = e4.w;
              mL[0] = f.x; mL[1] = f.y; mL[2] = f.z; mL[3] = f.w;
            }
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
              const int j = j4 * 2 + jj, e0i = jj * 2, e1i = jj * 2 + 1;
              const uint32_t s2 = bmul2(pack2(__uint_as_float(r1[2 * j]), __uint_as_float(r1[2 * j + 1])), scale2);
              const uint32_t d2 = pack2(__uint_as_float(r2[2 * j]), __uint_as_float(r2[2 * j + 1]));
              const float s0 = bf_lo(s2), s1 = bf_hi(s2), dp0 = bf_lo(d2), dp1 = bf_hi(d2);
              float e0 = ex2(fmaf(s0, LOG2E, -mL[e0i])), e1 = ex2(fmaf(s1, LOG2E, -mL[e1i]));
              bool k0 = true, k1 = true;                      // not masked
              if (diag) {
                if (MODE == MODE_DQ) { k0 = !(c0 + 2 * j > my); k1 = !(c0 + 2 * j + 1 > my); }
                else { k0 = !(my > c0 + 2 * j); k1 = !(my > c0 + 2 * j + 1); }
                if (!k0) e0 = 0.f;
                if (!k1) e1 = 0.f;
              }
              float ds0 = e0 * i2[e0i] * (dp0 - dd[e0i]), ds1 = e1 * i2[e1i] * (dp1 - dd[e1i]);
              if (k0 && s0 == mm[e0i]) ds0 -= mt[e0i];
              if (k1 && s1 == mm[e1i]) ds1 -= mt[e1i];
              // bf16(bf16(ds) * scale)
              ew[j] = bmul2(pack2(ds0, ds1), scale2);
              if (MODE == MODE_DKV) pw[j] = pack2(e0 * i1[e0i], e1 * i1[e1i]);
            }
          }
        }
        // over my own columns of the score buffer(s): nobody else reads them, and the next score product into this
        // buffer is issued after the output product that consumes these tiles
        if (MODE == MODE_DKV) tmem_st8(t1_col(buf) + lane_off + (uint32_t)ch, pw);
        tmem_st8((MODE == MODE_DKV ? t2_col(buf) : t1_col(buf)) + lane_off + (uint32_t)ch, ew);
      }
      if (!ok) break;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
#ifdef PCPB_ATC_TIMING
      if (lane == 0 && (warp == 2 || warp == 10)) ts_efull[buf] = clock64();
#endif
      if (lane == 0) mbar_arrive(efull_bar(buf));
      ATC_T1(12);
    }
    // ---- outputs: each warp stores 128 / NCG of the 128 output columns of its rows ----
    if (ok) ok = __all_sync(0xffffffffu, twait(19, out_bar, (uint32_t)k & 1u, p.err, tacc[8]));
    if (ok) {
      tc_fence_after();
      const long long grow = (long long)row_base + my;
      // HD output columns over the NCG warps of a lane quarter: HD / NCG each, in pieces of 32 (or one of 16)
      constexpr int CW = HD / NCG;
      if (CW >= 32) {
#pragma unroll
        for (int part = 0; part < CW / 32; ++part) {
          const int oc = cg * CW + part * 32;
          if (MODE == MODE_FWD) {
            store_out_cols<false>(out1 + lane_off + oc, p.o + grow * p.d + xq + oc);
          } else if (MODE == MODE_DQ) {
            store_out_cols<true>(out1 + lane_off + oc, p.dqkn + grow * (p.d + p.dkv) + xq + oc);
          } else {
            store_out_cols<true>(out1 + lane_off + oc, p.dqkv + grow * (p.d + 2 * p.dkv) + xv + oc);
            store_out_cols<true>(out2 + lane_off + oc, p.dqkn + grow * (p.d + p.dkv) + xk + oc);
          }
        }
      } else {
        const int oc = cg * CW;
        if (MODE == MODE_DQ) {
          store_out_cols16<true>(out1 + lane_off + oc, p.dqkn + grow * (p.d + p.dkv) + xq + oc);
        } else if (MODE == MODE_DKV) {
          store_out_cols16<true>(out1 + lane_off + oc, p.dqkv + grow * (p.d + 2 * p.dkv) + xv + oc);
          store_out_cols16<true>(out2 + lane_off + oc, p.dqkn + grow * (p.d + p.dkv) + xk + oc);
        } else {
          store_out_cols16<false>(out1 + lane_off + oc, p.o + grow * p.d + xq + oc);
        }
      }
      if (MODE == MODE_FWD && cg == 0) {
        const long long idx = ((long long)b * p.H + h) * p.T + my;
        p.mrow[idx] = m_run; p.lrow[idx] = l_run;
      }
      if (PERSIST) {
        // the accumulators are in registers / stored: the first output product of the next item may overwrite them
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(out_free_bar);
      }
    }
    gb += total_g;
    }                                                        // items
  }
#ifdef PCPB_ATC_TIMING
  if (lane == 0) {
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (tacc[c]) atomicAdd(&g_atc_t[MODE * 32 + 11 + c], (unsigned long long)tacc[c]);
  }
  if (threadIdx.x == 64) {
    atomicAdd(&g_atc_t[MODE * 32 + 0], (unsigned long long)(clock64() - t_cta0));
    atomicAdd(&g_atc_t[MODE * 32 + 1], 1ull);
    atomicAdd(&g_atc_t[MODE * 32 + 2], (unsigned long long)n_it);
  }
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

// D[b,h,i] = rowsum(do * o) * (l + 1e-4) / (l + 2e-4).  HD / 16 lanes per row, 16 elements (two 16-byte loads of each
// tensor) per lane: four (eight) rows per warp, 64 bytes in flight per thread.
template <int HD>
__global__ void __launch_bounds__(256) k_attn_tc_prep(const bf16* __restrict__ o, const bf16* __restrict__ dout,
                                                      const float* __restrict__ lrow, float* __restrict__ drow, int B, int T, int H,
                                                      const bf16* __restrict__ qkv, int Hkv) {
  __shared__ float sred[3][8];
  constexpr int LPROW = HD / 16, SHIFT = (HD == 128) ? 3 : 2;  // lanes per row
  const int sub = threadIdx.x & (LPROW - 1);
  const long long rows = (long long)B * H * T;
  // statistics for the bound on the adjoints that stay on the chip in the backward kernels (dP, dS): the largest
  // squared norm of a dO row and of a V row, the largest |D|; gathered per thread over its rows, then per block
  float m_do = 0.f, m_v = 0.f, m_d = 0.f;
  for (long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> SHIFT; gw < rows; gw += ((long long)gridDim.x * blockDim.x) >> SHIFT) {
    const int i = (int)(gw % T), bh = (int)(gw / T), b = bh / H, h = bh % H;
    const size_t off = ((size_t)b * T + i) * ((size_t)H * HD) + (size_t)h * HD + sub * 16;
    const uint4 a0 = *reinterpret_cast<const uint4*>(o + off), a1 = *reinterpret_cast<const uint4*>(o + off + 8);
    const uint4 c0 = *reinterpret_cast<const uint4*>(dout + off), c1 = *reinterpret_cast<const uint4*>(dout + off + 8);
    const uint32_t x[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t y[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float acc = 0.f, n_do = 0.f, n_v = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      acc += bf_lo(x[k]) * bf_lo(y[k]) + bf_hi(x[k]) * bf_hi(y[k]);
      n_do += bf_lo(y[k]) * bf_lo(y[k]) + bf_hi(y[k]) * bf_hi(y[k]);
    }
    if (h < Hkv) {
      const size_t voff = ((size_t)b * T + i) * ((size_t)(H + 2 * Hkv) * HD) + (size_t)(H + Hkv + h) * HD + sub * 16;
      const uint4 v0 = *reinterpret_cast<const uint4*>(qkv + voff), v1 = *reinterpret_cast<const uint4*>(qkv + voff + 8);
      const uint32_t z[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int k = 0; k < 8; ++k) n_v += bf_lo(z[k]) * bf_lo(z[k]) + bf_hi(z[k]) * bf_hi(z[k]);
    }
#pragma unroll
    for (int s = 1; s < LPROW; s <<= 1) {
      acc += __shfl_xor_sync(0xffffffffu, acc, s);
      n_do += __shfl_xor_sync(0xffffffffu, n_do, s);
      n_v += __shfl_xor_sync(0xffffffffu, n_v, s);
    }
    const float l = lrow[gw];
    const float D = acc * (l + PCPB_GUARD) / (l + 2.f * PCPB_GUARD);
    if (sub == 0) drow[gw] = D;
    // NaN must not be lost: a maximum that ignores NaN would hide it
    m_do = (n_do > m_do || n_do != n_do) ? n_do : m_do;
    m_v = (n_v > m_v || n_v != n_v) ? n_v : m_v;
    m_d = (fabsf(D) > m_d || D != D) ? fabsf(D) : m_d;
  }
  auto nmax = [](float a, float b) { return (b > a || b != b) ? b : a; };
#pragma unroll
  for (int s = 1; s <= 16; s <<= 1) {
    m_do = nmax(m_do, __shfl_xor_sync(0xffffffffu, m_do, s));
    m_v = nmax(m_v, __shfl_xor_sync(0xffffffffu, m_v, s));
    m_d = nmax(m_d, __shfl_xor_sync(0xffffffffu, m_d, s));
  }
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { sred[0][warp] = m_do; sred[1][warp] = m_d; sred[2][warp] = m_v; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float v = sred[threadIdx.x][0];
    for (int w = 1; w < 8; ++w) v = nmax(v, sred[threadIdx.x][w]);
    attn_bound_note((int)threadIdx.x, v);
  }
}

template <int MODE, int HD>
cudaError_t launch_mode(cudaStream_t st, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const AtcParams& p,
                        dim3 grid) {
  auto kern = k_attn_tc<MODE, HD>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AtcCfg<MODE, HD>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    // all of the SM's L1 / shared-memory array as shared memory: the forward kernel needs it to fit two CTAs per SM
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr[dev] = true;
  }
  kern<<<grid, AtcCfg<MODE, HD>::THREADS, AtcCfg<MODE, HD>::SMEM_BYTES, st>>>(a, b, c, p);
  return cudaGetLastError();
}

bool fill(const FlashArgs& a, int* err, AtcParams* p, CUtensorMap* mq, CUtensorMap* mv, CUtensorMap* md, bool need_do) {
  const int d = a.H * a.hd, dkv = a.Hkv * a.hd;
  const uint64_t M = (uint64_t)a.B * a.T;
  p->B = a.B; p->T = a.T; p->H = a.H; p->Hkv = a.Hkv; p->scale = a.scale; p->fwd_guard = a.no_guard ? 0.f : PCPB_GUARD; p->d = d; p->dkv = dkv;
  p->qkn = (const bf16*)a.qkn; p->dout = (const bf16*)a.dout;
  p->o = (bf16*)a.o; p->mrow = a.mrow; p->lrow = a.lrow; p->drow = a.drow; p->dqkn = (bf16*)a.dqkn; p->dqkv = (bf16*)a.dqkv;
  p->err = err; p->n_items = 1; p->bh_count = 1;
  bool ok = make_map(mq, a.qkn, (uint64_t)(d + dkv), M, (uint64_t)(d + dkv), 64) &&
            make_map(mv, a.qkv, (uint64_t)(d + 2 * dkv), M, (uint64_t)(d + 2 * dkv), 64);
  if (need_do) ok = ok && make_map(md, a.dout, (uint64_t)d, M, (uint64_t)d, 64);
  else *md = *mq;
  return ok;
}

}  // namespace

#ifdef PCPB_ATC_TIMING
extern "C" int pcpb_debug_atc_timing(unsigned long long* out96, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out96, g_atc_t, sizeof(unsigned long long) * 96);
  if (e == cudaSuccess && reset) { unsigned long long z[96] = {}; e = cudaMemcpyToSymbol(g_atc_t, z, sizeof z); }
  return e == cudaSuccess ? 0 : 2;
}
#endif

bool attn_tc_supported(const FlashArgs& a) {
  return (a.hd == 128 || a.hd == 64) && a.T % 128 == 0 && a.T >= 128 && a.H % a.Hkv == 0 && a.B > 0 && (long long)a.B * a.H <= 65535 &&
         ((((uintptr_t)a.qkn) | ((uintptr_t)a.qkv) | ((uintptr_t)a.o)) & 15) == 0 && encode_fn() != nullptr;
}

cudaError_t launch_attn_tc_fwd(cudaStream_t st, const FlashArgs& a, int* err_word) {
  AtcParams p;
  CUtensorMap mq, mv, md;
  if (!err_word || !fill(a, err_word, &p, &mq, &mv, &md, false)) return cudaErrorInvalidValue;
  // persistent: two CTAs per SM walk the work items, long row tiles first
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  p.bh_count = a.B * a.H; p.n_items = (a.T / 128) * p.bh_count;
  const int slots = sms * AtcCfg<MODE_FWD, 128>::CTAS_PER_SM;
  const dim3 grid(p.n_items < slots ? p.n_items : slots);
  return a.hd == 128 ? launch_mode<MODE_FWD, 128>(st, mq, mv, md, p, grid) : launch_mode<MODE_FWD, 64>(st, mq, mv, md, p, grid);
}

cudaError_t launch_attn_tc_bwd(cudaStream_t st, const FlashArgs& a, int* err_word) {
  AtcParams p;
  CUtensorMap mq, mv, md;
  if (!err_word || !fill(a, err_word, &p, &mq, &mv, &md, true)) return cudaErrorInvalidValue;
  const long long rows = (long long)a.B * a.H * a.T;
  {
    // a few rows per thread: the block-level statistics then cost three atomics per block
    const long long blocks = (rows * (a.hd / 16) + 255) / 256;
    const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
    if (a.hd == 128)
      k_attn_tc_prep<128><<<grid, 256, 0, st>>>((const bf16*)a.o, (const bf16*)a.dout, a.lrow, a.drow, a.B, a.T, a.H, (const bf16*)a.qkv, a.Hkv);
    else
      k_attn_tc_prep<64><<<grid, 256, 0, st>>>((const bf16*)a.o, (const bf16*)a.dout, a.lrow, a.drow, a.B, a.T, a.H, (const bf16*)a.qkv, a.Hkv);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  // persistent backward kernels: one CTA per SM walks the work items, long row tiles first
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  p.bh_count = a.B * a.Hkv; p.n_items = (a.T / 128) * p.bh_count;
  const dim3 g1(p.n_items < sms ? p.n_items : sms);
  e = a.hd == 128 ? launch_mode<MODE_DKV, 128>(st, mq, mv, md, p, g1) : launch_mode<MODE_DKV, 64>(st, mq, mv, md, p, g1);
  if (e != cudaSuccess) return e;
  p.bh_count = a.B * a.H; p.n_items = (a.T / 128) * p.bh_count;
  const dim3 g2(p.n_items < sms ? p.n_items : sms);
  return a.hd == 128 ? launch_mode<MODE_DQ, 128>(st, mq, mv, md, p, g2) : launch_mode<MODE_DQ, 64>(st, mq, mv, md, p, g2);
}

cudaError_t adj_status_fetch_attn_tc(cudaStream_t st, int* out, bool clear) { return adj_status_fetch_tu(st, out, clear); }

}  // namespace pcpb
