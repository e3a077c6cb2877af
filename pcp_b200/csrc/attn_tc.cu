// Causal attention (bf16, head_dim 128) on the 5th-generation tensor cores: tcgen05.mma with the score /
// gradient tiles and the output accumulators in tensor memory, operand tiles brought in by TMA.
//
// One CTA owns 128 "row-side" positions of one (batch, head) and streams 64-position "column-side" sub-tiles:
//   forward   rows = queries; per sub-tile of keys:  S = Q K^T  ->  P  ->  O += P V
//             (a first sweep over the keys computes the row max and row sum, so P is normalised BEFORE it is
//              rounded to bf16, exactly as the exported graph does)
//   dQ        rows = queries; per sub-tile of keys:  S = Q K^T, dP = dO V^T  ->  dS  ->  dQ += dS K
//   dK, dV    rows = keys;    per sub-tile of queries: S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T
//                                                       -> dV += P^T dO, dK += dS^T Q
// Warp roles (320 threads): warp 0 TMA producer (3-stage ring of sub-tile pairs), warp 1 MMA issuer and owner of the
// tensor-memory allocation, warps 2-9 element-wise: each thread owns one row and half of the 64 score columns, reads them with
// tcgen05.ld, does the softmax / softmax-backward arithmetic and writes the bf16 result into a 128-byte-swizzled
// shared-memory tile that the next MMA consumes as its A operand.  Score tiles are double-buffered in tensor memory
// so the MMAs of sub-tile i+1 overlap the arithmetic of sub-tile i.
//
// A streamed [64 x 128] sub-tile serves two roles with the same bytes: "K-major" B operand of the score product
// (contraction over head_dim) and "MN-major" B operand of the output product (contraction over its 64 rows).
//
// Numerics are those of attn_flash.cu / the generic kernels (scores rounded twice to bf16, guard terms 1e-4 / 2e-4,
// reduce-max term); D = rowsum(dO*O) (l+1e-4)/(l+2e-4) comes from k_attn_tc_prep.
// Every mbarrier wait is bounded; on expiry an error word is set and the CTA drains and frees its tensor memory.
#include "attn_tc.h"
#include "common.cuh"
#include "tc_common.cuh"

namespace pcpb {

namespace {

constexpr int HD = 128;
constexpr int NST = 3;                         // ring stages
constexpr int SUB_BYTES = 64 * HD * 2;         // one streamed sub-tile: 16 KB
constexpr int STAGE_BYTES = 2 * SUB_BYTES;     // (C1, C2)
constexpr int TILE_BYTES = 128 * HD * 2;       // one resident tile: 32 KB
constexpr int E_BYTES = 128 * 64 * 2;          // one element-wise result tile: 16 KB
constexpr float LOG2E = 1.4426950408889634f;

enum { MODE_FWD = 0, MODE_DQ = 1, MODE_DKV = 2 };

struct AtcParams {
  int B, T, H, Hkv;
  float scale;
  int d, dkv;                                  // model width, kv width
  bf16* o; float* mrow; float* lrow; const float* drow;
  bf16* dqkn; bf16* dqkv;
  int* err;
};

template <int MODE> struct AtcCfg {
  static constexpr int N_RES = (MODE == MODE_FWD) ? 1 : 2;
  static constexpr int N_E = (MODE == MODE_DKV) ? 2 : 1;
  static constexpr int STAT_BYTES = (MODE == MODE_DKV) ? 8 * 2 * 160 * 4 : 2 * 128 * 2 * 4;   // DKV: per warp, double-buffered; FWD: row-half exchange
  static constexpr int OFF_RING = N_RES * TILE_BYTES;
  static constexpr int OFF_E = OFF_RING + NST * STAGE_BYTES;
  static constexpr int OFF_STAT = OFF_E + N_E * E_BYTES;
  static constexpr int OFF_BAR = OFF_STAT + STAT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// f32 -> bf16 precision, round to nearest even, on the integer pipe (the conversion unit is the bottleneck of the
// element-wise warps; inputs are finite or +-inf)
__device__ __forceinline__ float r16(float x) {
  uint32_t u = __float_as_uint(x);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return __uint_as_float(u & 0xFFFF0000u);
}

// Optional instrumentation (-DPCPB_ATC_TIMING): cycles spent in each bounded wait, summed over warps and CTAs.
#ifdef PCPB_ATC_TIMING
__device__ unsigned long long g_atc_t[32];
#endif
__device__ __forceinline__ bool twait(int code, uint32_t bar, uint32_t parity, int* err) {
#ifdef PCPB_ATC_TIMING
  const long long t0 = clock64();
  const bool r = mbar_wait(bar, parity, err, code);
  if ((threadIdx.x & 31) == 0) atomicAdd(&g_atc_t[code], (unsigned long long)(clock64() - t0));
  return r;
#else
  return mbar_wait(bar, parity, err, code);
#endif
}

// Write 32 consecutive k-values (columns c0 .. c0+31 of row r) of a [128 x 64] bf16 A-operand tile (one 128-byte
// swizzle atom per row: 16-byte chunk j of row r lives at chunk position j ^ (r & 7)).
__device__ __forceinline__ void store_e32(uint32_t ebase, int r, int c0, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int kc = (c0 >> 3) + j;
    const uint32_t addr = ebase + (uint32_t)r * 128u + (uint32_t)((kc ^ (r & 7)) << 4);
    const uint32_t w0 = pack2(v[8 * j + 0], v[8 * j + 1]), w1 = pack2(v[8 * j + 2], v[8 * j + 3]);
    const uint32_t w2 = pack2(v[8 * j + 4], v[8 * j + 5]), w3 = pack2(v[8 * j + 6], v[8 * j + 7]);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
  }
}

// Store 64 consecutive output columns of one row (f32 accumulators in tensor memory at taddr) as bf16 to dst.
__device__ __forceinline__ void store_out_cols(uint32_t taddr, bf16* dst) {
#pragma unroll 1
  for (int c = 0; c < 64; c += 32) {
    uint32_t r[32];
    tmem_ld32(taddr + (uint32_t)c, r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 v;
      v.x = pack2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
      v.y = pack2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
      v.z = pack2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
      v.w = pack2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
      *reinterpret_cast<uint4*>(dst + c + 8 * j) = v;
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(320, 1)
k_attn_tc(const __grid_constant__ CUtensorMap tm_qkn, const __grid_constant__ CUtensorMap tm_qkv,
          const __grid_constant__ CUtensorMap tm_do, const AtcParams p) {
  using Cfg = AtcCfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sRes = base, sRing = base + Cfg::OFF_RING, sE = base + Cfg::OFF_E, sBar = base + Cfg::OFF_BAR;
  float* stat = reinterpret_cast<float*>(gen + Cfg::OFF_STAT);
  auto full_bar = [&](int s) { return sBar + 8u * s; };
  auto empty_bar = [&](int s) { return sBar + 8u * (NST + s); };
  auto tfull_bar = [&](int b) { return sBar + 8u * (2 * NST + b); };
  auto tempty_bar = [&](int b) { return sBar + 8u * (2 * NST + 2 + b); };
  const uint32_t efull_bar = sBar + 8u * (2 * NST + 4), eempty_bar = efull_bar + 8, out_bar = efull_bar + 16,
                 res_bar = efull_bar + 24, comb_bar = efull_bar + 32, tmem_slot = efull_bar + 40;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(gen + Cfg::OFF_BAR + 8 * (2 * NST + 4) + 40);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = p.H / p.Hkv;
#ifdef PCPB_ATC_TIMING
  const long long t_cta0 = clock64();
#endif
  // work of this CTA
  int b, h, hk, r0, n_it, n_q = 0;
  if (MODE == MODE_DKV) {
    const int bhk = blockIdx.y;
    b = bhk / p.Hkv; hk = bhk % p.Hkv; h = hk * grp;
    r0 = blockIdx.x * 128;                                   // first key of this CTA
    n_q = (p.T - r0) / 64;
    n_it = n_q * grp;
  } else {
    const int bh = blockIdx.y;
    b = bh / p.H; h = bh % p.H; hk = h / grp;
    r0 = (gridDim.x - 1 - blockIdx.x) * 128;                 // first query of this CTA, long rows first
    n_it = (r0 + 128) / 64;
  }
  const int total_g = (MODE == MODE_FWD) ? 2 * n_it : n_it;
  const int row_base = b * p.T;                              // first row of this batch element in [B*T, width]
  const int xq = h * HD, xk = p.d + hk * HD, xv = p.d + p.dkv + hk * HD;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(tfull_bar(t), 1); mbar_init(tempty_bar(t), 8); }
    mbar_init(efull_bar, 8); mbar_init(eempty_bar, 1); mbar_init(out_bar, 1); mbar_init(res_bar, 1); mbar_init(comb_bar, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot_gen;
  // tensor-memory columns: score buffers at 0 / 128 (T1 at +0, T2 at +64), outputs at 256 and 384
  auto t1_col = [&](int buf) { return tmem + (uint32_t)(buf * 128); };
  auto t2_col = [&](int buf) { return tmem + (uint32_t)(buf * 128 + 64); };
  const uint32_t out1 = tmem + 256u, out2 = tmem + 384u;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      auto load_tile128 = [&](uint32_t dst, const CUtensorMap* m, int x, int y) {
        tma_load_2d(dst, m, res_bar, x, y);           tma_load_2d(dst + 8192, m, res_bar, x, y + 64);
        tma_load_2d(dst + 16384, m, res_bar, x + 64, y); tma_load_2d(dst + 24576, m, res_bar, x + 64, y + 64);
      };
      mbar_expect_tx(res_bar, Cfg::N_RES * TILE_BYTES);
      if (MODE == MODE_FWD) load_tile128(sRes, &tm_qkn, xq, row_base + r0);
      if (MODE == MODE_DQ) { load_tile128(sRes, &tm_qkn, xq, row_base + r0); load_tile128(sRes + TILE_BYTES, &tm_do, xq, row_base + r0); }
      if (MODE == MODE_DKV) { load_tile128(sRes, &tm_qkn, xk, row_base + r0); load_tile128(sRes + TILE_BYTES, &tm_qkv, xv, row_base + r0); }
      int armed[NST] = {0, 0, 0};
      bool ok = true;
      for (int g = 0; g < total_g && ok; ++g) {
        const int s = g % NST;
        if (!(ok = twait(11, empty_bar(s), (((uint32_t)g / NST) & 1u) ^ 1u, p.err))) break;
        const uint32_t c1 = sRing + s * STAGE_BYTES, c2 = c1 + SUB_BYTES;
        const bool stats_pass = (MODE == MODE_FWD) && g < n_it;
        mbar_expect_tx(full_bar(s), stats_pass ? SUB_BYTES : STAGE_BYTES);
        armed[s] += 1;
        if (MODE == MODE_DKV) {
          const int hh = h + g / n_q, y = row_base + r0 + (g % n_q) * 64;
          tma_load_2d(c1, &tm_qkn, full_bar(s), hh * HD, y); tma_load_2d(c1 + 8192, &tm_qkn, full_bar(s), hh * HD + 64, y);
          tma_load_2d(c2, &tm_do, full_bar(s), hh * HD, y);  tma_load_2d(c2 + 8192, &tm_do, full_bar(s), hh * HD + 64, y);
        } else {
          const int y = row_base + ((MODE == MODE_FWD) ? (g % n_it) : g) * 64;
          tma_load_2d(c1, &tm_qkn, full_bar(s), xk, y); tma_load_2d(c1 + 8192, &tm_qkn, full_bar(s), xk + 64, y);
          if (!stats_pass) { tma_load_2d(c2, &tm_qkv, full_bar(s), xv, y); tma_load_2d(c2 + 8192, &tm_qkv, full_bar(s), xv + 64, y); }
        }
      }
      if (!ok) {
        for (int s = 0; s < NST; ++s)
          if (armed[s] > 0) {
            const uint32_t ph = (uint32_t)(armed[s] - 1) & 1u;
            for (uint32_t w = 0; w < (1u << 20); ++w) if (mbar_try(full_bar(s), ph)) break;
          }
        for (uint32_t w = 0; w < (1u << 20); ++w) if (mbar_try(res_bar, 0)) break;
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      // score products: M=128, N=64, A and B K-major; output products: M=128, N=128, A K-major, B MN-major
      constexpr uint32_t ID_T = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      constexpr uint32_t ID_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = twait(12, res_bar, 0, p.err);
      auto issue_T = [&](int g, bool release_stage) -> bool {
        const int s = g % NST, buf = g & 1;
        if (!twait(13, full_bar(s), ((uint32_t)g / NST) & 1u, p.err)) return false;
        if (!twait(14, tempty_bar(buf), (((uint32_t)g >> 1) & 1u) ^ 1u, p.err)) return false;
        tc_fence_after();
        const uint32_t c1 = sRing + s * STAGE_BYTES, c2 = c1 + SUB_BYTES;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t ao = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
          const uint32_t bo = (uint32_t)(ks >> 2) * 8192u + (uint32_t)(ks & 3) * 32u;
          mma_bf16(t1_col(buf), make_desc(sRes + ao, 16, 1024), make_desc(c1 + bo, 16, 1024), ID_T, ks > 0);
          if (MODE != MODE_FWD)
            mma_bf16(t2_col(buf), make_desc(sRes + TILE_BYTES + ao, 16, 1024), make_desc(c2 + bo, 16, 1024), ID_T, ks > 0);
        }
        if (release_stage) mma_commit(empty_bar(s));
        mma_commit(tfull_bar(buf));
        return true;
      };
      int g = 0;
      if (MODE == MODE_FWD)
        for (; g < n_it && ok; ++g) ok = issue_T(g, true);
      const int g0 = g;
      if (ok) ok = issue_T(g0, false);
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it && !(ok = issue_T(g0 + it + 1, false))) break;
        if (!(ok = twait(15, efull_bar, (uint32_t)it & 1u, p.err))) break;
        tc_fence_after();
        const int s = (g0 + it) % NST;
        const uint32_t c1 = sRing + s * STAGE_BYTES, c2 = c1 + SUB_BYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint32_t acc = (it > 0 || ks > 0) ? 1u : 0u;
          const uint64_t e1 = make_desc(sE + ks * 32u, 16, 1024);
          if (MODE == MODE_FWD) mma_bf16(out1, e1, make_desc(c2 + ks * 2048u, 8192, 1024), ID_O, acc);
          if (MODE == MODE_DQ) mma_bf16(out1, e1, make_desc(c1 + ks * 2048u, 8192, 1024), ID_O, acc);
          if (MODE == MODE_DKV) {
            mma_bf16(out1, e1, make_desc(c2 + ks * 2048u, 8192, 1024), ID_O, acc);
            mma_bf16(out2, make_desc(sE + E_BYTES + ks * 32u, 16, 1024), make_desc(c1 + ks * 2048u, 8192, 1024), ID_O, acc);
          }
        }
        mma_commit(empty_bar(s));
        mma_commit(eempty_bar);
      }
      if (ok) mma_commit(out_bar);
    }
  } else {
    // =========================== element-wise warps ===========================
    // Eight warps: two per tensor-memory lane quarter; each thread owns one row and one 32-column half of every
    // 64-column score sub-tile.
    const int q = warp & 3, row = q * 32 + lane, half = (warp - 2) >> 2, ch = half * 32;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int my = r0 + row;                                 // my query (FWD, DQ) or my key (DKV)
    bool ok = true;
    float m_run = -INFINITY, l_run = 0.f, inv1 = 0.f, inv2 = 0.f, Dr = 0.f, mterm = 0.f;
    if (MODE == MODE_DQ) {
      const long long idx = ((long long)b * p.H + h) * p.T + my;
      m_run = p.mrow[idx]; l_run = p.lrow[idx]; Dr = p.drow[idx];
      inv2 = 1.f / (l_run + 2.f * PCPB_GUARD);
      mterm = Dr * (2.f * PCPB_GUARD) * inv2;
    }
    int g = 0;
    if (MODE == MODE_FWD) {
      // ---- sweep 1: row max and row sum of exp over this thread's half of all keys ----
      for (; g < n_it; ++g) {
        const int buf = g & 1;
        ok = __all_sync(0xffffffffu, twait(16, tfull_bar(buf), ((uint32_t)g >> 1) & 1u, p.err));
        if (!ok) break;
        tc_fence_after();
        const int k0 = g * 64 + ch;
        const bool diag = (k0 + 31 > r0);
        uint32_t r[32];
        tmem_ld32(t1_col(buf) + lane_off + (uint32_t)ch, r);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));          // the values are in registers: release the buffer early
        float sv[32], cm = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = r16(r16(__uint_as_float(r[i])) * p.scale);
          if (diag && (k0 + i > my)) s = -INFINITY;
          sv[i] = s; cm = fmaxf(cm, s);
        }
        if (cm > m_run) { l_run *= ex2((m_run - cm) * LOG2E); m_run = cm; }
        if (m_run > -INFINITY) {
#pragma unroll
          for (int i = 0; i < 32; ++i) l_run += ex2((sv[i] - m_run) * LOG2E);
        }
      }
      // combine the two halves of each row through shared memory
      if (ok) {
        stat[(half * 128 + row) * 2] = m_run; stat[(half * 128 + row) * 2 + 1] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(comb_bar);
        ok = __all_sync(0xffffffffu, twait(20, comb_bar, 0, p.err));
      }
      if (ok) {
        const float mo = stat[((half ^ 1) * 128 + row) * 2], lo = stat[((half ^ 1) * 128 + row) * 2 + 1];
        const float mn = fmaxf(m_run, mo);
        l_run = l_run * ex2((m_run - mn) * LOG2E) + lo * ex2((mo - mn) * LOG2E);
        m_run = mn;
        inv1 = 1.f / (l_run + PCPB_GUARD);
      }
    }
    const int g0 = g;
    for (int it = 0; it < n_it && ok; ++it) {
      const int gg = g0 + it, buf = gg & 1;
      int c0 = 0;                                            // first column-side position of this thread's half
      // per-warp copy of the column statistics (no cross-warp barrier: a warp that gave up cannot block the others)
      float* st = stat + ((warp - 2) * 2 + (it & 1)) * 160;
      if (MODE == MODE_DKV) {
        const int hh = h + it / n_q;
        c0 = r0 + (it % n_q) * 64 + ch;
        const long long idx = ((long long)b * p.H + hh) * p.T + c0 + lane;
        const float mm = p.mrow[idx], ll = p.lrow[idx], dd = p.drow[idx];
        const float i2 = 1.f / (ll + 2.f * PCPB_GUARD);
        st[lane] = mm; st[32 + lane] = 1.f / (ll + PCPB_GUARD); st[64 + lane] = i2; st[96 + lane] = dd;
        st[128 + lane] = dd * (2.f * PCPB_GUARD) * i2;
        __syncwarp();
      } else {
        c0 = it * 64 + ch;
      }
      ok = __all_sync(0xffffffffu, twait(17, tfull_bar(buf), ((uint32_t)gg >> 1) & 1u, p.err));
      if (!ok) break;
      tc_fence_after();
      const bool diag = (MODE == MODE_DKV) ? (c0 < r0 + 128) : (c0 + 31 > r0);
      uint32_t r1[32];
      tmem_ld32(t1_col(buf) + lane_off + (uint32_t)ch, r1);
      float ev[32], e2v[32];
      if (MODE == MODE_FWD) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = r16(r16(__uint_as_float(r1[i])) * p.scale);
          const bool masked = diag && (c0 + i > my);
          ev[i] = masked ? 0.f : ex2((s - m_run) * LOG2E) * inv1;
        }
      } else {
        uint32_t r2[32];
        tmem_ld32(t2_col(buf) + lane_off + (uint32_t)ch, r2);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = r16(r16(__uint_as_float(r1[i])) * p.scale);
          const float dp = r16(__uint_as_float(r2[i]));
          float mm, i1, i2, dd, mt;
          bool masked;
          if (MODE == MODE_DQ) { mm = m_run; i1 = 0.f; i2 = inv2; dd = Dr; mt = mterm; masked = diag && (c0 + i > my); }
          else { mm = st[i]; i1 = st[32 + i]; i2 = st[64 + i]; dd = st[96 + i]; mt = st[128 + i]; masked = diag && (my > c0 + i); }
          const float e = masked ? 0.f : ex2((s - mm) * LOG2E);
          float dsf = e * i2 * (dp - dd);
          if (!masked && s == mm) dsf -= mt;
          // the second rounding of ds happens when the value is packed to bf16 for the result tile
          const float ds = masked ? 0.f : r16(dsf) * p.scale;
          if (MODE == MODE_DQ) ev[i] = ds; else { ev[i] = e * i1; e2v[i] = ds; }
        }
      }
      // the previous output products must have finished reading the result tile(s)
      ok = __all_sync(0xffffffffu, twait(18, eempty_bar, ((uint32_t)it & 1u) ^ 1u, p.err));
      if (!ok) break;
      store_e32(sE, row, ch, ev);
      if (MODE == MODE_DKV) store_e32(sE + E_BYTES, row, ch, e2v);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(efull_bar);
    }
    // ---- outputs: each warp stores 64 of the 128 output columns of its rows ----
    if (ok) ok = __all_sync(0xffffffffu, twait(19, out_bar, 0, p.err));
    if (ok) {
      tc_fence_after();
      const long long grow = (long long)row_base + my;
      const int oc = half * 64;
      if (MODE == MODE_FWD) {
        store_out_cols(out1 + lane_off + oc, p.o + grow * p.d + xq + oc);
        if (half == 0) {
          const long long idx = ((long long)b * p.H + h) * p.T + my;
          p.mrow[idx] = m_run; p.lrow[idx] = l_run;
        }
      } else if (MODE == MODE_DQ) {
        store_out_cols(out1 + lane_off + oc, p.dqkn + grow * (p.d + p.dkv) + xq + oc);
      } else {
        store_out_cols(out1 + lane_off + oc, p.dqkv + grow * (p.d + 2 * p.dkv) + xv + oc);
        store_out_cols(out2 + lane_off + oc, p.dqkn + grow * (p.d + p.dkv) + xk + oc);
      }
    }
  }
#ifdef PCPB_ATC_TIMING
  if (threadIdx.x == 64) {
    atomicAdd(&g_atc_t[0], (unsigned long long)(clock64() - t_cta0));
    atomicAdd(&g_atc_t[1], 1ull);
    atomicAdd(&g_atc_t[2], (unsigned long long)n_it);
  }
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// D[b,h,i] = rowsum(do * o) * (l + 1e-4) / (l + 2e-4).  One warp per row.
__global__ void k_attn_tc_prep(const bf16* __restrict__ o, const bf16* __restrict__ dout, const float* __restrict__ lrow,
                               float* __restrict__ drow, int B, int T, int H) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)B * H * T) return;
  const int i = (int)(gw % T), bh = (int)(gw / T), b = bh / H, h = bh % H;
  const size_t off = ((size_t)b * T + i) * ((size_t)H * HD) + (size_t)h * HD + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(o + off), c = *reinterpret_cast<const uint2*>(dout + off);
  float acc = __uint_as_float(a.x << 16) * __uint_as_float(c.x << 16) +
              __uint_as_float(a.x & 0xFFFF0000u) * __uint_as_float(c.x & 0xFFFF0000u) +
              __uint_as_float(a.y << 16) * __uint_as_float(c.y << 16) +
              __uint_as_float(a.y & 0xFFFF0000u) * __uint_as_float(c.y & 0xFFFF0000u);
  acc = warp_sum(acc);
  if (lane == 0) {
    const float l = lrow[gw];
    drow[gw] = acc * (l + PCPB_GUARD) / (l + 2.f * PCPB_GUARD);
  }
}

template <int MODE>
cudaError_t launch_mode(cudaStream_t st, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const AtcParams& p,
                        dim3 grid) {
  auto kern = k_attn_tc<MODE>;
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AtcCfg<MODE>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr[dev] = true;
  }
  kern<<<grid, 320, AtcCfg<MODE>::SMEM_BYTES, st>>>(a, b, c, p);
  return cudaGetLastError();
}

bool fill(const FlashArgs& a, int* err, AtcParams* p, CUtensorMap* mq, CUtensorMap* mv, CUtensorMap* md, bool need_do) {
  const int d = a.H * HD, dkv = a.Hkv * HD;
  const uint64_t M = (uint64_t)a.B * a.T;
  p->B = a.B; p->T = a.T; p->H = a.H; p->Hkv = a.Hkv; p->scale = a.scale; p->d = d; p->dkv = dkv;
  p->o = (bf16*)a.o; p->mrow = a.mrow; p->lrow = a.lrow; p->drow = a.drow; p->dqkn = (bf16*)a.dqkn; p->dqkv = (bf16*)a.dqkv;
  p->err = err;
  bool ok = make_map(mq, a.qkn, (uint64_t)(d + dkv), M, (uint64_t)(d + dkv), 64) &&
            make_map(mv, a.qkv, (uint64_t)(d + 2 * dkv), M, (uint64_t)(d + 2 * dkv), 64);
  if (need_do) ok = ok && make_map(md, a.dout, (uint64_t)d, M, (uint64_t)d, 64);
  else *md = *mq;
  return ok;
}

}  // namespace

#ifdef PCPB_ATC_TIMING
extern "C" int pcpb_debug_atc_timing(unsigned long long* out32, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out32, g_atc_t, sizeof(unsigned long long) * 32);
  if (e == cudaSuccess && reset) { unsigned long long z[32] = {}; e = cudaMemcpyToSymbol(g_atc_t, z, sizeof z); }
  return e == cudaSuccess ? 0 : 2;
}
#endif

bool attn_tc_supported(const FlashArgs& a) {
  return a.hd == HD && a.T % 128 == 0 && a.T >= 128 && a.H % a.Hkv == 0 && a.B > 0 && (long long)a.B * a.H <= 65535 &&
         ((((uintptr_t)a.qkn) | ((uintptr_t)a.qkv) | ((uintptr_t)a.o)) & 15) == 0 && encode_fn() != nullptr;
}

cudaError_t launch_attn_tc_fwd(cudaStream_t st, const FlashArgs& a, int* err_word) {
  AtcParams p;
  CUtensorMap mq, mv, md;
  if (!err_word || !fill(a, err_word, &p, &mq, &mv, &md, false)) return cudaErrorInvalidValue;
  return launch_mode<MODE_FWD>(st, mq, mv, md, p, dim3(a.T / 128, a.B * a.H));
}

cudaError_t launch_attn_tc_bwd(cudaStream_t st, const FlashArgs& a, int* err_word) {
  AtcParams p;
  CUtensorMap mq, mv, md;
  if (!err_word || !fill(a, err_word, &p, &mq, &mv, &md, true)) return cudaErrorInvalidValue;
  const long long rows = (long long)a.B * a.H * a.T;
  k_attn_tc_prep<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>((const bf16*)a.o, (const bf16*)a.dout, a.lrow, a.drow, a.B,
                                                                     a.T, a.H);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  e = launch_mode<MODE_DKV>(st, mq, mv, md, p, dim3(a.T / 128, a.B * a.Hkv));
  if (e != cudaSuccess) return e;
  return launch_mode<MODE_DQ>(st, mq, mv, md, p, dim3(a.T / 128, a.B * a.H));
}

}  // namespace pcpb
