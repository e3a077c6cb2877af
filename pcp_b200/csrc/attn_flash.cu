// Causal attention for bf16 models with head_dim 128, 64, 32 or 16, tiled so that the [T,T] score matrix never leaves
// the SM (forward) and is recomputed per tile (backward).  Tensor-core path: mma.sync m16n8k16 bf16 with
// ldmatrix-fed fragments; shared-memory tiles are filled with cp.async and XOR-swizzled per 16-byte chunk.
//
// Numerics (models/nanochat_d8_b8_t2048_bf16.mlir %106-%151 and the VJP rules they go through):
//   s = bf16(bf16(q.k) * scale_bf16); causal mask; softmax statistics in f32; l = sum exp(s - max)
//   o = bf16( sum_j bf16(exp(s_j - max)) v_j / (l + 1e-4) )
// One deliberate difference from the exported graph: the probability is rounded to bf16 before the division by
// (l + 1e-4) instead of after it (a single pass cannot know l earlier); the two differ by at most one bf16
// rounding of P.
// Backward: Pt = e/(l + 2e-4), dp = bf16(do.v), D = rowsum(do*o) (l+1e-4)/(l+2e-4),
//   dsf = Pt (dp - D) - [s == max] D 2e-4/(l+2e-4),  ds = bf16(bf16(dsf) * scale_bf16)
//   dv_j = sum_i bf16(P_ij) do_i,  dk_j = sum_i ds_ij q_i,  dq_i = sum_j ds_ij k_j
// dK/dV and dQ are produced by two kernels (one owns key blocks, one owns query blocks): no atomics, results
// are deterministic.
#include <cuda_bf16.h>
#include <stdint.h>

#define PCPB_ADJ_TU
#include "attn_flash.h"
#include "common.cuh"

namespace pcpb {

namespace {

// Every kernel and tile helper below is a template over the head dim HD (128, 64, 32 or 16 — the shipped nanochat
// graphs have 32-wide heads): a tile row is HD bf16 = HD/8 chunks of 16 bytes, the contraction over the head dim takes
// HD/16 mma k-steps and an output row has HD/8 n-tiles of 8 columns.
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// address of 16-byte chunk `chunk` (0..HD/8-1) of row `row` in a [rows][HD] bf16 tile.  The chunk index is XORed with
// a function of the row such that the 8 rows an ldmatrix phase reads (same chunk, consecutive rows) fall on the 8
// different 16-byte slots of a 128-byte bank line: rows of 128 bytes or more use the row's low three bits; shorter rows
// share a line (2 rows of 64 bytes, 4 of 32), which already separates them, and use the remaining row bits.
template <int HD>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
  constexpr int CPR = HD / 8;                                  // chunks per row
  constexpr int RPL = CPR >= 8 ? 1 : 8 / CPR;                  // rows per 128-byte line
  constexpr int MASK = (CPR >= 8 ? 8 : CPR) - 1;
  return base + (uint32_t)row * (HD * 2) + (uint32_t)((chunk ^ ((row / RPL) & MASK)) << 4);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Copy a [ROWS][HD] bf16 tile from global (row pitch `pitch` elements) into a swizzled smem tile.
template <int HD, int ROWS, int THREADS>
__device__ __forceinline__ void load_tile(uint32_t sbase, const bf16* __restrict__ g, long long pitch) {
  constexpr int CPR = HD / 8;                                  // 16-byte chunks per row
#pragma unroll
  for (int i = 0; i < (ROWS * CPR + THREADS - 1) / THREADS; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if ((ROWS * CPR) % THREADS != 0 && idx >= ROWS * CPR) break;
    const int row = idx / CPR, chunk = idx % CPR;
    cp_async16(tile_addr<HD>(sbase, row, chunk), g + (long long)row * pitch + chunk * 8);
  }
}

// A fragment (16 rows x 16 k) of a row-major tile: rows row0.., k chunk pair (2*ks, 2*ks+1)
template <int HD>
__device__ __forceinline__ void load_a(uint32_t sbase, int row0, int ks, uint32_t (&a)[4]) {
  const int lane = threadIdx.x & 31, id = lane >> 3, r = lane & 7;
  ldsm_x4(tile_addr<HD>(sbase, row0 + r + (id & 1) * 8, 2 * ks + (id >> 1)), a[0], a[1], a[2], a[3]);
}
// B fragments of two adjacent n-tiles (n0..n0+15) for k chunk pair ks, from a tile stored [n][k] (k contiguous)
template <int HD>
__device__ __forceinline__ void load_b_nk(uint32_t sbase, int n0, int ks, uint32_t (&b)[4]) {
  const int lane = threadIdx.x & 31, id = lane >> 3, r = lane & 7;
  ldsm_x4(tile_addr<HD>(sbase, n0 + r + (id >> 1) * 8, 2 * ks + (id & 1)), b[0], b[1], b[2], b[3]);
}
// B fragments of two adjacent n-tiles (n chunk nc, nc+1) for k rows k0..k0+15, from a tile stored [k][n] (n contiguous)
template <int HD>
__device__ __forceinline__ void load_b_kn(uint32_t sbase, int k0, int nc, uint32_t (&b)[4]) {
  const int lane = threadIdx.x & 31, id = lane >> 3, r = lane & 7;
  ldsm_x4_t(tile_addr<HD>(sbase, k0 + r + (id & 1) * 8, nc + (id >> 1)), b[0], b[1], b[2], b[3]);
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// ------------------------------------------------------------------------------------------------
// forward: CTA = 64 query rows of one (batch, head); 4 warps x 16 rows; key blocks of 64
// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(128) k_flash_fwd(FlashArgs a) {
  constexpr int ROWB = HD * 2, KS = HD / 16, NO = HD / 8;    // row bytes, head-dim k-steps, output n-tiles
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem), sK = sQ + 64 * ROWB, sV = sK + 2 * 64 * ROWB;
  const int qb = gridDim.x - 1 - blockIdx.x;                 // long rows first
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H, hk = h / (a.H / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int d = a.H * HD, dkv = a.Hkv * HD;
  const long long wqkn = d + dkv, wqkv = d + 2 * dkv;
  const int q0 = qb * 64;
  const bf16* Qg = (const bf16*)a.qkn + ((long long)b * a.T + q0) * wqkn + h * HD;
  const bf16* Kg = (const bf16*)a.qkn + (long long)b * a.T * wqkn + d + hk * HD;
  const bf16* Vg = (const bf16*)a.qkv + (long long)b * a.T * wqkv + d + dkv + hk * HD;

  load_tile<HD, 64, 128>(sQ, Qg, wqkn);
  load_tile<HD, 64, 128>(sK, Kg, wqkn);
  load_tile<HD, 64, 128>(sV, Vg, wqkv);
  cp_async_commit();

  float o[NO][4];
#pragma unroll
  for (int i = 0; i < NO; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int nkb = qb + 1;
  const int row_lo = q0 + warp * 16 + g;                     // this thread's rows: row_lo and row_lo + 8
  const uint32_t scale2 = pack2(a.scale, a.scale);

  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nkb) {
      load_tile<HD, 64, 128>(sK + (buf ^ 1) * 64 * ROWB, Kg + (long long)(kb + 1) * 64 * wqkn, wqkn);
      load_tile<HD, 64, 128>(sV + (buf ^ 1) * 64 * ROWB, Vg + (long long)(kb + 1) * 64 * wqkv, wqkv);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t cK = sK + buf * 64 * ROWB, cV = sV + buf * 64 * ROWB;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t af[4];
      load_a<HD>(sQ, warp * 16, ks, af);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bfr[4];
        load_b_nk<HD>(cK, np * 16, ks, bfr);
        mma16816(s[2 * np], af[0], af[1], af[2], af[3], bfr[0], bfr[1]);
        mma16816(s[2 * np + 1], af[0], af[1], af[2], af[3], bfr[2], bfr[3]);
      }
    }
    // scale (both roundings of the exported graph), causal mask on the diagonal block
    const bool diag = (kb == nkb - 1);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        // two adjacent columns at a time: packed convert + bf16x2 multiply instead of four scalar converts
        const uint32_t s2 = bmul2(pack2(s[nt][2 * r], s[nt][2 * r + 1]), scale2);
        float v0 = bf_lo(s2), v1 = bf_hi(s2);
        if (diag) {
          const int col = kb * 64 + nt * 8 + 2 * t;
          const int row = row_lo + r * 8;
          if (col > row) v0 = -INFINITY;
          if (col + 1 > row) v1 = -INFINITY;
        }
        s[nt][2 * r] = v0; s[nt][2 * r + 1] = v1;
        mx[r] = fmaxf(mx[r], fmaxf(v0, v1));
      }
    }
    float alpha[2], mnew[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = quad_max(mx[r]);
      mnew[r] = fmaxf(m_run[r], mx[r]);
      alpha[r] = exp2f((m_run[r] - mnew[r]) * LOG2E);
      m_run[r] = mnew[r];
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = exp2f((s[nt][e] - mnew[e >> 1]) * LOG2E);
        s[nt][e] = p;
        rs[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + quad_sum(rs[r]);
#pragma unroll
    for (int i = 0; i < NO; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < KS; ++np) {
        uint32_t bfr[4];
        load_b_kn<HD>(cV, kk * 16, 2 * np, bfr);
        mma16816(o[2 * np], a0, a1, a2, a3, bfr[0], bfr[1]);
        mma16816(o[2 * np + 1], a0, a1, a2, a3, bfr[2], bfr[3]);
      }
    }
    __syncthreads();
  }
  // finish: o / (l + 1e-4)
  bf16* Og = (bf16*)a.o + ((long long)b * a.T) * d + h * HD;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_lo + r * 8;
    const float inv = 1.f / (l_run[r] + PCPB_GUARD);
#pragma unroll
    for (int nt = 0; nt < NO; ++nt) {
      const uint32_t v = pack_bf16(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
      *reinterpret_cast<uint32_t*>(Og + (long long)row * d + nt * 8 + 2 * t) = v;
    }
    if (t == 0) {
      a.mrow[(long long)bh * a.T + row] = m_run[r];
      a.lrow[(long long)bh * a.T + row] = l_run[r];
    }
  }
}

// D[b,h,i] = rowsum(do * o) * (l + 1e-4) / (l + 2e-4).  One warp per row.
__global__ void k_flash_prep(FlashArgs a) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)a.B * a.H * a.T;
  if (gw >= rows) return;
  const int i = (int)(gw % a.T), bh = (int)(gw / a.T), b = bh / a.H, h = bh % a.H;
  const int HD = a.hd, d = a.H * HD;
  const bf16* op = (const bf16*)a.o + ((long long)b * a.T + i) * d + h * HD;
  const bf16* dp = (const bf16*)a.dout + ((long long)b * a.T + i) * d + h * HD;
  // a lane takes HD/32 consecutive elements (4 or 8 bytes of each row)
  // n_do, n_v: squared norms of the dO row and (kv heads) of the V row, for the bound on the adjoints dP = dO V^T and
  // dS that stay in registers in the backward kernels
  float acc = 0.f, n_do = 0.f, n_v = 0.f;
  const bf16* vp = (const bf16*)a.qkv + ((long long)b * a.T + i) * (long long)(d + 2 * a.Hkv * HD) + d + a.Hkv * HD + h * HD;
  if (HD == 128) {
    const uint2 x = *reinterpret_cast<const uint2*>(op + lane * 4), y = *reinterpret_cast<const uint2*>(dp + lane * 4);
    acc = bf_lo(x.x) * bf_lo(y.x) + bf_hi(x.x) * bf_hi(y.x) + bf_lo(x.y) * bf_lo(y.y) + bf_hi(x.y) * bf_hi(y.y);
    n_do = bf_lo(y.x) * bf_lo(y.x) + bf_hi(y.x) * bf_hi(y.x) + bf_lo(y.y) * bf_lo(y.y) + bf_hi(y.y) * bf_hi(y.y);
    if (h < a.Hkv) {
      const uint2 z = *reinterpret_cast<const uint2*>(vp + lane * 4);
      n_v = bf_lo(z.x) * bf_lo(z.x) + bf_hi(z.x) * bf_hi(z.x) + bf_lo(z.y) * bf_lo(z.y) + bf_hi(z.y) * bf_hi(z.y);
    }
  } else if (HD == 64) {
    const uint32_t x = *reinterpret_cast<const uint32_t*>(op + lane * 2), y = *reinterpret_cast<const uint32_t*>(dp + lane * 2);
    acc = bf_lo(x) * bf_lo(y) + bf_hi(x) * bf_hi(y);
    n_do = bf_lo(y) * bf_lo(y) + bf_hi(y) * bf_hi(y);
    if (h < a.Hkv) {
      const uint32_t z = *reinterpret_cast<const uint32_t*>(vp + lane * 2);
      n_v = bf_lo(z) * bf_lo(z) + bf_hi(z) * bf_hi(z);
    }
  } else if (lane < HD) {                                      // 32 or 16: one element per lane
    const float x = to_f(op[lane]), y = to_f(dp[lane]);
    acc = x * y;
    n_do = y * y;
    if (h < a.Hkv) { const float z = to_f(vp[lane]); n_v = z * z; }
  }
  acc = warp_sum(acc); n_do = warp_sum(n_do); n_v = warp_sum(n_v);
  if (lane == 0) {
    const float l = a.lrow[gw];
    const float D = acc * (l + PCPB_GUARD) / (l + 2.f * PCPB_GUARD);
    a.drow[gw] = D;
    // what the backward kernels need per query row, divisions done once here: max, 1/(l+1e-4), 1/(l+2e-4), D
    a.stat4[gw] = make_float4(a.mrow[gw], 1.f / (l + PCPB_GUARD), 1.f / (l + 2.f * PCPB_GUARD), D);
    attn_bound_note(0, n_do); attn_bound_note(1, D); attn_bound_note(2, n_v);
  }
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared by both backward kernels: two adjacent fragment elements (columns c, c+1 of one row) from raw scores / raw dp
// to the packed bf16 pairs (P, P') and (ds, ds').  st0 / st1 = (m, 1/(l+1e-4), 1/(l+2e-4), D) of the query row of each
// element.  Roundings to bf16 are done two at a time (one packed convert or one bf16x2 multiply per op of the graph):
// scalar float -> bf16 converts run on the quarter-rate XU pipe, which they kept 70 % busy.
__device__ __forceinline__ void bwd_pair(float s0raw, float s1raw, float dp0raw, float dp1raw, uint32_t scale2, const float4 st0,
                                         const float4 st1, bool m0, bool m1, uint32_t& p2, uint32_t& ds2) {
  const uint32_t s2 = bmul2(pack2(s0raw, s1raw), scale2);             // bf16(bf16(q.k) * scale)
  const float s0 = bf_lo(s2), s1 = bf_hi(s2);
  const float e0 = m0 ? 0.f : ex2_approx(fmaf(s0, LOG2E, -st0.x * LOG2E));
  const float e1 = m1 ? 0.f : ex2_approx(fmaf(s1, LOG2E, -st1.x * LOG2E));
  const uint32_t d2 = pack2(dp0raw, dp1raw);                          // bf16(do.v)
  float f0 = e0 * st0.z * (bf_lo(d2) - st0.w), f1 = e1 * st1.z * (bf_hi(d2) - st1.w);
  if (!m0 && s0 == st0.x) f0 -= st0.w * (2.f * PCPB_GUARD) * st0.z;
  if (!m1 && s1 == st1.x) f1 -= st1.w * (2.f * PCPB_GUARD) * st1.z;
  p2 = pack2(e0 * st0.y, e1 * st1.y);
  ds2 = bmul2(pack2(m0 ? 0.f : f0, m1 ? 0.f : f1), scale2);           // bf16(bf16(dsf) * scale)
}

// ------------------------------------------------------------------------------------------------
// backward, dK / dV: CTA = 128 keys of one (batch, kv head); 8 warps x 16 keys; query blocks of 64.
// Works on the transposed tiles S^T = K Q^T and dP^T = V dO^T so that P^T and dS^T come out of the tensor
// cores already in the A-operand register layout of the next two products.
// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(256) k_flash_bwd_dkv(FlashArgs a) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) attn_bound_check_and_clear();   // bound gathered by k_flash_prep
  constexpr int ROWB = HD * 2, KS = HD / 16, NO = HD / 8;    // row bytes, head-dim k-steps, output n-tiles
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sK = smem_u32(smem), sV = sK + 128 * ROWB, sQ = sV + 128 * ROWB, sDO = sQ + 2 * 64 * ROWB;
  float4* sstat = reinterpret_cast<float4*>(smem + 2 * 128 * ROWB + 4 * 64 * ROWB);     // [2 bufs][64] row records
  const int kb = blockIdx.x;
  const int bhk = blockIdx.y, b = bhk / a.Hkv, hk = bhk % a.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int d = a.H * HD, dkv = a.Hkv * HD, grp = a.H / a.Hkv;
  const long long wqkn = d + dkv, wqkv = d + 2 * dkv;
  const int j0 = kb * 128;
  const bf16* Kg = (const bf16*)a.qkn + ((long long)b * a.T + j0) * wqkn + d + hk * HD;
  const bf16* Vg = (const bf16*)a.qkv + ((long long)b * a.T + j0) * wqkv + d + dkv + hk * HD;
  load_tile<HD, 128, 256>(sK, Kg, wqkn);
  load_tile<HD, 128, 256>(sV, Vg, wqkv);
  cp_async_commit();

  float dk[NO][4], dv[NO][4];
#pragma unroll
  for (int i = 0; i < NO; ++i) { dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f; dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f; }

  const int nqb = a.T / 64, qb_first = j0 / 64;
  const int per_head = nqb - qb_first;
  const int total = per_head * grp;
  const int key_lo = j0 + warp * 16 + g;                     // this thread's keys: key_lo and key_lo + 8
  const uint32_t scale2 = pack2(a.scale, a.scale);

  auto issue = [&](int it, int buf) {
    const int h = hk * grp + it / per_head, qb = qb_first + it % per_head;
    const bf16* Qg = (const bf16*)a.qkn + ((long long)b * a.T + qb * 64) * wqkn + h * HD;
    const bf16* DOg = (const bf16*)a.dout + ((long long)b * a.T + qb * 64) * d + h * HD;
    load_tile<HD, 64, 256>(sQ + buf * 64 * ROWB, Qg, wqkn);
    load_tile<HD, 64, 256>(sDO + buf * 64 * ROWB, DOg, d);
    if (threadIdx.x < 64)
      cp_async16(smem_u32(sstat + buf * 64 + threadIdx.x), a.stat4 + ((long long)b * a.H + h) * a.T + qb * 64 + threadIdx.x);
    cp_async_commit();
  };
  issue(0, 0);

  for (int it = 0; it < total; ++it) {
    const int buf = it & 1;
    if (it + 1 < total) { issue(it + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const int qb = qb_first + it % per_head;
    const uint32_t cQ = sQ + buf * 64 * ROWB, cDO = sDO + buf * 64 * ROWB;
    const float4* st = sstat + buf * 64;

    float sT[8][4], dpT[8][4];                               // [16 keys] x [64 queries]
#pragma unroll
    for (int i = 0; i < 8; ++i) { sT[i][0] = sT[i][1] = sT[i][2] = sT[i][3] = 0.f; dpT[i][0] = dpT[i][1] = dpT[i][2] = dpT[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t ak[4], av[4];
      load_a<HD>(sK, warp * 16, ks, ak);
      load_a<HD>(sV, warp * 16, ks, av);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bq[4], bd[4];
        load_b_nk<HD>(cQ, np * 16, ks, bq);
        load_b_nk<HD>(cDO, np * 16, ks, bd);
        mma16816(sT[2 * np], ak[0], ak[1], ak[2], ak[3], bq[0], bq[1]);
        mma16816(sT[2 * np + 1], ak[0], ak[1], ak[2], ak[3], bq[2], bq[3]);
        mma16816(dpT[2 * np], av[0], av[1], av[2], av[3], bd[0], bd[1]);
        mma16816(dpT[2 * np + 1], av[0], av[1], av[2], av[3], bd[2], bd[3]);
      }
    }
    const bool diag = (qb * 64 < j0 + 128);                  // some (key, query) pairs of this tile are masked
    uint32_t P2[8][2], DS2[8][2];                            // packed pairs: [n-tile][row half]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int qi = nt * 8 + 2 * t;                         // query index inside the block (tile column) of the pair
      const float4 st0 = st[qi], st1 = st[qi + 1];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int key = key_lo + r * 8;
        const bool m0 = diag && (key > qb * 64 + qi), m1 = diag && (key > qb * 64 + qi + 1);
        bwd_pair(sT[nt][2 * r], sT[nt][2 * r + 1], dpT[nt][2 * r], dpT[nt][2 * r + 1], scale2, st0, st1, m0, m1, P2[nt][r], DS2[nt][r]);
      }
    }
    // dV += P^T dO ; dK += dS^T Q     (contraction over the 64 queries)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t p0 = P2[2 * kk][0], p1 = P2[2 * kk][1], p2 = P2[2 * kk + 1][0], p3 = P2[2 * kk + 1][1];
      const uint32_t s0 = DS2[2 * kk][0], s1 = DS2[2 * kk][1], s2 = DS2[2 * kk + 1][0], s3 = DS2[2 * kk + 1][1];
#pragma unroll
      for (int np = 0; np < KS; ++np) {
        uint32_t bd[4], bq[4];
        load_b_kn<HD>(cDO, kk * 16, 2 * np, bd);
        load_b_kn<HD>(cQ, kk * 16, 2 * np, bq);
        mma16816(dv[2 * np], p0, p1, p2, p3, bd[0], bd[1]);
        mma16816(dv[2 * np + 1], p0, p1, p2, p3, bd[2], bd[3]);
        mma16816(dk[2 * np], s0, s1, s2, s3, bq[0], bq[1]);
        mma16816(dk[2 * np + 1], s0, s1, s2, s3, bq[2], bq[3]);
      }
    }
    __syncthreads();
  }
  // dk -> k part of dqkn (gradient wrt the normalised roped k), dv -> v part of dqkv
  bf16* dKg = (bf16*)a.dqkn + ((long long)b * a.T) * wqkn + d + hk * HD;
  bf16* dVg = (bf16*)a.dqkv + ((long long)b * a.T) * wqkv + d + dkv + hk * HD;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int key = key_lo + r * 8;
#pragma unroll
    for (int nt = 0; nt < NO; ++nt) {
      *reinterpret_cast<uint32_t*>(dKg + (long long)key * wqkn + nt * 8 + 2 * t) = adj_edge2(pack_bf16(dk[nt][2 * r], dk[nt][2 * r + 1]));
      *reinterpret_cast<uint32_t*>(dVg + (long long)key * wqkv + nt * 8 + 2 * t) = adj_edge2(pack_bf16(dv[nt][2 * r], dv[nt][2 * r + 1]));
    }
  }
}

// ------------------------------------------------------------------------------------------------
// backward, dQ: CTA = 64 query rows of one (batch, head); 4 warps x 16 rows; key blocks of 64
// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(128) k_flash_bwd_dq(FlashArgs a) {
  constexpr int ROWB = HD * 2, KS = HD / 16, NO = HD / 8;    // row bytes, head-dim k-steps, output n-tiles
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem), sDO = sQ + 64 * ROWB, sK = sDO + 64 * ROWB, sV = sK + 2 * 64 * ROWB;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H, hk = h / (a.H / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int d = a.H * HD, dkv = a.Hkv * HD;
  const long long wqkn = d + dkv, wqkv = d + 2 * dkv;
  const int q0 = qb * 64;
  const bf16* Qg = (const bf16*)a.qkn + ((long long)b * a.T + q0) * wqkn + h * HD;
  const bf16* DOg = (const bf16*)a.dout + ((long long)b * a.T + q0) * d + h * HD;
  const bf16* Kg = (const bf16*)a.qkn + (long long)b * a.T * wqkn + d + hk * HD;
  const bf16* Vg = (const bf16*)a.qkv + (long long)b * a.T * wqkv + d + dkv + hk * HD;
  load_tile<HD, 64, 128>(sQ, Qg, wqkn);
  load_tile<HD, 64, 128>(sDO, DOg, d);
  load_tile<HD, 64, 128>(sK, Kg, wqkn);
  load_tile<HD, 64, 128>(sV, Vg, wqkv);
  cp_async_commit();

  const int row_lo = q0 + warp * 16 + g;
  const uint32_t scale2 = pack2(a.scale, a.scale);
  float4 rst[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) rst[r] = a.stat4[(long long)bh * a.T + row_lo + r * 8];
  float dq[NO][4];
#pragma unroll
  for (int i = 0; i < NO; ++i) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }
  const int nkb = qb + 1;
  for (int kb = 0; kb < nkb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < nkb) {
      load_tile<HD, 64, 128>(sK + (buf ^ 1) * 64 * ROWB, Kg + (long long)(kb + 1) * 64 * wqkn, wqkn);
      load_tile<HD, 64, 128>(sV + (buf ^ 1) * 64 * ROWB, Vg + (long long)(kb + 1) * 64 * wqkv, wqkv);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t cK = sK + buf * 64 * ROWB, cV = sV + buf * 64 * ROWB;
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t aq[4], ad[4];
      load_a<HD>(sQ, warp * 16, ks, aq);
      load_a<HD>(sDO, warp * 16, ks, ad);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bk[4], bv[4];
        load_b_nk<HD>(cK, np * 16, ks, bk);
        load_b_nk<HD>(cV, np * 16, ks, bv);
        mma16816(s[2 * np], aq[0], aq[1], aq[2], aq[3], bk[0], bk[1]);
        mma16816(s[2 * np + 1], aq[0], aq[1], aq[2], aq[3], bk[2], bk[3]);
        mma16816(dp[2 * np], ad[0], ad[1], ad[2], ad[3], bv[0], bv[1]);
        mma16816(dp[2 * np + 1], ad[0], ad[1], ad[2], ad[3], bv[2], bv[3]);
      }
    }
    const bool diag = (kb == nkb - 1);
    uint32_t DS2[8][2];                                      // packed pairs: [n-tile][row half]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int col = kb * 64 + nt * 8 + 2 * t;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const bool m0 = diag && (col > row_lo + r * 8), m1 = diag && (col + 1 > row_lo + r * 8);
        uint32_t p2;
        bwd_pair(s[nt][2 * r], s[nt][2 * r + 1], dp[nt][2 * r], dp[nt][2 * r + 1], scale2, rst[r], rst[r], m0, m1, p2, DS2[nt][r]);
      }
    }
    // dQ += dS K    (contraction over the 64 keys)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t a0 = DS2[2 * kk][0], a1 = DS2[2 * kk][1], a2 = DS2[2 * kk + 1][0], a3 = DS2[2 * kk + 1][1];
#pragma unroll
      for (int np = 0; np < KS; ++np) {
        uint32_t bk[4];
        load_b_kn<HD>(cK, kk * 16, 2 * np, bk);
        mma16816(dq[2 * np], a0, a1, a2, a3, bk[0], bk[1]);
        mma16816(dq[2 * np + 1], a0, a1, a2, a3, bk[2], bk[3]);
      }
    }
    __syncthreads();
  }
  bf16* dQg = (bf16*)a.dqkn + ((long long)b * a.T) * wqkn + h * HD;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_lo + r * 8;
#pragma unroll
    for (int nt = 0; nt < NO; ++nt)
      *reinterpret_cast<uint32_t*>(dQg + (long long)row * wqkn + nt * 8 + 2 * t) = adj_edge2(pack_bf16(dq[nt][2 * r], dq[nt][2 * r + 1]));
  }
}

template <int HD> struct FlashSmem {
  static constexpr int ROWB = HD * 2;
  static constexpr int FWD = 64 * ROWB + 4 * 64 * ROWB;                          // Q + 2x(K,V): 80 KB at HD = 128
  static constexpr int DKV = 2 * 128 * ROWB + 4 * 64 * ROWB + 2 * 64 * 16;       // K,V + 2x(Q,dO) + row records: 130 KB
  static constexpr int DQ = 2 * 64 * ROWB + 4 * 64 * ROWB;                       // Q,dO + 2x(K,V): 96 KB
};

template <int HD> cudaError_t set_attrs() {
  static bool attr[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr[dev]) {
    cudaError_t e = cudaFuncSetAttribute(k_flash_fwd<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem<HD>::FWD);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_flash_bwd_dkv<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem<HD>::DKV);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_flash_bwd_dq<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, FlashSmem<HD>::DQ);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr[dev] = true;
  }
  return cudaSuccess;
}

template <int HD> cudaError_t flash_fwd(cudaStream_t st, const FlashArgs& a) {
  cudaError_t e0 = set_attrs<HD>();
  if (e0 != cudaSuccess) return e0;
  dim3 grid(a.T / 64, a.B * a.H);
  k_flash_fwd<HD><<<grid, 128, FlashSmem<HD>::FWD, st>>>(a);
  return cudaGetLastError();
}

template <int HD> cudaError_t flash_bwd(cudaStream_t st, const FlashArgs& a) {
  cudaError_t e0 = set_attrs<HD>();
  if (e0 != cudaSuccess) return e0;
  const long long rows = (long long)a.B * a.H * a.T;
  k_flash_prep<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dim3 g1(a.T / 128, a.B * a.Hkv);
  k_flash_bwd_dkv<HD><<<g1, 256, FlashSmem<HD>::DKV, st>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dim3 g2(a.T / 64, a.B * a.H);
  k_flash_bwd_dq<HD><<<g2, 128, FlashSmem<HD>::DQ, st>>>(a);
  return cudaGetLastError();
}

}  // namespace

bool flash_supported(const FlashArgs& a) {
  return (a.hd == 128 || a.hd == 64 || a.hd == 32 || a.hd == 16) && a.T % 128 == 0 && a.T >= 128 && a.H % a.Hkv == 0 && a.B > 0 &&
         ((a.H * a.hd) % 8 == 0) && (long long)a.B * a.H <= 65535 && (long long)a.B * a.Hkv <= 65535;
}

cudaError_t launch_flash_fwd(cudaStream_t st, const FlashArgs& a) {
  switch (a.hd) {
    case 128: return flash_fwd<128>(st, a);
    case 64: return flash_fwd<64>(st, a);
    case 32: return flash_fwd<32>(st, a);
    default: return flash_fwd<16>(st, a);
  }
}

cudaError_t launch_flash_bwd(cudaStream_t st, const FlashArgs& a) {
  switch (a.hd) {
    case 128: return flash_bwd<128>(st, a);
    case 64: return flash_bwd<64>(st, a);
    case 32: return flash_bwd<32>(st, a);
    default: return flash_bwd<16>(st, a);
  }
}

cudaError_t adj_status_fetch_attn_flash(cudaStream_t st, int* out, bool clear) { return adj_status_fetch_tu(st, out, clear); }

}  // namespace pcpb
