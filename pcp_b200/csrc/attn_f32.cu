// Causal attention for f32 models with 16-, 32-, 64- or 128-wide heads (64: the nanoGPT-small fp32 configuration; the
// others: the shipped f32 graphs), forward and backward, tiled for the SIMT pipes.  The f32 models must stay f32-exact,
// so the score / probability / gradient tiles are f32 FMAs: 64 x 64 score tiles, 256 threads, a 4 x 4 register block per
// thread (4 x HD/16 for the head-dim-wide outputs), operands in shared memory in a k-major layout read with 16-byte
// loads.  They replace the one-block-per-query-row kernels of kernels.cu (k_attn_*_generic) for these shapes: those took
// 60 ms of the 135 ms nanoGPT-small step (one scalar dot product per thread and key, atomics in the backward).
//   forward   one CTA per (64 queries, batch, head): S = Q K^T per key tile, running row max / sum, O += P V,
//             O / (l + 1e-4) at the end.  f32 has no rounding between the ops of the graph, so normalising after the
//             sum is the graph's P = e / (l + 1e-4), O = P V up to the order of the f32 additions.
//   dQ        one CTA per (64 queries, batch, head);  dK, dV: one CTA per (64 keys, batch, kv head), which walks the
//             query heads of its group and the query tiles at or after it: no atomics, the result does not depend on
//             timing (the generic kernel adds into dK / dV with float atomics).
// Arithmetic of the backward as in k_attn_bwd_generic (kernels.cu): Pt = e / (l + 2e-4), dp = edge(dO . v),
// dsf = Pt (dp - D) - [s == max] D 2e-4 / (l + 2e-4), ds = edge(dsf * scale), outputs through the edge step; D is
// rowsum(dO * O) (l + 1e-4) / (l + 2e-4), which equals sum_j Pt_j dp_j while no dp is clamped (the tensor-core kernels
// use the same identity); a clamped dp or an out-of-range dsf sets ADJ_INTERNAL.
#define PCPB_ADJ_TU
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace pcpb {

namespace {

constexpr int TL = 64;                 // tile edge: queries and keys per tile
// k-major operand tile [k][W]: element (k, c) at k * W + (((c / 4) ^ (k % 8)) * 4 + c % 4) (for W < 32 the XOR uses
// fewer bits of k).  The XOR spreads the transposing stores (lanes along k, fixed c) over several bank groups; 16-byte
// reads of a 4-element group stay aligned.  W = 64 for tiles whose columns are queries or keys, W = HD for tiles whose
// columns are head-dim elements.
template <int W> __device__ __forceinline__ int swz(int k, int c) {
  constexpr int M = (W / 4 < 8 ? W / 4 : 8) - 1;
  return k * W + ((((c >> 2) ^ (k & M)) << 2) | (c & 3));
}

// acc[i][j] += sum_{k < KD} At(k, 4 ty + i) * Bt(k, 4 tx + j); both tiles 64 wide
template <int KD>
__device__ __forceinline__ void mm_s(const float* __restrict__ At, const float* __restrict__ Bt, int ty, int tx, float (&acc)[4][4]) {
#pragma unroll 8
  for (int k = 0; k < KD; ++k) {
    const float4 a = *reinterpret_cast<const float4*>(At + k * TL + ((ty ^ (k & 7)) << 2));
    const float4 b = *reinterpret_cast<const float4*>(Bt + k * TL + ((tx ^ (k & 7)) << 2));
    const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}
// acc[i][j] += sum_{k < 64} At(k, 4 ty + i) * Bt(k, NC tx + j): At 64 wide, Bt HD wide, NC = HD / 16 columns per thread
template <int HD>
__device__ __forceinline__ void mm_o(const float* __restrict__ At, const float* __restrict__ Bt, int ty, int tx, float (&acc)[4][HD / 16]) {
  constexpr int NC = HD / 16;
  constexpr int M = (HD / 4 < 8 ? HD / 4 : 8) - 1;
#pragma unroll 8
  for (int k = 0; k < TL; ++k) {
    const float4 a = *reinterpret_cast<const float4*>(At + k * TL + ((ty ^ (k & 7)) << 2));
    const float av[4] = {a.x, a.y, a.z, a.w};
    float bv[NC];
    const float* br = Bt + k * HD;
    if (NC >= 4) {
#pragma unroll
      for (int q = 0; q < NC / 4; ++q) {
        const float4 b = *reinterpret_cast<const float4*>(br + (((tx * (NC / 4) + q) ^ (k & M)) << 2));
        bv[(4 * q) % NC] = b.x; bv[(4 * q + 1) % NC] = b.y; bv[(4 * q + 2) % NC] = b.z; bv[(4 * q + 3) % NC] = b.w;
      }
    } else if (NC == 2) {
      const float2 b = *reinterpret_cast<const float2*>(br + ((((tx >> 1) ^ (k & M)) << 2) | ((tx & 1) << 1)));
      bv[0] = b.x; bv[1 % NC] = b.y;
    } else {
      bv[0] = br[(((tx >> 2) ^ (k & M)) << 2) | (tx & 3)];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

// 64 rows x HD columns of a row-major global matrix (row stride ld) into shared memory.
// TRANS: element (r, e) -> 64-wide tile (k = e, c = r);  else -> HD-wide tile (k = r, c = e).
template <bool TRANS, int HD>
__device__ __forceinline__ void load_tile(const float* __restrict__ g, long long ld, float* __restrict__ t) {
  for (int idx = threadIdx.x; idx < TL * HD; idx += 256) {
    const int r = idx / HD, e = idx % HD;
    const float v = g[(size_t)r * ld + e];
    t[TRANS ? swz<TL>(e, r) : swz<HD>(r, e)] = v;
  }
}
template <int N> __device__ __forceinline__ void zero4(float (&a)[4][N]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) a[i][j] = 0.f;
}
// NC consecutive floats of an output row
template <int NC> __device__ __forceinline__ void store_row(float* __restrict__ dst, const float (&v)[NC]) {
  if (NC % 4 == 0) {
#pragma unroll
    for (int q = 0; q < NC / 4; ++q)
      *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(v[(4 * q) % NC], v[(4 * q + 1) % NC], v[(4 * q + 2) % NC], v[(4 * q + 3) % NC]);
  } else if (NC == 2) {
    *reinterpret_cast<float2*>(dst) = make_float2(v[0], v[1 % NC]);
  } else {
    dst[0] = v[0];
  }
}
// reductions over the 16 threads (tx) that share a row: they are the low or the high half of a warp
__device__ __forceinline__ float max16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float sum16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct Dims {
  int d, dkv, wqkn, wqkv;
};
__device__ __forceinline__ Dims dims(const AttnArgs& a) {
  Dims x;
  x.d = a.H * a.hd; x.dkv = a.Hkv * a.hd; x.wqkn = x.d + x.dkv; x.wqkv = x.d + 2 * x.dkv;
  return x;
}

template <int HD>
__global__ void __launch_bounds__(256) k_attn_f32_fwd(AttnArgs a) {
  constexpr int NC = HD / 16;
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;                      // [HD][64]  (k = e, c = query)
  float* Kt = Qt + HD * TL;            // [HD][64]  (k = e, c = key)
  float* Vs = Kt + HD * TL;            // [64][HD]  (k = key, c = e)
  float* Pt = Vs + TL * HD;            // [64][64]  (k = key, c = query)
  const Dims x = dims(a);
  const int it = gridDim.x - 1 - blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H, hk = h / (a.H / a.Hkv);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float* qkn = (const float*)a.qkn;
  const float* qkv = (const float*)a.qkv;
  const size_t row0 = (size_t)b * a.T + (size_t)it * TL;
  load_tile<true, HD>(qkn + row0 * x.wqkn + h * HD, x.wqkn, Qt);
  float m[4], l[4], O[4][NC];
#pragma unroll
  for (int i = 0; i < 4; ++i) { m[i] = -INFINITY; l[i] = 0.f; }
  zero4(O);
  for (int jt = 0; jt <= it; ++jt) {
    const size_t key0 = (size_t)b * a.T + (size_t)jt * TL;
    __syncthreads();                                           // the previous tile's products are done
    load_tile<true, HD>(qkn + key0 * x.wqkn + x.d + hk * HD, x.wqkn, Kt);
    load_tile<false, HD>(qkv + key0 * x.wqkv + x.d + x.dkv + hk * HD, x.wqkv, Vs);
    __syncthreads();
    float S[4][4];
    zero4(S);
    mm_s<HD>(Qt, Kt, ty, tx, S);
    float p[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = ty * 4 + i;
      float tm = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool keep = jt < it || tx * 4 + j <= row;
        S[i][j] = keep ? S[i][j] * a.scale : -INFINITY;
        tm = fmaxf(tm, S[i][j]);
      }
      tm = max16(tm);
      const float mn = fmaxf(m[i], tm);                        // finite: the diagonal is never masked
      const float c = expf(m[i] - mn);                          // 0 for the first tile
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { p[i][j] = expf(S[i][j] - mn); rs += p[i][j]; }
      rs = sum16(rs);
      l[i] = l[i] * c + rs;
      m[i] = mn;
#pragma unroll
      for (int j = 0; j < NC; ++j) O[i][j] *= c;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = tx * 4 + j;
      *reinterpret_cast<float4*>(Pt + k * TL + ((ty ^ (k & 7)) << 2)) = make_float4(p[0][j], p[1][j], p[2][j], p[3][j]);
    }
    __syncthreads();
    mm_o<HD>(Pt, Vs, ty, tx, O);
  }
  float* o = (float*)a.o;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t row = row0 + ty * 4 + i;
    const float inv = 1.f / (l[i] + PCPB_GUARD);
    float v[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) v[j] = O[i][j] * inv;
    store_row<NC>(o + row * x.d + h * HD + tx * NC, v);
    if (tx == 0) {
      a.mrow[(size_t)bh * a.T + it * TL + ty * 4 + i] = m[i];
      a.lrow[(size_t)bh * a.T + it * TL + ty * 4 + i] = l[i];
    }
  }
}

// D per (batch, head, row): rowsum(dO * O) (l + 1e-4) / (l + 2e-4).  One warp per row.
__global__ void __launch_bounds__(256) k_attn_f32_prep(AttnArgs a, float* __restrict__ drow) {
  const Dims x = dims(a);
  const int w = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int total = a.B * a.H * a.T;
  if (w >= total) return;
  const int bh = w / a.T, i = w % a.T, b = bh / a.H, h = bh % a.H;
  const size_t row = (size_t)b * a.T + i;
  const float* o = (const float*)a.o + row * x.d + h * a.hd;
  const float* go = (const float*)a.dout + row * x.d + h * a.hd;
  float s = 0.f;
  for (int e = lane; e < a.hd; e += 32) s += o[e] * go[e];
  s = warp_sum(s);
  if (lane == 0) {
    const float l = a.lrow[w];
    drow[w] = s * (l + PCPB_GUARD) / (l + 2.f * PCPB_GUARD);
  }
}

// Gradient of one score tile: from S (raw dot products) and dP to Pf = e / (l + 1e-4) and dS, in place.
// masked entries give 0.  st: per-row statistics in shared memory [3][64]: max, l, D.
__device__ __forceinline__ void score_grad(const AttnArgs& a, bool diag, int ty, int tx, const float* __restrict__ st, float (&S)[4][4],
                                           float (&dP)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = ty * 4 + i;
    const float mx = st[row], l = st[TL + row], D = st[2 * TL + row];
    const float den1 = l + PCPB_GUARD, den2 = l + 2.f * PCPB_GUARD;
    const float mterm = D * (2.f * PCPB_GUARD) / den2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool keep = !diag || tx * 4 + j <= row;
      const float s = S[i][j] * a.scale;
      const float ex = keep ? expf(s - mx) : 0.f;
      const float dpr = dP[i][j];
      const float dp = adj_edge<float>(dpr);                   // dP: an output of the dot_general VJP
      if (keep && dp != dpr) adj_note(ADJ_INTERNAL);           // D was formed from the unclamped dP
      const float pt = ex / den2;
      const float dsf = pt * (dp - D) - ((keep && s == mx) ? mterm : 0.f);
      if (keep && !(fabsf(dsf) <= PCPB_ADJ_CLIP)) adj_note(ADJ_INTERNAL);
      S[i][j] = ex / den1;                                     // forward probability
      dP[i][j] = keep ? adj_edge<float>(dsf * a.scale) : 0.f;  // dS
    }
  }
}
__device__ __forceinline__ void load_stats(const AttnArgs& a, const float* __restrict__ drow, size_t base, float* __restrict__ st) {
  if (threadIdx.x < TL) {
    st[threadIdx.x] = a.mrow[base + threadIdx.x];
    st[TL + threadIdx.x] = a.lrow[base + threadIdx.x];
    st[2 * TL + threadIdx.x] = drow[base + threadIdx.x];
  }
}

template <int HD>
__global__ void __launch_bounds__(256) k_attn_f32_dq(AttnArgs a, const float* __restrict__ drow) {
  constexpr int NC = HD / 16;
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;                      // [HD][64]  (k = e, c = query)
  float* dOt = Qt + HD * TL;           // [HD][64]  (k = e, c = query)
  float* Kt = dOt + HD * TL;           // [HD][64]  (k = e, c = key)
  float* Vt = Kt + HD * TL;            // [HD][64]  (k = e, c = key)
  float* Ks = Vt + HD * TL;            // [64][HD]  (k = key, c = e)
  float* dSt = Ks + TL * HD;           // [64][64]  (k = key, c = query)
  float* st = dSt + TL * TL;           // [3][64]
  const Dims x = dims(a);
  const int it = gridDim.x - 1 - blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H, hk = h / (a.H / a.Hkv);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float* qkn = (const float*)a.qkn;
  const float* qkv = (const float*)a.qkv;
  const size_t row0 = (size_t)b * a.T + (size_t)it * TL;
  load_tile<true, HD>(qkn + row0 * x.wqkn + h * HD, x.wqkn, Qt);
  load_tile<true, HD>((const float*)a.dout + row0 * x.d + h * HD, x.d, dOt);
  load_stats(a, drow, (size_t)bh * a.T + (size_t)it * TL, st);
  float dQ[4][NC];
  zero4(dQ);
  for (int jt = 0; jt <= it; ++jt) {
    const size_t key0 = (size_t)b * a.T + (size_t)jt * TL;
    __syncthreads();
    load_tile<true, HD>(qkn + key0 * x.wqkn + x.d + hk * HD, x.wqkn, Kt);
    load_tile<false, HD>(qkn + key0 * x.wqkn + x.d + hk * HD, x.wqkn, Ks);
    load_tile<true, HD>(qkv + key0 * x.wqkv + x.d + x.dkv + hk * HD, x.wqkv, Vt);
    __syncthreads();
    float S[4][4], dP[4][4];
    zero4(S); zero4(dP);
    mm_s<HD>(Qt, Kt, ty, tx, S);
    mm_s<HD>(dOt, Vt, ty, tx, dP);
    score_grad(a, jt == it, ty, tx, st, S, dP);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = tx * 4 + j;
      *reinterpret_cast<float4*>(dSt + k * TL + ((ty ^ (k & 7)) << 2)) = make_float4(dP[0][j], dP[1][j], dP[2][j], dP[3][j]);
    }
    __syncthreads();
    mm_o<HD>(dSt, Ks, ty, tx, dQ);
  }
  float* dqkn = (float*)a.dqkn;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t row = row0 + ty * 4 + i;
    float v[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) v[j] = adj_edge<float>(dQ[i][j]);
    store_row<NC>(dqkn + row * x.wqkn + h * HD + tx * NC, v);
  }
}

template <int HD>
__global__ void __launch_bounds__(256) k_attn_f32_dkv(AttnArgs a, const float* __restrict__ drow) {
  constexpr int NC = HD / 16;
  extern __shared__ __align__(16) float sm[];
  float* Kt = sm;                      // [HD][64]  (k = e, c = key), resident
  float* Vt = Kt + HD * TL;            // [HD][64]  (k = e, c = key), resident
  float* Qt = Vt + HD * TL;            // [HD][64]  (k = e, c = query)
  float* dOt = Qt + HD * TL;           // [HD][64]  (k = e, c = query)
  float* Qs = dOt + HD * TL;           // [64][HD]  (k = query, c = e)
  float* dOs = Qs + TL * HD;           // [64][HD]  (k = query, c = e)
  float* Ps = dOs + TL * HD;           // [64][64]  (k = query, c = key)
  float* dSs = Ps + TL * TL;           // [64][64]  (k = query, c = key)
  float* st = dSs + TL * TL;           // [3][64]
  const Dims x = dims(a);
  const int jt = blockIdx.x, bhk = blockIdx.y, b = bhk / a.Hkv, hk = bhk % a.Hkv, grp = a.H / a.Hkv;
  const int nt = a.T / TL;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const float* qkn = (const float*)a.qkn;
  const float* qkv = (const float*)a.qkv;
  const size_t key0 = (size_t)b * a.T + (size_t)jt * TL;
  load_tile<true, HD>(qkn + key0 * x.wqkn + x.d + hk * HD, x.wqkn, Kt);
  load_tile<true, HD>(qkv + key0 * x.wqkv + x.d + x.dkv + hk * HD, x.wqkv, Vt);
  float dK[4][NC], dV[4][NC];
  zero4(dK); zero4(dV);
  for (int g = 0; g < grp; ++g) {
    const int h = hk * grp + g, bh = b * a.H + h;
    for (int it = jt; it < nt; ++it) {
      const size_t row0 = (size_t)b * a.T + (size_t)it * TL;
      __syncthreads();
      load_tile<true, HD>(qkn + row0 * x.wqkn + h * HD, x.wqkn, Qt);
      load_tile<false, HD>(qkn + row0 * x.wqkn + h * HD, x.wqkn, Qs);
      load_tile<true, HD>((const float*)a.dout + row0 * x.d + h * HD, x.d, dOt);
      load_tile<false, HD>((const float*)a.dout + row0 * x.d + h * HD, x.d, dOs);
      load_stats(a, drow, (size_t)bh * a.T + (size_t)it * TL, st);
      __syncthreads();
      float S[4][4], dP[4][4];
      zero4(S); zero4(dP);
      mm_s<HD>(Qt, Kt, ty, tx, S);                              // rows = queries, columns = keys, as in the other kernels
      mm_s<HD>(dOt, Vt, ty, tx, dP);
      score_grad(a, it == jt, ty, tx, st, S, dP);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int k = ty * 4 + i;
        *reinterpret_cast<float4*>(Ps + k * TL + ((tx ^ (k & 7)) << 2)) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
        *reinterpret_cast<float4*>(dSs + k * TL + ((tx ^ (k & 7)) << 2)) = make_float4(dP[i][0], dP[i][1], dP[i][2], dP[i][3]);
      }
      __syncthreads();
      mm_o<HD>(Ps, dOs, ty, tx, dV);                            // dV[key][e] += P[query][key] dO[query][e]
      mm_o<HD>(dSs, Qs, ty, tx, dK);                            // dK[key][e] += dS[query][key] Q[query][e]
    }
  }
  float* dqkn = (float*)a.dqkn;
  float* dqkv = (float*)a.dqkv;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const size_t row = key0 + ty * 4 + i;
    float vk[NC], vv[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) { vk[j] = adj_edge<float>(dK[i][j]); vv[j] = adj_edge<float>(dV[i][j]); }
    store_row<NC>(dqkn + row * x.wqkn + x.d + hk * HD + tx * NC, vk);
    store_row<NC>(dqkv + row * x.wqkv + x.d + x.dkv + hk * HD + tx * NC, vv);
  }
}

template <int HD> struct Smem {
  static constexpr size_t FWD = (size_t)(3 * HD * TL + TL * TL) * sizeof(float);
  static constexpr size_t DQ = (size_t)(5 * HD * TL + TL * TL + 3 * TL) * sizeof(float);
  static constexpr size_t DKV = (size_t)(6 * HD * TL + 2 * TL * TL + 3 * TL) * sizeof(float);
  static_assert(DKV <= 232448, "more shared memory than a CTA can have");
};

template <int HD> cudaError_t set_attrs() {
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(k_attn_f32_fwd<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<HD>::FWD);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_f32_dq<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<HD>::DQ);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_attn_f32_dkv<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<HD>::DKV);
  if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
  return e;
}

template <int HD> cudaError_t fwd(cudaStream_t st, const AttnArgs& a) {
  cudaError_t e = set_attrs<HD>();
  if (e != cudaSuccess) return e;
  k_attn_f32_fwd<HD><<<dim3(a.T / TL, a.B * a.H), 256, Smem<HD>::FWD, st>>>(a);
  return cudaGetLastError();
}
template <int HD> cudaError_t bwd(cudaStream_t st, const AttnArgs& a, float* drow) {
  cudaError_t e = set_attrs<HD>();
  if (e != cudaSuccess) return e;
  const int rows = a.B * a.H * a.T;
  k_attn_f32_prep<<<(rows + 7) / 8, 256, 0, st>>>(a, drow);
  k_attn_f32_dkv<HD><<<dim3(a.T / TL, a.B * a.Hkv), 256, Smem<HD>::DKV, st>>>(a, drow);
  k_attn_f32_dq<HD><<<dim3(a.T / TL, a.B * a.H), 256, Smem<HD>::DQ, st>>>(a, drow);
  return cudaGetLastError();
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

bool attn_f32_supported(int dt, const AttnArgs& a) {
  static int off = -1;
  if (off < 0) { const char* e = getenv("PCPB_ATTN_F32"); off = (e && !strcmp(e, "generic")) ? 1 : 0; }
  if (off || dt != DT_F32 || a.T % TL || a.B <= 0 || a.H % a.Hkv) return false;
  if (a.hd != 16 && a.hd != 32 && a.hd != 64 && a.hd != 128) return false;
  if ((long long)a.B * a.H > 65535) return false;
  // 16-byte accesses: every head starts on a 16-byte boundary in every buffer (row widths are multiples of 16 floats)
  return aligned16(a.qkn) && aligned16(a.qkv) && aligned16(a.o) && (!a.dout || aligned16(a.dout)) &&
         (!a.dqkn || aligned16(a.dqkn)) && (!a.dqkv || aligned16(a.dqkv));
}

cudaError_t launch_attn_f32_fwd(cudaStream_t st, const AttnArgs& a) {
  switch (a.hd) {
    case 128: return fwd<128>(st, a);
    case 64: return fwd<64>(st, a);
    case 32: return fwd<32>(st, a);
    default: return fwd<16>(st, a);
  }
}

// drow: f32 scratch of at least B * H * T elements
cudaError_t launch_attn_f32_bwd(cudaStream_t st, const AttnArgs& a, float* drow) {
  switch (a.hd) {
    case 128: return bwd<128>(st, a, drow);
    case 64: return bwd<64>(st, a, drow);
    case 32: return bwd<32>(st, a, drow);
    default: return bwd<16>(st, a, drow);
  }
}

cudaError_t adj_status_fetch_attn_f32(cudaStream_t st, int* out, bool clear) { return adj_status_fetch_tu(st, out, clear); }

}  // namespace pcpb
