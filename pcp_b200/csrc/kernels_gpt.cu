// Kernels specific to the nanoGPT model family (tools/generate_nanogpt_small.py,
// tools/generate_nanogpt_medium_bf16.py; graphs models/nanogpt_small.mlir, models/nanogpt_medium_bf16.mlir):
// learned position embedding, LayerNorm with scale and shift whose variance is computed in f64, lm_head bias.
//
// LayerNorm as exported (every divide carries the sanitiser's +1e-4, src/compiler/sanitizer.zig:8-111):
//   xf = f32(x);  mean64 = sum(f64(xf)) / (d + 1e-4);  var = f32( sum((f64(xf) - mean64)^2) / (d + 1e-4) )
//   mean = sum(xf) / (f32(d) + 1e-4);  r = rsqrt(var + 1e-5);  y = T( (xf - mean) * r * gamma + beta )
// Backward through the same ops with the VJP rules' own guards (src/autodiff/vjp_rules.zig:154,1529):
//   dxhat = dy * gamma;  dc = dxhat * r;  dr = sum(dxhat * (xf - mean));  dt = -0.5 dr rsqrt(t + 1e-4)^3
//   f64 branch: dS2 = dt / (d + 2e-4);  dc64 = 2 dS2 c64;  dmean64 = -sum(dc64);  dx64 = dc64 + dmean64 / (d + 2e-4)
//   f32 branch: dmean = -sum(dc);  dx = dc + dmean / (f32(d) + 2e-4) + f32(dx64)
#define PCPB_ADJ_TU
#include "common.cuh"
#include "kernels.h"

namespace pcpb {

#define DISPATCH_DT(dt, ...)                                   \
  do {                                                         \
    if ((dt) == DT_F32) { typedef float T; __VA_ARGS__; }      \
    else if ((dt) == DT_BF16) { typedef bf16 T; __VA_ARGS__; } \
    else return cudaErrorInvalidValue;                         \
  } while (0)

static inline unsigned cdiv(size_t a, size_t b) { return (unsigned)((a + b - 1) / b); }

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- token + position embedding ----------------------------------------------------------------------
template <typename T>
__global__ void k_embed_pos_fwd(const T* __restrict__ wte, const T* __restrict__ wpe, const long long* __restrict__ idx,
                                int M, int Tlen, int d, int V, T* __restrict__ x) {
  const size_t n = (size_t)M * d;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / d), j = (int)(i % d);
    long long row = idx[m];
    row = row < 0 ? 0 : (row >= V ? V - 1 : row);
    x[i] = from_f<T>(to_f(wte[(size_t)row * d + j]) + to_f(wpe[(size_t)(m % Tlen) * d + j]));
  }
}
// dwte[idx[m]] += dx[m] (atomic, f32);  dwpe[t] = sum_b dx[b*T + t] (in batch order)
template <typename T>
__global__ void k_embed_pos_bwd(const long long* __restrict__ idx, int B, int Tlen, int d, int V, const T* __restrict__ dx,
                                float* __restrict__ dwte, float* __restrict__ dwpe) {
  const size_t n = (size_t)Tlen * d;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / d), j = (int)(i % d);
    float acc = 0.f;
    for (int b = 0; b < B; ++b) {
      const size_t m = (size_t)b * Tlen + t;
      const float g = to_f(dx[m * d + j]);
      acc += g;
      if (dwte) {                                             // else: summed per token by launch_embed_scatter_sorted
        long long row = idx[m];
        row = row < 0 ? 0 : (row >= V ? V - 1 : row);
        atomicAdd(dwte + (size_t)row * d + j, g);
      }
    }
    dwpe[i] = acc;
  }
}
cudaError_t launch_embed_pos_fwd(cudaStream_t st, int dt, const void* wte, const void* wpe, const long long* idx, int M,
                                 int Tlen, int d, int V, void* x) {
  if (M == 0) return cudaSuccess;
  DISPATCH_DT(dt, (k_embed_pos_fwd<T><<<min(cdiv((size_t)M * d, 256), 148u * 8), 256, 0, st>>>((const T*)wte, (const T*)wpe,
                                                                                             idx, M, Tlen, d, V, (T*)x)));
  return cudaGetLastError();
}
cudaError_t launch_embed_pos_bwd(cudaStream_t st, int dt, const long long* idx, int B, int Tlen, int d, int V, const void* dx,
                                 float* dwte, float* dwpe) {
  if (B == 0) return cudaSuccess;
  DISPATCH_DT(dt, (k_embed_pos_bwd<T><<<min(cdiv((size_t)Tlen * d, 256), 148u * 8), 256, 0, st>>>(idx, B, Tlen, d, V,
                                                                                               (const T*)dx, dwte, dwpe)));
  return cudaGetLastError();
}

// ---- LayerNorm forward: one warp per row -----------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) k_layernorm_fwd(const T* __restrict__ x, const T* __restrict__ gamma,
                                                       const T* __restrict__ beta, int M, int d, T* __restrict__ y,
                                                       float* __restrict__ mean_out, float* __restrict__ t_out,
                                                       double* __restrict__ mean64_out) {
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (m >= M) return;
  const T* xr = x + (size_t)m * d;
  float s32 = 0.f;
  double s64 = 0.0;
  for (int j = lane; j < d; j += 32) { const float v = to_f(xr[j]); s32 += v; s64 += (double)v; }
  s32 = warp_sum(s32);
  s64 = warp_sum_d(s64);
  const double dd = (double)d + 1e-4;
  const double mean64 = s64 / dd;
  double v64 = 0.0;
  for (int j = lane; j < d; j += 32) { const double c = (double)to_f(xr[j]) - mean64; v64 += c * c; }
  v64 = warp_sum_d(v64) / dd;
  const float var = (float)v64;
  const float mean = s32 / ((float)d + PCPB_GUARD);
  const float t = var + 1e-5f;
  const float r = rsqrtf(t);
  if (lane == 0) { mean_out[m] = mean; t_out[m] = t; mean64_out[m] = mean64; }
  T* yr = y + (size_t)m * d;
  for (int j = lane; j < d; j += 32)
    yr[j] = from_f<T>(((to_f(xr[j]) - mean) * r) * to_f(gamma[j]) + to_f(beta[j]));
}
// Vectorised variant for d = 256 * NCH: a lane owns 8 consecutive columns of every 256-column chunk and keeps the row
// in registers over the three passes (one 16-byte read per chunk); arithmetic per element as above.
template <typename T, int NCH>
__global__ void __launch_bounds__(256) k_layernorm_fwd_vec(const T* __restrict__ x, const T* __restrict__ gamma,
                                                           const T* __restrict__ beta, int M, T* __restrict__ y,
                                                           float* __restrict__ mean_out, float* __restrict__ t_out,
                                                           double* __restrict__ mean64_out) {
  constexpr int d = 256 * NCH;
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (m >= M) return;
  const T* xr = x + (size_t)m * d;
  float xv[NCH][8];
#pragma unroll
  for (int k = 0; k < NCH; ++k) ld8<T>(xr + k * 256 + lane * 8, xv[k]);
  float s32 = 0.f;
  double s64 = 0.0;
#pragma unroll
  for (int k = 0; k < NCH; ++k)
#pragma unroll
    for (int e = 0; e < 8; ++e) { s32 += xv[k][e]; s64 += (double)xv[k][e]; }
  s32 = warp_sum(s32);
  s64 = warp_sum_d(s64);
  const double dd = (double)d + 1e-4;
  const double mean64 = s64 / dd;
  double v64 = 0.0;
#pragma unroll
  for (int k = 0; k < NCH; ++k)
#pragma unroll
    for (int e = 0; e < 8; ++e) { const double c = (double)xv[k][e] - mean64; v64 += c * c; }
  v64 = warp_sum_d(v64) / dd;
  const float var = (float)v64;
  const float mean = s32 / ((float)d + PCPB_GUARD);
  const float t = var + 1e-5f;
  const float r = rsqrtf(t);
  if (lane == 0) { mean_out[m] = mean; t_out[m] = t; mean64_out[m] = mean64; }
  T* yr = y + (size_t)m * d;
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    float g[8], bt[8], o[8];
    ld8<T>(gamma + k * 256 + lane * 8, g);
    ld8<T>(beta + k * 256 + lane * 8, bt);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = ((xv[k][e] - mean) * r) * g[e] + bt[e];
    st8<T>(yr + k * 256 + lane * 8, o);
  }
}
cudaError_t launch_layernorm_fwd(cudaStream_t st, int dt, const void* x, const void* gamma, const void* beta, int M, int d,
                                 void* y, float* mean, float* tsave, double* mean64) {
  if (M == 0) return cudaSuccess;
  const bool aligned = ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)gamma) | ((uintptr_t)beta)) & 31) == 0;
#define PCPB_LNF_VEC(NCH)                                                                                              \
  if (aligned && d == 256 * NCH) {                                                                                     \
    DISPATCH_DT(dt, (k_layernorm_fwd_vec<T, NCH><<<cdiv(M, 8), 256, 0, st>>>((const T*)x, (const T*)gamma, (const T*)beta, M, \
                                                                            (T*)y, mean, tsave, mean64)));             \
    return cudaGetLastError();                                                                                         \
  }
  PCPB_LNF_VEC(1) PCPB_LNF_VEC(2) PCPB_LNF_VEC(3) PCPB_LNF_VEC(4)
#undef PCPB_LNF_VEC
  DISPATCH_DT(dt, (k_layernorm_fwd<T><<<cdiv(M, 8), 256, 0, st>>>((const T*)x, (const T*)gamma, (const T*)beta, M, d, (T*)y,
                                                                  mean, tsave, mean64)));
  return cudaGetLastError();
}

// ---- LayerNorm backward ----------------------------------------------------------------------------------
// Block = 8 warps, LN_ROWS rows per block (one warp per row at a time).  Each warp keeps the column sums of
// dgamma / dbeta over the rows it handled in its own shared-memory slice (a lane owns columns lane + 32 k); the
// 8 slices are combined and written as one partial per block.
constexpr int LN_ROWS = 64;
// The generic kernel (widths that are not a multiple of 256, e.g. 384) has no loads in flight beyond the row a warp works
// on, so it wants many resident warps instead: 16 rows per block (two per warp), 1024 blocks at 16384 rows.  With 64 rows
// per block it took 148 us per launch at [16384, 384] f32 (100 MB of traffic: 15 us at the copy bandwidth).
constexpr int LN_ROWS_GENERIC = 16;

template <typename T>
__global__ void __launch_bounds__(256) k_layernorm_bwd(const T* __restrict__ x, const T* __restrict__ gamma,
                                                       const float* __restrict__ mean_in, const float* __restrict__ t_in,
                                                       const double* __restrict__ mean64_in, const T* __restrict__ dy,
                                                       const T* __restrict__ dres, int M, int d, T* __restrict__ dx,
                                                       float* __restrict__ partial, int rows_per_block) {
  extern __shared__ float sm[];                  // [8 warps][2][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nc = (d + 31) / 32;
  float* dgw = sm + (size_t)(warp * 2 + 0) * d;     // this warp's column sums; lane owns columns lane + 32 k
  float* dbw = sm + (size_t)(warp * 2 + 1) * d;
  for (int j = lane; j < d; j += 32) { dgw[j] = 0.f; dbw[j] = 0.f; }
  const double dd2 = ((double)d + 1e-4) + 1e-4;
  const float df2 = ((float)d + PCPB_GUARD) + PCPB_GUARD;
  for (int rr = warp; rr < rows_per_block; rr += 8) {
    const int m = blockIdx.x * rows_per_block + rr;
    if (m >= M) break;
    const T* xr = x + (size_t)m * d; const T* dyr = dy + (size_t)m * d;
    const float mean = mean_in[m], t = t_in[m], r = rsqrtf(t);
    const double mean64 = mean64_in[m];
    float A = 0.f, Bc = 0.f;
    double C64 = 0.0;
    for (int k = 0; k < nc; ++k) {
      const int j = lane + 32 * k;
      if (j < d) {
        const float xv = to_f(xr[j]), g = to_f(dyr[j]);
        const float dxh = g * to_f(gamma[j]);
        A += dxh * (xv - mean);
        Bc += dxh * r;
        C64 += (double)xv - mean64;
        dgw[j] += g * ((xv - mean) * r);
        dbw[j] += g;
      }
    }
    A = warp_sum(A); Bc = warp_sum(Bc); C64 = warp_sum_d(C64);
    const float rp = rsqrtf(t + PCPB_GUARD);
    const float dtv = adj_edge<float>((A * -0.5f) * ((rp * rp) * rp));      // rsqrt VJP output: an adjoint edge
    const double dS2 = (double)dtv / dd2;
    const double dsum64 = (-2.0 * dS2 * C64) / dd2;
    const float dsum32 = (-Bc) / df2;
    for (int k = 0; k < nc; ++k) {
      const int j = lane + 32 * k;
      if (j < d) {
        const float xv = to_f(xr[j]);
        const float dc = (to_f(dyr[j]) * to_f(gamma[j])) * r;
        const double dx64 = 2.0 * dS2 * ((double)xv - mean64) + dsum64;
        // the three contributions are edges of the f32 statistics graph, their sum crosses the f32 -> T convert edge
        float o = adj_edge<float>(dc) + adj_edge<float>(dsum32) + adj_edge<float>((float)dx64);
        o = adj_edge<T>(o);
        if (dres) o += to_f(dres[(size_t)m * d + j]);
        dx[(size_t)m * d + j] = from_f<T>(o);
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) {
    const int which = i / d, j = i % d;
    float acc = 0.f;
    for (int w = 0; w < 8; ++w) acc += sm[(w * 2 + which) * d + j];
    partial[((size_t)blockIdx.x * 2 + which) * d + j] = acc;
  }
}
// Vectorised variant for d = 256 * NCH (NCH <= 4): a lane owns 8 consecutive columns of every 256-column chunk, reads
// x and dy once with 16-byte loads and keeps them in registers between the statistics pass and the output pass; the
// per-element arithmetic is that of k_layernorm_bwd.
template <typename T, int NCH>
__global__ void __launch_bounds__(256) k_layernorm_bwd_vec(const T* __restrict__ x, const T* __restrict__ gamma,
                                                           const float* __restrict__ mean_in, const float* __restrict__ t_in,
                                                           const double* __restrict__ mean64_in, const T* __restrict__ dy,
                                                           const T* __restrict__ dres, int M, T* __restrict__ dx,
                                                           float* __restrict__ partial) {
  constexpr int d = 256 * NCH;
  extern __shared__ float sm[];                  // [8 warps][2][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* dgw = sm + (size_t)(warp * 2 + 0) * d;
  float* dbw = sm + (size_t)(warp * 2 + 1) * d;
  for (int j = lane; j < d; j += 32) { dgw[j] = 0.f; dbw[j] = 0.f; }
  __syncwarp();
  const double dd2 = ((double)d + 1e-4) + 1e-4;
  const float df2 = ((float)d + PCPB_GUARD) + PCPB_GUARD;
  float gam[NCH][8];
#pragma unroll
  for (int k = 0; k < NCH; ++k) ld8<T>(gamma + k * 256 + lane * 8, gam[k]);
  for (int rr = warp; rr < LN_ROWS; rr += 8) {
    const int m = blockIdx.x * LN_ROWS + rr;
    if (m >= M) break;
    const T* xr = x + (size_t)m * d; const T* dyr = dy + (size_t)m * d;
    const float mean = mean_in[m], t = t_in[m], r = rsqrtf(t);
    const double mean64 = mean64_in[m];
    float xv[NCH][8], g[NCH][8];
#pragma unroll
    for (int k = 0; k < NCH; ++k) { ld8<T>(xr + k * 256 + lane * 8, xv[k]); ld8<T>(dyr + k * 256 + lane * 8, g[k]); }
    float A = 0.f, Bc = 0.f;
    double C64 = 0.0;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      float4* pg = reinterpret_cast<float4*>(dgw + k * 256 + lane * 8);
      float4* pb = reinterpret_cast<float4*>(dbw + k * 256 + lane * 8);
      float ag[8], ab[8];
      *reinterpret_cast<float4*>(ag) = pg[0]; *reinterpret_cast<float4*>(ag + 4) = pg[1];
      *reinterpret_cast<float4*>(ab) = pb[0]; *reinterpret_cast<float4*>(ab + 4) = pb[1];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float dxh = g[k][e] * gam[k][e];
        A += dxh * (xv[k][e] - mean);
        Bc += dxh * r;
        C64 += (double)xv[k][e] - mean64;
        ag[e] += g[k][e] * ((xv[k][e] - mean) * r);
        ab[e] += g[k][e];
      }
      pg[0] = *reinterpret_cast<float4*>(ag); pg[1] = *reinterpret_cast<float4*>(ag + 4);
      pb[0] = *reinterpret_cast<float4*>(ab); pb[1] = *reinterpret_cast<float4*>(ab + 4);
    }
    A = warp_sum(A); Bc = warp_sum(Bc); C64 = warp_sum_d(C64);
    const float rp = rsqrtf(t + PCPB_GUARD);
    const float dtv = adj_edge<float>((A * -0.5f) * ((rp * rp) * rp));      // rsqrt VJP output: an adjoint edge
    const double dS2 = (double)dtv / dd2;
    const double dsum64 = (-2.0 * dS2 * C64) / dd2;
    const float dsum32 = (-Bc) / df2;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      float o[8], res[8];
      if (dres) ld8<T>(dres + (size_t)m * d + k * 256 + lane * 8, res);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float dc = (g[k][e] * gam[k][e]) * r;
        const double dx64 = 2.0 * dS2 * ((double)xv[k][e] - mean64) + dsum64;
        o[e] = adj_edge<T>(adj_edge<float>(dc) + adj_edge<float>(dsum32) + adj_edge<float>((float)dx64));
        if (dres) o[e] += res[e];
      }
      st8<T>(dx + (size_t)m * d + k * 256 + lane * 8, o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) {
    const int which = i / d, j = i % d;
    float acc = 0.f;
    for (int w = 0; w < 8; ++w) acc += sm[(w * 2 + which) * d + j];
    partial[((size_t)blockIdx.x * 2 + which) * d + j] = acc;
  }
}
// bf16 form of the vectorised kernel: x, dy and gamma stay packed (four registers per eight elements), so a warp can hold
// the next row's x and dy, fetched before the current row is worked on, beside the current one.
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float (&f)[8]) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}
template <int NCH>
__global__ void __launch_bounds__(256) k_layernorm_bwd_bf16(const bf16* __restrict__ x, const bf16* __restrict__ gamma,
                                                            const float* __restrict__ mean_in, const float* __restrict__ t_in,
                                                            const double* __restrict__ mean64_in, const bf16* __restrict__ dy,
                                                            const bf16* __restrict__ dres, int M, bf16* __restrict__ dx,
                                                            float* __restrict__ partial) {
  constexpr int d = 256 * NCH;
  extern __shared__ float sm[];                  // [8 warps][2][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* dgw = sm + (size_t)(warp * 2 + 0) * d;
  float* dbw = sm + (size_t)(warp * 2 + 1) * d;
  for (int j = lane; j < d; j += 32) { dgw[j] = 0.f; dbw[j] = 0.f; }
  __syncwarp();
  const double dd2 = ((double)d + 1e-4) + 1e-4;
  const float df2 = ((float)d + PCPB_GUARD) + PCPB_GUARD;
  uint4 gam[NCH], nx[NCH], ny[NCH];
#pragma unroll
  for (int k = 0; k < NCH; ++k) gam[k] = *reinterpret_cast<const uint4*>(gamma + k * 256 + lane * 8);
  const int m_first = blockIdx.x * LN_ROWS + warp;
  if (m_first < M) {
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      nx[k] = *reinterpret_cast<const uint4*>(x + (size_t)m_first * d + k * 256 + lane * 8);
      ny[k] = *reinterpret_cast<const uint4*>(dy + (size_t)m_first * d + k * 256 + lane * 8);
    }
  }
  for (int rr = warp; rr < LN_ROWS; rr += 8) {
    const int m = blockIdx.x * LN_ROWS + rr;
    if (m >= M) break;
    uint4 cx[NCH], cy[NCH];
#pragma unroll
    for (int k = 0; k < NCH; ++k) { cx[k] = nx[k]; cy[k] = ny[k]; }
    const int mn = m + 8;
    if (rr + 8 < LN_ROWS && mn < M) {
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        nx[k] = *reinterpret_cast<const uint4*>(x + (size_t)mn * d + k * 256 + lane * 8);
        ny[k] = *reinterpret_cast<const uint4*>(dy + (size_t)mn * d + k * 256 + lane * 8);
      }
    }
    const float mean = mean_in[m], t = t_in[m], r = rsqrtf(t);
    const double mean64 = mean64_in[m];
    float A = 0.f, Bc = 0.f;
    double C64 = 0.0;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      float xv[8], g[8], gm[8];
      unpack_bf16x8(cx[k], xv); unpack_bf16x8(cy[k], g); unpack_bf16x8(gam[k], gm);
      float4* pg = reinterpret_cast<float4*>(dgw + k * 256 + lane * 8);
      float4* pb = reinterpret_cast<float4*>(dbw + k * 256 + lane * 8);
      float ag[8], ab[8];
      *reinterpret_cast<float4*>(ag) = pg[0]; *reinterpret_cast<float4*>(ag + 4) = pg[1];
      *reinterpret_cast<float4*>(ab) = pb[0]; *reinterpret_cast<float4*>(ab + 4) = pb[1];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float dxh = g[e] * gm[e];
        A += dxh * (xv[e] - mean);
        Bc += dxh * r;
        C64 += (double)xv[e] - mean64;
        ag[e] += g[e] * ((xv[e] - mean) * r);
        ab[e] += g[e];
      }
      pg[0] = *reinterpret_cast<float4*>(ag); pg[1] = *reinterpret_cast<float4*>(ag + 4);
      pb[0] = *reinterpret_cast<float4*>(ab); pb[1] = *reinterpret_cast<float4*>(ab + 4);
    }
    A = warp_sum(A); Bc = warp_sum(Bc); C64 = warp_sum_d(C64);
    const float rp = rsqrtf(t + PCPB_GUARD);
    const float dtv = adj_edge<float>((A * -0.5f) * ((rp * rp) * rp));      // rsqrt VJP output: an adjoint edge
    const double dS2 = (double)dtv / dd2;
    const double dsum64 = (-2.0 * dS2 * C64) / dd2;
    const float dsum32 = (-Bc) / df2;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      float xv[8], g[8], gm[8], o[8], res[8];
      unpack_bf16x8(cx[k], xv); unpack_bf16x8(cy[k], g); unpack_bf16x8(gam[k], gm);
      if (dres) ld8<bf16>(dres + (size_t)m * d + k * 256 + lane * 8, res);
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        const float dc0 = (g[e] * gm[e]) * r, dc1 = (g[e + 1] * gm[e + 1]) * r;
        const double a0 = 2.0 * dS2 * ((double)xv[e] - mean64) + dsum64, a1 = 2.0 * dS2 * ((double)xv[e + 1] - mean64) + dsum64;
        const uint32_t o2 = adj_edge2(pack2(dc0 + dsum32 + (float)a0, dc1 + dsum32 + (float)a1));      // the bf16 rounding of dx, as an adjoint edge
        o[e] = bf_lo(o2); o[e + 1] = bf_hi(o2);
        if (dres) { o[e] += res[e]; o[e + 1] += res[e + 1]; }
      }
      st8<bf16>(dx + (size_t)m * d + k * 256 + lane * 8, o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) {
    const int which = i / d, j = i % d;
    float acc = 0.f;
    for (int w = 0; w < 8; ++w) acc += sm[(w * 2 + which) * d + j];
    partial[((size_t)blockIdx.x * 2 + which) * d + j] = acc;
  }
}
// dgamma[j], dbeta[j] = sum over blocks (in block order), rounded to the model dtype, finite-guarded, clamped
// Block = 32 columns x 8 row groups: a thread sums the partials b = group, group + 8, ... in that order, the eight group
// sums are added in group order (a fixed summation tree: deterministic).
template <typename T>
__global__ void __launch_bounds__(256) k_ln_param_grads(const float* __restrict__ partial, int nblk, int d,
                                                        float* __restrict__ dgamma, float* __restrict__ dbeta, float clip) {
  __shared__ float sm[8][33];
  const int col = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + col;                       // over 2 * d columns: dgamma then dbeta
  float acc = 0.f;
  if (i < 2 * d) {
    const int which = i / d, j = i % d;
    for (int b = grp; b < nblk; b += 8) acc += partial[((size_t)b * 2 + which) * d + j];
  }
  sm[grp][col] = acc;
  __syncthreads();
  if (grp == 0 && i < 2 * d) {
    float tot = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) tot += sm[g][col];
    float v = rnd<T>(tot);
    if (!((v - v) == 0.f)) v = 0.f;
    v = fminf(fmaxf(v, -clip), clip);
    (i / d == 0 ? dgamma : dbeta)[i % d] = v;
  }
}
size_t layernorm_bwd_scratch_floats(int M, int d) { return (size_t)((M + LN_ROWS_GENERIC - 1) / LN_ROWS_GENERIC) * 2 * d; }

cudaError_t launch_layernorm_bwd(cudaStream_t st, int dt, const void* x, const void* gamma, const float* mean,
                                 const float* tsave, const double* mean64, const void* dy, const void* dres, int M, int d,
                                 void* dx, float* partial, float* dgamma, float* dbeta) {
  if (M == 0) return cudaSuccess;
  if ((size_t)8 * 2 * d * sizeof(float) > 200 * 1024) return cudaErrorInvalidValue;
  int nblk = (M + LN_ROWS - 1) / LN_ROWS;
  const size_t smem = (size_t)8 * 2 * d * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = (dt == DT_F32)
        ? cudaFuncSetAttribute(k_layernorm_bwd<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : cudaFuncSetAttribute(k_layernorm_bwd<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  const bool aligned = ((((uintptr_t)x) | ((uintptr_t)dy) | ((uintptr_t)dx) | ((uintptr_t)gamma) | ((uintptr_t)dres)) & 31) == 0;
  bool done = false;
#define PCPB_LN_VEC(NCH)                                                                                                  \
  if (!done && aligned && d == 256 * NCH) {                                                                               \
    if (smem > 48 * 1024) {                                                                                               \
      cudaError_t ea = (dt == DT_F32)                                                                                     \
          ? cudaFuncSetAttribute(k_layernorm_bwd_vec<float, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) \
          : cudaFuncSetAttribute(k_layernorm_bwd_vec<bf16, NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (ea != cudaSuccess) return ea;                                                                                   \
    }                                                                                                                     \
    DISPATCH_DT(dt, (k_layernorm_bwd_vec<T, NCH><<<nblk, 256, smem, st>>>((const T*)x, (const T*)gamma, mean, tsave, mean64, \
                                                                         (const T*)dy, (const T*)dres, M, (T*)dx, partial))); \
    done = true;                                                                                                          \
  }
#define PCPB_LN_BF16(NCH)                                                                                                 \
  if (!done && aligned && dt == DT_BF16 && d == 256 * NCH) {                                                              \
    if (smem > 48 * 1024) {                                                                                               \
      cudaError_t ea = cudaFuncSetAttribute(k_layernorm_bwd_bf16<NCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (ea != cudaSuccess) return ea;                                                                                   \
    }                                                                                                                     \
    k_layernorm_bwd_bf16<NCH><<<nblk, 256, smem, st>>>((const bf16*)x, (const bf16*)gamma, mean, tsave, mean64, (const bf16*)dy, \
                                                       (const bf16*)dres, M, (bf16*)dx, partial);                        \
    done = true;                                                                                                          \
  }
  PCPB_LN_BF16(1) PCPB_LN_BF16(2) PCPB_LN_BF16(3) PCPB_LN_BF16(4)
#undef PCPB_LN_BF16
  PCPB_LN_VEC(1) PCPB_LN_VEC(2) PCPB_LN_VEC(3) PCPB_LN_VEC(4)
#undef PCPB_LN_VEC
  if (!done) {
    nblk = (M + LN_ROWS_GENERIC - 1) / LN_ROWS_GENERIC;
    DISPATCH_DT(dt, (k_layernorm_bwd<T><<<nblk, 256, smem, st>>>((const T*)x, (const T*)gamma, mean, tsave, mean64,
                                                                 (const T*)dy, (const T*)dres, M, d, (T*)dx, partial, LN_ROWS_GENERIC)));
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  DISPATCH_DT(dt, (k_ln_param_grads<T><<<cdiv(2 * d, 32), 256, 0, st>>>(partial, nblk, d, dgamma, dbeta, 100.f)));
  return cudaGetLastError();
}

// ---- column sum of a [M, V] matrix (lm_head bias gradient): per-block partials, then an ordered reduction ----
constexpr int CS_ROWS = 256;
template <typename T>
__global__ void k_colsum_partial(const T* __restrict__ z, int M, int V, float* __restrict__ partial) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= V) return;
  const int m0 = blockIdx.y * CS_ROWS, m1 = min(m0 + CS_ROWS, M);
  float acc = 0.f;
  for (int m = m0; m < m1; ++m) acc += to_f(z[(size_t)m * V + v]);
  partial[(size_t)blockIdx.y * V + v] = acc;
}
template <typename T>
__global__ void k_colsum_final(const float* __restrict__ partial, int nblk, int V, float* __restrict__ out, float clip) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= V) return;
  float acc = 0.f;
  for (int b = 0; b < nblk; ++b) acc += partial[(size_t)b * V + v];
  float r = rnd<T>(acc);
  if (!((r - r) == 0.f)) r = 0.f;
  out[v] = fminf(fmaxf(r, -clip), clip);
}
size_t colsum_scratch_floats(int M, int V) { return (size_t)((M + CS_ROWS - 1) / CS_ROWS) * V; }
cudaError_t launch_colsum(cudaStream_t st, int dt, const void* z, int M, int V, float* partial, float* out) {
  if (M == 0 || V == 0) return cudaSuccess;
  const int nblk = (M + CS_ROWS - 1) / CS_ROWS;
  dim3 grid(cdiv(V, 128), nblk);
  DISPATCH_DT(dt, (k_colsum_partial<T><<<grid, 128, 0, st>>>((const T*)z, M, V, partial)));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  DISPATCH_DT(dt, (k_colsum_final<T><<<cdiv(V, 128), 128, 0, st>>>(partial, nblk, V, out, 100.f)));
  return cudaGetLastError();
}

// ---- strided 2-D copy (q|k columns between the qkv and qkn layouts) --------------------------------------
template <typename T>
__global__ void k_copy_cols(const T* __restrict__ src, long long sp, T* __restrict__ dst, long long dp, int M, int ncols) {
  const size_t n = (size_t)M * ncols;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / ncols, c = i % ncols;
    dst[m * dp + c] = src[m * sp + c];
  }
}
// the same in 16-byte words (pitches, width and base addresses multiples of 16 bytes)
__global__ void k_copy_cols16(const uint4* __restrict__ src, long long sp, uint4* __restrict__ dst, long long dp, int M, int nw) {
  const size_t n = (size_t)M * nw;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / nw, c = i % nw;
    dst[m * dp + c] = src[m * sp + c];
  }
}
cudaError_t launch_copy_cols(cudaStream_t st, int dt, const void* src, long long src_pitch, void* dst, long long dst_pitch,
                             int M, int ncols) {
  if (M == 0 || ncols == 0) return cudaSuccess;
  const size_t es = (dt == DT_F32) ? 4 : 2, per = 16 / es;
  if (ncols % per == 0 && src_pitch % per == 0 && dst_pitch % per == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
    const int nw = (int)(ncols / per);
    k_copy_cols16<<<min(cdiv((size_t)M * nw, 256), 148u * 16), 256, 0, st>>>((const uint4*)src, src_pitch / (long long)per, (uint4*)dst,
                                                                             dst_pitch / (long long)per, M, nw);
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_copy_cols<T><<<min(cdiv((size_t)M * ncols, 256), 148u * 8), 256, 0, st>>>((const T*)src, src_pitch, (T*)dst,
                                                                                            dst_pitch, M, ncols)));
  return cudaGetLastError();
}

cudaError_t adj_status_fetch_kernels_gpt(cudaStream_t st, int* out, bool clear) { return adj_status_fetch_tu(st, out, clear); }

}  // namespace pcpb
