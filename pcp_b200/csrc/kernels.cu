// Training-step kernels, generic path: correct for every shape and both model dtypes (f32, bf16).
// The tensor-core kernels in gemm_tc.cu / attn_tc.cu take over for bf16 shapes they support.
//
// Numerical contract (what the reference's compiled graph computes; see the file:line notes):
//  * values of model dtype are rounded per op exactly where the exported graph has an op of that
//    type (models/nanochat_d8_b8_t2048_bf16.mlir), statistics / softmax / loss are f32;
//  * forward divides and logs carry +1e-4 (src/compiler/sanitizer.zig:8-111), the divide / log /
//    rsqrt VJP rules carry another +1e-4 (src/autodiff/vjp_rules.zig:198,1510,1543).
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

// =================================================================================================
// conversions, batching
// =================================================================================================
template <typename T>
__global__ void k_convert_f32(const float* __restrict__ in, T* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = from_f<T>(in[i]);
}
template <typename T>
__global__ void k_widen_f32(const T* __restrict__ in, float* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = to_f<T>(in[i]);
}
cudaError_t launch_convert_f32(cudaStream_t st, int dt, const float* in, void* out, size_t n) {
  if (n == 0) return cudaSuccess;
  unsigned grid = min(cdiv(n, 256), 148u * 16);
  DISPATCH_DT(dt, (k_convert_f32<T><<<grid, 256, 0, st>>>(in, (T*)out, n)));
  return cudaGetLastError();
}
cudaError_t launch_widen_to_f32(cudaStream_t st, int dt, const void* in, float* out, size_t n) {
  if (n == 0) return cudaSuccess;
  unsigned grid = min(cdiv(n, 256), 148u * 16);
  DISPATCH_DT(dt, (k_widen_f32<T><<<grid, 256, 0, st>>>((const T*)in, out, n)));
  return cudaGetLastError();
}

// FIFO batch: inputs = window[0:BT], targets = window[1:BT+1], widened to i64
// (src/data/loader.zig:555-589).
__global__ void k_fifo_batch(const uint16_t* __restrict__ tok, long long cursor, long long bt,
                             long long* __restrict__ x, long long* __restrict__ y) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < bt; i += stride) {
    x[i] = (long long)tok[cursor + i];
    y[i] = (long long)tok[cursor + i + 1];
  }
}
cudaError_t launch_fifo_batch(cudaStream_t st, const uint16_t* tokens, long long cursor, long long bt,
                              long long* inputs, long long* targets) {
  if (bt == 0) return cudaSuccess;
  k_fifo_batch<<<min(cdiv(bt, 256), 148u * 8), 256, 0, st>>>(tokens, cursor, bt, inputs, targets);
  return cudaGetLastError();
}

// Random-window batch: row b takes `block` tokens from starts[b], targets are the same window shifted by one,
// widened to i64 (U16TokenDataset / TextDataset / ByteTextDataset .getBatchImpl, src/data/loader.zig:276-307,
// 366-397, 457-486).  TOK: uint16_t (pre-tokenised streams) or uint32_t (char / byte tokenizers).
template <typename TOK>
__global__ void k_window_batch(const TOK* __restrict__ tok, const unsigned long long* __restrict__ starts, int batch,
                               long long block, long long* __restrict__ x, long long* __restrict__ y) {
  const long long total = (long long)batch * block;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const long long b = i / block, t = i - b * block;
    const unsigned long long s = starts[b] + (unsigned long long)t;
    x[i] = (long long)tok[s];
    y[i] = (long long)tok[s + 1];
  }
}
cudaError_t launch_window_batch(cudaStream_t st, const void* tokens, int token_bytes, const unsigned long long* starts,
                                int batch, long long block, long long* inputs, long long* targets) {
  const long long total = (long long)batch * block;
  if (total == 0) return cudaSuccess;
  const unsigned grid = min(cdiv(total, 256), 148u * 8);
  if (token_bytes == 2) k_window_batch<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)tokens, starts, batch, block, inputs, targets);
  else k_window_batch<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)tokens, starts, batch, block, inputs, targets);
  return cudaGetLastError();
}

// =================================================================================================
// RMSNorm (parameter free).  y = x * T(rsqrt(sum(x^2)/(d+1e-4) + 1e-5)); tsave = the rsqrt argument.
// =================================================================================================
template <typename T>
__device__ __forceinline__ void rmsnorm_row_fwd(const T* __restrict__ xr, T* __restrict__ yr, int d,
                                                float* tsave_slot, float* red) {
  float ss = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) { float v = to_f(xr[j]); ss += v * v; }
  ss = block_sum(ss, red);
  const float t = ss / ((float)d + PCPB_GUARD) + 1e-5f;
  const float r = rnd<T>(rsqrtf(t));
  if (threadIdx.x == 0 && tsave_slot) *tsave_slot = t;
  for (int j = threadIdx.x; j < d; j += blockDim.x) yr[j] = from_f<T>(to_f(xr[j]) * r);
}

template <typename T>
__global__ void k_rmsnorm_fwd(const T* __restrict__ x, int d, T* __restrict__ y, float* __restrict__ tsave) {
  __shared__ float red[32];
  const size_t m = blockIdx.x;
  rmsnorm_row_fwd<T>(x + m * d, y + m * d, d, tsave ? tsave + m : nullptr, red);
}
template <typename T>
__global__ void k_embed_norm_fwd(const T* __restrict__ wte, const long long* __restrict__ idx, int d, int V,
                                 T* __restrict__ y, float* __restrict__ tsave) {
  __shared__ float red[32];
  const size_t m = blockIdx.x;
  long long row = idx[m];
  row = row < 0 ? 0 : (row >= V ? V - 1 : row);       // gather clamps start indices
  rmsnorm_row_fwd<T>(wte + (size_t)row * d, y + m * d, d, tsave + m, red);
}

// Backward of y = x * T(r), r = rsqrt(t), t = sum(x^2)/(d+1e-4) + 1e-5:
//   multiply VJP:   dx1 = T(dy * T(r));   dr = T(sum_j T(dy_j * x_j))
//   rsqrt VJP:      dt = (dr * -0.5) * rsqrt(t + 1e-4)^3
//   divide VJP:     ds = dt / ((d + 1e-4) + 1e-4)
//   power VJP:      dx2 = T(ds * 2 * x)      (x^2/x == x up to one ulp; 0 at x == 0)
// Every one of these values is an adjoint edge of the reference's engine (finite guard, clamp to +-100, cast:
// adj_edge); the edges between them that only reshape, broadcast or convert repeat a clamp already applied.
template <typename T>
__device__ __forceinline__ float rmsnorm_row_ds(const T* __restrict__ xr, const T* __restrict__ dyr, int d,
                                                float t, float* red) {
  float acc = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) acc += adj_edge<T>(to_f(dyr[j]) * to_f(xr[j]));
  acc = block_sum(acc, red);
  const float dr = adj_edge<T>(acc);
  const float rp = rsqrtf(t + PCPB_GUARD);
  const float dt = adj_edge<float>((dr * -0.5f) * ((rp * rp) * rp));
  return adj_edge<float>(dt / (((float)d + PCPB_GUARD) + PCPB_GUARD));
}

template <typename T>
__global__ void k_rmsnorm_bwd(const T* __restrict__ x, const float* __restrict__ tsave, const T* __restrict__ dy,
                              const T* __restrict__ dres, int d, T* __restrict__ dx) {
  __shared__ float red[32];
  const size_t m = blockIdx.x;
  const T* xr = x + m * d; const T* dyr = dy + m * d;
  const float t = tsave[m];
  const float ds = rmsnorm_row_ds<T>(xr, dyr, d, t, red);
  const float r = rnd<T>(rsqrtf(t));
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    const float xv = to_f(xr[j]);
    float g = adj_edge<T>(to_f(dyr[j]) * r) + adj_edge<T>(ds * (2.f * xv));
    if (dres) g += to_f(dres[m * d + j]);
    dx[m * d + j] = from_f<T>(g);
  }
}
template <typename T>
__global__ void k_embed_norm_bwd(const T* __restrict__ wte, const long long* __restrict__ idx, int d, int V,
                                 const T* __restrict__ dy, const float* __restrict__ tsave,
                                 float* __restrict__ dwte, T* __restrict__ rows) {
  __shared__ float red[32];
  const size_t m = blockIdx.x;
  long long row = idx[m];
  row = row < 0 ? 0 : (row >= V ? V - 1 : row);
  const T* xr = wte + (size_t)row * d; const T* dyr = dy + m * d;
  const float t = tsave[m];
  const float ds = rmsnorm_row_ds<T>(xr, dyr, d, t, red);
  const float r = rnd<T>(rsqrtf(t));
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    const float xv = to_f(xr[j]);
    const float g = rnd<T>(adj_edge<T>(to_f(dyr[j]) * r) + adj_edge<T>(ds * (2.f * xv)));
    if (rows) rows[m * d + j] = from_f<T>(g);                    // summed per token by launch_embed_scatter_sorted
    else atomicAdd(dwte + (size_t)row * d + j, g);
  }
}


// ---- vectorised variants: one warp per row, 16-byte accesses, used when d % 8 == 0 ------------------
template <typename T>
__global__ void __launch_bounds__(256) k_rmsnorm_fwd_vec(const T* __restrict__ x, const T* __restrict__ wte,
                                                         const long long* __restrict__ idx, int M, int d, int V,
                                                         T* __restrict__ y, float* __restrict__ tsave) {
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (m >= M) return;
  const T* xr;
  if (idx) {
    long long row = idx[m];
    row = row < 0 ? 0 : (row >= V ? V - 1 : row);
    xr = wte + (size_t)row * d;
  } else {
    xr = x + (size_t)m * d;
  }
  const int nv = d >> 3;
  float ss = 0.f;
  for (int v = lane; v < nv; v += 32) {
    float f[8];
    ld8<T>(xr + v * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float t = ss / ((float)d + PCPB_GUARD) + 1e-5f;
  const float r = rnd<T>(rsqrtf(t));
  if (lane == 0 && tsave) tsave[m] = t;
  T* yr = y + (size_t)m * d;
  for (int v = lane; v < nv; v += 32) {
    float f[8];
    ld8<T>(xr + v * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= r;
    st8<T>(yr + v * 8, f);
  }
}

// dwte != nullptr: embedding variant (x rows come from wte[idx], gradient rows are atomically added to dwte)
// dst[0..3] += (a, b, c, e) as one reduction (dst 16-byte aligned); no value is returned, so the adds are performed at L2.
__device__ __forceinline__ void red_add_v4(float* dst, float a, float b, float c, float e) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(e) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(256) k_rmsnorm_bwd_vec(const T* __restrict__ x, const T* __restrict__ wte,
                                                         const long long* __restrict__ idx, const float* __restrict__ tsave,
                                                         const T* __restrict__ dy, const T* __restrict__ dres, int M, int d,
                                                         int V, T* __restrict__ dx, float* __restrict__ dwte) {
  const int m = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (m >= M) return;
  const T* xr;
  long long row = 0;
  if (idx) {
    row = idx[m];
    row = row < 0 ? 0 : (row >= V ? V - 1 : row);
    xr = wte + (size_t)row * d;
  } else {
    xr = x + (size_t)m * d;
  }
  const T* dyr = dy + (size_t)m * d;
  const int nv = d >> 3;
  // Adjoint edges (see rmsnorm_row_ds).  The element-wise ones are products of dy with x, with r and of ds with 2x:
  // the largest |dy| and |x| of the row bound them all, so the guard / clamp code only runs for a row whose bound fails
  // (then it is exact); a row inside the bound is untouched by it, as in the reference.
  float acc = 0.f;
  uint32_t mg = 0u;
  for (int v = lane; v < nv; v += 32) {
    float a[8], g[8];
    ld8<T>(xr + v * 8, a);
    ld8<T>(dyr + v * 8, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc += rnd<T>(g[i] * a[i]); adj_track(mg, g[i]); }
  }
  mg = __reduce_max_sync(0xffffffffu, mg);
  const float t = tsave[m];
  // |x_j| <= sqrt(sum x^2) = sqrt((t - 1e-5) (d + 1e-4)), from the statistic the forward saved (NaN if x had one)
  const float gmax = __uint_as_float(mg), amax = sqrtf(fmaxf(t - 1e-5f, 0.f) * ((float)d + PCPB_GUARD));
  if (!(gmax * amax <= PCPB_ADJ_CLIP)) {                         // some product may be beyond the clamp (or not finite)
    acc = 0.f;
    for (int v = lane; v < nv; v += 32) {
      float a[8], g[8];
      ld8<T>(xr + v * 8, a);
      ld8<T>(dyr + v * 8, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += adj_edge<T>(g[i] * a[i]);
    }
  }
  acc = warp_sum(acc);
  const float dr = adj_edge<T>(acc);
  const float rp = rsqrtf(t + PCPB_GUARD);
  const float ds = adj_edge<float>(adj_edge<float>((dr * -0.5f) * ((rp * rp) * rp)) / (((float)d + PCPB_GUARD) + PCPB_GUARD));
  const float r = rnd<T>(rsqrtf(t));
  const bool plain = (gmax * r <= PCPB_ADJ_CLIP) && (fabsf(ds) * 2.f * amax <= PCPB_ADJ_CLIP);
  for (int v = lane; v < nv; v += 32) {
    float a[8], g[8], o[8];
    ld8<T>(xr + v * 8, a);
    ld8<T>(dyr + v * 8, g);
    if (plain) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = rnd<T>(g[i] * r) + rnd<T>(ds * (2.f * a[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = adj_edge<T>(g[i] * r) + adj_edge<T>(ds * (2.f * a[i]));
    }
    if (dwte) {
      // scatter into the f32 embedding gradient: two 16-byte vector reductions instead of eight scalar atomics
      float* dst = dwte + (size_t)row * d + v * 8;
      red_add_v4(dst, rnd<T>(o[0]), rnd<T>(o[1]), rnd<T>(o[2]), rnd<T>(o[3]));
      red_add_v4(dst + 4, rnd<T>(o[4]), rnd<T>(o[5]), rnd<T>(o[6]), rnd<T>(o[7]));
    } else {
      if (dres) {
        float e[8];
        ld8<T>(dres + (size_t)m * d + v * 8, e);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += e[i];
      }
      st8<T>(dx + (size_t)m * d + v * 8, o);
    }
  }
}

static inline bool vec_ok(int d, const void* a, const void* b = nullptr, const void* c = nullptr, const void* e = nullptr) {
  return d % 8 == 0 && ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c) | ((uintptr_t)e)) & 15) == 0;
}

static inline int norm_threads(int d) { return d >= 1024 ? 256 : (d >= 256 ? 128 : 64); }

cudaError_t launch_rmsnorm_fwd(cudaStream_t st, int dt, const void* x, int M, int d, void* y, float* tsave) {
  if (M == 0) return cudaSuccess;
  if (vec_ok(d, x, y)) {
    DISPATCH_DT(dt, (k_rmsnorm_fwd_vec<T><<<cdiv(M, 8), 256, 0, st>>>((const T*)x, nullptr, nullptr, M, d, 0, (T*)y, tsave)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_rmsnorm_fwd<T><<<M, norm_threads(d), 0, st>>>((const T*)x, d, (T*)y, tsave)));
  return cudaGetLastError();
}
cudaError_t launch_embed_norm_fwd(cudaStream_t st, int dt, const void* wte, const long long* idx, int M, int d,
                                  int V, void* x, float* tsave) {
  if (M == 0) return cudaSuccess;
  if (vec_ok(d, wte, x)) {
    DISPATCH_DT(dt, (k_rmsnorm_fwd_vec<T><<<cdiv(M, 8), 256, 0, st>>>(nullptr, (const T*)wte, idx, M, d, V, (T*)x, tsave)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_embed_norm_fwd<T><<<M, norm_threads(d), 0, st>>>((const T*)wte, idx, d, V, (T*)x, tsave)));
  return cudaGetLastError();
}
cudaError_t launch_rmsnorm_bwd(cudaStream_t st, int dt, const void* x, const float* tsave, const void* dy,
                               const void* dres, int M, int d, void* dx) {
  if (M == 0) return cudaSuccess;
  if (vec_ok(d, x, dy, dres, dx)) {
    DISPATCH_DT(dt, (k_rmsnorm_bwd_vec<T><<<cdiv(M, 8), 256, 0, st>>>((const T*)x, nullptr, nullptr, tsave, (const T*)dy,
                                                                    (const T*)dres, M, d, 0, (T*)dx, nullptr)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_rmsnorm_bwd<T><<<M, norm_threads(d), 0, st>>>((const T*)x, tsave, (const T*)dy,
                                                                    (const T*)dres, d, (T*)dx)));
  return cudaGetLastError();
}
cudaError_t launch_embed_norm_bwd(cudaStream_t st, int dt, const void* wte, const long long* idx, int M, int d,
                                  int V, const void* dy, const float* tsave, float* dwte) {
  if (M == 0) return cudaSuccess;
  if (vec_ok(d, wte, dy, dwte)) {
    DISPATCH_DT(dt, (k_rmsnorm_bwd_vec<T><<<cdiv(M, 8), 256, 0, st>>>(nullptr, (const T*)wte, idx, tsave, (const T*)dy,
                                                                    nullptr, M, d, V, nullptr, dwte)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_embed_norm_bwd<T><<<M, norm_threads(d), 0, st>>>((const T*)wte, idx, d, V, (const T*)dy,
                                                                       tsave, dwte, (T*)nullptr)));
  return cudaGetLastError();
}
cudaError_t launch_embed_norm_bwd_rows(cudaStream_t st, int dt, const void* wte, const long long* idx, int M, int d, int V,
                                       const void* dy, const float* tsave, void* rows) {
  if (M == 0) return cudaSuccess;
  if (vec_ok(d, wte, dy, rows)) {
    // the embedding form of the RMSNorm backward with the row written instead of scattered (same values: the sum of the
    // two rounded terms, rounded to the model dtype by the store)
    DISPATCH_DT(dt, (k_rmsnorm_bwd_vec<T><<<cdiv(M, 8), 256, 0, st>>>(nullptr, (const T*)wte, idx, tsave, (const T*)dy,
                                                                    nullptr, M, d, V, (T*)rows, nullptr)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_embed_norm_bwd<T><<<M, norm_threads(d), 0, st>>>((const T*)wte, idx, d, V, (const T*)dy, tsave,
                                                                       (float*)nullptr, (T*)rows)));
  return cudaGetLastError();
}

// =================================================================================================
// RoPE (half split, bf16 tables) + per-head RMSNorm of q and k.  One warp per (token, head).
// =================================================================================================
template <typename T>
__device__ __forceinline__ float table_val(const uint16_t* tab, size_t i) {
  // tables are bf16; an f32 model converts them to f32 (exact), a bf16 model uses them as they are
  return __uint_as_float(((uint32_t)tab[i]) << 16);
}

template <typename T>
__global__ void k_rope_qknorm_fwd(const T* __restrict__ qkv, const uint16_t* __restrict__ cosT,
                                  const uint16_t* __restrict__ sinT, int M, int Tlen, int H, int Hkv, int hd,
                                  T* __restrict__ qkn, float* __restrict__ tq) {
  const int heads = H + Hkv;
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)M * heads) return;
  const int m = (int)(gw / heads), h = (int)(gw % heads);
  const int wqkv = (H + 2 * Hkv) * hd, wqkn = heads * hd;
  const T* src = qkv + (size_t)m * wqkv + (size_t)h * hd;          // q heads then k heads are contiguous
  T* dst = qkn + (size_t)m * wqkn + (size_t)h * hd;
  const int half = hd >> 1, pos = m % Tlen;
  float ss = 0.f;
  for (int i = lane; i < half; i += 32) {
    const float x1 = to_f(src[i]), x2 = to_f(src[i + half]);
    const float c = table_val<T>(cosT, (size_t)pos * half + i), s = table_val<T>(sinT, (size_t)pos * half + i);
    const float y1 = rnd<T>(rnd<T>(x1 * c) + rnd<T>(x2 * s));
    const float y2 = rnd<T>(rnd<T>(x1 * (-s)) + rnd<T>(x2 * c));
    ss += y1 * y1 + y2 * y2;
  }
  ss = warp_sum(ss);
  const float t = ss / ((float)hd + PCPB_GUARD) + 1e-5f;
  const float r = rnd<T>(rsqrtf(t));
  if (lane == 0) tq[(size_t)m * heads + h] = t;
  for (int i = lane; i < half; i += 32) {
    const float x1 = to_f(src[i]), x2 = to_f(src[i + half]);
    const float c = table_val<T>(cosT, (size_t)pos * half + i), s = table_val<T>(sinT, (size_t)pos * half + i);
    const float y1 = rnd<T>(rnd<T>(x1 * c) + rnd<T>(x2 * s));
    const float y2 = rnd<T>(rnd<T>(x1 * (-s)) + rnd<T>(x2 * c));
    dst[i] = from_f<T>(y1 * r);
    dst[i + half] = from_f<T>(y2 * r);
  }
}

template <typename T>
__global__ void k_rope_qknorm_bwd(const T* __restrict__ qkv, const T* __restrict__ dqkn,
                                  const float* __restrict__ tq, const uint16_t* __restrict__ cosT,
                                  const uint16_t* __restrict__ sinT, int M, int Tlen, int H, int Hkv, int hd,
                                  T* __restrict__ dqkv) {
  const int heads = H + Hkv;
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)M * heads) return;
  const int m = (int)(gw / heads), h = (int)(gw % heads);
  const int wqkv = (H + 2 * Hkv) * hd, wqkn = heads * hd;
  const T* src = qkv + (size_t)m * wqkv + (size_t)h * hd;
  const T* dyp = dqkn + (size_t)m * wqkn + (size_t)h * hd;
  T* dst = dqkv + (size_t)m * wqkv + (size_t)h * hd;
  const int half = hd >> 1, pos = m % Tlen;
  const float t = tq[(size_t)m * heads + h];
  // pass 1: dr = T(sum T(dy * y)) over the head
  float acc = 0.f;
  for (int i = lane; i < half; i += 32) {
    const float x1 = to_f(src[i]), x2 = to_f(src[i + half]);
    const float c = table_val<T>(cosT, (size_t)pos * half + i), s = table_val<T>(sinT, (size_t)pos * half + i);
    const float y1 = rnd<T>(rnd<T>(x1 * c) + rnd<T>(x2 * s));
    const float y2 = rnd<T>(rnd<T>(x1 * (-s)) + rnd<T>(x2 * c));
    acc += adj_edge<T>(to_f(dyp[i]) * y1) + adj_edge<T>(to_f(dyp[i + half]) * y2);
  }
  acc = warp_sum(acc);
  const float dr = adj_edge<T>(acc);
  const float rp = rsqrtf(t + PCPB_GUARD);
  const float dtt = adj_edge<float>((dr * -0.5f) * ((rp * rp) * rp));
  const float ds = adj_edge<float>(dtt / (((float)hd + PCPB_GUARD) + PCPB_GUARD));
  const float r = rnd<T>(rsqrtf(t));
  for (int i = lane; i < half; i += 32) {
    const float x1 = to_f(src[i]), x2 = to_f(src[i + half]);
    const float c = table_val<T>(cosT, (size_t)pos * half + i), s = table_val<T>(sinT, (size_t)pos * half + i);
    const float y1 = rnd<T>(rnd<T>(x1 * c) + rnd<T>(x2 * s));
    const float y2 = rnd<T>(rnd<T>(x1 * (-s)) + rnd<T>(x2 * c));
    // gradient wrt the roped value y
    const float g1 = rnd<T>(adj_edge<T>(to_f(dyp[i]) * r) + adj_edge<T>(ds * (2.f * y1)));
    const float g2 = rnd<T>(adj_edge<T>(to_f(dyp[i + half]) * r) + adj_edge<T>(ds * (2.f * y2)));
    // y1 = x1*c + x2*s ; y2 = x1*(-s) + x2*c
    dst[i] = from_f<T>(adj_edge<T>(g1 * c) + adj_edge<T>(g2 * (-s)));
    dst[i + half] = from_f<T>(adj_edge<T>(g1 * s) + adj_edge<T>(g2 * c));
  }
}


// ---- vectorised RoPE + QK-norm: each thread owns 8 rotation pairs; hd/16 threads per head ---------------
template <typename T>
__device__ __forceinline__ void rope8(const float (&x1)[8], const float (&x2)[8], const float (&c)[8], const float (&s)[8],
                                      float (&y1)[8], float (&y2)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    y1[i] = rnd<T>(rnd<T>(x1[i] * c[i]) + rnd<T>(x2[i] * s[i]));
    y2[i] = rnd<T>(rnd<T>(x1[i] * (-s[i])) + rnd<T>(x2[i] * c[i]));
  }
}
__device__ __forceinline__ float group_sum(float v, int tph) {
  for (int o = tph >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__global__ void __launch_bounds__(256) k_rope_qknorm_fwd_vec(const T* __restrict__ qkv, const uint16_t* __restrict__ cosT,
                                                             const uint16_t* __restrict__ sinT, int M, int Tlen, int H,
                                                             int Hkv, int hd, T* __restrict__ qkn, float* __restrict__ tq) {
  const int heads = H + Hkv, half = hd >> 1, tph = half >> 3;
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long slot = gt / tph;
  const int sub = (int)(gt % tph);
  const bool live = slot < (long long)M * heads;
  const int m = live ? (int)(slot / heads) : 0, h = live ? (int)(slot % heads) : 0;
  const T* src = qkv + (size_t)m * ((H + 2 * Hkv) * hd) + (size_t)h * hd + sub * 8;
  const int pos = m % Tlen;
  float x1[8], x2[8], c[8], s[8], y1[8], y2[8];
  ld8<T>(src, x1);
  ld8<T>(src + half, x2);
  ld8<bf16>(reinterpret_cast<const bf16*>(cosT) + (size_t)pos * half + sub * 8, c);
  ld8<bf16>(reinterpret_cast<const bf16*>(sinT) + (size_t)pos * half + sub * 8, s);
  rope8<T>(x1, x2, c, s, y1, y2);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += y1[i] * y1[i] + y2[i] * y2[i];
  ss = group_sum(ss, tph);
  const float t = ss / ((float)hd + PCPB_GUARD) + 1e-5f;
  const float r = rnd<T>(rsqrtf(t));
  if (!live) return;
  if (sub == 0) tq[(size_t)m * heads + h] = t;
#pragma unroll
  for (int i = 0; i < 8; ++i) { y1[i] *= r; y2[i] *= r; }
  T* dst = qkn + (size_t)m * (heads * hd) + (size_t)h * hd + sub * 8;
  st8<T>(dst, y1);
  st8<T>(dst + half, y2);
}

template <typename T>
__global__ void __launch_bounds__(256) k_rope_qknorm_bwd_vec(const T* __restrict__ qkv, const T* __restrict__ dqkn,
                                                             const float* __restrict__ tq, const uint16_t* __restrict__ cosT,
                                                             const uint16_t* __restrict__ sinT, int M, int Tlen, int H, int Hkv,
                                                             int hd, T* __restrict__ dqkv) {
  const int heads = H + Hkv, half = hd >> 1, tph = half >> 3;
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long slot = gt / tph;
  const int sub = (int)(gt % tph);
  const bool live = slot < (long long)M * heads;
  const int m = live ? (int)(slot / heads) : 0, h = live ? (int)(slot % heads) : 0;
  const size_t wqkv = (size_t)(H + 2 * Hkv) * hd;
  const T* src = qkv + (size_t)m * wqkv + (size_t)h * hd + sub * 8;
  const T* dyp = dqkn + (size_t)m * (heads * hd) + (size_t)h * hd + sub * 8;
  const int pos = m % Tlen;
  float x1[8], x2[8], c[8], s[8], y1[8], y2[8], d1[8], d2[8];
  ld8<T>(src, x1);
  ld8<T>(src + half, x2);
  ld8<bf16>(reinterpret_cast<const bf16*>(cosT) + (size_t)pos * half + sub * 8, c);
  ld8<bf16>(reinterpret_cast<const bf16*>(sinT) + (size_t)pos * half + sub * 8, s);
  ld8<T>(dyp, d1);
  ld8<T>(dyp + half, d2);
  rope8<T>(x1, x2, c, s, y1, y2);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc += adj_edge<T>(d1[i] * y1[i]) + adj_edge<T>(d2[i] * y2[i]);
  acc = group_sum(acc, tph);
  const float t = tq[(size_t)m * heads + h];
  const float dr = adj_edge<T>(acc);
  const float rp = rsqrtf(t + PCPB_GUARD);
  const float ds = adj_edge<float>(adj_edge<float>((dr * -0.5f) * ((rp * rp) * rp)) / (((float)hd + PCPB_GUARD) + PCPB_GUARD));
  const float r = rnd<T>(rsqrtf(t));
  if (!live) return;
  float o1[8], o2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float g1 = rnd<T>(adj_edge<T>(d1[i] * r) + adj_edge<T>(ds * (2.f * y1[i])));
    const float g2 = rnd<T>(adj_edge<T>(d2[i] * r) + adj_edge<T>(ds * (2.f * y2[i])));
    o1[i] = adj_edge<T>(g1 * c[i]) + adj_edge<T>(g2 * (-s[i]));
    o2[i] = adj_edge<T>(g1 * s[i]) + adj_edge<T>(g2 * c[i]);
  }
  T* dst = dqkv + (size_t)m * wqkv + (size_t)h * hd + sub * 8;
  st8<T>(dst, o1);
  st8<T>(dst + half, o2);
}

// ---- bf16 RoPE + QK-norm on bf16 pairs: the same op sequence as the templates above (each mul / add of the graph
// is one mul.bf16x2 / add.bf16x2), a third of their instruction count.  Eight rotation pairs per thread.
__global__ void __launch_bounds__(256) k_rope_qknorm_fwd_bf16x2(const bf16* __restrict__ qkv, const uint16_t* __restrict__ cosT,
                                                                const uint16_t* __restrict__ sinT, int M, int Tlen, int H,
                                                                int Hkv, int hd, bf16* __restrict__ qkn, float* __restrict__ tq) {
  const int heads = H + Hkv, half = hd >> 1, tph = half >> 3;
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long slot = gt / tph;
  const int sub = (int)(gt % tph);
  const bool live = slot < (long long)M * heads;
  const int m = live ? (int)(slot / heads) : 0, h = live ? (int)(slot % heads) : 0;
  const bf16* src = qkv + (size_t)m * ((H + 2 * Hkv) * hd) + (size_t)h * hd + sub * 8;
  const int pos = m % Tlen;
  const uint4 X1 = *reinterpret_cast<const uint4*>(src), X2 = *reinterpret_cast<const uint4*>(src + half);
  const uint4 Cw = *reinterpret_cast<const uint4*>(cosT + (size_t)pos * half + sub * 8);
  const uint4 Sw = *reinterpret_cast<const uint4*>(sinT + (size_t)pos * half + sub * 8);
  const uint32_t x1[4] = {X1.x, X1.y, X1.z, X1.w}, x2[4] = {X2.x, X2.y, X2.z, X2.w};
  const uint32_t c[4] = {Cw.x, Cw.y, Cw.z, Cw.w}, sn[4] = {Sw.x, Sw.y, Sw.z, Sw.w};
  uint32_t y1[4], y2[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    y1[i] = badd2(bmul2(x1[i], c[i]), bmul2(x2[i], sn[i]));
    y2[i] = badd2(bmul2(x1[i], sn[i] ^ 0x80008000u), bmul2(x2[i], c[i]));
    const float a0 = bf_lo(y1[i]), b0 = bf_lo(y2[i]), a1 = bf_hi(y1[i]), b1 = bf_hi(y2[i]);
    ss += a0 * a0 + b0 * b0;
    ss += a1 * a1 + b1 * b1;
  }
  ss = group_sum(ss, tph);
  const float t = ss / ((float)hd + PCPB_GUARD) + 1e-5f;
  const uint32_t r2 = pack2(rsqrtf(t), rsqrtf(t));
  if (!live) return;
  if (sub == 0) tq[(size_t)m * heads + h] = t;
  bf16* dst = qkn + (size_t)m * (heads * hd) + (size_t)h * hd + sub * 8;
  *reinterpret_cast<uint4*>(dst) = make_uint4(bmul2(y1[0], r2), bmul2(y1[1], r2), bmul2(y1[2], r2), bmul2(y1[3], r2));
  *reinterpret_cast<uint4*>(dst + half) = make_uint4(bmul2(y2[0], r2), bmul2(y2[1], r2), bmul2(y2[2], r2), bmul2(y2[3], r2));
}

__global__ void __launch_bounds__(256, 4) k_rope_qknorm_bwd_bf16x2(const bf16* __restrict__ qkv, const bf16* __restrict__ dqkn,
                                                                const float* __restrict__ tq, const uint16_t* __restrict__ cosT,
                                                                const uint16_t* __restrict__ sinT, int M, int Tlen, int H, int Hkv,
                                                                int hd, bf16* __restrict__ dqkv) {
  const int heads = H + Hkv, half = hd >> 1, tph = half >> 3;
  const long long gt = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long slot = gt / tph;
  const int sub = (int)(gt % tph);
  const bool live = slot < (long long)M * heads;
  const int m = live ? (int)(slot / heads) : 0, h = live ? (int)(slot % heads) : 0;
  const size_t wqkv = (size_t)(H + 2 * Hkv) * hd;
  const bf16* src = qkv + (size_t)m * wqkv + (size_t)h * hd + sub * 8;
  const bf16* dyp = dqkn + (size_t)m * (heads * hd) + (size_t)h * hd + sub * 8;
  const int pos = m % Tlen;
  const uint4 X1 = *reinterpret_cast<const uint4*>(src), X2 = *reinterpret_cast<const uint4*>(src + half);
  const uint4 Cw = *reinterpret_cast<const uint4*>(cosT + (size_t)pos * half + sub * 8);
  const uint4 Sw = *reinterpret_cast<const uint4*>(sinT + (size_t)pos * half + sub * 8);
  const uint4 D1 = *reinterpret_cast<const uint4*>(dyp), D2 = *reinterpret_cast<const uint4*>(dyp + half);
  const uint32_t x1[4] = {X1.x, X1.y, X1.z, X1.w}, x2[4] = {X2.x, X2.y, X2.z, X2.w};
  const uint32_t c[4] = {Cw.x, Cw.y, Cw.z, Cw.w}, sn[4] = {Sw.x, Sw.y, Sw.z, Sw.w};
  const uint32_t d1[4] = {D1.x, D1.y, D1.z, D1.w}, d2[4] = {D2.x, D2.y, D2.z, D2.w};
  uint32_t y1[4], y2[4];
  // Adjoint edges: d*y products, dr, ds, d*r, ds*2y, and the products with cos / sin (|cos|, |sin| <= 1).  The largest
  // |d| and |y| of the head row bound all the element-wise ones; the guard / clamp code runs only for a head row whose
  // bound fails (and is exact there).
  float acc = 0.f;
  uint32_t md = 0u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    y1[i] = badd2(bmul2(x1[i], c[i]), bmul2(x2[i], sn[i]));
    y2[i] = badd2(bmul2(x1[i], sn[i] ^ 0x80008000u), bmul2(x2[i], c[i]));
    const uint32_t p1 = bmul2(d1[i], y1[i]), p2 = bmul2(d2[i], y2[i]);
    acc += bf_lo(p1) + bf_lo(p2);
    acc += bf_hi(p1) + bf_hi(p2);
    adj_track2(md, d1[i]); adj_track2(md, d2[i]);
  }
  // largest |d| over the head row (the tph lanes of this group; NaN is kept by the packed maximum); |y_i| is bounded by
  // sqrt(sum y^2) = sqrt((t - 1e-5) (hd + 1e-4)) from the statistic the forward saved (NaN if y had one)
  for (int o = tph >> 1; o > 0; o >>= 1) adj_track2(md, __shfl_xor_sync(0xffffffffu, md, o));
  const float t = tq[(size_t)m * heads + h];
  const float dmax = fmaxf(bf_lo(md), bf_hi(md)), ymax = sqrtf(fmaxf(t - 1e-5f, 0.f) * ((float)hd + PCPB_GUARD));
  const bool nan_in = (bf_lo(md) != bf_lo(md)) || (bf_hi(md) != bf_hi(md)) || (t != t);
  if (nan_in || !(dmax * ymax <= PCPB_ADJ_CLIP)) {
    acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t p1 = adj_edge2(bmul2(d1[i], y1[i])), p2 = adj_edge2(bmul2(d2[i], y2[i]));
      acc += bf_lo(p1) + bf_lo(p2);
      acc += bf_hi(p1) + bf_hi(p2);
    }
  }
  acc = group_sum(acc, tph);
  const float dr = adj_edge<bf16>(acc);
  const float rp = rsqrtf(t + PCPB_GUARD);
  const float ds = adj_edge<float>(adj_edge<float>((dr * -0.5f) * ((rp * rp) * rp)) / (((float)hd + PCPB_GUARD) + PCPB_GUARD));
  const float rr = rsqrtf(t);
  const uint32_t r2 = pack2(rr, rr);
  if (!live) return;
  // bound on d*r, ds*2y and on their sum g (which the cos / sin products cannot exceed)
  const bool plain = !nan_in && (dmax * rr + fabsf(ds) * 2.f * ymax <= PCPB_ADJ_CLIP);
  uint32_t o1[4], o2[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // gradient wrt the roped value: bf16(bf16(d * r) + bf16(ds * (2 * y))), ds in f32
    uint32_t t1 = pack2(ds * (2.f * bf_lo(y1[i])), ds * (2.f * bf_hi(y1[i])));
    uint32_t t2 = pack2(ds * (2.f * bf_lo(y2[i])), ds * (2.f * bf_hi(y2[i])));
    if (plain) {
      const uint32_t g1 = badd2(bmul2(d1[i], r2), t1), g2 = badd2(bmul2(d2[i], r2), t2);
      // y1 = x1*c + x2*s ; y2 = x1*(-s) + x2*c
      o1[i] = badd2(bmul2(g1, c[i]), bmul2(g2, sn[i] ^ 0x80008000u));
      o2[i] = badd2(bmul2(g1, sn[i]), bmul2(g2, c[i]));
    } else {
      t1 = adj_edge2(t1); t2 = adj_edge2(t2);
      const uint32_t g1 = badd2(adj_edge2(bmul2(d1[i], r2)), t1), g2 = badd2(adj_edge2(bmul2(d2[i], r2)), t2);
      o1[i] = badd2(adj_edge2(bmul2(g1, c[i])), adj_edge2(bmul2(g2, sn[i] ^ 0x80008000u)));
      o2[i] = badd2(adj_edge2(bmul2(g1, sn[i])), adj_edge2(bmul2(g2, c[i])));
    }
  }
  bf16* dst = dqkv + (size_t)m * wqkv + (size_t)h * hd + sub * 8;
  *reinterpret_cast<uint4*>(dst) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
  *reinterpret_cast<uint4*>(dst + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
}

static inline bool rope_vec_ok(int hd, const void* a, const void* b, const void* c, const void* d) {
  const int tph = hd / 16;
  return hd % 16 == 0 && tph >= 1 && tph <= 32 && (tph & (tph - 1)) == 0 &&
         ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c) | ((uintptr_t)d)) & 15) == 0;
}

cudaError_t launch_rope_qknorm_fwd(cudaStream_t st, int dt, const void* qkv, const uint16_t* c, const uint16_t* s,
                                   int M, int Tlen, int H, int Hkv, int hd, void* qkn, float* tq) {
  const long long warps = (long long)M * (H + Hkv);
  if (warps == 0) return cudaSuccess;
  if (rope_vec_ok(hd, qkv, qkn, c, s)) {
    const long long threads = warps * (hd / 16);
    if (dt == DT_BF16) {
      k_rope_qknorm_fwd_bf16x2<<<cdiv(threads, 256), 256, 0, st>>>((const bf16*)qkv, c, s, M, Tlen, H, Hkv, hd, (bf16*)qkn, tq);
      return cudaGetLastError();
    }
    DISPATCH_DT(dt, (k_rope_qknorm_fwd_vec<T><<<cdiv(threads, 256), 256, 0, st>>>((const T*)qkv, c, s, M, Tlen, H, Hkv, hd,
                                                                                  (T*)qkn, tq)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_rope_qknorm_fwd<T><<<cdiv(warps * 32, 256), 256, 0, st>>>((const T*)qkv, c, s, M, Tlen, H, Hkv,
                                                                                hd, (T*)qkn, tq)));
  return cudaGetLastError();
}
cudaError_t launch_rope_qknorm_bwd(cudaStream_t st, int dt, const void* qkv, const void* dqkn, const float* tq,
                                   const uint16_t* c, const uint16_t* s, int M, int Tlen, int H, int Hkv, int hd,
                                   void* dqkv) {
  const long long warps = (long long)M * (H + Hkv);
  if (warps == 0) return cudaSuccess;
  if (rope_vec_ok(hd, qkv, dqkn, dqkv, c) && (((uintptr_t)s) & 15) == 0) {
    const long long threads = warps * (hd / 16);
    if (dt == DT_BF16) {
      k_rope_qknorm_bwd_bf16x2<<<cdiv(threads, 256), 256, 0, st>>>((const bf16*)qkv, (const bf16*)dqkn, tq, c, s, M, Tlen, H, Hkv,
                                                                   hd, (bf16*)dqkv);
      return cudaGetLastError();
    }
    DISPATCH_DT(dt, (k_rope_qknorm_bwd_vec<T><<<cdiv(threads, 256), 256, 0, st>>>((const T*)qkv, (const T*)dqkn, tq, c, s, M,
                                                                                  Tlen, H, Hkv, hd, (T*)dqkv)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_rope_qknorm_bwd<T><<<cdiv(warps * 32, 256), 256, 0, st>>>((const T*)qkv, (const T*)dqkn, tq, c,
                                                                                s, M, Tlen, H, Hkv, hd, (T*)dqkv)));
  return cudaGetLastError();
}

// =================================================================================================
// Generic GEMM: 64x64 tile, BK=16, 256 threads, 4x4 per thread, f32 accumulate.
// =================================================================================================
template <typename T>
__device__ __forceinline__ void gemm_epilogue(const GemmArgs& g, int m, int n, float acc) {
  const size_t o = (size_t)m * g.ldc + n;
  switch (g.epi) {
    case EPI_STORE:
      // g.adj: the product is an activation gradient (dot_general VJP output), i.e. an adjoint edge
      ((T*)g.C)[o] = from_f<T>(g.adj ? adj_edge<T>(acc) : acc);
      break;
    case EPI_RESID:
      ((T*)g.C)[o] = from_f<T>(to_f(((const T*)g.R)[o]) + rnd<T>(acc));
      break;
    case EPI_RELU2: {
      const T u = from_f<T>(acc);
      ((T*)g.C)[o] = u;
      const float r = fmaxf(to_f(u), 0.f);
      ((T*)g.C2)[o] = from_f<T>(r * r);
      break;
    }
    case EPI_DRELU2: {
      // a = power(max(u,0), 2).  power VJP (src/autodiff/vjp_rules.zig:252): g * (2 * (a / r)), 0 at r == 0;
      // maximum VJP (:499): pass where u > 0.
      const float da = adj_edge<T>(acc);
      const float u = to_f(((const T*)g.R)[o]);
      const float r = fmaxf(u, 0.f);
      float out = 0.f;
      if (u > 0.f) {
        const float y = rnd<T>(r * r);
        const float q = rnd<T>(y / r);
        out = adj_edge<T>(da * rnd<T>(2.f * q));
      }
      ((T*)g.C)[o] = from_f<T>(out);
      break;
    }
    case EPI_WGRAD: {
      float v = rnd<T>(acc);
      if (!((v - v) == 0.f)) v = 0.f;                       // finite guard
      v = fminf(fmaxf(v, -g.clip), g.clip);
      ((float*)g.C)[o] = v;
      break;
    }
    case EPI_RELU: {
      const T u = from_f<T>(acc);
      ((T*)g.C)[o] = u;
      ((T*)g.C2)[o] = from_f<T>(fmaxf(to_f(u), 0.f));
      break;
    }
    case EPI_DRELU:
      ((T*)g.C)[o] = (to_f(((const T*)g.R)[o]) > 0.f) ? from_f<T>(adj_edge<T>(acc)) : from_f<T>(0.f);
      break;
    case EPI_BIAS:
      ((T*)g.C)[o] = from_f<T>(acc + to_f(((const T*)g.R)[n]));
      break;
    case EPI_GELU: {
      const T u = from_f<T>(acc);
      ((T*)g.C)[o] = u;
      ((T*)g.C2)[o] = from_f<T>(gelu_fwd<T>(to_f(u)));
      break;
    }
    case EPI_DGELU:
      ((T*)g.C)[o] = from_f<T>(adj_edge<T>(adj_edge<T>(acc) * gelu_grad<T>(to_f(((const T*)g.R)[o]))));
      break;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) k_gemm_generic(GemmArgs g) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64 + 4];
  const T* __restrict__ A = (const T*)g.A;
  const T* __restrict__ B = (const T*)g.B;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const bool a_kfast = (g.sak == 1), b_nfast = (g.sbn == 1);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.K; k0 += 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      int mm, kk;
      if (a_kfast) { kk = idx & 15; mm = idx >> 4; } else { mm = idx & 63; kk = idx >> 6; }
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < g.M && gk < g.K) ? to_f(A[(size_t)gm * g.sam + (size_t)gk * g.sak]) : 0.f;
      int nn, kb;
      if (b_nfast) { nn = idx & 63; kb = idx >> 6; } else { kb = idx & 15; nn = idx >> 4; }
      const int gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < g.N && gkb < g.K) ? to_f(B[(size_t)gkb * g.sbk + (size_t)gn * g.sbn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < g.N) gemm_epilogue<T>(g, m, n, acc[i][j]);
    }
  }
}

// ---- f32 operands as sums of three bf16 values, packed for one bf16 GEMM over 6 K (see kernels.h) ----
template <bool ROWFAST>
__global__ void __launch_bounds__(256) k_split3_pack(const float* __restrict__ src, long long s_row, long long s_k, int rows, int K,
                                                     int bpat, __nv_bfloat16* __restrict__ dst) {
  __shared__ float tile[32][33];                                // [row][k]
  const int r0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    if (ROWFAST) {                                              // rows are contiguous in memory: read along the rows
      const int r = r0 + threadIdx.x, k = k0 + i;
      tile[threadIdx.x][i] = (r < rows && k < K) ? src[(size_t)r * s_row + (size_t)k * s_k] : 0.f;
    } else {
      const int r = r0 + i, k = k0 + threadIdx.x;
      tile[i][threadIdx.x] = (r < rows && k < K) ? src[(size_t)r * s_row + (size_t)k * s_k] : 0.f;
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, k = k0 + threadIdx.x;
    if (r >= rows || k >= K) continue;
    const float x = tile[i][threadIdx.x];
    const __nv_bfloat16 p1 = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(p1);
    const __nv_bfloat16 p2 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(p2);
    const __nv_bfloat16 p3 = __float2bfloat16_rn(r2);
    __nv_bfloat16* d = dst + (size_t)r * 6 * K + k;
    // smallest products first, a1 b1 last (see kernels.h)
    if (bpat == 0) { d[0] = p3; d[K] = p2; d[2 * (size_t)K] = p1; d[3 * (size_t)K] = p2; d[4 * (size_t)K] = p1; d[5 * (size_t)K] = p1; }
    else           { d[0] = p1; d[K] = p2; d[2 * (size_t)K] = p3; d[3 * (size_t)K] = p1; d[4 * (size_t)K] = p2; d[5 * (size_t)K] = p1; }
  }
}
cudaError_t launch_split3_pack(cudaStream_t st, const float* src, long long s_row, long long s_k, int rows, int K, int b_pattern,
                               void* dst_bf16) {
  if (rows == 0 || K == 0) return cudaSuccess;
  const dim3 grid(cdiv(K, 32), cdiv(rows, 32)), block(32, 8);
  if (s_row == 1 && s_k != 1) k_split3_pack<true><<<grid, block, 0, st>>>(src, s_row, s_k, rows, K, b_pattern, (__nv_bfloat16*)dst_bf16);
  else k_split3_pack<false><<<grid, block, 0, st>>>(src, s_row, s_k, rows, K, b_pattern, (__nv_bfloat16*)dst_bf16);
  return cudaGetLastError();
}
__global__ void __launch_bounds__(256) k_gemm_epilogue_f32(GemmArgs g, const float* __restrict__ acc) {
  const size_t mn = (size_t)g.M * g.N;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += (size_t)gridDim.x * blockDim.x)
    gemm_epilogue<float>(g, (int)(i / g.N), (int)(i % g.N), acc[i]);
}
cudaError_t launch_gemm_epilogue_f32(cudaStream_t st, const GemmArgs& g, const float* acc) {
  if (g.M == 0 || g.N == 0) return cudaSuccess;
  const size_t mn = (size_t)g.M * g.N;
  unsigned blocks = (unsigned)((mn + 255) / 256);
  if (blocks > 148u * 16) blocks = 148u * 16;
  k_gemm_epilogue_f32<<<blocks, 256, 0, st>>>(g, acc);
  return cudaGetLastError();
}

cudaError_t launch_gemm_generic(cudaStream_t st, int dt, const GemmArgs& g) {
  if (g.M == 0 || g.N == 0) return cudaSuccess;
  dim3 grid(cdiv(g.N, 64), cdiv(g.M, 64));
  DISPATCH_DT(dt, (k_gemm_generic<T><<<grid, 256, 0, st>>>(g)));
  return cudaGetLastError();
}

// =================================================================================================
// Generic causal attention.  One block per (query row, batch*head).
//   s_j = T(T(q.k_j) * scale), masked (j > i) entries contribute 0;  P = T(e / (l + 1e-4));
//   o = T(sum_j P_j v_j).
// Backward (softmax through the guarded divide, exp, subtract and reduce-max rules):
//   Pt_j = e_j / (l + 2e-4);  dp_j = T(do . v_j);  D = sum_j Pt_j dp_j;
//   dsf_j = Pt_j (dp_j - D) - [s_j == max] D 2e-4/(l + 2e-4);  ds_j = T(T(dsf_j) * scale).
// =================================================================================================
template <typename T>
__global__ void __launch_bounds__(128) k_attn_fwd_generic(AttnArgs a) {
  extern __shared__ float sm[];
  float* sc = sm;                 // [T]
  float* qrow = sm + a.T;         // [hd]
  __shared__ float red[32];
  const int i = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int hk = h / (a.H / a.Hkv);
  const int d = a.H * a.hd, dkv = a.Hkv * a.hd, wqkn = d + dkv, wqkv = d + 2 * dkv;
  const T* qkn = (const T*)a.qkn; const T* qkv = (const T*)a.qkv;
  const size_t mi = (size_t)b * a.T + i;
  for (int e = threadIdx.x; e < a.hd; e += blockDim.x) qrow[e] = to_f(qkn[mi * wqkn + h * a.hd + e]);
  __syncthreads();
  float mx = -INFINITY;
  for (int j = threadIdx.x; j <= i; j += blockDim.x) {
    const T* kr = qkn + ((size_t)b * a.T + j) * wqkn + d + hk * a.hd;
    float dot = 0.f;
    for (int e = 0; e < a.hd; ++e) dot = fmaf(qrow[e], to_f(kr[e]), dot);
    const float s = rnd<T>(rnd<T>(dot) * a.scale);
    sc[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_max(mx, red);
  float l = 0.f;
  for (int j = threadIdx.x; j <= i; j += blockDim.x) { const float e = expf(sc[j] - mx); sc[j] = e; l += e; }
  l = block_sum(l, red);
  const float inv = 1.f / (l + PCPB_GUARD);
  for (int j = threadIdx.x; j <= i; j += blockDim.x) sc[j] = rnd<T>(sc[j] / (l + PCPB_GUARD));
  (void)inv;
  __syncthreads();
  if (threadIdx.x == 0) { a.mrow[(size_t)bh * a.T + i] = mx; a.lrow[(size_t)bh * a.T + i] = l; }
  for (int e = threadIdx.x; e < a.hd; e += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j <= i; ++j)
      acc = fmaf(sc[j], to_f(qkv[((size_t)b * a.T + j) * wqkv + d + dkv + hk * a.hd + e]), acc);
    ((T*)a.o)[mi * d + h * a.hd + e] = from_f<T>(acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) k_attn_bwd_generic(AttnArgs a) {
  extern __shared__ float sm[];
  float* ds = sm;                    // [T]  scaled score gradients
  float* pf = sm + a.T;              // [T]  forward probabilities (model dtype values)
  float* qrow = sm + 2 * a.T;        // [hd]
  float* dorow = qrow + a.hd;        // [hd]
  __shared__ float red[32];
  const int i = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int hk = h / (a.H / a.Hkv);
  const int d = a.H * a.hd, dkv = a.Hkv * a.hd, wqkn = d + dkv, wqkv = d + 2 * dkv;
  const T* qkn = (const T*)a.qkn; const T* qkv = (const T*)a.qkv; const T* dout = (const T*)a.dout;
  const size_t mi = (size_t)b * a.T + i;
  for (int e = threadIdx.x; e < a.hd; e += blockDim.x) {
    qrow[e] = to_f(qkn[mi * wqkn + h * a.hd + e]);
    dorow[e] = to_f(dout[mi * d + h * a.hd + e]);
  }
  __syncthreads();
  const float mx = a.mrow[(size_t)bh * a.T + i], l = a.lrow[(size_t)bh * a.T + i];
  const float den2 = l + 2.f * PCPB_GUARD;
  float Dp = 0.f;
  for (int j = threadIdx.x; j <= i; j += blockDim.x) {
    const T* kr = qkn + ((size_t)b * a.T + j) * wqkn + d + hk * a.hd;
    const T* vr = qkv + ((size_t)b * a.T + j) * wqkv + d + dkv + hk * a.hd;
    float dot = 0.f, dp = 0.f;
    for (int e = 0; e < a.hd; ++e) {
      dot = fmaf(qrow[e], to_f(kr[e]), dot);
      dp = fmaf(dorow[e], to_f(vr[e]), dp);
    }
    const float s = rnd<T>(rnd<T>(dot) * a.scale);
    const float ex = expf(s - mx);
    dp = adj_edge<T>(dp);                         // dP: an output of the dot_general VJP
    pf[j] = rnd<T>(ex / (l + PCPB_GUARD));
    const float pt = ex / den2;
    Dp += pt * dp;
    ds[j] = pt;                       // stash Pt, finish after D is known
    sm[2 * a.T + 2 * a.hd + j] = dp;  // [T] dp
    sm[3 * a.T + 2 * a.hd + j] = (s == mx) ? 1.f : 0.f;
  }
  const float D = block_sum(Dp, red);
  const float mterm = D * (2.f * PCPB_GUARD) / den2;
  for (int j = threadIdx.x; j <= i; j += blockDim.x) {
    const float dp = sm[2 * a.T + 2 * a.hd + j];
    const float dsf = ds[j] * (dp - D) - sm[3 * a.T + 2 * a.hd + j] * mterm;
    // the softmax backward is evaluated in closed form: its inner edges cannot be clamped one by one, only noted
    const float dsr = rnd<T>(dsf);
    if (!(fabsf(dsr) <= PCPB_ADJ_CLIP)) adj_note(ADJ_INTERNAL);
    ds[j] = adj_edge<T>(dsr * a.scale);
  }
  __syncthreads();
  // dq_i = T(sum_j ds_j k_j)
  for (int e = threadIdx.x; e < a.hd; e += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j <= i; ++j) acc = fmaf(ds[j], to_f(qkn[((size_t)b * a.T + j) * wqkn + d + hk * a.hd + e]), acc);
    ((T*)a.dqkn)[mi * wqkn + h * a.hd + e] = from_f<T>(adj_edge<T>(acc));
  }
  // dk_j += ds_j q_i ; dv_j += P_j do_i   (f32 accumulators shared by the heads of one kv group)
  for (int idx = threadIdx.x; idx < (i + 1) * a.hd; idx += blockDim.x) {
    const int j = idx / a.hd, e = idx % a.hd;
    float* dst = a.dkv_acc + ((size_t)b * a.T + j) * (2 * dkv);
    atomicAdd(dst + hk * a.hd + e, ds[j] * qrow[e]);
    atomicAdd(dst + dkv + hk * a.hd + e, pf[j] * dorow[e]);
  }
}

template <typename T>
__global__ void k_attn_bwd_finish(const float* __restrict__ acc, int M, int d, int dkv, T* __restrict__ dqkn,
                                  T* __restrict__ dqkv) {
  const size_t n = (size_t)M * 2 * dkv;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / (2 * dkv); const int c = (int)(i % (2 * dkv));
    if (c < dkv) dqkn[m * (d + dkv) + d + c] = from_f<T>(adj_edge<T>(acc[i]));
    else dqkv[m * (d + 2 * dkv) + d + c] = from_f<T>(adj_edge<T>(acc[i]));     // c in [dkv, 2dkv) -> column d + dkv + (c-dkv)
  }
}

cudaError_t launch_attn_fwd_generic(cudaStream_t st, int dt, const AttnArgs& a) {
  if (a.B == 0 || a.T == 0) return cudaSuccess;
  dim3 grid(a.T, a.B * a.H);
  const size_t smem = (size_t)(a.T + a.hd) * sizeof(float);
  DISPATCH_DT(dt, (k_attn_fwd_generic<T><<<grid, 128, smem, st>>>(a)));
  return cudaGetLastError();
}
cudaError_t launch_attn_bwd_generic(cudaStream_t st, int dt, const AttnArgs& a) {
  if (a.B == 0 || a.T == 0) return cudaSuccess;
  const int M = a.B * a.T, d = a.H * a.hd, dkv = a.Hkv * a.hd;
  cudaError_t e = cudaMemsetAsync(a.dkv_acc, 0, (size_t)M * 2 * dkv * sizeof(float), st);
  if (e != cudaSuccess) return e;
  dim3 grid(a.T, a.B * a.H);
  const size_t smem = (size_t)(4 * a.T + 2 * a.hd) * sizeof(float);
  if (smem > 48 * 1024) {
    if (dt == DT_F32) e = cudaFuncSetAttribute(k_attn_bwd_generic<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    else e = cudaFuncSetAttribute(k_attn_bwd_generic<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  DISPATCH_DT(dt, (k_attn_bwd_generic<T><<<grid, 128, smem, st>>>(a)));
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  DISPATCH_DT(dt, (k_attn_bwd_finish<T><<<min(cdiv((size_t)M * 2 * dkv, 256), 148u * 8), 256, 0, st>>>(
                      a.dkv_acc, M, d, dkv, (T*)a.dqkn, (T*)a.dqkv)));
  return cudaGetLastError();
}

// =================================================================================================
// Soft-capped cross entropy, forward + backward in one pass pair per row.
//   c = cap * tanh(z / (cap + 1e-4));  sh = c - max;  se = sum exp(sh);  logp = sh - log(se + 1e-4)
//   loss = sum_valid(-logp[target]) / (count + 1e-4)
// Backward (dtot = 1/(count + 2e-4)):
//   dc_j = dtot * (exp(sh_j)/(se + 2e-4) - [j == target] + [c_j == max] * 2e-4/(se + 2e-4))
//   dz_j = T(dc_j * cap * (1 - tanh^2) / (cap + 2e-4))
// =================================================================================================
__global__ void k_count_valid(const long long* __restrict__ tg, int M, long long ignore, float* __restrict__ count) {
  __shared__ float red[32];
  float c = 0.f;
  for (int i = threadIdx.x; i < M; i += blockDim.x) c += (tg[i] != ignore) ? 1.f : 0.f;
  c = block_sum(c, red);                      // counts are integers < 2^24 per partial: exact in f32
  if (threadIdx.x == 0) *count = c;
}
cudaError_t launch_count_valid(cudaStream_t st, const long long* targets, int M, long long ignore, float* count) {
  k_count_valid<<<1, 1024, 0, st>>>(targets, M, ignore, count);
  return cudaGetLastError();
}

template <typename T>
__global__ void __launch_bounds__(256) k_softcap_ce(T* __restrict__ logits, const long long* __restrict__ tg, int V,
                                                    float cap, long long ignore, const float* __restrict__ count,
                                                    float* __restrict__ rowloss, int write_grad, float seed) {
  __shared__ float red[32];
  const size_t m = blockIdx.x;
  T* z = logits + m * V;
  const long long t = tg[m];
  const bool valid = (t != ignore);
  const float capg = cap + PCPB_GUARD;
  const bool capped = cap > 0.f;                      // cap == 0: plain cross entropy (nanoGPT family)
  auto capf = [&](float x) { return capped ? tanhf(x / capg) * cap : x; };
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < V; j += blockDim.x) mx = fmaxf(mx, capf(to_f(z[j])));
  mx = block_max(mx, red);
  float se = 0.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) se += expf(capf(to_f(z[j])) - mx);
  se = block_sum(se, red);
  if (threadIdx.x == 0) {
    float nll = 0.f;
    if (valid) {
      long long tt = t < 0 ? 0 : (t >= V ? V - 1 : t);
      nll = -((capf(to_f(z[tt])) - mx) - logf(se + PCPB_GUARD));
    }
    rowloss[m] = nll;
  }
  if (!write_grad) return;
  __syncthreads();
  // seed = d(loss) given by the caller.  The factors that follow (softmax probabilities, 1 - tanh^2, cap / (cap + 2e-4))
  // never exceed one in magnitude, so once this first edge is inside the clamp every later edge of the loss is too.
  const float dtot = valid ? adj_edge<float>(seed / (*count + 2.f * PCPB_GUARD)) : 0.f;
  const float den = se + 2.f * PCPB_GUARD;
  const float dzscale = capped ? cap / (capg + PCPB_GUARD) : 1.f;
  for (int j = threadIdx.x; j < V; j += blockDim.x) {
    const float zj = to_f(z[j]);
    const float th = capped ? tanhf(zj / capg) : 0.f;
    const float c = capped ? th * cap : zj;
    float dc = expf(c - mx) / den;
    if ((long long)j == t) dc -= 1.f;
    if (c == mx) dc += (2.f * PCPB_GUARD) / den;
    dc *= dtot;
    z[j] = from_f<T>(adj_edge<T>(dc * dzscale * (1.f - th * th)));
  }
}

// Vectorised variant (V % 8 == 0): online max / sum in one pass over the row, gradient in a second pass.
template <typename T>
__global__ void __launch_bounds__(512) k_softcap_ce_vec(T* __restrict__ logits, const long long* __restrict__ tg, int V,
                                                        float cap, long long ignore, const float* __restrict__ count,
                                                        float* __restrict__ rowloss, int write_grad, float seed) {
  __shared__ float red[32];
  const size_t m = blockIdx.x;
  T* z = logits + m * V;
  const long long t = tg[m];
  const bool valid = (t != ignore);
  const float capg = cap + PCPB_GUARD, icapg = 1.f / capg;
  const bool capped = cap > 0.f;                      // cap == 0: plain cross entropy (nanoGPT family)
  const int nv = V >> 3;
  float mx = -INFINITY, se = 0.f;
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float f[8];
    ld8<T>(z + v * 8, f);
    float c[8], cm = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      c[i] = capped ? m_tanh<T>(sizeof(T) == 4 ? f[i] / capg : f[i] * icapg) * cap : f[i];
      cm = fmaxf(cm, c[i]);
    }
    if (cm > mx) { se *= m_exp<T>(mx - cm); mx = cm; }
#pragma unroll
    for (int i = 0; i < 8; ++i) se += m_exp<T>(c[i] - mx);
  }
  const float gmx = block_max(mx, red);
  se *= (mx == -INFINITY) ? 0.f : m_exp<T>(mx - gmx);
  se = block_sum(se, red);
  mx = gmx;
  if (threadIdx.x == 0) {
    float nll = 0.f;
    if (valid) {
      long long tt = t < 0 ? 0 : (t >= V ? V - 1 : t);
      const float zt = to_f(z[tt]);
      const float c = capped ? m_tanh<T>(sizeof(T) == 4 ? zt / capg : zt * icapg) * cap : zt;
      nll = -((c - mx) - logf(se + PCPB_GUARD));
    }
    rowloss[m] = nll;
  }
  if (!write_grad) return;
  __syncthreads();                                  // the target logit was read above before anyone overwrites it
  const float dtot = valid ? adj_edge<float>(seed / (*count + 2.f * PCPB_GUARD)) : 0.f;     // the one edge that can grow
  const float iden = 1.f / (se + 2.f * PCPB_GUARD);
  const float dzscale = capped ? cap / (capg + PCPB_GUARD) : 1.f;
  for (int v = threadIdx.x; v < nv; v += blockDim.x) {
    float f[8], o[8];
    ld8<T>(z + v * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float th = capped ? m_tanh<T>(sizeof(T) == 4 ? f[i] / capg : f[i] * icapg) : 0.f;
      const float c = capped ? th * cap : f[i];
      float dc = m_exp<T>(c - mx) * iden;
      if ((long long)(v * 8 + i) == t) dc -= 1.f;
      if (c == mx) dc += (2.f * PCPB_GUARD) * iden;
      o[i] = dc * dtot * dzscale * (1.f - th * th);
    }
    st8<T>(z + v * 8, o);
  }
  // every value above is bounded by |dtot| <= 100 unless a logit was not finite, and a logit that is not finite makes
  // the row's sum of exponentials not finite; only then the row is passed through the guard / clamp of the output
  // edge (non-finite -> 0)
  if (!(fabsf(se) < INFINITY) || !(fabsf(mx) < INFINITY)) {
    __syncthreads();
    for (int j = threadIdx.x; j < V; j += blockDim.x) z[j] = from_f<T>(adj_edge<T>(to_f(z[j])));
  }
}
cudaError_t launch_softcap_ce(cudaStream_t st, int dt, void* logits, const long long* targets, int M, int V,
                              float cap, long long ignore, const float* count, float* rowloss, int write_grad, float seed) {
  if (M == 0) return cudaSuccess;
  if (V % 8 == 0 && (((uintptr_t)logits) & 15) == 0) {
    const int threads = V >= 16384 ? 512 : 128;
    DISPATCH_DT(dt, (k_softcap_ce_vec<T><<<M, threads, 0, st>>>((T*)logits, targets, V, cap, ignore, count, rowloss, write_grad, seed)));
    return cudaGetLastError();
  }
  DISPATCH_DT(dt, (k_softcap_ce<T><<<M, 256, 0, st>>>((T*)logits, targets, V, cap, ignore, count, rowloss, write_grad, seed)));
  return cudaGetLastError();
}

__global__ void k_loss_finalize(const float* __restrict__ rowloss, int M, const float* __restrict__ count,
                                float* __restrict__ loss) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < M; i += blockDim.x) s += rowloss[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) *loss = s / (*count + PCPB_GUARD);
}
cudaError_t adj_status_fetch_kernels(cudaStream_t st, int* out, bool clear) { return adj_status_fetch_tu(st, out, clear); }

cudaError_t launch_loss_finalize(cudaStream_t st, const float* rowloss, int M, const float* count, float* loss) {
  k_loss_finalize<<<1, 1024, 0, st>>>(rowloss, M, count, loss);
  return cudaGetLastError();
}

// =================================================================================================
// Fused multi-tensor AdamW (src/optimizers/adam_mlir.zig:50-149), f32, op order kept (no FMA
// contraction) so results match an op-by-op f32 evaluation.
//   pass 1: per-chunk sum of clamp(g,+-1000)^2 -> partial[chunk]
//   pass 2: per-tensor sum of its partials in chunk order -> normsq[tensor]
//   pass 3: update
// =================================================================================================
__global__ void __launch_bounds__(256) k_adam_sumsq(const TensorSeg* __restrict__ segs, const int* __restrict__ c2s,
                                                    float* __restrict__ partial) {
  __shared__ float red[32];
  const int chunk = blockIdx.x;
  const TensorSeg s = segs[c2s[chunk]];
  const long long base = (long long)(chunk - s.first_chunk) * ADAM_CHUNK;
  const long long end = min(base + (long long)ADAM_CHUNK, s.n);
  float acc = 0.f;
  if ((((uintptr_t)s.g) & 15) == 0 && ((end - base) & 3) == 0) {
    for (long long i = base + 4 * threadIdx.x; i < end; i += 4 * blockDim.x) {
      const float4 g4 = *reinterpret_cast<const float4*>(s.g + i);
      const float a = fminf(fmaxf(g4.x, -1000.f), 1000.f), b = fminf(fmaxf(g4.y, -1000.f), 1000.f);
      const float c = fminf(fmaxf(g4.z, -1000.f), 1000.f), d = fminf(fmaxf(g4.w, -1000.f), 1000.f);
      acc += a * a; acc += b * b; acc += c * c; acc += d * d;
    }
  } else {
    for (long long i = base + threadIdx.x; i < end; i += blockDim.x) {
      const float g = fminf(fmaxf(s.g[i], -1000.f), 1000.f);
      acc += g * g;
    }
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) partial[chunk] = acc;
}
__global__ void k_adam_norm(const TensorSeg* __restrict__ segs, const float* __restrict__ partial,
                            float* __restrict__ normsq) {
  __shared__ float red[32];
  const TensorSeg s = segs[blockIdx.x];
  float acc = 0.f;
  for (int c = threadIdx.x; c < s.num_chunks; c += blockDim.x) acc += partial[s.first_chunk + c];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) normsq[blockIdx.x] = acc;
}
__device__ __forceinline__ void adam_elem(float p, float g, float m, float v, float scale, float omb1, float omb2,
                                          const AdamHyper& h, float& pn, float& mn, float& vn) {
  const float gc = __fmul_rn(g, scale);
  mn = __fadd_rn(__fmul_rn(h.beta1, m), __fmul_rn(omb1, gc));
  vn = __fadd_rn(__fmul_rn(h.beta2, v), __fmul_rn(omb2, __fmul_rn(gc, gc)));
  const float mh = __fdiv_rn(mn, h.m_corr), vh = __fdiv_rn(vn, h.v_corr);
  const float ratio = __fdiv_rn(mh, __fadd_rn(__fsqrt_rn(vh), h.eps));
  pn = __fsub_rn(p, __fmul_rn(h.lr, __fadd_rn(ratio, __fmul_rn(h.wd, p))));
}

template <typename T>
__global__ void __launch_bounds__(256) k_adam_update(const TensorSeg* __restrict__ segs, const int* __restrict__ c2s,
                                                     const float* __restrict__ normsq, AdamHyper h, int has_shadow) {
  const int chunk = blockIdx.x;
  const int si = c2s[chunk];
  const TensorSeg s = segs[si];
  const long long base = (long long)(chunk - s.first_chunk) * ADAM_CHUNK;
  const long long end = min(base + (long long)ADAM_CHUNK, s.n);
  const float norm = __fadd_rn(__fsqrt_rn(normsq[si]), h.eps);
  const float scale = __fdiv_rn(h.max_norm, fmaxf(norm, h.max_norm));
  const float omb1 = __fsub_rn(1.f, h.beta1), omb2 = __fsub_rn(1.f, h.beta2);
  const bool shadow = has_shadow && s.shadow;
  const uintptr_t al = (uintptr_t)s.p | (uintptr_t)s.g | (uintptr_t)s.m | (uintptr_t)s.v | (uintptr_t)s.p_out |
                       (uintptr_t)s.m_out | (uintptr_t)s.v_out | (shadow ? (uintptr_t)s.shadow : 0);
  if ((al & 15) == 0 && ((end - base) & 3) == 0) {
    // 16-byte path: four elements per thread and access
    for (long long i = base + 4 * threadIdx.x; i < end; i += 4 * blockDim.x) {
      const float4 p4 = *reinterpret_cast<const float4*>(s.p + i), g4 = *reinterpret_cast<const float4*>(s.g + i);
      const float4 m4 = *reinterpret_cast<const float4*>(s.m + i), v4 = *reinterpret_cast<const float4*>(s.v + i);
      float4 pn, mn, vn;
      adam_elem(p4.x, g4.x, m4.x, v4.x, scale, omb1, omb2, h, pn.x, mn.x, vn.x);
      adam_elem(p4.y, g4.y, m4.y, v4.y, scale, omb1, omb2, h, pn.y, mn.y, vn.y);
      adam_elem(p4.z, g4.z, m4.z, v4.z, scale, omb1, omb2, h, pn.z, mn.z, vn.z);
      adam_elem(p4.w, g4.w, m4.w, v4.w, scale, omb1, omb2, h, pn.w, mn.w, vn.w);
      *reinterpret_cast<float4*>(s.p_out + i) = pn;
      *reinterpret_cast<float4*>(s.m_out + i) = mn;
      *reinterpret_cast<float4*>(s.v_out + i) = vn;
      if (shadow) {
        T* sh = (T*)s.shadow + i;
        if (sizeof(T) == 2) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(pn.x, pn.y), hi = __floats2bfloat162_rn(pn.z, pn.w);
          uint2 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(sh) = pk;
        } else {
          sh[0] = from_f<T>(pn.x); sh[1] = from_f<T>(pn.y); sh[2] = from_f<T>(pn.z); sh[3] = from_f<T>(pn.w);
        }
      }
    }
    return;
  }
  for (long long i = base + threadIdx.x; i < end; i += blockDim.x) {
    float pn, mn, vn;
    adam_elem(s.p[i], s.g[i], s.m[i], s.v[i], scale, omb1, omb2, h, pn, mn, vn);
    s.p_out[i] = pn; s.m_out[i] = mn; s.v_out[i] = vn;
    if (shadow) ((T*)s.shadow)[i] = from_f<T>(pn);
  }
}
cudaError_t launch_adamw(cudaStream_t st, int shadow_dt, const TensorSeg* segs, int nseg, const int* chunk2seg,
                         int nchunks, float* partial, float* normsq, AdamHyper h) {
  if (nseg == 0 || nchunks == 0) return cudaSuccess;
  k_adam_sumsq<<<nchunks, 256, 0, st>>>(segs, chunk2seg, partial);
  k_adam_norm<<<nseg, 256, 0, st>>>(segs, partial, normsq);
  if (shadow_dt == DT_BF16) k_adam_update<bf16><<<nchunks, 256, 0, st>>>(segs, chunk2seg, normsq, h, 1);
  else k_adam_update<float><<<nchunks, 256, 0, st>>>(segs, chunk2seg, normsq, h, shadow_dt == DT_F32 ? 1 : 0);
  return cudaGetLastError();
}

__global__ void k_axpy(float* __restrict__ acc, const float* __restrict__ g, float alpha, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) acc[i] = __fadd_rn(acc[i], __fmul_rn(alpha, g[i]));
}
__global__ void k_scale(float* __restrict__ x, float alpha, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] = __fmul_rn(x[i], alpha);
}
cudaError_t launch_axpy_f32(cudaStream_t st, float* acc, const float* g, float alpha, size_t n) {
  if (n == 0) return cudaSuccess;
  k_axpy<<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(acc, g, alpha, n);
  return cudaGetLastError();
}
cudaError_t launch_scale_f32(cudaStream_t st, float* x, float alpha, size_t n) {
  if (n == 0) return cudaSuccess;
  k_scale<<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(x, alpha, n);
  return cudaGetLastError();
}
template <typename T>
__global__ void k_round_guard(float* __restrict__ x, size_t n, float clip) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = rnd<T>(x[i]);
    if (!((v - v) == 0.f)) v = 0.f;
    x[i] = fminf(fmaxf(v, -clip), clip);
  }
}
cudaError_t launch_round_guard_f32(cudaStream_t st, int dt, float* x, size_t n, float clip) {
  if (n == 0) return cudaSuccess;
  DISPATCH_DT(dt, (k_round_guard<T><<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(x, n, clip)));
  return cudaGetLastError();
}
__global__ void k_check_finite(const float* __restrict__ x, size_t n, int* __restrict__ flag) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  int bad = 0;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) { const float v = x[i]; bad |= !((v - v) == 0.f); }
  if (bad) *flag = 1;
}
cudaError_t launch_check_finite(cudaStream_t st, const float* x, size_t n, int* flag) {
  if (n == 0) return cudaSuccess;
  k_check_finite<<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(x, n, flag);
  return cudaGetLastError();
}

// =================================================================================================
// DiLoCo outer step (src/nodes/workers/worker.zig:1371-1412, src/algorithms/diloco.zig:929-1055,
// src/optimizers/nesterov.zig:82-97)
// =================================================================================================
__global__ void k_delta(const float* __restrict__ t0, const float* __restrict__ t1, float* __restrict__ d, size_t n,
                        int trunc) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = __fsub_rn(t0[i], t1[i]);
    d[i] = trunc ? trunc_bf16(v) : v;
  }
}
cudaError_t launch_delta(cudaStream_t st, const float* theta0, const float* theta, float* delta, size_t n, int trunc) {
  if (n == 0) return cudaSuccess;
  k_delta<<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(theta0, theta, delta, n, trunc);
  return cudaGetLastError();
}

__global__ void __launch_bounds__(256) k_nesterov_shard(OuterArgs a) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float div = (float)a.ncontrib;
  for (; i < a.n; i += stride) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < a.ncontrib) acc = __fadd_rn(acc, a.deltas[w][i]);
    acc = __fdiv_rn(acc, div);
    if (!a.keep_nonfinite && !((acc - acc) == 0.f)) acc = 0.f;
    const float vn = __fadd_rn(__fmul_rn(a.mu, a.vel[i]), acc);
    a.vel[i] = vn;
    float th = __fsub_rn(a.master[i], __fmul_rn(a.lr, __fadd_rn(acc, __fmul_rn(a.mu, vn))));
    if (a.trunc) th = trunc_bf16(th);
    a.master[i] = th;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < a.nouts) a.outs[w][i] = th;
  }
}
// The same arithmetic on four elements per thread with 16-byte accesses (local and peer memory alike): used when every
// pointer is 16-byte aligned, which the shard layout guarantees (shard offsets are multiples of 256 elements).
__global__ void __launch_bounds__(256) k_nesterov_shard_v4(OuterArgs a, long long n4) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float div = (float)a.ncontrib;
  for (; i < n4; i += stride) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < a.ncontrib) {
        const float4 d = reinterpret_cast<const float4*>(a.deltas[w])[i];
        acc[0] = __fadd_rn(acc[0], d.x); acc[1] = __fadd_rn(acc[1], d.y); acc[2] = __fadd_rn(acc[2], d.z); acc[3] = __fadd_rn(acc[3], d.w);
      }
    const float4 v4 = reinterpret_cast<const float4*>(a.vel)[i], m4 = reinterpret_cast<const float4*>(a.master)[i];
    const float vel[4] = {v4.x, v4.y, v4.z, v4.w}, mas[4] = {m4.x, m4.y, m4.z, m4.w};
    float vn[4], th[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float g = __fdiv_rn(acc[k], div);
      if (!a.keep_nonfinite && !((g - g) == 0.f)) g = 0.f;
      vn[k] = __fadd_rn(__fmul_rn(a.mu, vel[k]), g);
      th[k] = __fsub_rn(mas[k], __fmul_rn(a.lr, __fadd_rn(g, __fmul_rn(a.mu, vn[k]))));
      if (a.trunc) th[k] = trunc_bf16(th[k]);
    }
    reinterpret_cast<float4*>(a.vel)[i] = make_float4(vn[0], vn[1], vn[2], vn[3]);
    const float4 out = make_float4(th[0], th[1], th[2], th[3]);
    reinterpret_cast<float4*>(a.master)[i] = out;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < a.nouts) reinterpret_cast<float4*>(a.outs[w])[i] = out;
  }
}
// Streaming DiLoCo worker side (src/nodes/workers/worker.zig:2433-2437 and :2583-2600), f32, no FMA contraction.
__global__ void k_stream_delta(float* __restrict__ snap, const float* __restrict__ theta, float* __restrict__ d, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float cur = theta[i];
    d[i] = __fsub_rn(snap[i], cur);
    snap[i] = cur;
  }
}
__global__ void k_stream_merge(float* __restrict__ theta, const float* __restrict__ glob, float* __restrict__ snap, float alpha,
                               size_t n) {
  const float om = __fsub_rn(1.0f, alpha);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float v = __fadd_rn(__fmul_rn(alpha, theta[i]), __fmul_rn(om, glob[i]));
    theta[i] = v;
    snap[i] = v;
  }
}
cudaError_t launch_stream_delta(cudaStream_t st, float* snapshot, const float* theta, float* delta, size_t n) {
  if (n == 0) return cudaSuccess;
  k_stream_delta<<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(snapshot, theta, delta, n);
  return cudaGetLastError();
}
cudaError_t launch_stream_merge(cudaStream_t st, float* theta, const float* global, float* snapshot, float alpha, size_t n) {
  if (n == 0) return cudaSuccess;
  k_stream_merge<<<min(cdiv(n, 256), 148u * 16), 256, 0, st>>>(theta, global, snapshot, alpha, n);
  return cudaGetLastError();
}

cudaError_t launch_nesterov_shard(cudaStream_t st, const OuterArgs& a) {
  if (a.n == 0) return cudaSuccess;
  uintptr_t all = (uintptr_t)a.vel | (uintptr_t)a.master;
  for (int w = 0; w < a.ncontrib; ++w) all |= (uintptr_t)a.deltas[w];
  for (int w = 0; w < a.nouts; ++w) all |= (uintptr_t)a.outs[w];
  const long long n4 = ((all & 15) == 0) ? a.n / 4 : 0;
  if (n4 > 0) {
    k_nesterov_shard_v4<<<min(cdiv((size_t)n4, 256), 148u * 8), 256, 0, st>>>(a, n4);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || n4 * 4 == a.n) return e;
    OuterArgs t = a;                                       // the last one to three elements
    const long long done = n4 * 4;
    for (int w = 0; w < t.ncontrib; ++w) t.deltas[w] += done;
    for (int w = 0; w < t.nouts; ++w) t.outs[w] += done;
    t.vel += done; t.master += done; t.n = a.n - done;
    k_nesterov_shard<<<1, 32, 0, st>>>(t);
    return cudaGetLastError();
  }
  k_nesterov_shard<<<min(cdiv((size_t)a.n, 256), 148u * 8), 256, 0, st>>>(a);
  return cudaGetLastError();
}

}  // namespace pcpb
