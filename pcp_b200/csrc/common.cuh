// Shared device helpers for the PCP training-step kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pcpb {

// Element-type codes follow the order of DType in the reference (src/core/tensor.zig:9-62).
enum : int { DT_F32 = 0, DT_F64 = 1, DT_F16 = 2, DT_BF16 = 3, DT_I32 = 4, DT_I64 = 5, DT_BOOL = 6 };

static inline size_t dtype_size(int dt) {
  switch (dt) {
    case DT_F32: case DT_I32: return 4;
    case DT_F64: case DT_I64: return 8;
    case DT_F16: case DT_BF16: return 2;
    default: return 1;
  }
}

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

// Round a float to the model dtype and widen again: the value a model-dtype op would hold.
template <typename T> __device__ __forceinline__ float rnd(float x) { return to_f<T>(from_f<T>(x)); }

// f32 -> bf16 by dropping the low 16 bits (the reference's truncating store of deltas and master
// weights, src/nodes/workers/worker.zig:1384, src/algorithms/diloco.zig:1038).
__device__ __forceinline__ float trunc_bf16(float x) {
  return __uint_as_float(__float_as_uint(x) & 0xFFFF0000u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions; `red` is shared memory of >= 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// 8-element vector access (16 bytes of bf16, 32 bytes of f32); p must be 16-byte aligned.
template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&f)[8]);
template <> __device__ __forceinline__ void ld8<float>(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void ld8<bf16>(const bf16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&f)[8]);
template <> __device__ __forceinline__ void st8<float>(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <> __device__ __forceinline__ void st8<bf16>(bf16* p, const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162 h;
  h = __floats2bfloat162_rn(f[0], f[1]); v.x = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(f[2], f[3]); v.y = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(f[4], f[5]); v.z = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(f[6], f[7]); v.w = *reinterpret_cast<uint32_t*>(&h);
  *reinterpret_cast<uint4*>(p) = v;
}

// Transcendentals: accurate for f32 models (1e-4 parity), hardware approximations for bf16 models.
template <typename T> __device__ __forceinline__ float m_tanh(float x) { return tanhf(x); }
template <> __device__ __forceinline__ float m_tanh<bf16>(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T> __device__ __forceinline__ float m_exp(float x) { return expf(x); }
template <> __device__ __forceinline__ float m_exp<bf16>(float x) { return __expf(x); }

// Guard constant the reference adds to every divide / log denominator in the forward graph
// (src/compiler/sanitizer.zig:8-111) and again inside the divide / log / rsqrt VJP rules
// (src/autodiff/vjp_rules.zig:198,1510,1543).
// ---- bf16 pairs in one 32-bit word (low half = first element) ------------------------------------------
// add / mul / max on pairs are single bf16 operations: exact result rounded once to nearest even, which is what
// an op of the exported bf16 graphs computes.
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// Two bf16 products at once: each lane of d = bf16(a * b), round to nearest even.
__device__ __forceinline__ uint32_t bmul2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t badd2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bmax2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }


// ---- tanh-approximated GELU (nanoGPT family, optional activation) ---------------------------------------
// The exported graph writes it as nine ops of model dtype T:
//   x2 = u*u; x3 = x2*u; k = c2*x3; s = u + k; z = c1*s; t = tanh(z); p = t + 1; h = 0.5*u; a = h*p
// with c1 = T(sqrt(2/pi)), c2 = T(0.044715).  gelu_fwd rounds after every op as the graph does.  gelu_grad is
// da/du of the same expression evaluated once in f32 (the reverse-mode graph of the reference sums five adjoint
// contributions in T; for bf16 the single rounding here is the more accurate of the two and inside its tolerance).
#define PCPB_GELU_C1 0.7978845608028654f
#define PCPB_GELU_C2 0.044715f
template <typename T> __device__ __forceinline__ float gelu_fwd(float u) {
  const float c1 = rnd<T>(PCPB_GELU_C1), c2 = rnd<T>(PCPB_GELU_C2);
  const float x2 = rnd<T>(u * u);
  const float x3 = rnd<T>(x2 * u);
  const float k = rnd<T>(c2 * x3);
  const float s = rnd<T>(u + k);
  const float z = rnd<T>(c1 * s);
  const float t = rnd<T>(tanhf(z));                  // accurate also for bf16: the approximation would flip roundings of t
  const float p = rnd<T>(t + 1.f);
  const float h = rnd<T>(0.5f * u);
  return rnd<T>(h * p);
}
template <typename T> __device__ __forceinline__ float gelu_grad(float u) {
  const float c1 = rnd<T>(PCPB_GELU_C1), c2 = rnd<T>(PCPB_GELU_C2);
  const float u2 = u * u;
  const float t = m_tanh<T>(c1 * (u + c2 * u2 * u));
  return 0.5f * (1.f + t) + 0.5f * u * (1.f - t * t) * c1 * (1.f + 3.f * c2 * u2);
}

#define PCPB_GUARD 1e-4f

// ---- adjoint edges ------------------------------------------------------------------------------------------
// The reference's AD engine passes every adjoint a VJP rule produces through the same three steps before it is
// accumulated (src/autodiff/engine.zig:622-682): non-finite -> 0 (tested as (g - g) == 0 in the edge's element type),
// clamp to [-100, 100] in f32, cast back to the element type.  adj_edge<T> is that step for a value computed in f32
// that the rule would hold in T; adj_edge2 the same on a pair of bf16 values.  On healthy models the step changes
// nothing; when it does, bit ADJ_CLAMPED of the status word is set so that the host can tell.  ADJ_INTERNAL is set
// for the fused attention kernels when the adjoints that never leave the chip (dP, dS) cannot be shown to stay inside
// the limit: those kernels use an algebraically fused backward that cannot apply the clamp per edge, so past that
// point their gradients are those of the unclamped arithmetic, clamped where they leave the kernel.
#define PCPB_ADJ_CLIP 100.f
enum : int { ADJ_CLAMPED = 1, ADJ_INTERNAL = 2 };
#ifdef PCPB_ADJ_TU
static __device__ int g_adj_status = 0;       // one per translation unit and device; read through adj_status_fetch()
__device__ __forceinline__ void adj_note(int bit) {
  if (!(*(volatile int*)&g_adj_status & bit)) atomicOr(&g_adj_status, bit);
}
template <typename T> __device__ __forceinline__ float adj_edge(float v) {
  const float r = rnd<T>(v);
  const float c = fminf(fmaxf(((r - r) == 0.f) ? r : 0.f, -PCPB_ADJ_CLIP), PCPB_ADJ_CLIP);
  if (c != r) adj_note(ADJ_CLAMPED);            // also taken for NaN (NaN != anything)
  return c;
}
__device__ __forceinline__ uint32_t bmin2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("min.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t adj_edge2(uint32_t w) {
  // 100.0 = 0x42C8 in bf16.  min / max return one of their operands, so an in-range finite pair comes back bit for bit
  const uint32_t c = bmin2(bmax2(w, 0xC2C8C2C8u), 0x42C842C8u);
  if (c == w) return w;
  adj_note(ADJ_CLAMPED);
  const float lo = bf_lo(w), hi = bf_hi(w);
  const float cl = fminf(fmaxf(((lo - lo) == 0.f) ? lo : 0.f, -PCPB_ADJ_CLIP), PCPB_ADJ_CLIP);
  const float ch = fminf(fmaxf(((hi - hi) == 0.f) ? hi : 0.f, -PCPB_ADJ_CLIP), PCPB_ADJ_CLIP);
  return pack2(cl, ch);
}
// Cheap form for hot loops: compute without the guard while tracking the largest magnitude seen, and only when the
// tracker ends beyond the limit (or saw a NaN / Inf) redo the row / chunk through adj_edge.  The tracker holds |v| as
// a bit pattern: non-negative floats order like unsigned integers, NaN and Inf above every finite value.
__device__ __forceinline__ void adj_track(uint32_t& mx, float v) { mx = max(mx, __float_as_uint(v) & 0x7FFFFFFFu); }
__device__ __forceinline__ bool adj_over(uint32_t mx) { return mx > 0x42C80000u; }             // > 100.0f, NaN, Inf
// the same on bf16 pairs: a packed running maximum of |lo|, |hi| that keeps NaN
__device__ __forceinline__ void adj_track2(uint32_t& mx2, uint32_t w) {
  asm("max.NaN.bf16x2 %0, %0, %1;" : "+r"(mx2) : "r"(w & 0x7FFF7FFFu));
}
__device__ __forceinline__ bool adj_over2(uint32_t mx2) { return (mx2 & 0xFFFFu) > 0x42C8u || (mx2 >> 16) > 0x42C8u; }
// Bound for the adjoints that never leave the fused attention backward (dP = dO V^T and dS = P (dP - D)):
// |dP_ij| <= |dO_i| |V_j| and |dS_ij| <= |dP_ij| + |D_i| (P <= 1), so max|dO_i| max|V_j| + max|D_i| <= 100 proves that
// the reference's clamp on those edges is inactive without touching the kernels' inner loops.  The row statistics are
// gathered by the kernel that prepares D (squared norms and |D| as float bit patterns, combined with atomicMax) and
// evaluated, then cleared, by the first thread of the backward kernel that follows it on the stream.
static __device__ unsigned g_attn_bound[3] = {0u, 0u, 0u};      // max |dO_i|^2, max |D_i|, max |V_j|^2
__device__ __forceinline__ void attn_bound_note(int which, float v) {
  const unsigned bits = __float_as_uint(fabsf(v));             // NaN sorts above every finite value
  if (bits > *(volatile unsigned*)&g_attn_bound[which]) atomicMax(&g_attn_bound[which], bits);
}
__device__ __forceinline__ void attn_bound_check_and_clear() {
  const float a = __uint_as_float(g_attn_bound[0]), dmax = __uint_as_float(g_attn_bound[1]), v = __uint_as_float(g_attn_bound[2]);
  if (!(sqrtf(a) * sqrtf(v) + dmax <= PCPB_ADJ_CLIP)) adj_note(ADJ_INTERNAL);
  g_attn_bound[0] = 0u; g_attn_bound[1] = 0u; g_attn_bound[2] = 0u;
}
// Host access to this translation unit's status word on the current device.
static inline cudaError_t adj_status_fetch_tu(cudaStream_t st, int* out, bool clear) {
  cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_adj_status, sizeof(int), 0, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e == cudaSuccess && clear && *out) {
    const int zero = 0;
    e = cudaMemcpyToSymbolAsync(g_adj_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  }
  return e;
}
#endif

}  // namespace pcpb
