// Rollout generation on the device: batched prefill and greedy decode of a Qwen3-shaped decoder with a paged KV
// cache.  Replaces the reference's one-token-per-call loop with a dense host-side cache
// (src/nodes/workers/generation_engine.zig:174-332) and its host sampler (src/core/math.zig:21-73, greedy branch); the
// arithmetic is that of the decode-step graph the reference exports (tools/export_qwen3_generation.py):
//   weighted RMSNorm -> q / k / v projections -> per-head RMSNorm of q and k -> RoPE (rotate-half, theta 1e6)
//   -> attention over the cache as it was BEFORE the step (the step's own key / value row is written afterwards, so
//      slot `pos` contributes a zero key -- score 0 -- and a zero value; generation_engine.zig:285-312)
//   -> output projection + residual -> weighted RMSNorm -> SwiGLU MLP + residual; final RMSNorm, LM head, argmax.
// bf16 values are rounded where an op of the exported graph would round them (linear layers: f32 accumulation, one
// rounding; the softmax in f32, probabilities rounded after normalisation).
//
// Data layout in HBM
//   weights     one flat bf16 buffer in the argument order of the exported function (= named_parameters() of the
//               Hugging Face model): embed, per layer q k v o q_norm k_norm gate up down input_ln post_ln, norm, lm_head.
//               q, k, v are adjacent, and so are gate, up: each group is one [N, K] panel for one GEMM.
//   KV cache    pages of PAGE tokens: kpages / vpages [layer][page][kv_head][PAGE][head_dim] bf16; block_table
//               [sequence][logical page] -> physical page.  Pages are handed out round-robin over the sequences, so a
//               sequence's pages are not contiguous.
//   decode      activations of the <= 16 sequences in 16-row buffers; every decode step is one CUDA graph launch
//               (token ids and positions live on the device, so the graph does not change from step to step).
//
// Kernels
//   k_gemv16     C[16, N] = X[16, K] W[N, K]^T for the decode step: HBM-bound (every weight byte is read once per
//                step and used for 16 rows).  A CTA owns 8 output columns, its 8 warps split K; a lane streams 16-byte
//                pieces of one weight row and feeds them to mma.sync m16n8k16 with X as the 16-row operand (the k index
//                is permuted the same way for both operands, so no shuffles are needed); partial sums meet in shared
//                memory in warp order (deterministic).  Epilogues: store, residual add, SwiGLU (two panels).
//   prefill GEMMs run on the tcgen05 kernels of gemm_tc.cu (M = prompt tokens, padded to 128).
//   k_attn_rows  one CTA per (token row, kv head): scores of the row's query heads against the cached keys below its
//                position (one key per thread), f32 softmax over them and the zero slot, probabilities rounded to bf16,
//                P V with the keys split over the warps.  Used for prefill rows and decode rows alike.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <stdlib.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../include/pcp_b200.h"
#include "attn_flash.h"
#include "attn_tc.h"
#include "common.cuh"
#include "gemm_tc.h"
#include "kernels.h"

using namespace pcpb;

namespace {

constexpr int ROWS = 16;            // rows of the decode-step operand (sequences per step)
constexpr int PER_LAYER = 11;       // q k v o q_norm k_norm gate up down input_ln post_ln

enum { GV_STORE = 0, GV_RESID = 1, GV_SWIGLU = 2 };
// Warps per GEMV CTA (each takes K / GV_WARPS of the contraction).  Eight warps at <= 64 registers: four resident CTAs
// per SM, 592 slots, so the 512-CTA launches of a layer (N = 4096) run as one wave (at 70 registers ncu showed 444
// slots and a 15 %-full second wave).  Measured alternatives: 4-warp CTAs (8 per SM) were slower for the N = 4096 and
// the SwiGLU launches (30 against 19 us, 67 against 52 us); a cluster of 8 CTAs splitting K with X staged in shared
// memory and a distributed-shared-memory reduction was slower still.
constexpr int GV_WARPS = 8;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ld_stream(const void* p) {      // weights: read once, keep them out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float silu_bf16(float g) { return bf16_round(g / (1.f + expf(-g))); }
// Programmatic dependent launch: the kernels of a decode step are launched so that the next one may start while the
// previous one drains.  A kernel first lets its own dependents go, does whatever does not depend on its predecessor
// (the GEMV: the first pieces of its weight rows, which nothing in a decode step writes), and only then waits for the
// predecessor's results.  Both instructions do nothing in a kernel launched the ordinary way (the prefill).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// C[16, N] (+ epilogue) = X[16, K] * W[N, K]^T.  grid = N / 8, block = GV_WARPS warps, each K / GV_WARPS of the contraction.
// K % 512 == 0 (a warp's share is a multiple of 64), N % 8 == 0.  X rows beyond the batch are zero.
// A lane reads 32 consecutive bytes (16 k values) of its weight row per step, so the four lanes of a row cover a whole
// 128-byte line; those 16 values serve four k16 MMA steps, and X is read with the same permutation of k.
// Which k values a warp takes does not matter for the result's definition (the partial sums are added in warp order):
// by default warp w takes the contiguous slice [w K / 8, (w + 1) K / 8); with kmap_slices == 0 the warps interleave (in
// step i warp w reads the 64 k values at (GV_WARPS i + w) * 64, so that the CTA reads 512 contiguous bytes of each of its
// 8 weight rows at a time), which measured 1 - 2 % slower per decode step.
template <int EPI>
__global__ void __launch_bounds__(GV_WARPS * 32, 4) k_gemv16(const bf16* __restrict__ X, const bf16* __restrict__ W, const bf16* __restrict__ W2,
                                                int N, int K, bf16* __restrict__ C, long long ldc, const bf16* __restrict__ R,
                                                int kmap_slices) {
  __shared__ float red[GV_WARPS][ROWS * 8 * (EPI == GV_SWIGLU ? 2 : 1)];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * 8;
  const int kslice = K / GV_WARPS;
  // element offset of this warp's step at position kb of its slice: contiguous slice, or interleaved 64-element pieces
  const int k0 = kmap_slices ? warp * kslice : warp * 64;
  const int kmul = kmap_slices ? 1 : GV_WARPS;
  const bf16* wrow = W + (size_t)(n0 + g) * K + k0 + 16 * q;
  const bf16* w2row = (EPI == GV_SWIGLU) ? W2 + (size_t)(n0 + g) * K + k0 + 16 * q : nullptr;
  const bf16* xlo = X + (size_t)g * K + k0 + 16 * q;
  const bf16* xhi = X + (size_t)(g + 8) * K + k0 + 16 * q;
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
  constexpr int U = (EPI == GV_SWIGLU) ? 2 : 4;                 // 32-byte weight pieces in flight per lane and panel
  uint4 wv[U][2], w2v[U][2];
  auto load_w = [&](int kb) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool in = kb + 64 * u < kslice;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        wv[u][hlf] = in ? ld_stream(wrow + (kb + 64 * u) * kmul + 8 * hlf) : make_uint4(0, 0, 0, 0);
        if (EPI == GV_SWIGLU) w2v[u][hlf] = in ? ld_stream(w2row + (kb + 64 * u) * kmul + 8 * hlf) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  pdl_launch_dependents();
  load_w(0);                                                    // weights do not depend on the previous kernel
  pdl_wait();                                                   // X (and R) do
  for (int kb = 0; kb < kslice; kb += 64 * U) {
    if (kb > 0) load_w(kb);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (kb + 64 * u >= kslice) break;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        // 8 consecutive k values serve two k16 steps: elements {0,1,2,3} and {4,5,6,7}; the operand X is read with
        // the same permutation of k, so the products line up
        const uint4 a = *reinterpret_cast<const uint4*>(xlo + (kb + 64 * u) * kmul + 8 * hlf);
        const uint4 b = *reinterpret_cast<const uint4*>(xhi + (kb + 64 * u) * kmul + 8 * hlf);
        mma16816(acc, a.x, b.x, a.y, b.y, wv[u][hlf].x, wv[u][hlf].y);
        mma16816(acc, a.z, b.z, a.w, b.w, wv[u][hlf].z, wv[u][hlf].w);
        if (EPI == GV_SWIGLU) {
          mma16816(acc2, a.x, b.x, a.y, b.y, w2v[u][hlf].x, w2v[u][hlf].y);
          mma16816(acc2, a.z, b.z, a.w, b.w, w2v[u][hlf].z, w2v[u][hlf].w);
        }
      }
    }
  }
  // accumulator layout: acc[0], acc[1] = (row g, cols 2q, 2q+1); acc[2], acc[3] = (row g + 8, same cols)
  float* mine = red[warp];
  mine[g * 8 + 2 * q] = acc[0]; mine[g * 8 + 2 * q + 1] = acc[1];
  mine[(g + 8) * 8 + 2 * q] = acc[2]; mine[(g + 8) * 8 + 2 * q + 1] = acc[3];
  if (EPI == GV_SWIGLU) {
    float* m2 = mine + ROWS * 8;
    m2[g * 8 + 2 * q] = acc2[0]; m2[g * 8 + 2 * q + 1] = acc2[1];
    m2[(g + 8) * 8 + 2 * q] = acc2[2]; m2[(g + 8) * 8 + 2 * q + 1] = acc2[3];
  }
  __syncthreads();
  if (threadIdx.x < ROWS * 8) {
    const int r = threadIdx.x >> 3, c = threadIdx.x & 7;
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int w = 0; w < GV_WARPS; ++w) {                        // warp order: the sum does not depend on timing
      s += red[w][threadIdx.x];
      if (EPI == GV_SWIGLU) s2 += red[w][ROWS * 8 + threadIdx.x];
    }
    const size_t o = (size_t)r * ldc + n0 + c;
    float v = bf16_round(s);
    if (EPI == GV_RESID) v = bf16_round(to_f(R[o]) + v);
    if (EPI == GV_SWIGLU) v = bf16_round(silu_bf16(v) * bf16_round(s2));
    C[o] = from_f<bf16>(v);
  }
}

// Wide form of the same product: a CTA of 8 warps owns 64 output columns (warp w the 8 columns n0 + 8 w ..) and the k
// range [blockIdx.y kc, (blockIdx.y + 1) kc); the operand X of that range is staged in shared memory once per CTA (in
// pieces of GW_KC columns) and shared by the 8 warps.  In the 8-column form every CTA fetches all of X: two bytes of X
// from L2 for every weight byte from HBM (ncu: 273 MB into the SMs for 101 MB of DRAM reads), and the X loads sit
// between the arrival of a batch of weights and the issue of the next.  Here X costs a quarter of a byte per weight
// byte and comes out of shared memory.
// The contraction is split over gridDim.y CTAs so that small matrices still fill the GPU.  Partial sums go to `part`
// ([gridDim.y][16][N] f32, a second panel behind it for SwiGLU); the CTA that finds the column block's counter at
// gridDim.y - 1 adds the partials in split order (the result does not depend on which CTA that is), applies the epilogue
// and puts the counter back to 0.  No CTA waits for another.
constexpr int GW_KC = 1024;                                     // columns of X staged at a time
constexpr int GW_LD = GW_KC + 32;                               // shared-memory row stride (elements): rows 64 bytes apart modulo a bank line, so
                                                                // that the 16-byte reads of two rows (8 lanes) miss each other
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
template <int EPI>
__global__ void __launch_bounds__(256, 4) k_gemv16w(const bf16* __restrict__ X, const bf16* __restrict__ W, const bf16* __restrict__ W2,
                                                    int N, int K, int kc, bf16* __restrict__ C, long long ldc, const bf16* __restrict__ R,
                                                    float* __restrict__ part, int* __restrict__ counters) {
  extern __shared__ __align__(16) uint8_t gw_smem[];
  bf16* xs = reinterpret_cast<bf16*>(gw_smem);                  // [16][GW_LD]
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * 64 + warp * 8;
  const bool active = n0 < N;                                   // N % 8 == 0: a warp's 8 columns are all in or all out
  const int kbeg = blockIdx.y * kc;
  const int klen = min(kc, K - kbeg);                           // the last k range may be shorter
  const int nsteps = klen / 64;
  // Per 64-column step a lane reads two 16-byte pieces of its weight row: columns [8 q, 8 q + 8) and [32 + 8 q, 40 + 8 q).
  // The four lanes of a row then cover 64 contiguous bytes, two whole 32-byte sectors, with each load instruction.
  // (With 32 contiguous bytes per lane, one half per instruction, every sector crossed from L2 to the SM twice: ncu
  // showed 241 MB into the SMs for the 101 MB matrix.)  Which k values a lane takes does not matter as long as X is read
  // with the same assignment.
  const bf16* wrow = W + (size_t)(active ? n0 + g : 0) * K + kbeg + 8 * q;
  const bf16* w2row = (EPI == GV_SWIGLU) ? W2 + (size_t)(active ? n0 + g : 0) * K + kbeg + 8 * q : nullptr;
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
  constexpr int U = (EPI == GV_SWIGLU) ? 2 : 4;                 // 32-byte weight pieces in flight per lane and panel
  uint4 wv[U][2], w2v[U][2];
  auto load_w = [&](int s) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool in = active && s + u < nsteps;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        wv[u][hlf] = in ? ld_stream(wrow + (s + u) * 64 + 32 * hlf) : make_uint4(0, 0, 0, 0);
        if (EPI == GV_SWIGLU) w2v[u][hlf] = in ? ld_stream(w2row + (s + u) * 64 + 32 * hlf) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  pdl_launch_dependents();
  load_w(0);                                                    // weights do not depend on the previous kernel
  pdl_wait();                                                   // X (and R, part, counters) do
  for (int s = 0; s < nsteps; s += U) {
    if (s > 0) load_w(s);
    if ((s * 64) % GW_KC == 0) {                                // next piece of X (GW_KC is a multiple of 64 U)
      if (s > 0) __syncthreads();                               // every warp is done with the previous piece
      const int len = min(GW_KC, klen - s * 64);
      const bf16* src = X + kbeg + s * 64;
      for (int i = threadIdx.x; i < ROWS * (len / 8); i += blockDim.x) {
        const int row = i / (len / 8), c8 = i % (len / 8);
        cp_async16(xs + row * GW_LD + c8 * 8, src + (size_t)row * K + c8 * 8);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (s + u >= nsteps) break;
      const int xc = ((s + u) * 64) % GW_KC + 8 * q;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        // 8 consecutive k values serve two k16 steps: elements {0,1,2,3} and {4,5,6,7}; the operand X is read with
        // the same permutation of k, so the products line up
        const uint4 a = *reinterpret_cast<const uint4*>(xs + g * GW_LD + xc + 32 * hlf);
        const uint4 b = *reinterpret_cast<const uint4*>(xs + (g + 8) * GW_LD + xc + 32 * hlf);
        mma16816(acc, a.x, b.x, a.y, b.y, wv[u][hlf].x, wv[u][hlf].y);
        mma16816(acc, a.z, b.z, a.w, b.w, wv[u][hlf].z, wv[u][hlf].w);
        if (EPI == GV_SWIGLU) {
          mma16816(acc2, a.x, b.x, a.y, b.y, w2v[u][hlf].x, w2v[u][hlf].y);
          mma16816(acc2, a.z, b.z, a.w, b.w, w2v[u][hlf].z, w2v[u][hlf].w);
        }
      }
    }
  }
  // accumulator layout: acc[0], acc[1] = (row g, cols 2q, 2q+1); acc[2], acc[3] = (row g + 8, same cols)
  const int splits = gridDim.y;
  const int col = n0 + 2 * q;
  if (splits > 1) {
    if (active) {
      float* mine = part + (size_t)blockIdx.y * ROWS * N;
      *reinterpret_cast<float2*>(mine + (size_t)g * N + col) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(mine + (size_t)(g + 8) * N + col) = make_float2(acc[2], acc[3]);
      if (EPI == GV_SWIGLU) {
        float* m2 = mine + (size_t)splits * ROWS * N;
        *reinterpret_cast<float2*>(m2 + (size_t)g * N + col) = make_float2(acc2[0], acc2[1]);
        *reinterpret_cast<float2*>(m2 + (size_t)(g + 8) * N + col) = make_float2(acc2[2], acc2[3]);
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const int seen = atomicAdd(counters + blockIdx.x, 1);
      s_last = (seen == splits - 1);
      if (s_last) counters[blockIdx.x] = 0;                     // ready for the next launch (launches are serialised)
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (active) {
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      acc2[0] = acc2[1] = acc2[2] = acc2[3] = 0.f;
      for (int sp = 0; sp < splits; ++sp) {                     // split order: the sum does not depend on timing
        const float* src = part + (size_t)sp * ROWS * N;
        const float2 lo = __ldcg(reinterpret_cast<const float2*>(src + (size_t)g * N + col));
        const float2 hi = __ldcg(reinterpret_cast<const float2*>(src + (size_t)(g + 8) * N + col));
        acc[0] += lo.x; acc[1] += lo.y; acc[2] += hi.x; acc[3] += hi.y;
        if (EPI == GV_SWIGLU) {
          const float* s2 = src + (size_t)splits * ROWS * N;
          const float2 lo2 = __ldcg(reinterpret_cast<const float2*>(s2 + (size_t)g * N + col));
          const float2 hi2 = __ldcg(reinterpret_cast<const float2*>(s2 + (size_t)(g + 8) * N + col));
          acc2[0] += lo2.x; acc2[1] += lo2.y; acc2[2] += hi2.x; acc2[3] += hi2.y;
        }
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int hlf = 0; hlf < 2; ++hlf) {
    const size_t o = (size_t)(g + 8 * hlf) * ldc + col;
    float v0 = bf16_round(acc[2 * hlf]), v1 = bf16_round(acc[2 * hlf + 1]);
    if (EPI == GV_RESID) {
      const __nv_bfloat162 rr = *reinterpret_cast<const __nv_bfloat162*>(R + o);
      v0 = bf16_round(__bfloat162float(rr.x) + v0); v1 = bf16_round(__bfloat162float(rr.y) + v1);
    }
    if (EPI == GV_SWIGLU) {
      v0 = bf16_round(silu_bf16(v0) * bf16_round(acc2[2 * hlf]));
      v1 = bf16_round(silu_bf16(v1) * bf16_round(acc2[2 * hlf + 1]));
    }
    *reinterpret_cast<__nv_bfloat162*>(C + o) = __floats2bfloat162_rn(v0, v1);
  }
}

// rows of the embedding table -> h [M, d]; tokens outside the table are clamped like a gather's start indices
__global__ void k_embed_rows(const bf16* __restrict__ emb, const long long* __restrict__ tok, int M, int d, int V,
                             bf16* __restrict__ h) {
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x;
  if (m >= M) return;
  long long t = tok[m];
  t = t < 0 ? 0 : (t >= V ? V - 1 : t);
  const uint4* src = reinterpret_cast<const uint4*>(emb + (size_t)t * d);
  uint4* dst = reinterpret_cast<uint4*>(h + (size_t)m * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

// Qwen3RMSNorm: y = w * bf16(x * rsqrt(mean(x^2) + eps)), statistics in f32.  One block per row; a thread keeps its
// 16-byte pieces of the row in registers between the statistics and the output (one read of the row).  `gather`
// (optional) selects the source row of output row m.  d % 8 == 0, d <= 8 * 4 * blockDim.
__global__ void __launch_bounds__(256) k_rmsnorm_w(const bf16* __restrict__ x, const bf16* __restrict__ w, const int* __restrict__ gather,
                                                   int M, int d, float eps, bf16* __restrict__ y) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x;
  const bf16* xr = x + (size_t)(gather ? gather[m] : m) * d;
  const int nv = d >> 3;
  constexpr int MAXV = 4;
  float f[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nv) {
      ld8<bf16>(xr + v * 8, f[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[k][i] * f[k][i];
    }
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)d + eps);
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nv) {
      float wf[8], o[8];
      ld8<bf16>(w + v * 8, wf);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = wf[i] * bf16_round(f[k][i] * r);
      st8<bf16>(y + (size_t)m * d + v * 8, o);
    }
  }
}

// act = bf16(silu(gate)) * up on [M, 2f] -> [M, f] (prefill; the decode step has this in the GEMV epilogue); f % 8 == 0
__global__ void k_swiglu(const bf16* __restrict__ gu, int M, int f, bf16* __restrict__ act) {
  const size_t nv = (size_t)M * (f >> 3), fv = (size_t)(f >> 3);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / fv, c = (i % fv) * 8;
    float g[8], u[8], o[8];
    ld8<bf16>(gu + m * 2 * f + c, g);
    ld8<bf16>(gu + m * 2 * f + f + c, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = silu_bf16(g[k]) * u[k];
    st8<bf16>(act + m * (size_t)f + c, o);
  }
}

struct RowMap {                     // which sequence and position a token row belongs to
  const int* seq;                   // [M]
  const int* pos;                   // [M]
};

// Per (row, head): q and k heads get the weighted RMSNorm over head_dim, then RoPE; q is divided by sqrt(head_dim) and
// stored to qbuf [M, H*hd]; k and v go into the row's cache slot.  One warp per head, head_dim = 128 or 64.
__global__ void __launch_bounds__(256) k_qknorm_rope_cache(const bf16* __restrict__ qkv, const bf16* __restrict__ qn, const bf16* __restrict__ kn,
                                                           const bf16* __restrict__ cosT, const bf16* __restrict__ sinT, RowMap map, int M, int H,
                                                           int Hkv, int hd, float eps, const int* __restrict__ block_table,
                                                           int max_pages, int page, bf16* __restrict__ kpages, bf16* __restrict__ vpages,
                                                           bf16* __restrict__ qbuf, bf16* __restrict__ sqk, bf16* __restrict__ sqv, int Tseq) {
  pdl_launch_dependents();
  pdl_wait();
  const int heads = H + 2 * Hkv;
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)M * heads) return;
  const int m = (int)(gw / heads), h = (int)(gw % heads);
  const int sq = map.seq[m], pos = map.pos[m];
  if (sq < 0) return;                                           // padding row
  const int per = hd / 32;                                      // elements per lane: 4 (hd 128) or 2 (hd 64)
  const bf16* src = qkv + (size_t)m * heads * hd + (size_t)h * hd + lane * per;
  float v[4];
  for (int i = 0; i < per; ++i) v[i] = to_f(src[i]);
  const int pg = block_table[sq * max_pages + pos / page], off = pos % page;
  // sqk / sqv (prefill on the tensor-core attention kernel): q of row m in row m, k and v of row m in row m + 1 of the
  // same sequence -- with a zero row at position 0 the ordinary causal kernel then sees, for the query at position p,
  // the zero slot and the keys below p, which is what the exported step attends to
  const bool stage_next = sqk && pos + 1 < Tseq;
  if (h >= H + Hkv) {                                           // value head: stored as projected
    bf16* dst = vpages + (((size_t)pg * Hkv + (h - H - Hkv)) * page + off) * hd + lane * per;
    for (int i = 0; i < per; ++i) dst[i] = from_f<bf16>(v[i]);
    if (stage_next) {
      bf16* d2 = sqv + (size_t)(m + 1) * (H + 2 * Hkv) * hd + (size_t)h * hd + lane * per;
      for (int i = 0; i < per; ++i) d2[i] = from_f<bf16>(v[i]);
    }
    return;
  }
  const bf16* wn = (h < H) ? qn : kn;
  float ss = 0.f;
  for (int i = 0; i < per; ++i) ss += v[i] * v[i];
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)hd + eps);
  float y[4];
  for (int i = 0; i < per; ++i) y[i] = bf16_round(to_f(wn[lane * per + i]) * bf16_round(v[i] * r));
  // rotate_half: element i pairs with i + hd/2 (lanes 16 apart); out = y*cos + rot*sin, rot = -y[i+half] (i < half), y[i-half] else
  const bool low = lane < 16;
  float o[4];
  for (int i = 0; i < per; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, y[i], 16);
    const int e = lane * per + i;
    const float c = to_f(cosT[(size_t)pos * hd + e]), s = to_f(sinT[(size_t)pos * hd + e]);
    const float rot = low ? -partner : partner;
    o[i] = bf16_round(bf16_round(y[i] * c) + bf16_round(rot * s));
  }
  if (h < H) {
    const float sc = sqrtf((float)hd);
    bf16* dst = sqk ? sqk + (size_t)m * (H + Hkv) * hd + (size_t)h * hd + lane * per
                    : qbuf + (size_t)m * H * hd + (size_t)h * hd + lane * per;
    for (int i = 0; i < per; ++i) dst[i] = from_f<bf16>(o[i] / sc);
  } else {
    bf16* dst = kpages + (((size_t)pg * Hkv + (h - H)) * page + off) * hd + lane * per;
    for (int i = 0; i < per; ++i) dst[i] = from_f<bf16>(o[i]);
    if (stage_next) {
      bf16* d2 = sqk + (size_t)(m + 1) * (H + Hkv) * hd + (size_t)h * hd + lane * per;
      for (int i = 0; i < per; ++i) d2[i] = from_f<bf16>(o[i]);
    }
  }
}

// Attention of one token row against the cache below its position, for the G query heads of one kv head.
// grid = (M, Hkv), block = ATT_THREADS.  Dynamic shared memory: q [G][hd] f32, p [G][npos_max] f32, partial out [warps][G][hd] f32.
// ATT_THREADS: 1024 for the decode step (few CTAs, hundreds of keys each: the keys of both passes are spread over 32
// warps), 256 for prefill rows (thousands of CTAs with few keys each).
template <int HD, int G, int ATT_THREADS>
__global__ void __launch_bounds__(ATT_THREADS) k_attn_rows(const bf16* __restrict__ qbuf, RowMap map, int H, int Hkv, const int* __restrict__ block_table,
                                                   int max_pages, int page, const bf16* __restrict__ kpages, const bf16* __restrict__ vpages,
                                                   int npos_max, bf16* __restrict__ out) {
  extern __shared__ float sm[];
  constexpr int ATT_WARPS = ATT_THREADS / 32;
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x, kvh = blockIdx.y;
  const int sq = map.seq[m], pos = map.pos[m];
  if (sq < 0) return;
  float* qs = sm;                          // [G][HD]
  float* ps = qs + G * HD;                 // [G][npos_max]
  float* po = ps + (size_t)G * npos_max;   // [ATT_WARPS][G][HD]
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x)
    qs[i] = to_f(qbuf[(size_t)m * H * HD + (size_t)(kvh * G) * HD + i]);
  __syncthreads();
  const int* bt = block_table + sq * max_pages;
  // pass 1: one key per thread, G dot products per key; the product of the matmul is a bf16 value
  for (int j = threadIdx.x; j < pos; j += blockDim.x) {
    const bf16* kr = kpages + (((size_t)bt[j / page] * Hkv + kvh) * page + (j % page)) * HD;
    float d[G];
#pragma unroll
    for (int g = 0; g < G; ++g) d[g] = 0.f;
#pragma unroll 4
    for (int c = 0; c < HD / 8; ++c) {
      float kf[8];
      ld8<bf16>(kr + c * 8, kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float* qg = qs + g * HD + c * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) d[g] = fmaf(qg[e], kf[e], d[g]);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) ps[(size_t)g * npos_max + j] = bf16_round(d[g]);
  }
  __syncthreads();
  // softmax in f32 over the keys below pos and the zero slot at pos (score 0, value 0); later slots carry -1e4 on a
  // zero score and underflow to weight 0.  All G heads are reduced together: two block-wide exchanges in all.
  {
    const int warp_ = threadIdx.x >> 5, lane_ = threadIdx.x & 31;
    float mx[G], se[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      mx[g] = 0.f;                                               // the zero slot
      const float* pg = ps + (size_t)g * npos_max;
      for (int j = threadIdx.x; j < pos; j += blockDim.x) mx[g] = fmaxf(mx[g], pg[j]);
      mx[g] = warp_max(mx[g]);
      if (lane_ == 0) po[warp_ * G + g] = mx[g];
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float m = 0.f;
      for (int w = 0; w < ATT_WARPS; ++w) m = fmaxf(m, po[w * G + g]);
      mx[g] = m;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* pg = ps + (size_t)g * npos_max;
      float sum = 0.f;
      for (int j = threadIdx.x; j < pos; j += blockDim.x) { const float e = expf(pg[j] - mx[g]); pg[j] = e; sum += e; }
      sum = warp_sum(sum);
      if (lane_ == 0) po[warp_ * G + g] = sum;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sum = 0.f;
      for (int w = 0; w < ATT_WARPS; ++w) sum += po[w * G + g];     // warp order: the same sum in every thread
      se[g] = sum + expf(0.f - mx[g]);
    }
    // a thread normalises the entries it wrote itself: no barrier needed in between
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float* pg = ps + (size_t)g * npos_max;
      for (int j = threadIdx.x; j < pos; j += blockDim.x) pg[j] = bf16_round(pg[j] / se[g]);
    }
  }
  __syncthreads();
  // pass 2: P V.  The keys are split over the warps; a lane owns HD / 32 consecutive output elements of every head.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int PER = HD / 32;
  float acc[G][PER];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[g][e] = 0.f;
#pragma unroll 8
  for (int j = warp; j < pos; j += ATT_WARPS) {
    const bf16* vr = vpages + (((size_t)bt[j / page] * Hkv + kvh) * page + (j % page)) * HD + lane * PER;
    float vf[PER];
    if (PER == 4) {
      const uint2 raw = *reinterpret_cast<const uint2*>(vr);          // one 8-byte load per lane: a 256-byte row per warp
      vf[0] = bf_lo(raw.x); vf[1] = bf_hi(raw.x); vf[2 % PER] = bf_lo(raw.y); vf[3 % PER] = bf_hi(raw.y);
    } else {
      const uint32_t raw = *reinterpret_cast<const uint32_t*>(vr);
      vf[0] = bf_lo(raw); vf[1] = bf_hi(raw);
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float p = ps[(size_t)g * npos_max + j];
#pragma unroll
      for (int e = 0; e < PER; ++e) acc[g][e] = fmaf(p, vf[e], acc[g][e]);
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < PER; ++e) po[((size_t)warp * G + g) * HD + lane * PER + e] = acc[g][e];
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    float s = 0.f;
    for (int w = 0; w < ATT_WARPS; ++w) s += po[(size_t)w * G * HD + i];
    out[(size_t)m * H * HD + (size_t)(kvh * G) * HD + i] = from_f<bf16>(s);
  }
}

// Sampler.argmax (src/core/math.zig:61-73): the first maximum wins, NaN never wins.  Two stages: ARG_CHUNKS blocks per
// row each find the first maximum of a slice of the row (16-byte loads), then one warp per row picks the first maximum
// among the slices; the winner becomes the row's next input token, is recorded at out[row][step] and the row's position
// advances.
constexpr int ARG_CHUNKS = 32;
__device__ __forceinline__ bool arg_better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }
__global__ void __launch_bounds__(256) k_argmax_part(const bf16* __restrict__ logits, int V, long long ldl, float* __restrict__ pval,
                                                     int* __restrict__ pidx) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const bf16* z = logits + (size_t)row * ldl;
  const int nv = V >> 3, per = (nv + ARG_CHUNKS - 1) / ARG_CHUNKS;
  const int v0 = chunk * per, v1 = min(nv, v0 + per);
  float best = -INFINITY;
  int at = 0x7fffffff;
  for (int v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    float f[8];
    ld8<bf16>(z + v * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (f[i] > best) { best = f[i]; at = v * 8 + i; }          // ascending scan: the lowest index of the maximum
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, at, o);
    if (arg_better(ov, oi, best, at)) { best = ov; at = oi; }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) { bv[w] = best; bi[w] = at; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; ++k)
      if (arg_better(bv[k], bi[k], best, at)) { best = bv[k]; at = bi[k]; }
    pval[row * ARG_CHUNKS + chunk] = best; pidx[row * ARG_CHUNKS + chunk] = at;
  }
}
__global__ void __launch_bounds__(32) k_argmax_advance(const float* __restrict__ pval, const int* __restrict__ pidx, long long* __restrict__ cur_tok,
                                                       int* __restrict__ cur_pos, long long* __restrict__ out, int max_new,
                                                       const int* __restrict__ step, int advance) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x;
  float best = lane < ARG_CHUNKS ? pval[row * ARG_CHUNKS + lane] : -INFINITY;
  int at = lane < ARG_CHUNKS ? pidx[row * ARG_CHUNKS + lane] : 0x7fffffff;
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, at, o);
    if (arg_better(ov, oi, best, at)) { best = ov; at = oi; }
  }
  if (lane == 0) {
    const long long tok = (at == 0x7fffffff) ? 0 : at;         // all -inf / NaN: index 0, as the reference's scan
    const int s = *step;
    if (s < max_new) out[(size_t)row * max_new + s] = tok;
    cur_tok[row] = tok;
    if (advance) cur_pos[row] += 1;
  }
}
__global__ void k_bump(int* step) {
  pdl_launch_dependents();
  pdl_wait();
  *step += 1;
}

// N(0, std) bf16 weights from a counter-based generator: for benchmark set-up only (the reference loads a weight
// blob; generating 8 x 10^9 values on the host would take minutes).
__global__ void k_random_normal_bf16(bf16* __restrict__ w, size_t n, unsigned long long seed, float std) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u1 = ((float)(z >> 40) + 1.f) * (1.f / 16777216.f), u2 = (float)((z >> 16) & 0xFFFFFF) * (1.f / 16777216.f);
    w[i] = from_f<bf16>(std * sqrtf(-2.f * logf(u1)) * cosf(6.2831853f * u2));
  }
}
__global__ void k_fill_bf16(bf16* __restrict__ w, size_t n, float v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) w[i] = from_f<bf16>(v);
}
__global__ void k_f32_to_bf16(const float* __restrict__ in, bf16* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = from_f<bf16>(in[i]);
}

}  // namespace

struct pcpb_rollout {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::string err;
  pcpb_rollout_cfg cfg{};
  std::vector<void*> allocs;
  bf16* wflat = nullptr;
  std::vector<size_t> woff;          // element offset of every tensor in wflat
  size_t nweights = 0;
  bool have_weights = false;
  // geometry
  int hq = 0, hk = 0, max_rows = 0, max_pages = 0, n_pages = 0;
  // activations: prefill-sized (max_rows rows) and the 16-row decode set
  bf16 *h = nullptr, *h2 = nullptr, *x = nullptr, *qkv = nullptr, *q = nullptr, *att = nullptr, *gu = nullptr, *act = nullptr;
  bf16 *dh = nullptr, *dh2 = nullptr, *dx = nullptr, *dqkv = nullptr, *dq = nullptr, *datt = nullptr, *dact = nullptr, *logits = nullptr;
  bf16 *kpages = nullptr, *vpages = nullptr, *cosT = nullptr, *sinT = nullptr;
  bf16 *sqk = nullptr, *sqv = nullptr;   // prefill staging for the tensor-core attention: [rows, hq + hk] (q | shifted k), [rows, hq + 2 hk] (v part: shifted v)
  float *att_m = nullptr, *att_l = nullptr;
  int *block_table = nullptr, *row_seq = nullptr, *row_pos = nullptr, *last_row = nullptr, *drow_seq = nullptr, *cur_pos = nullptr,
      *step = nullptr, *tc_err = nullptr;
  long long *row_tok = nullptr, *cur_tok = nullptr, *out_tok = nullptr;
  float* arg_val = nullptr;          // [16][ARG_CHUNKS] first maxima of the logit slices
  int* arg_idx = nullptr;
  int out_cap = 0;
  cudaGraphExec_t graph = nullptr;
  int graph_batch = 0, graph_maxnew = 0;
  long long graph_launches = 0;      // kernels in one replay of the decode-step graph
  float* gv_part = nullptr;          // split-K partial sums of the wide decode GEMV
  int* gv_cnt = nullptr;             // one arrival counter per 64-column block (back at 0 after every launch)
  int gv_wide = 1, gv_slots = 592;        // PCPB_ROLLOUT_GEMV=narrow: the 8-column kernel; gv_slots: resident CTAs (4 per SM)
  int kmap_slices = 1;               // 1: every warp one contiguous K / 8 slice (default); 0: interleaved 128-byte pieces
  bool no_tc_prefill = false;             // PCPB_ROLLOUT_PREFILL=rows: the row kernel also for aligned prompts
  bool use_pdl = true, pdl_now = false;   // programmatic dependent launch inside the decode step (PCPB_ROLLOUT_PDL=0: off)
  cudaEvent_t e0 = nullptr, e1 = nullptr, e2 = nullptr;
  long long launches = 0;
};

namespace {

int rfail(pcpb_rollout* r, int code, const std::string& msg) {
  if (r) r->err = msg;
  return code;
}
#define RCK(r, call)                                                                                         \
  do {                                                                                                       \
    cudaError_t e__ = (call);                                                                                \
    if (e__ != cudaSuccess) {                                                                                \
      char m__[384];                                                                                         \
      snprintf(m__, sizeof m__, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
      (r)->err = m__;                                                                                        \
      return PCPB_E_CUDA;                                                                                    \
    }                                                                                                        \
  } while (0)

template <typename P> int ralloc(pcpb_rollout* r, P** out, size_t bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    char m[200];
    snprintf(m, sizeof m, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    r->err = m;
    return PCPB_E_CUDA;
  }
  r->allocs.push_back(p);
  *out = (P*)p;
  return PCPB_OK;
}
#define RA(r, ptr, bytes) do { int rc__ = ralloc(r, &(ptr), (bytes)); if (rc__) return rc__; } while (0)

struct Guard {
  int prev = -1;
  explicit Guard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
  ~Guard() { if (prev >= 0) cudaSetDevice(prev); }
};

// Kernel launch on the engine's stream.  While a decode step is being enqueued (r->pdl_now) the launch carries the
// programmatic-serialisation attribute, so that the kernel may start while its predecessor drains; the kernels wait
// for their predecessor themselves (pdl_wait) before they touch anything it produces.
template <typename... KA, typename... A>
cudaError_t klaunch(pcpb_rollout* r, void (*kern)(KA...), dim3 grid, dim3 block, size_t smem, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = r->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = r->pdl_now ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KA>(args)...);
}

std::vector<std::vector<long long>> param_shapes(const pcpb_rollout_cfg& c) {
  const long long d = c.d_model, hq = (long long)c.n_head * c.head_dim, hk = (long long)c.n_kv_head * c.head_dim, f = c.d_ff;
  std::vector<std::vector<long long>> s;
  s.push_back({c.vocab, d});
  for (int l = 0; l < c.n_layer; ++l) {
    s.push_back({hq, d}); s.push_back({hk, d}); s.push_back({hk, d}); s.push_back({d, hq});
    s.push_back({c.head_dim}); s.push_back({c.head_dim});
    s.push_back({f, d}); s.push_back({f, d}); s.push_back({d, f}); s.push_back({d}); s.push_back({d});
  }
  s.push_back({d}); s.push_back({c.vocab, d});
  return s;
}

const bf16* W(const pcpb_rollout* r, int i) { return r->wflat + r->woff[i]; }

// C[M, N] = A[M, K] Wt[N, K]^T (+ residual) on the tcgen05 kernels (prefill); falls back to the generic kernel
int big_gemm(pcpb_rollout* r, const bf16* A, const bf16* Wt, bf16* C, int M, int N, int K, int epi, const bf16* R) {
  GemmArgs g;
  g.A = A; g.sam = K; g.sak = 1; g.B = Wt; g.sbk = 1; g.sbn = K; g.C = C; g.ldc = N; g.R = R; g.C2 = nullptr;
  g.M = M; g.N = N; g.K = K; g.epi = epi; g.clip = 100.f; g.err_word = r->tc_err;
  r->launches += 1;
  if (gemm_tc_supported(g)) RCK(r, launch_gemm_tc(r->stream, g));
  else RCK(r, launch_gemm_generic(r->stream, DT_BF16, g));
  return PCPB_OK;
}

// Split of the contraction for the wide GEMV into k ranges of `kc` columns (a multiple of 64; the last range may be
// shorter).  Matrices with fewer column blocks than CTA slots (4 per SM): as many ranges as keep the launch within one
// wave of resident CTAs, so that no second, mostly empty wave follows (768 CTAs on 592 slots ran as two).  Larger
// matrices (the LM head): ranges of at most 256 KB of weights per CTA, many waves.
struct GvPlan { int splits, kc; };
GvPlan gv_plan(int N, int K, bool swiglu, int slots) {
  const int blocks = (N + 63) / 64, steps = K / 64;
  int sp;
  if (blocks <= slots) sp = std::max(1, std::min(steps, slots / blocks));
  else sp = std::max(1, (int)(((size_t)64 * K * 2 * (swiglu ? 2 : 1) + 256 * 1024 - 1) / (256 * 1024)));
  const int kc_steps = (steps + sp - 1) / sp;
  return GvPlan{(steps + kc_steps - 1) / kc_steps, kc_steps * 64};
}
size_t gv_part_elems(int N, int K, bool swiglu, int slots) {
  const GvPlan pl = gv_plan(N, K, swiglu, slots);
  return pl.splits > 1 ? (size_t)pl.splits * ROWS * N * (swiglu ? 2 : 1) : 0;
}

int gemv(pcpb_rollout* r, int epi, const bf16* X, const bf16* Wt, const bf16* W2, int N, int K, bf16* C, long long ldc, const bf16* R) {
  r->launches += 1;
  const bf16* none = nullptr;
  if (r->gv_wide) {
    const GvPlan pl = gv_plan(N, K, epi == GV_SWIGLU, r->gv_slots);
    const int kc = pl.kc;
    const dim3 grid((N + 63) / 64, pl.splits), block(256);
    const size_t smem = (size_t)ROWS * GW_LD * 2;
    if (epi == GV_STORE) RCK(r, klaunch(r, k_gemv16w<GV_STORE>, grid, block, smem, X, Wt, none, N, K, kc, C, ldc, none, r->gv_part, r->gv_cnt));
    else if (epi == GV_RESID) RCK(r, klaunch(r, k_gemv16w<GV_RESID>, grid, block, smem, X, Wt, none, N, K, kc, C, ldc, R, r->gv_part, r->gv_cnt));
    else RCK(r, klaunch(r, k_gemv16w<GV_SWIGLU>, grid, block, smem, X, Wt, W2, N, K, kc, C, ldc, none, r->gv_part, r->gv_cnt));
    return PCPB_OK;
  }
  if (epi == GV_STORE) RCK(r, klaunch(r, k_gemv16<GV_STORE>, dim3(N / 8), dim3(GV_WARPS * 32), 0, X, Wt, none, N, K, C, ldc, none, r->kmap_slices));
  else if (epi == GV_RESID) RCK(r, klaunch(r, k_gemv16<GV_RESID>, dim3(N / 8), dim3(GV_WARPS * 32), 0, X, Wt, none, N, K, C, ldc, R, r->kmap_slices));
  else RCK(r, klaunch(r, k_gemv16<GV_SWIGLU>, dim3(N / 8), dim3(GV_WARPS * 32), 0, X, Wt, W2, N, K, C, ldc, none, r->kmap_slices));
  return PCPB_OK;
}

size_t attn_smem(const pcpb_rollout_cfg& c, int threads = 1024) {
  const int G = c.n_head / c.n_kv_head;
  return ((size_t)G * c.head_dim + (size_t)G * c.max_seq + (size_t)(threads / 32) * G * c.head_dim) * sizeof(float);
}

template <int HD, int G>
void attn_launch(pcpb_rollout* r, const bf16* q, RowMap map, int M, const bf16* kp, const bf16* vp, bf16* out, bool set_attr) {
  const pcpb_rollout_cfg& c = r->cfg;
  if (set_attr) {
    cudaFuncSetAttribute(k_attn_rows<HD, G, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem(c, 1024));
    cudaFuncSetAttribute(k_attn_rows<HD, G, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem(c, 256));
    return;
  }
  if (M <= ROWS)
    klaunch(r, k_attn_rows<HD, G, 1024>, dim3(M, c.n_kv_head), dim3(1024), attn_smem(c, 1024), q, map, c.n_head, c.n_kv_head,
            (const int*)r->block_table, r->max_pages, c.page_tokens, kp, vp, c.max_seq, out);
  else
    klaunch(r, k_attn_rows<HD, G, 256>, dim3(M, c.n_kv_head), dim3(256), attn_smem(c, 256), q, map, c.n_head, c.n_kv_head,
            (const int*)r->block_table, r->max_pages, c.page_tokens, kp, vp, c.max_seq, out);
}
template <int HD>
void attn_dispatch(pcpb_rollout* r, const bf16* q, RowMap map, int M, const bf16* kp, const bf16* vp, bf16* out, bool set_attr) {
  switch (r->cfg.n_head / r->cfg.n_kv_head) {
    case 1: attn_launch<HD, 1>(r, q, map, M, kp, vp, out, set_attr); break;
    case 2: attn_launch<HD, 2>(r, q, map, M, kp, vp, out, set_attr); break;
    case 4: attn_launch<HD, 4>(r, q, map, M, kp, vp, out, set_attr); break;
    default: attn_launch<HD, 8>(r, q, map, M, kp, vp, out, set_attr); break;
  }
}
// kp / vp: the layer's pages
int attention(pcpb_rollout* r, const bf16* q, const int* rs, const int* rp, int M, const bf16* kp, const bf16* vp, bf16* out,
              bool set_attr = false) {
  RowMap map{rs, rp};
  if (!set_attr) r->launches += 1;
  if (r->cfg.head_dim == 128) attn_dispatch<128>(r, q, map, M, kp, vp, out, set_attr);
  else attn_dispatch<64>(r, q, map, M, kp, vp, out, set_attr);
  RCK(r, cudaGetLastError());
  return PCPB_OK;
}

// One pass over the layers for M token rows.  decode: the 16-row buffers and the GEMV kernels; else prefill.
// tc_T > 0 (prefill only): every sequence has tc_T prompt rows, a multiple of 128, and head_dim is 128: the attention runs
// on the tcgen05 kernel over staged q / shifted k, v buffers instead of the row kernel.
int layers(pcpb_rollout* r, bool decode, int M, const int* rs, const int* rp, int tc_T = 0) {
  const pcpb_rollout_cfg& c = r->cfg;
  const bool tc_attn = !decode && tc_T > 0;
  if (tc_attn) {
    // position 0 of every sequence: the zero slot (k and v parts of the first row of each sequence)
    const size_t wk = (size_t)(c.n_head + c.n_kv_head) * c.head_dim, wv = (size_t)(c.n_head + 2 * c.n_kv_head) * c.head_dim;
    RCK(r, cudaMemset2DAsync(r->sqk + (size_t)c.n_head * c.head_dim, (size_t)tc_T * wk * 2, 0, (size_t)c.n_kv_head * c.head_dim * 2,
                             (size_t)(M / tc_T), r->stream));
    RCK(r, cudaMemset2DAsync(r->sqv + (size_t)(c.n_head + c.n_kv_head) * c.head_dim, (size_t)tc_T * wv * 2, 0,
                             (size_t)c.n_kv_head * c.head_dim * 2, (size_t)(M / tc_T), r->stream));
  }
  const int d = c.d_model, f = c.d_ff, hq = r->hq, hk = r->hk, nqkv = hq + 2 * hk;
  cudaStream_t st = r->stream;
  bf16 *h = decode ? r->dh : r->h, *h2 = decode ? r->dh2 : r->h2, *x = decode ? r->dx : r->x, *qkv = decode ? r->dqkv : r->qkv;
  bf16 *q = decode ? r->dq : r->q, *att = decode ? r->datt : r->att, *act = decode ? r->dact : r->act;
  const int Mp = decode ? ROWS : (M + 127) / 128 * 128;          // rows the GEMMs run over
  RowMap map{rs, rp};
  for (int l = 0; l < c.n_layer; ++l) {
    const int p0 = 1 + PER_LAYER * l;
    int rc;
    r->launches += 1;
    RCK(r, klaunch(r, k_rmsnorm_w, dim3(M), dim3(256), 0, (const bf16*)h, W(r, p0 + 9), (const int*)nullptr, M, d, c.rms_eps, x));
    if (decode) { if ((rc = gemv(r, GV_STORE, x, W(r, p0), nullptr, nqkv, d, qkv, nqkv, nullptr))) return rc; }
    else if ((rc = big_gemm(r, x, W(r, p0), qkv, Mp, nqkv, d, EPI_STORE, nullptr))) return rc;
    const long long warps = (long long)M * (c.n_head + 2 * c.n_kv_head);
    const size_t layer_pages = (size_t)l * r->n_pages * c.n_kv_head * c.page_tokens * c.head_dim;
    bf16 *kp = r->kpages + layer_pages, *vp = r->vpages + layer_pages;
    r->launches += 1;
    RCK(r, klaunch(r, k_qknorm_rope_cache, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, (const bf16*)qkv, W(r, p0 + 4),
                   W(r, p0 + 5), (const bf16*)r->cosT, (const bf16*)r->sinT, map, M, c.n_head, c.n_kv_head, c.head_dim, c.rms_eps,
                   (const int*)r->block_table, r->max_pages, c.page_tokens, kp, vp, q, tc_attn ? r->sqk : (bf16*)nullptr,
                   tc_attn ? r->sqv : (bf16*)nullptr, tc_T));
    // the row's own key / value are in the cache now, but its attention reads only the slots below its position
    if (tc_attn) {
      FlashArgs fa{};
      fa.qkn = r->sqk; fa.qkv = r->sqv; fa.o = att; fa.mrow = r->att_m; fa.lrow = r->att_l;
      fa.B = M / tc_T; fa.T = tc_T; fa.H = c.n_head; fa.Hkv = c.n_kv_head; fa.hd = c.head_dim; fa.scale = 1.f; fa.no_guard = 1;
      r->launches += 1;
      RCK(r, launch_attn_tc_fwd(st, fa, r->tc_err));
    } else if ((rc = attention(r, q, rs, rp, M, kp, vp, att))) return rc;
    if (decode) { if ((rc = gemv(r, GV_RESID, att, W(r, p0 + 3), nullptr, d, hq, h2, d, h))) return rc; }
    else if ((rc = big_gemm(r, att, W(r, p0 + 3), h2, Mp, d, hq, EPI_RESID, h))) return rc;
    r->launches += 1;
    RCK(r, klaunch(r, k_rmsnorm_w, dim3(M), dim3(256), 0, (const bf16*)h2, W(r, p0 + 10), (const int*)nullptr, M, d, c.rms_eps, x));
    if (decode) {
      if ((rc = gemv(r, GV_SWIGLU, x, W(r, p0 + 6), W(r, p0 + 7), f, d, act, f, nullptr))) return rc;
      if ((rc = gemv(r, GV_RESID, act, W(r, p0 + 8), nullptr, d, f, h, d, h2))) return rc;
    } else {
      if ((rc = big_gemm(r, x, W(r, p0 + 6), r->gu, Mp, 2 * f, d, EPI_STORE, nullptr))) return rc;
      r->launches += 1;
      k_swiglu<<<148 * 8, 256, 0, st>>>(r->gu, M, f, act);
      if ((rc = big_gemm(r, act, W(r, p0 + 8), h, Mp, d, f, EPI_RESID, h2))) return rc;
    }
  }
  RCK(r, cudaGetLastError());
  return PCPB_OK;
}

// final norm of the given rows (gathered), LM head, argmax -> next tokens
int head_and_sample(pcpb_rollout* r, const bf16* hsrc, const int* gather, int B, int max_new, int advance) {
  const pcpb_rollout_cfg& c = r->cfg;
  r->launches += 4;
  RCK(r, klaunch(r, k_rmsnorm_w, dim3(B), dim3(256), 0, hsrc, W(r, (int)r->nweights - 2), gather, B, c.d_model, c.rms_eps, r->dx));
  int rc = gemv(r, GV_STORE, r->dx, W(r, (int)r->nweights - 1), nullptr, c.vocab, c.d_model, r->logits, c.vocab, nullptr);
  if (rc) return rc;
  RCK(r, klaunch(r, k_argmax_part, dim3(ARG_CHUNKS, B), dim3(256), 0, (const bf16*)r->logits, c.vocab, (long long)c.vocab, r->arg_val, r->arg_idx));
  RCK(r, klaunch(r, k_argmax_advance, dim3(B), dim3(32), 0, (const float*)r->arg_val, (const int*)r->arg_idx, r->cur_tok, r->cur_pos, r->out_tok,
                 max_new, (const int*)r->step, advance));
  RCK(r, klaunch(r, k_bump, dim3(1), dim3(1), 0, r->step));
  RCK(r, cudaGetLastError());
  return PCPB_OK;
}

int decode_step_enqueue(pcpb_rollout* r, int B, int max_new) {
  const pcpb_rollout_cfg& c = r->cfg;
  r->launches += 1;
  r->pdl_now = r->use_pdl;
  cudaError_t e = klaunch(r, k_embed_rows, dim3(B), dim3(128), 0, W(r, 0), (const long long*)r->cur_tok, B, c.d_model, c.vocab, r->dh);
  int rc = PCPB_OK;
  if (e != cudaSuccess) rc = rfail(r, PCPB_E_CUDA, std::string("decode step launch failed: ") + cudaGetErrorString(e));
  if (!rc) rc = layers(r, true, B, r->drow_seq, r->cur_pos);
  if (!rc) rc = head_and_sample(r, r->dh, nullptr, B, max_new, 1);
  r->pdl_now = false;
  return rc;
}

}  // namespace

extern "C" {

const char* pcpb_rollout_last_error(const pcpb_rollout* r) { return r ? r->err.c_str() : "null rollout engine"; }

void pcpb_rollout_destroy(pcpb_rollout* r) {
  if (!r) return;
  Guard g(r->device);
  if (r->stream) cudaStreamSynchronize(r->stream);
  if (r->graph) cudaGraphExecDestroy(r->graph);
  for (void* p : r->allocs) cudaFree(p);
  for (cudaEvent_t e : {r->e0, r->e1, r->e2}) if (e) cudaEventDestroy(e);
  if (r->stream) cudaStreamDestroy(r->stream);
  delete r;
}

long long pcpb_rollout_num_params(const pcpb_rollout_cfg* c) {
  if (!c) return -1;
  long long n = 0;
  for (auto& s : param_shapes(*c)) { long long e = 1; for (long long v : s) e *= v; n += e; }
  return n;
}

int pcpb_rollout_create(int device, const pcpb_rollout_cfg* cfg, pcpb_rollout** out) {
  if (!out || !cfg) return PCPB_E_INVALID;
  pcpb_rollout* r = new pcpb_rollout();
  *out = r;                                            // returned even on failure so that the message can be read
  r->device = device; r->cfg = *cfg;
  const pcpb_rollout_cfg& c = r->cfg;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return rfail(r, PCPB_E_CUDA, "no CUDA device");
  if (device < 0 || device >= ndev) return rfail(r, PCPB_E_INVALID, "device ordinal out of range");
  if (c.vocab < 8 || c.d_model < 256 || c.n_layer < 1 || c.n_head < 1 || c.n_kv_head < 1 || c.d_ff < 256 || c.max_seq < 2 ||
      c.page_tokens < 1 || c.max_batch < 1 || c.max_prompt < 1)
    return rfail(r, PCPB_E_INVALID, "bad rollout configuration");
  if (c.head_dim != 128 && c.head_dim != 64) return rfail(r, PCPB_E_INVALID, "head_dim must be 64 or 128");
  {
    const int G = c.n_head % c.n_kv_head ? 0 : c.n_head / c.n_kv_head;
    if (G != 1 && G != 2 && G != 4 && G != 8) return rfail(r, PCPB_E_INVALID, "query heads must be 1, 2, 4 or 8 times the kv heads");
  }
  if (c.max_batch > ROWS) return rfail(r, PCPB_E_TOO_LARGE, "at most 16 sequences per step");
  r->hq = c.n_head * c.head_dim; r->hk = c.n_kv_head * c.head_dim;
  // the decode GEMV splits K over 8 warps in pieces of 64 and N in pieces of 8
  if (c.d_model % 512 || c.d_ff % 512 || r->hq % 512 || c.vocab % 8 || r->hk % 8)
    return rfail(r, PCPB_E_INVALID, "d_model, d_ff and n_head*head_dim must be multiples of 512, vocab of 8");
  if (c.max_prompt > c.max_seq) return rfail(r, PCPB_E_INVALID, "max_prompt exceeds max_seq");
  if (c.d_model > 8 * 4 * 256) return rfail(r, PCPB_E_TOO_LARGE, "d_model beyond 8192 is not supported by the norm kernel");
  Guard g(device);
  RCK(r, cudaSetDevice(device));
  cudaDeviceProp prop;
  RCK(r, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return rfail(r, PCPB_E_CUDA, "this library is built for sm_100a (B200) only");
  if (attn_smem(c) > 200 * 1024) return rfail(r, PCPB_E_TOO_LARGE, "max_seq too long for the attention kernel's shared memory");
  RCK(r, cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking));
  RCK(r, cudaEventCreate(&r->e0)); RCK(r, cudaEventCreate(&r->e1)); RCK(r, cudaEventCreate(&r->e2));
  // weights
  size_t off = 0;
  for (auto& s : param_shapes(c)) {
    size_t n = 1; for (long long v : s) n *= (size_t)v;
    r->woff.push_back(off);
    off += (n + 7) / 8 * 8;                                   // every tensor starts on a 16-byte boundary
  }
  r->nweights = r->woff.size();
  RA(r, r->wflat, off * sizeof(bf16));
  r->woff.push_back(off);
  // geometry of the buffers
  r->max_rows = ((size_t)c.max_batch * c.max_prompt + 127) / 128 * 128;
  r->max_pages = (c.max_seq + c.page_tokens - 1) / c.page_tokens;
  r->n_pages = r->max_pages * c.max_batch;
  const size_t d = c.d_model, f = c.d_ff, nqkv = r->hq + 2 * r->hk, MR = r->max_rows;
  RA(r, r->h, MR * d * 2); RA(r, r->h2, MR * d * 2); RA(r, r->x, MR * d * 2); RA(r, r->qkv, MR * nqkv * 2);
  RA(r, r->q, MR * r->hq * 2); RA(r, r->att, MR * r->hq * 2);
  if (c.head_dim == 128) {
    RA(r, r->sqk, MR * (size_t)(r->hq + r->hk) * 2); RA(r, r->sqv, MR * nqkv * 2);
    RA(r, r->att_m, MR * (size_t)c.n_head * 4); RA(r, r->att_l, MR * (size_t)c.n_head * 4);
  } RA(r, r->gu, MR * 2 * f * 2); RA(r, r->act, MR * f * 2);
  RA(r, r->dh, ROWS * d * 2); RA(r, r->dh2, ROWS * d * 2); RA(r, r->dx, ROWS * d * 2); RA(r, r->dqkv, ROWS * nqkv * 2);
  RA(r, r->dq, ROWS * (size_t)r->hq * 2); RA(r, r->datt, ROWS * (size_t)r->hq * 2); RA(r, r->dact, ROWS * f * 2);
  RA(r, r->logits, ROWS * (size_t)c.vocab * 2);
  const size_t cache = (size_t)c.n_layer * r->n_pages * c.n_kv_head * c.page_tokens * c.head_dim;
  RA(r, r->kpages, cache * 2); RA(r, r->vpages, cache * 2);
  RA(r, r->cosT, (size_t)c.max_seq * c.head_dim * 2); RA(r, r->sinT, (size_t)c.max_seq * c.head_dim * 2);
  RA(r, r->block_table, (size_t)c.max_batch * r->max_pages * 4);
  RA(r, r->row_seq, MR * 4); RA(r, r->row_pos, MR * 4); RA(r, r->row_tok, MR * 8); RA(r, r->last_row, ROWS * 4);
  RA(r, r->drow_seq, ROWS * 4); RA(r, r->cur_pos, ROWS * 4); RA(r, r->cur_tok, ROWS * 8); RA(r, r->step, 4); RA(r, r->tc_err, 4);
  RCK(r, cudaMemset(r->tc_err, 0, 4));
  RA(r, r->arg_val, ROWS * ARG_CHUNKS * 4); RA(r, r->arg_idx, ROWS * ARG_CHUNKS * 4);
  {
    const char* e = getenv("PCPB_ROLLOUT_GEMV");
    r->gv_wide = !(e && !strcmp(e, "narrow"));
    {
      int sms = 148;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, r->device);
      r->gv_slots = 4 * (sms > 0 ? sms : 148);
    }
    e = getenv("PCPB_ROLLOUT_GEMV_CTAS");                  // for comparisons
    if (e && atoi(e) > 0) r->gv_slots = atoi(e);
    const int mc = r->gv_slots, nqkv = r->hq + 2 * r->hk;
    size_t pe = gv_part_elems(nqkv, (int)d, false, mc);
    pe = std::max(pe, gv_part_elems((int)d, r->hq, false, mc));
    pe = std::max(pe, gv_part_elems(c.d_ff, (int)d, true, mc));
    pe = std::max(pe, gv_part_elems((int)d, c.d_ff, false, mc));
    pe = std::max(pe, gv_part_elems(c.vocab, (int)d, false, mc));
    RA(r, r->gv_part, pe * 4);
    const size_t nb = (size_t)(std::max(std::max(nqkv, c.d_ff), c.vocab) + 63) / 64;
    RA(r, r->gv_cnt, nb * 4);
    RCK(r, cudaMemset(r->gv_cnt, 0, nb * 4));
  }
  // rows beyond the batch stay zero in the 16-row operands of the decode GEMV
  RCK(r, cudaMemset(r->dh, 0, ROWS * d * 2)); RCK(r, cudaMemset(r->dh2, 0, ROWS * d * 2)); RCK(r, cudaMemset(r->dx, 0, ROWS * d * 2));
  RCK(r, cudaMemset(r->dq, 0, ROWS * (size_t)r->hq * 2)); RCK(r, cudaMemset(r->datt, 0, ROWS * (size_t)r->hq * 2));
  RCK(r, cudaMemset(r->dact, 0, ROWS * f * 2)); RCK(r, cudaMemset(r->dqkv, 0, ROWS * nqkv * 2));
  // RoPE tables: cos / sin of pos * theta^(-2i/hd) in f32, emb = cat(freqs, freqs), rounded to bf16
  {
    const int half = c.head_dim / 2;
    std::vector<uint16_t> ct((size_t)c.max_seq * c.head_dim), stb(ct.size());
    auto tobf = [](float v) { uint32_t u; memcpy(&u, &v, 4); u = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16; return (uint16_t)u; };
    for (int p = 0; p < c.max_seq; ++p)
      for (int i = 0; i < half; ++i) {
        const float inv = (float)(1.0 / pow((double)c.rope_theta, 2.0 * i / c.head_dim));
        const float fr = (float)p * inv;
        const uint16_t cv = tobf(cosf(fr)), sv = tobf(sinf(fr));
        ct[(size_t)p * c.head_dim + i] = ct[(size_t)p * c.head_dim + half + i] = cv;
        stb[(size_t)p * c.head_dim + i] = stb[(size_t)p * c.head_dim + half + i] = sv;
      }
    RCK(r, cudaMemcpy(r->cosT, ct.data(), ct.size() * 2, cudaMemcpyHostToDevice));
    RCK(r, cudaMemcpy(r->sinT, stb.data(), stb.size() * 2, cudaMemcpyHostToDevice));
  }
  { int rc = attention(r, nullptr, nullptr, nullptr, 0, nullptr, nullptr, nullptr, true); if (rc) return rc; }
  {
    const char* e = getenv("PCPB_ROLLOUT_KMAP");          // "interleave": 128-byte pieces of a row go round the warps (for comparisons)
    r->kmap_slices = (e && !strcmp(e, "interleave")) ? 0 : 1;
    e = getenv("PCPB_ROLLOUT_PREFILL");
    r->no_tc_prefill = e && !strcmp(e, "rows");
    e = getenv("PCPB_ROLLOUT_PDL");
    r->use_pdl = !(e && e[0] == '0');
  }
  return PCPB_OK;
}

int pcpb_rollout_load_weights(pcpb_rollout* r, const void* blob, size_t nbytes, int dtype) {
  if (!r || !r->stream) return PCPB_E_INVALID;
  if (!blob) return rfail(r, PCPB_E_INVALID, "null weight blob");
  if (dtype != PCPB_F32 && dtype != PCPB_BF16) return rfail(r, PCPB_E_INVALID, "weight blob must be f32 or bf16");
  Guard g(r->device);
  const size_t es = dtype == PCPB_F32 ? 4 : 2;
  const long long total = pcpb_rollout_num_params(&r->cfg);
  if (nbytes != (size_t)total * es) return rfail(r, PCPB_E_INVALID, "weight blob has the wrong length");
  // tensor after tensor in argument order, tightly packed (generation_engine.zig:101-113); f32 is rounded to bf16
  auto shapes = param_shapes(r->cfg);
  size_t src = 0;
  float* stage = nullptr;
  size_t stage_cap = 0;
  for (size_t i = 0; i < shapes.size(); ++i) {
    size_t n = 1; for (long long v : shapes[i]) n *= (size_t)v;
    if (dtype == PCPB_BF16) {
      RCK(r, cudaMemcpyAsync(r->wflat + r->woff[i], (const char*)blob + src * 2, n * 2, cudaMemcpyHostToDevice, r->stream));
    } else {
      if (stage_cap < n) {
        if (stage) { RCK(r, cudaStreamSynchronize(r->stream)); cudaFree(stage); }
        RCK(r, cudaMalloc(&stage, n * 4));
        stage_cap = n;
      }
      RCK(r, cudaMemcpyAsync(stage, (const char*)blob + src * 4, n * 4, cudaMemcpyHostToDevice, r->stream));
      k_f32_to_bf16<<<148 * 8, 256, 0, r->stream>>>(stage, r->wflat + r->woff[i], n);
    }
    src += n;
  }
  RCK(r, cudaStreamSynchronize(r->stream));
  if (stage) cudaFree(stage);
  r->have_weights = true;
  return PCPB_OK;
}

int pcpb_rollout_random_weights(pcpb_rollout* r, uint64_t seed, float std) {
  if (!r || !r->stream) return PCPB_E_INVALID;
  Guard g(r->device);
  auto shapes = param_shapes(r->cfg);
  for (size_t i = 0; i < shapes.size(); ++i) {
    size_t n = 1; for (long long v : shapes[i]) n *= (size_t)v;
    if (shapes[i].size() == 1) k_fill_bf16<<<64, 256, 0, r->stream>>>(r->wflat + r->woff[i], n, 1.f);       // norm weights at 1
    else k_random_normal_bf16<<<148 * 16, 256, 0, r->stream>>>(r->wflat + r->woff[i], n, seed + 0x1000003ull * i, std);
  }
  RCK(r, cudaGetLastError());
  RCK(r, cudaStreamSynchronize(r->stream));
  r->have_weights = true;
  return PCPB_OK;
}

int pcpb_rollout_generate(pcpb_rollout* r, const int64_t* prompts, const int* prompt_lens, int batch, int prompt_stride,
                          int max_new_tokens, int64_t eos_token, float temperature, int64_t* tokens_out, int* n_generated,
                          int* finish_reason, double* prefill_ms, double* decode_ms) {
  if (!r || !r->stream) return PCPB_E_INVALID;
  const pcpb_rollout_cfg& c = r->cfg;
  if (!r->have_weights) return rfail(r, PCPB_E_STATE, "no weights loaded (pcpb_rollout_load_weights)");
  if (!prompts || !prompt_lens || !tokens_out || !n_generated || batch < 1 || batch > c.max_batch || max_new_tokens < 1)
    return rfail(r, PCPB_E_INVALID, "bad generate arguments");
  if (!(temperature < 1e-6f)) return rfail(r, PCPB_E_INVALID, "only greedy decoding (temperature < 1e-6) runs on the device");
  Guard g(r->device);
  // token rows of the prefill: an empty prompt is the single input token 0 (generation_engine.zig:233-240)
  std::vector<int> rs, rp, last(batch), lens(batch);
  std::vector<long long> rt;
  for (int b = 0; b < batch; ++b) {
    const int len = prompt_lens[b];
    if (len < 0 || len > c.max_prompt || len > prompt_stride) return rfail(r, PCPB_E_INVALID, "prompt length out of range");
    lens[b] = len > 0 ? len : 1;
    if (lens[b] + max_new_tokens - 1 > c.max_seq) return rfail(r, PCPB_E_TOO_LARGE, "prompt + new tokens exceed max_seq");
    for (int p = 0; p < lens[b]; ++p) { rs.push_back(b); rp.push_back(p); rt.push_back(len > 0 ? prompts[(size_t)b * prompt_stride + p] : 0); }
    last[b] = (int)rs.size() - 1;
  }
  const int M = (int)rs.size();
  if (M > r->max_rows) return rfail(r, PCPB_E_TOO_LARGE, "more prompt tokens than max_batch * max_prompt");
  // pages: handed out round-robin over the sequences, so that no sequence's pages are contiguous
  std::vector<int> bt((size_t)c.max_batch * r->max_pages, 0);
  {
    int next = 0;
    for (int lp = 0; lp < r->max_pages; ++lp)
      for (int b = 0; b < batch; ++b)
        if (lp * c.page_tokens < lens[b] + max_new_tokens) bt[(size_t)b * r->max_pages + lp] = next++;
    if (next > r->n_pages) return rfail(r, PCPB_E_TOO_LARGE, "KV cache pages exhausted");
  }
  if (r->out_cap < ROWS * max_new_tokens) { RA(r, r->out_tok, (size_t)ROWS * max_new_tokens * 8); r->out_cap = ROWS * max_new_tokens; }
  cudaStream_t st = r->stream;
  std::vector<int> dseq(ROWS, -1), dpos(ROWS, 0);
  for (int b = 0; b < batch; ++b) { dseq[b] = b; dpos[b] = lens[b]; }
  RCK(r, cudaMemcpyAsync(r->block_table, bt.data(), bt.size() * 4, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemcpyAsync(r->row_seq, rs.data(), (size_t)M * 4, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemcpyAsync(r->row_pos, rp.data(), (size_t)M * 4, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemcpyAsync(r->row_tok, rt.data(), (size_t)M * 8, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemcpyAsync(r->last_row, last.data(), (size_t)batch * 4, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemcpyAsync(r->drow_seq, dseq.data(), ROWS * 4, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemcpyAsync(r->cur_pos, dpos.data(), ROWS * 4, cudaMemcpyHostToDevice, st));
  RCK(r, cudaMemsetAsync(r->step, 0, 4, st));
  RCK(r, cudaMemsetAsync(r->out_tok, 0, (size_t)ROWS * max_new_tokens * 8, st));
  // ---- prefill: all prompt tokens at once; the first new token comes from each sequence's last prompt row ----
  RCK(r, cudaEventRecord(r->e0, st));
  const int Mp = (M + 127) / 128 * 128;
  if (Mp > M) RCK(r, cudaMemsetAsync(r->h + (size_t)M * c.d_model, 0, (size_t)(Mp - M) * c.d_model * 2, st));
  r->launches += 1;
  k_embed_rows<<<M, 128, 0, st>>>(W(r, 0), r->row_tok, M, c.d_model, c.vocab, r->h);
  // equal prompt lengths that are a multiple of 128 (and head_dim 128): prefill attention on the tensor-core kernel
  int tc_T = 0;
  {
    bool same = r->sqk != nullptr && lens[0] % 128 == 0 && !r->no_tc_prefill;
    for (int b = 1; b < batch && same; ++b) same = lens[b] == lens[0];
    if (same) {
      FlashArgs fa{};
      fa.qkn = r->sqk; fa.qkv = r->sqv; fa.o = r->att; fa.B = batch; fa.T = lens[0]; fa.H = c.n_head; fa.Hkv = c.n_kv_head; fa.hd = c.head_dim;
      if (attn_tc_supported(fa)) tc_T = lens[0];
    }
  }
  int rc = layers(r, false, M, r->row_seq, r->row_pos, tc_T);
  if (rc) return rc;
  if ((rc = head_and_sample(r, r->h, r->last_row, batch, max_new_tokens, 0))) return rc;
  RCK(r, cudaEventRecord(r->e1, st));
  // ---- decode: one graph launch per step ----
  if (max_new_tokens > 1) {
    if (!r->graph || r->graph_batch != batch || r->graph_maxnew != max_new_tokens) {
      if (r->graph) { cudaGraphExecDestroy(r->graph); r->graph = nullptr; }
      cudaGraph_t gr = nullptr;
      RCK(r, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
      const long long before = r->launches;
      rc = decode_step_enqueue(r, batch, max_new_tokens);
      r->graph_launches = r->launches - before;
      r->launches = before;
      cudaError_t ce = cudaStreamEndCapture(st, &gr);
      if (rc) { if (gr) cudaGraphDestroy(gr); return rc; }
      RCK(r, ce);
      ce = cudaGraphInstantiate(&r->graph, gr, 0);
      cudaGraphDestroy(gr);
      RCK(r, ce);
      r->graph_batch = batch; r->graph_maxnew = max_new_tokens;
    }
    for (int s = 1; s < max_new_tokens; ++s) RCK(r, cudaGraphLaunch(r->graph, st));
    r->launches += r->graph_launches * (max_new_tokens - 1);
  }
  RCK(r, cudaEventRecord(r->e2, st));
  std::vector<long long> host((size_t)ROWS * max_new_tokens);
  RCK(r, cudaMemcpyAsync(host.data(), r->out_tok, host.size() * 8, cudaMemcpyDeviceToHost, st));
  int tcerr = 0;
  RCK(r, cudaMemcpyAsync(&tcerr, r->tc_err, 4, cudaMemcpyDeviceToHost, st));
  RCK(r, cudaStreamSynchronize(st));
  if (tcerr) { cudaMemset(r->tc_err, 0, 4); return rfail(r, PCPB_E_CUDA, "a tensor-core kernel gave up waiting on a barrier during prefill"); }
  float ms = 0.f;
  if (prefill_ms) { RCK(r, cudaEventElapsedTime(&ms, r->e0, r->e1)); *prefill_ms = ms; }
  if (decode_ms) { RCK(r, cudaEventElapsedTime(&ms, r->e1, r->e2)); *decode_ms = ms; }
  // the host loop's stopping rule (generation_engine.zig:270-276): stop at eos_token, else after max_new_tokens
  for (int b = 0; b < batch; ++b) {
    int n = max_new_tokens, why = 0;                           // 0 = "length", 1 = "stop"
    for (int s = 0; s < max_new_tokens; ++s) {
      tokens_out[(size_t)b * max_new_tokens + s] = host[(size_t)b * max_new_tokens + s];
      if (host[(size_t)b * max_new_tokens + s] == eos_token) { n = s + 1; why = 1; break; }
    }
    for (int s = n; s < max_new_tokens; ++s) tokens_out[(size_t)b * max_new_tokens + s] = 0;
    n_generated[b] = n;
    if (finish_reason) finish_reason[b] = why;
  }
  return PCPB_OK;
}

int pcpb_rollout_read_logits(pcpb_rollout* r, int row, float* dst, size_t n) {
  if (!r || !r->stream || !dst || row < 0 || row >= ROWS || n != (size_t)r->cfg.vocab) return PCPB_E_INVALID;
  Guard g(r->device);
  std::vector<uint16_t> tmp(n);
  RCK(r, cudaMemcpyAsync(tmp.data(), r->logits + (size_t)row * r->cfg.vocab, n * 2, cudaMemcpyDeviceToHost, r->stream));
  RCK(r, cudaStreamSynchronize(r->stream));
  for (size_t i = 0; i < n; ++i) { const uint32_t u = (uint32_t)tmp[i] << 16; memcpy(dst + i, &u, 4); }
  return PCPB_OK;
}

long long pcpb_rollout_launch_count(const pcpb_rollout* r) { return r ? r->launches : 0; }

}  // extern "C"
