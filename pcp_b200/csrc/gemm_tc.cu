// bf16 GEMM on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the accumulator in tensor
// memory, operand tiles staged in shared memory by TMA (128-byte swizzle), one persistent CTA per SM.
//
//   C[M,N] = sum_k A(m,k) B(k,n)       A, B bf16; f32 accumulate; epilogues of kernels.h
//
// Tile 128 x BN (BN = 256 or 128) x 64.  Warp roles (320 threads):
//   warp 0      TMA producer: fills the NSTAGE-deep ring of (A tile, B tile) pairs
//   warp 1      allocates tensor memory; one elected lane issues tcgen05.mma and commits
//   warps 2..9  epilogue: tcgen05.ld of one accumulator buffer (32 lanes per warp, half of the columns), epilogue
//               math, stores; the residual / pre-activation operand is prefetched while the MMAs run
// Two accumulator buffers of BN columns each let the epilogue of tile i overlap the MMAs of tile i+1.
//
// Operand layouts.  Either operand may be "K-major" (contraction index contiguous in memory) or
// "MN-major" (the M / N index contiguous); the three GEMMs of a linear layer need all combinations:
//   forward   Y = X W^T      A K-major,  B K-major
//   dgrad     dX = dY W      A K-major,  B MN-major
//   wgrad     dW = dY^T X    A MN-major, B MN-major      (long contraction: split over CTAs, f32 slabs)
// K-major tile in shared memory: rows of 64 elements (128 B), 8-row groups 1024 B apart.
// MN-major tile: chunks of 64 M/N-elements; inside a chunk one 128 B row per k, 8-row groups 1024 B apart,
// chunks 8192 B apart.
//
// Every mbarrier wait is bounded: after the limit the kernel sets an error word, stops issuing work, waits
// (bounded) for its own TMA copies still in flight, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define PCPB_ADJ_TU
#include "gemm_tc.h"
#include "tc_common.cuh"

namespace pcpb {

namespace {

constexpr int BM = 128, BK = 64;
constexpr int N_EPI = 8;                                  // epilogue warps
constexpr int GEMM_THREADS = 64 + 32 * N_EPI;
constexpr int A_TILE_BYTES = BM * BK * 2;                 // 16 KB

struct TcParams {
  int M, N, K;                 // output rows, output cols, contraction length
  int tiles_m, tiles_n, splits, kb_per_split;
  int group_m;                 // row tiles per group of the tile order (1 = plain row-major order)
  int epi;
  int adj;                     // EPI_STORE: the output is an activation gradient (an adjoint edge: guard + clamp)
  int wide;                    // 1: rows of C / C2 / R start on 32-byte boundaries, so 256-bit accesses may be used
  void* C; long long ldc;
  const void* R; void* C2;
  float clip;
  float* slab;                 // split-K partial sums [splits][M][N] (f32)
  int* err;
};

// Epilogue of 32 consecutive columns of one output row held as f32 bit patterns in r[].
// rpre: the 32 values of the per-element operand R for these columns (residual / pre-activation), loaded by the
// caller ahead of time; only read by the epilogues that have such an operand.
__device__ __forceinline__ void epilogue_chunk(const TcParams& p, int row, int col, const uint32_t (&r)[32], const uint4* rpre) {
  float acc[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(r[i]);
  const size_t o = (size_t)row * p.ldc + col;
  if (p.epi == EPI_WGRAD || p.epi < 0) {                      // f32 outputs
    float* dst = (p.epi < 0) ? p.slab + o : (float*)p.C + o;
    if (p.epi == EPI_WGRAD) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float v = bf16_round(acc[i]);
        if (!((v - v) == 0.f)) v = 0.f;
        acc[i] = fminf(fmaxf(v, -p.clip), p.clip);
      }
    }
    if (p.wide) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 lo = make_uint4(__float_as_uint(acc[8 * i]), __float_as_uint(acc[8 * i + 1]), __float_as_uint(acc[8 * i + 2]), __float_as_uint(acc[8 * i + 3]));
        const uint4 hi = make_uint4(__float_as_uint(acc[8 * i + 4]), __float_as_uint(acc[8 * i + 5]), __float_as_uint(acc[8 * i + 6]), __float_as_uint(acc[8 * i + 7]));
        st_global_256(dst + 8 * i, lo, hi);
      }
      return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<float4*>(dst)[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
    return;
  }
  // bf16 outputs, two per 32-bit word.  Every step after the packing is one bf16 operation of the exported graph:
  // the dot result is rounded to bf16, and add / mul / max on bf16 pairs round their exact result once, as its ops do.
  __nv_bfloat16* C = (__nv_bfloat16*)p.C + o;
  if (p.epi == EPI_BIAS) {
    // the graph adds the bias to the f32 dot result and rounds once
    const uint4* bp = reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.R + col);      // bias[N], model dtype
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float xb[8];
      unpack8(bp[q], xb);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[8 * q + i] += xb[i];
    }
  }
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) w[j] = pack2(acc[2 * j], acc[2 * j + 1]);
  const uint32_t* x = reinterpret_cast<const uint32_t*>(rpre);     // per-element operand, when the epilogue has one
  // The product of a backward GEMM is an output of the dot_general VJP, i.e. an adjoint edge of the reference's engine
  // (src/autodiff/engine.zig:622-682): non-finite -> 0, clamp to +-100.  One min and one max per pair when in range.
  // Hot path: a running maximum of the magnitudes (two instructions per pair), one test per 32 columns; the guard and
  // clamp themselves only run for a chunk that needs them.
  const bool backward = p.adj || p.epi == EPI_DRELU || p.epi == EPI_DRELU2 || p.epi == EPI_DGELU;
  if (backward) {
    uint32_t mx2 = 0u;
#pragma unroll
    for (int j = 0; j < 16; ++j) adj_track2(mx2, w[j]);
    if (adj_over2(mx2)) {
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] = adj_edge2(w[j]);
    }
  }
  if (p.epi == EPI_RESID) {
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = badd2(x[j], w[j]);
  } else if (p.epi == EPI_DRELU) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t lo = bf_lo(x[j]) > 0.f ? (w[j] & 0xFFFFu) : 0u, hi = bf_hi(x[j]) > 0.f ? (w[j] & 0xFFFF0000u) : 0u;
      w[j] = lo | hi;
    }
  } else if (p.epi == EPI_DRELU2) {
    // backward of a = power(max(u,0), 2):  da * bf16(2 * bf16(bf16(r*r) / r)), r = max(u, 0); zero where u <= 0.
    // The quotient of two bf16 values is never a rounding tie of bf16 and is at least 2^-17 (relative) away from
    // one, so y * rcp(r) (2 ulp of f32) rounds to the same bf16 as the exact division.
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t r2 = bmax2(x[j], 0u);
      const uint32_t y2 = bmul2(r2, r2);
      const float q0 = bf_lo(y2) * rcp_approx(fmaxf(bf_lo(r2), 1e-30f)), q1 = bf_hi(y2) * rcp_approx(fmaxf(bf_hi(r2), 1e-30f));
      const uint32_t t2 = bmul2(pack2(q0, q1), 0x40004000u);           // 2 * q
      w[j] = bmul2(w[j], t2);                                           // the power VJP's output: an edge, checked below
    }
  } else if (p.epi == EPI_DGELU) {
    // backward of the tanh GELU: bf16(da * gelu'(u)), the derivative evaluated once in f32
#pragma unroll
    for (int j = 0; j < 16; ++j)
      w[j] = pack2(bf_lo(w[j]) * gelu_grad<__nv_bfloat16>(bf_lo(x[j])), bf_hi(w[j]) * gelu_grad<__nv_bfloat16>(bf_hi(x[j])));
  }
  if (p.epi == EPI_DRELU2 || p.epi == EPI_DGELU) {               // the activation VJP's output edge
    uint32_t mx2 = 0u;
#pragma unroll
    for (int j = 0; j < 16; ++j) adj_track2(mx2, w[j]);
    if (adj_over2(mx2)) {
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] = adj_edge2(w[j]);
    }
  }
  if (p.wide) {
    st_global_256(C, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
    st_global_256(C + 16, make_uint4(w[8], w[9], w[10], w[11]), make_uint4(w[12], w[13], w[14], w[15]));
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(C)[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
  }
  if (p.epi == EPI_RELU2 || p.epi == EPI_RELU || p.epi == EPI_GELU) {
    // second output: max(u, 0), its square, or the tanh GELU, from u as stored
    __nv_bfloat16* C2 = (__nv_bfloat16*)p.C2 + o;
    if (p.epi == EPI_GELU) {
      // the nine bf16 ops of the exported activation, two elements at a time; tanh in f32, rounded once
      const uint32_t c1 = pack2(PCPB_GELU_C1, PCPB_GELU_C1), c2 = pack2(PCPB_GELU_C2, PCPB_GELU_C2);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t u = w[j];
        const uint32_t z = bmul2(c1, badd2(u, bmul2(c2, bmul2(bmul2(u, u), u))));
        const uint32_t t = pack2(tanhf(bf_lo(z)), tanhf(bf_hi(z)));
        w[j] = bmul2(bmul2(0x3F003F00u, u), badd2(t, 0x3F803F80u));     // (0.5 * u) * (t + 1)
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t r2 = bmax2(w[j], 0u);
        w[j] = (p.epi == EPI_RELU2) ? bmul2(r2, r2) : r2;
      }
    }
    if (p.wide) {
      st_global_256(C2, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]));
      st_global_256(C2 + 16, make_uint4(w[8], w[9], w[10], w[11]), make_uint4(w[12], w[13], w[14], w[15]));
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) reinterpret_cast<uint4*>(C2)[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
  }
}

// Output tile of a work item.  Tiles are numbered so that tiles running at the same time share operands in L2: when
// there are many column tiles (the LM head: every row tile would otherwise stream the whole weight matrix through
// L2), groups of row tiles walk the columns together; otherwise columns vary fastest.
__device__ __forceinline__ void tile_coords(const TcParams& p, int tile, int* tm, int* tn) {
  if (p.group_m <= 1) { *tm = tile / p.tiles_n; *tn = tile % p.tiles_n; return; }
  const int per_group = p.group_m * p.tiles_n;
  const int g = tile / per_group, rem = tile % per_group;
  const int gm = min(p.group_m, p.tiles_m - g * p.group_m);       // the last group may be short
  *tm = g * p.group_m + rem % gm;
  *tn = rem / gm;
}

template <int BN> struct TcCfg {
  static constexpr int B_TILE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int NSTAGE = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const TcParams p) {
  using Cfg = TcCfg<BN>;
  constexpr int NSTAGE = Cfg::NSTAGE;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;          // 1024 B alignment for the swizzle atoms
  const uint32_t bar_base = base + NSTAGE * Cfg::STAGE_BYTES;
  // barrier layout (8 B each): full[NSTAGE], empty[NSTAGE], tmem_full[2], tmem_empty[2], then the tmem address
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * NSTAGE + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * NSTAGE + 4);
  uint8_t* smem_gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + NSTAGE * Cfg::STAGE_BYTES + 8 * (2 * NSTAGE + 4));

  const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
  const int total_items = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), N_EPI); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // All 32 lanes run the loop, so its addresses and coordinates are warp-uniform values; one elected lane issues.
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      const int tile = item / p.splits, split = item % p.splits;
      int tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const int m0 = tm * BM, n0 = tn * BN;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = min(kb0 + p.kb_per_split, p.K / BK);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % NSTAGE;
        const uint32_t ph = (it / NSTAGE) & 1u;
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1u, p.err, 1)))) break;
        mbar_expect_tx_elect(full_bar(s), Cfg::STAGE_BYTES);
        const uint32_t sa = base + s * Cfg::STAGE_BYTES, sb = sa + A_TILE_BYTES;
        const int k0 = kb * BK;
        if (!A_MN) tma_load_2d_elect(sa, &tma_a, full_bar(s), k0, m0);
        else {
#pragma unroll
          for (int c = 0; c < BM / 64; ++c) tma_load_2d_elect(sa + c * 8192, &tma_a, full_bar(s), m0 + c * 64, k0);
        }
        if (!B_MN) tma_load_2d_elect(sb, &tma_b, full_bar(s), k0, n0);
        else {
#pragma unroll
          for (int c = 0; c < BN / 64; ++c) tma_load_2d_elect(sb + c * 8192, &tma_b, full_bar(s), n0 + c * 64, k0);
        }
      }
    }
    if (!ok) {
      // error path: `it` loads were armed; let the ones still in flight land before the CTA goes away (bounded)
      for (uint32_t j = (it > (uint32_t)NSTAGE ? it - NSTAGE : 0u); j < it; ++j) {
        const uint32_t ph = (j / NSTAGE) & 1u;
        for (uint32_t w = 0; w < (1u << 20); ++w) if (mbar_try(full_bar(j % NSTAGE), ph)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the loops and the waits; one elected lane issues the MMAs and the commits.
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                               ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    constexpr uint32_t A_LBO = A_MN ? 8192u : 16u, B_LBO = B_MN ? 8192u : 16u;
    constexpr uint32_t A_KSTEP = A_MN ? 2048u : 32u, B_KSTEP = B_MN ? 2048u : 32u;
    uint32_t it = 0;
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++local) {
      const int split = item % p.splits;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = min(kb0 + p.kb_per_split, p.K / BK);
      const int acc = local & 1;
      const uint32_t aph = ((uint32_t)local >> 1) & 1u;
      if (!(ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(acc), aph ^ 1u, p.err, 2)))) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % NSTAGE;
        const uint32_t ph = (it / NSTAGE) & 1u;
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.err, 3)))) break;
        tc_fence_after();
        const uint32_t sa = base + s * Cfg::STAGE_BYTES, sb = sa + A_TILE_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t da = make_desc(sa + k * A_KSTEP, A_LBO, 1024u);
          const uint64_t db = make_desc(sb + k * B_KSTEP, B_LBO, 1024u);
          mma_bf16_elect(tmem_d, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        mma_commit_elect(empty_bar(s));               // frees the stage when these MMAs have read it
      }
      if (ok) mma_commit_elect(tfull_bar(acc));       // accumulator complete
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // Eight warps: two per tensor-memory lane quarter, each with one half of the BN accumulator columns; a thread owns
    // one output row.  The per-element operand of the epilogue (residual or pre-activation) does not depend on the
    // accumulator, so it is fetched before the wait and its latency is spent under the MMAs of the tile.
    constexpr int NCH = BN / 64;                    // 32-column chunks per warp
    const int q = warp & 3, half = (warp - 2) >> 2;
    const bool reads_r = (p.splits == 1) && (p.epi == EPI_RESID || p.epi == EPI_DRELU2 || p.epi == EPI_DRELU || p.epi == EPI_DGELU);
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++local) {
      const int tile = item / p.splits, split = item % p.splits;
      int tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const int m0 = tm * BM, n0 = tn * BN + half * (BN / 2);
      const int acc = local & 1;
      const uint32_t aph = ((uint32_t)local >> 1) & 1u;
      const int row = m0 + q * 32 + lane;
      uint4 rpre[NCH * 4];
      if (reads_r) {
        const uint4* rp = reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.R + (size_t)row * p.ldc + n0);
        if (p.wide) {
#pragma unroll
          for (int i = 0; i < NCH * 2; ++i) ld_global_256(rp + 2 * i, rpre[2 * i], rpre[2 * i + 1]);
        } else {
#pragma unroll
          for (int i = 0; i < NCH * 4; ++i) rpre[i] = __ldg(rp + i);
        }
      }
      ok = mbar_wait(tfull_bar(acc), aph, p.err, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      TcParams pe = p;
      if (p.splits > 1) { pe.epi = -1; pe.slab = p.slab + (size_t)split * p.M * p.N; pe.ldc = p.N; }
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * (BN / 2) + c * 32), r);
        epilogue_chunk(pe, row, n0 + c * 32, r, rpre + c * 4);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
  }
}

// =====================================================================================================
// Two-CTA variant: a cluster of two CTAs (one SM each) computes a 256 x 256 tile with tcgen05.mma.cta_group::2.
// CTA r of the pair holds rows [128r, 128r+128) of the A tile, rows [128r, 128r+128) of the B tile (its half of
// the N columns) and the accumulators of its 128 output rows, so every operand byte is loaded once per pair and
// each SM reads half as much shared memory per FLOP as in the one-CTA kernel.
//   warp 0 (both CTAs)   TMA producer for its own halves; the bytes of both CTAs are counted on CTA 0's full barrier
//   warp 1, CTA 0        waits for a full stage, issues the MMAs for the pair; the commit arrives on the empty /
//                        accumulator-full barriers of both CTAs
//   warps 2..9 (both)    epilogue of the CTA's 128 rows; release the accumulator on CTA 0's barrier
// =====================================================================================================
constexpr int NSTAGE2 = 6;
constexpr int STAGE2_BYTES = 2 * A_TILE_BYTES;                  // A half + B half: 32 KB
constexpr int SMEM2_BYTES = NSTAGE2 * STAGE2_BYTES + 1024 + 256;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_gemm_tc2(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const TcParams p) {
  constexpr int BN = 256, NSTAGE = NSTAGE2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = base + NSTAGE * STAGE2_BYTES;
  // barriers (8 B each): full[NSTAGE] (used in CTA 0), empty[NSTAGE], tmem_full[2], tmem_empty[2] (CTA 0), tmem address
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (2 * NSTAGE + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (3 * NSTAGE + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (3 * NSTAGE + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (3 * NSTAGE + 4);
  uint8_t* smem_gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + NSTAGE * STAGE2_BYTES + 8 * (3 * NSTAGE + 4));

  const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                      // 0 = leader
  const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;
  const int total_items = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 2 * N_EPI); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();                                           // barriers of both CTAs initialised, tensor memory allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ------------------------------ TMA producer (own halves) ------------------------------
    uint32_t it = 0;
    bool ok = true;
    const uint32_t full0 = map_to_cta(full_bar(0), 0);          // CTA 0's full barriers, cluster address
    for (int item = cluster_id; item < total_items && ok; item += n_clusters) {
      const int tile = item / p.splits, split = item % p.splits;
      int tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const int m0 = tm * 256 + (int)rank * 128, n0 = tn * BN + (int)rank * 128;
      const int kb0 = split * p.kb_per_split;
      const int kb1 = min(kb0 + p.kb_per_split, p.K / BK);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % NSTAGE;
        const uint32_t ph = (it / NSTAGE) & 1u;
        if (!(ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1u, p.err, 1)))) break;
        // CTA 0 arms its barrier with the bytes of both CTAs; CTA 1's copies count on it as well (its own stage is
        // free: the commit that freed it came after CTA 0's barrier had completed the previous use of this stage)
        if (rank == 0) mbar_expect_tx_elect(full_bar(s), 2 * STAGE2_BYTES);
        const uint32_t fb = full0 + 8u * s;
        const uint32_t sa = base + s * STAGE2_BYTES, sb = sa + A_TILE_BYTES;
        const int k0 = kb * BK;
        if (!A_MN) tma_load_2d_pair_elect(sa, &tma_a, fb, k0, m0);
        else {
          tma_load_2d_pair_elect(sa, &tma_a, fb, m0, k0);
          tma_load_2d_pair_elect(sa + 8192, &tma_a, fb, m0 + 64, k0);
        }
        if (!B_MN) tma_load_2d_pair_elect(sb, &tma_b, fb, k0, n0);
        else {
          tma_load_2d_pair_elect(sb, &tma_b, fb, n0, k0);
          tma_load_2d_pair_elect(sb + 8192, &tma_b, fb, n0 + 64, k0);
        }
      }
    }
    if (!ok && rank == 0) {
      // error path: let the copies already issued (by both CTAs) land before the pair goes away (bounded)
      for (uint32_t j = (it > (uint32_t)NSTAGE ? it - NSTAGE : 0u); j < it; ++j) {
        const uint32_t ph = (j / NSTAGE) & 1u;
        for (uint32_t w = 0; w < (1u << 20); ++w) if (mbar_try(full_bar(j % NSTAGE), ph)) break;
      }
    }
  } else if (warp == 1) {
    uint32_t it = 0;
    int local = 0;
    bool ok = true;
    if (rank != 0) {
      // CTA 1 has no MMA work: CTA 0 issues for the pair
    } else {
      // ------------------------------ CTA 0: MMA issuer for the pair ------------------------------
      constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                 ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
      constexpr uint32_t A_LBO = A_MN ? 8192u : 16u, B_LBO = B_MN ? 8192u : 16u;
      constexpr uint32_t A_KSTEP = A_MN ? 2048u : 32u, B_KSTEP = B_MN ? 2048u : 32u;
      for (int item = cluster_id; item < total_items && ok; item += n_clusters, ++local) {
        const int split = item % p.splits;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, p.K / BK);
        const int acc = local & 1;
        const uint32_t aph = ((uint32_t)local >> 1) & 1u;
        if (!(ok = __all_sync(0xffffffffu, mbar_wait_cluster(tempty_bar(acc), aph ^ 1u, p.err, 2)))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1u;
          if (!(ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, p.err, 3)))) break;
          tc_fence_after();
          const uint32_t sa = base + s * STAGE2_BYTES, sb = sa + A_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_desc(sa + k * A_KSTEP, A_LBO, 1024u);
            const uint64_t db = make_desc(sb + k * B_KSTEP, B_LBO, 1024u);
            mma2_bf16_elect(tmem_d, da, db, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          mma2_commit_multicast_elect(empty_bar(s), 3);         // frees the stage in both CTAs
        }
        if (ok) mma2_commit_multicast_elect(tfull_bar(acc), 3); // accumulators of both CTAs complete
      }
    }
  } else {
    // ------------------------------ epilogue of this CTA's 128 rows ------------------------------
    constexpr int NCH = BN / 64;
    const int q = warp & 3, half = (warp - 2) >> 2;
    const bool reads_r = (p.splits == 1) && (p.epi == EPI_RESID || p.epi == EPI_DRELU2 || p.epi == EPI_DRELU || p.epi == EPI_DGELU);
    const uint32_t tempty_leader = map_to_cta(tempty_bar(0), 0);  // tempty_bar(a) of CTA 0 = this + 8a
    int local = 0;
    bool ok = true;
    for (int item = cluster_id; item < total_items && ok; item += n_clusters, ++local) {
      const int tile = item / p.splits, split = item % p.splits;
      int tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const int m0 = tm * 256 + (int)rank * 128, n0 = tn * BN + half * (BN / 2);
      const int acc = local & 1;
      const uint32_t aph = ((uint32_t)local >> 1) & 1u;
      const int row = m0 + q * 32 + lane;
      uint4 rpre[NCH * 4];
      if (reads_r) {
        const uint4* rp = reinterpret_cast<const uint4*>((const __nv_bfloat16*)p.R + (size_t)row * p.ldc + n0);
        if (p.wide) {
#pragma unroll
          for (int i = 0; i < NCH * 2; ++i) ld_global_256(rp + 2 * i, rpre[2 * i], rpre[2 * i + 1]);
        } else {
#pragma unroll
          for (int i = 0; i < NCH * 4; ++i) rpre[i] = __ldg(rp + i);
        }
      }
      ok = mbar_wait(tfull_bar(acc), aph, p.err, 4);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      TcParams pe = p;
      if (p.splits > 1) { pe.epi = -1; pe.slab = p.slab + (size_t)split * p.M * p.N; pe.ldc = p.N; }
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * (BN / 2) + c * 32), r);
        epilogue_chunk(pe, row, n0 + c * 32, r, rpre + c * 4);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + 8u * acc);
    }
  }
  tc_fence_before();
  cluster_sync_all();                                           // nobody may still be signalling this CTA's barriers
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Sum of the split-K slabs in split order, then the weight-gradient epilogue.
__global__ void k_splitk_reduce(const float* __restrict__ slab, int splits, size_t mn, int N, float* __restrict__ C,
                                long long ldc, int epi, float clip) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < mn; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += slab[(size_t)s * mn + i];
    if (epi == EPI_WGRAD) {
      float v = bf16_round(acc);
      if (!((v - v) == 0.f)) v = 0.f;
      acc = fminf(fmaxf(v, -clip), clip);
    }
    C[(i / N) * ldc + (i % N)] = acc;
  }
}

struct Plan {
  bool ok = false;
  bool pair = false;            // two-CTA kernel (256 x 256 tiles)
  bool a_mn = false, b_mn = false;
  long long lda = 0, ldb = 0;
  int bn = 0, splits = 1, kb_per_split = 0;
};

int g_sm_count = 0;

// Split-K factor of a weight-gradient GEMM with few output tiles: the one (1..8, at least 8 k-blocks per split) whose
// tiles x splits work items fill whole rounds of 148 CTAs best; each extra split costs a little for its f32 slab.
// PCPB_GEMM_PAIR=0 keeps every GEMM on the one-CTA kernel.
bool pair_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("PCPB_GEMM_PAIR"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

// Longest contraction the two-CTA kernel is used for (PCPB_GEMM_PAIR_MAXK overrides).
int pair_max_k() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("PCPB_GEMM_PAIR_MAXK"); v = e ? atoi(e) : (1 << 30); if (v <= 0) v = 1 << 30; }
  return v;
}

int pick_splits(int tiles, int kblocks, int slots = 148) {
  if (tiles >= 2 * slots) return 1;
  int best = 1;
  double best_score = -1.0;
  for (int s = 1; s <= 8; ++s) {
    if (s > 1 && kblocks / s < 8) break;
    const int items = tiles * s, rounds = (items + slots - 1) / slots;
    const double score = (double)items / ((double)rounds * slots) - 0.01 * s;
    if (score > best_score) { best_score = score; best = s; }
  }
  return best;
}

Plan plan_for(const GemmArgs& g) {
  Plan pl;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return pl;
  if (g.M % BM || g.K % BK || g.N % 128) return pl;
  if (g.sak == 1 && g.sam >= g.K) { pl.a_mn = false; pl.lda = g.sam; }
  else if (g.sam == 1 && g.sak >= g.M) { pl.a_mn = true; pl.lda = g.sak; }
  else return pl;
  if (g.sbk == 1 && g.sbn >= g.K) { pl.b_mn = false; pl.ldb = g.sbn; }
  else if (g.sbn == 1 && g.sbk >= g.N) { pl.b_mn = true; pl.ldb = g.sbk; }
  else return pl;
  if (pl.a_mn && !pl.b_mn) return pl;                            // combination not instantiated
  if (pl.lda % 8 || pl.ldb % 8 || g.ldc % 8) return pl;
  if (((uintptr_t)g.A | (uintptr_t)g.B | (uintptr_t)g.C) & 15) return pl;
  if (g.R && ((uintptr_t)g.R & 15)) return pl;
  if (g.C2 && ((uintptr_t)g.C2 & 15)) return pl;
  if (g.epi < EPI_STORE || g.epi > EPI_RAWF32) return pl;
  pl.bn = (g.N % 256 == 0) ? 256 : 128;
  pl.pair = pair_enabled() && g.M % 256 == 0 && g.N % 256 == 0 && g.K <= pair_max_k();
  const int tiles = (g.M / (pl.pair ? 256 : BM)) * (g.N / pl.bn), kblocks = g.K / BK;
  pl.splits = (g.epi == EPI_WGRAD || g.epi == EPI_RAWF32) ? pick_splits(tiles, kblocks, pl.pair ? 74 : 148) : 1;
  // the f32 slabs must fit the caller's scratch
  while (pl.splits > 1 && (size_t)pl.splits * g.M * g.N * sizeof(float) > g.scratch_bytes) --pl.splits;
  pl.kb_per_split = (kblocks + pl.splits - 1) / pl.splits;
  pl.splits = (kblocks + pl.kb_per_split - 1) / pl.kb_per_split;
  pl.ok = true;
  return pl;
}

template <int BN, bool A_MN, bool B_MN>
cudaError_t launch_variant(cudaStream_t st, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int grid) {
  auto kern = k_gemm_tc<BN, A_MN, B_MN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<BN>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  kern<<<grid, GEMM_THREADS, TcCfg<BN>::SMEM_BYTES, st>>>(ma, mb, p);
  return cudaGetLastError();
}

template <bool A_MN, bool B_MN>
cudaError_t launch_pair(cudaStream_t st, const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p, int items) {
  auto kern = k_gemm_tc2<A_MN, B_MN>;
  static bool attr_set[64] = {};
  static int max_clusters[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = SMEM2_BYTES; cfg.stream = st; cfg.attrs = at; cfg.numAttrs = 1;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
    if (e != cudaSuccess) return e;
    cfg.gridDim = dim3(2 * 74);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) return e;
    if (n < 1) return cudaErrorInvalidConfiguration;
    max_clusters[dev] = n < 74 ? n : 74;
    attr_set[dev] = true;
  }
  const int clusters = items < max_clusters[dev] ? items : max_clusters[dev];
  cfg.gridDim = dim3(2 * clusters);
  return cudaLaunchKernelEx(&cfg, kern, ma, mb, p);
}

}  // namespace

bool gemm_tc_supported(const GemmArgs& g) { return g.err_word != nullptr && plan_for(g).ok && encode_fn() != nullptr; }
int gemm_tc_launches(const GemmArgs& g) { return plan_for(g).splits > 1 ? 2 : 1; }

size_t gemm_tc_scratch_wanted(int M, int N, int K) {
  if (M % BM || N % 128 || K % BK) return 0;
  const int bn = (N % 256 == 0) ? 256 : 128;
  const int tiles = (M / BM) * (N / bn), kblocks = K / BK;
  int s = pick_splits(tiles, kblocks);
  if (M % 256 == 0 && N % 256 == 0) { const int s2 = pick_splits((M / 256) * (N / 256), kblocks, 74); if (s2 > s) s = s2; }
  return s > 1 ? (size_t)s * M * N * sizeof(float) : 0;
}

cudaError_t launch_gemm_tc(cudaStream_t st, const GemmArgs& g) {
  const Plan pl = plan_for(g);
  if (!pl.ok) return cudaErrorInvalidValue;
  if (!g_sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  int* err = g.err_word;
  if (!err) return cudaErrorInvalidValue;
  cudaError_t e = cudaSuccess;
  CUtensorMap ma, mb;
  bool ok;
  if (!pl.a_mn) ok = make_map(&ma, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)pl.lda, BM);
  else ok = make_map(&ma, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)pl.lda, 64);
  if (!pl.b_mn) ok = ok && make_map(&mb, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)pl.ldb, pl.pair ? 128u : (uint32_t)pl.bn);
  else ok = ok && make_map(&mb, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)pl.ldb, 64);
  if (!ok) return cudaErrorInvalidValue;
  TcParams p;
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.tiles_m = g.M / (pl.pair ? 256 : BM); p.tiles_n = g.N / pl.bn; p.splits = pl.splits; p.kb_per_split = pl.kb_per_split;
  {
    // Row tiles that walk the columns together (LM-head forward).  Every group streams the whole weight matrix, which
    // does not stay in L2 next to the output stream, so DRAM reads are about (row tiles / group) x |W|; the group's rows
    // of A must stay in L2 (group x 0.65 MB at K = 1280).  Measured at 32768 x 65536 x 1280 (128 row tiles): 8 -> 4.8 GB
    // read, 3.85 ms; 32 -> 1.5 GB, 3.62 ms; 64 -> 2.9 GB, 3.73 ms.  PCPB_GEMM_GROUP_M overrides it for such comparisons.
    static int group_env = -1;
    if (group_env < 0) { const char* e = getenv("PCPB_GEMM_GROUP_M"); group_env = e ? atoi(e) : 0; }
    p.group_m = (p.tiles_n >= 32 && p.splits == 1) ? (group_env > 0 ? group_env : 32) : 1;
  }
  {
    // 256-bit epilogue accesses need every row segment to start on a 32-byte boundary (16 bf16 / 8 f32 elements)
    const uintptr_t all = (uintptr_t)g.C | (uintptr_t)g.R | (uintptr_t)g.C2 | (uintptr_t)g.scratch;
    p.wide = ((all & 31) == 0 && g.ldc % 16 == 0 && g.N % 16 == 0) ? 1 : 0;
  }
  p.epi = g.epi; p.C = g.C; p.ldc = g.ldc; p.R = g.R; p.C2 = g.C2; p.clip = g.clip; p.adj = g.adj; p.slab = nullptr; p.err = err;
  if (pl.splits > 1) p.slab = (float*)g.scratch;
  else if (g.epi == EPI_RAWF32) { p.epi = -1; p.slab = (float*)g.C; }     // the accumulators as they are, like a split-K slab
  const int items = p.tiles_m * p.tiles_n * p.splits;
  const int grid = items < g_sm_count ? items : g_sm_count;
  if (pl.pair) {
    if (!pl.a_mn && !pl.b_mn) e = launch_pair<false, false>(st, ma, mb, p, items);
    else if (!pl.a_mn && pl.b_mn) e = launch_pair<false, true>(st, ma, mb, p, items);
    else e = launch_pair<true, true>(st, ma, mb, p, items);
  } else if (pl.bn == 256) {
    if (!pl.a_mn && !pl.b_mn) e = launch_variant<256, false, false>(st, ma, mb, p, grid);
    else if (!pl.a_mn && pl.b_mn) e = launch_variant<256, false, true>(st, ma, mb, p, grid);
    else e = launch_variant<256, true, true>(st, ma, mb, p, grid);
  } else {
    if (!pl.a_mn && !pl.b_mn) e = launch_variant<128, false, false>(st, ma, mb, p, grid);
    else if (!pl.a_mn && pl.b_mn) e = launch_variant<128, false, true>(st, ma, mb, p, grid);
    else e = launch_variant<128, true, true>(st, ma, mb, p, grid);
  }
  if (e != cudaSuccess) return e;
  if (pl.splits > 1) {
    const size_t mn = (size_t)g.M * g.N;
    unsigned blocks = (unsigned)((mn + 255) / 256);
    if (blocks > 148u * 16) blocks = 148u * 16;
    k_splitk_reduce<<<blocks, 256, 0, st>>>((const float*)g.scratch, pl.splits, mn, g.N, (float*)g.C, g.ldc, g.epi, g.clip);
    e = cudaGetLastError();
  }
  return e;
}

cudaError_t adj_status_fetch_gemm_tc(cudaStream_t st, int* out, bool clear) { return adj_status_fetch_tu(st, out, clear); }

}  // namespace pcpb
