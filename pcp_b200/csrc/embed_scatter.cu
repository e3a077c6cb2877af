// Embedding gradient as a sort + segmented sum instead of floating-point atomics: the order in which the rows of one
// token are added is fixed, so f32 gradients are bit-identical from run to run.
//   1. key[m] = clamp(idx[m]) (the gather clamps its start indices), pos[m] = m
//   2. stable radix sort of the pairs by key (cub::DeviceRadixSort): positions stay ascending within a token
//   3. k_embed_chunk_sums: one block per 128 sorted entries adds the rows of every run of equal keys inside its chunk in
//      position order; a run that lies inside the chunk is written to dwte[key]; a run that crosses a chunk border
//      leaves a partial sum (P0: the run came in from the previous chunk; P1: it starts here and goes on)
//   4. k_embed_join_runs: for every run that crosses a border, the block of the chunk it starts in adds P1 and the P0 of
//      the following chunks in chunk order
// A token that fills a tenth of a 65536-token batch (Zipf) is spread over 50 blocks this way.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "kernels.h"

namespace pcpb {

namespace {

constexpr int CH = 128;                                         // sorted entries per block

__global__ void k_embed_keys(const long long* __restrict__ idx, int M, int V, int* __restrict__ key, int* __restrict__ pos) {
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  long long row = idx[m];
  row = row < 0 ? 0 : (row >= V ? V - 1 : row);
  key[m] = (int)row;
  pos[m] = m;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) k_embed_chunk_sums(const int* __restrict__ key, const int* __restrict__ pos, int M, int d,
                                                          const T* __restrict__ rows, float* __restrict__ dwte, float* __restrict__ P0,
                                                          float* __restrict__ P1) {
  __shared__ int sk[CH + 2], sp[CH];                            // keys of the chunk with one neighbour on either side
  const int c = blockIdx.x, s = c * CH, e = min(M, s + CH), n = e - s;
  for (int i = threadIdx.x; i < n; i += blockDim.x) { sk[i + 1] = key[s + i]; sp[i] = pos[s + i]; }
  if (threadIdx.x == 0) {
    sk[0] = s > 0 ? key[s - 1] : -1;
    sk[n + 1] = e < M ? key[e] : -1;
  }
  __syncthreads();
  if (VEC) {
    // 8 columns per thread, 16-byte loads (d a multiple of 8, rows 16-byte aligned)
    for (int j = threadIdx.x * 8; j < d; j += blockDim.x * 8) {
      int a = 0;
      while (a < n) {
        const int k = sk[a + 1];
        int b = a + 1;
        while (b < n && sk[b + 1] == k) ++b;                    // run [a, b): the same for every thread
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        int i = a;
        for (; i + 4 <= b; i += 4) {                            // four rows in flight; added in position order
          float x0[8], x1[8], x2[8], x3[8];
          ld8<T>(rows + (size_t)sp[i] * d + j, x0); ld8<T>(rows + (size_t)sp[i + 1] * d + j, x1);
          ld8<T>(rows + (size_t)sp[i + 2] * d + j, x2); ld8<T>(rows + (size_t)sp[i + 3] * d + j, x3);
#pragma unroll
          for (int q = 0; q < 8; ++q) { acc[q] += x0[q]; acc[q] += x1[q]; acc[q] += x2[q]; acc[q] += x3[q]; }
        }
        for (; i < b; ++i) {
          float x0[8];
          ld8<T>(rows + (size_t)sp[i] * d + j, x0);
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] += x0[q];
        }
        const bool from_before = (a == 0 && sk[0] == k), goes_on = (b == n && sk[n + 1] == k);
        float* dst = from_before ? P0 + (size_t)c * d + j : goes_on ? P1 + (size_t)c * d + j : dwte + (size_t)k * d + j;
        st8<float>(dst, acc);
        a = b;
      }
    }
    return;
  }
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    int a = 0;                                                  // first entry of the current run (chunk-relative)
    while (a < n) {
      const int k = sk[a + 1];
      int b = a + 1;
      while (b < n && sk[b + 1] == k) ++b;                      // run [a, b): the same for every thread
      float acc = 0.f;
      int i = a;
      for (; i + 4 <= b; i += 4) {                              // four rows in flight; added in position order
        const float x0 = to_f(rows[(size_t)sp[i] * d + j]), x1 = to_f(rows[(size_t)sp[i + 1] * d + j]);
        const float x2 = to_f(rows[(size_t)sp[i + 2] * d + j]), x3 = to_f(rows[(size_t)sp[i + 3] * d + j]);
        acc += x0; acc += x1; acc += x2; acc += x3;
      }
      for (; i < b; ++i) acc += to_f(rows[(size_t)sp[i] * d + j]);
      const bool from_before = (a == 0 && sk[0] == k), goes_on = (b == n && sk[n + 1] == k);
      if (from_before) P0[(size_t)c * d + j] = acc;
      else if (goes_on) P1[(size_t)c * d + j] = acc;
      else dwte[(size_t)k * d + j] = acc;
      a = b;
    }
  }
}

// One block per chunk whose last run starts in it and goes on into the next chunk.
__global__ void __launch_bounds__(256) k_embed_join_runs(const int* __restrict__ key, int M, int d, const float* __restrict__ P0,
                                                         const float* __restrict__ P1, float* __restrict__ dwte) {
  const int c = blockIdx.x, s = c * CH, e = min(M, s + CH);
  if (e >= M) return;
  const int k = key[e - 1];
  if (key[e] != k) return;                                      // the last run ends with the chunk
  if (key[s] == k && s > 0 && key[s - 1] == k) return;          // the whole chunk belongs to a run that started earlier
  int last = c + 1;                                             // chunks c + 1 .. last carry the rest of the run in P0
  while ((last + 1) * CH < M && key[(last + 1) * CH] == k) ++last;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float acc = P1[(size_t)c * d + j];
    for (int q = c + 1; q <= last; ++q) acc += P0[(size_t)q * d + j];     // chunk order
    dwte[(size_t)k * d + j] = acc;
  }
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

size_t sort_temp_bytes(int M) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr, M);
  return bytes;
}

}  // namespace

size_t embed_scatter_scratch_bytes(int M, int d) {
  if (M <= 0) return 0;
  const size_t chunks = (size_t)(M + CH - 1) / CH;
  return 4 * align256((size_t)M * sizeof(int)) + 2 * align256(chunks * d * sizeof(float)) + align256(sort_temp_bytes(M));
}

cudaError_t launch_embed_scatter_sorted(cudaStream_t st, int dt, const long long* idx, int M, int d, int V, const void* rows,
                                        void* scratch, size_t scratch_bytes, float* dwte) {
  if (M == 0) return cudaSuccess;
  if (!scratch || scratch_bytes < embed_scatter_scratch_bytes(M, d)) return cudaErrorInvalidValue;
  const size_t seg = align256((size_t)M * sizeof(int));
  const int chunks = (M + CH - 1) / CH;
  const size_t pseg = align256((size_t)chunks * d * sizeof(float));
  char* base = (char*)scratch;
  int* key_in = (int*)base; int* key_out = (int*)(base + seg); int* pos_in = (int*)(base + 2 * seg); int* pos_out = (int*)(base + 3 * seg);
  float* P0 = (float*)(base + 4 * seg); float* P1 = (float*)(base + 4 * seg + pseg);
  void* temp = base + 4 * seg + 2 * pseg;
  size_t temp_bytes = scratch_bytes - (4 * seg + 2 * pseg);
  k_embed_keys<<<(M + 255) / 256, 256, 0, st>>>(idx, M, V, key_in, pos_in);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  int bits = 1;
  while (bits < 31 && (1LL << bits) < (long long)V) ++bits;     // keys are below V
  e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, key_in, key_out, pos_in, pos_out, M, 0, bits, st);
  if (e != cudaSuccess) return e;
  const int threads = d >= 256 ? 256 : (d >= 128 ? 128 : 64);
  const bool vec = d % 8 == 0 && ((((uintptr_t)rows) | ((uintptr_t)dwte)) & 15) == 0;
  if (dt == DT_F32 && vec) k_embed_chunk_sums<float, true><<<chunks, threads, 0, st>>>(key_out, pos_out, M, d, (const float*)rows, dwte, P0, P1);
  else if (dt == DT_F32) k_embed_chunk_sums<float, false><<<chunks, threads, 0, st>>>(key_out, pos_out, M, d, (const float*)rows, dwte, P0, P1);
  else if (dt == DT_BF16 && vec) k_embed_chunk_sums<bf16, true><<<chunks, threads, 0, st>>>(key_out, pos_out, M, d, (const bf16*)rows, dwte, P0, P1);
  else if (dt == DT_BF16) k_embed_chunk_sums<bf16, false><<<chunks, threads, 0, st>>>(key_out, pos_out, M, d, (const bf16*)rows, dwte, P0, P1);
  else return cudaErrorInvalidValue;
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  k_embed_join_runs<<<chunks, threads, 0, st>>>(key_out, M, d, P0, P1, dwte);
  return cudaGetLastError();
}

}  // namespace pcpb
