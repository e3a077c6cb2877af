// AdamW step for callers that must not allocate device memory.
//
// The regular optimiser entry (pcpb_execute "apply_optimizer") allocates its output buffers and a small
// descriptor table on every call, and the fused worker path keeps its reduction scratch in a workspace
// obtained with cudaMalloc.  Some hosts cannot accept that: a runtime that hands this library slices of one
// arena it reserved up front and accounts for every byte (memory-planned runtimes work this way; the reference
// compiles its modules for one and even bounds the size of a single allocation at compile time with
// --iree-stream-resource-max-allocation-size, src/mlir/context.zig:238-239), or a service whose step loop
// forbids allocation calls because cudaMalloc / cudaFree synchronise the whole device.  For them
// pcpb_adamw_step_noalloc runs the same three AdamW kernels on caller-owned tensors with the per-chunk
// reduction scratch and the launch descriptors placed in a fixed array inside the library image.
//
// Limits and rules (also stated at the declaration in include/pcp_b200.h):
//   * at most PCPB_NOALLOC_MAX_ELEMS elements per call; larger tensors are refused with PCPB_E_TOO_LARGE;
//   * the array (about 64 KB) exists once per GPU that loads the library and lives until the process exits;
//   * every call uses the same array and finds the previous call's contents in it: the call rewrites the
//     descriptor and the chunk map and overwrites every partial sum it later reads, nothing else is assumed;
//   * two calls whose GPU work overlaps (different streams, different threads) race on the array: callers
//     serialise them;
//   * the first call on each device looks up the device address of the array (cudaGetSymbolAddress).  Make
//     that first call before starting any stream capture.
#include <math.h>
#include <stdio.h>

#include <mutex>

#include "../../include/pcp_b200.h"
#include "common.cuh"
#include "kernels.h"

using namespace pcpb;

namespace {

constexpr long long MAX_ELEMS = PCPB_NOALLOC_MAX_ELEMS;
constexpr int MAX_CHUNKS = (int)(MAX_ELEMS / ADAM_CHUNK);

// layout of the static scratch
struct NoAllocScratch {
  TensorSeg seg;                 // descriptor of the one tensor of this call
  float normsq[16];              // [0] used
  int chunk2seg[MAX_CHUNKS];     // all zero: every chunk belongs to segment 0
  float partial[MAX_CHUNKS];     // per-chunk sums of squares
};

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

__global__ void k_noalloc_setup(NoAllocScratch* s, TensorSeg seg, int nchunks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) { s->seg = seg; s->normsq[0] = 0.f; }
  if (i < nchunks) s->chunk2seg[i] = 0;
}

std::mutex g_mu;
NoAllocScratch* g_dev_ptr[64] = {};

int set_err(char* err, size_t cap, int code, const char* msg) {
  if (err && cap) snprintf(err, cap, "%s", msg);
  return code;
}

}  // namespace

extern "C" int pcpb_adamw_step_noalloc(void* stream, const float* p, const float* g, const float* m, const float* v,
                                       float* p_out, float* m_out, float* v_out, long long n,
                                       const pcpb_adam_conf* conf, float timestep, char* err, size_t err_cap) {
  if (err && err_cap) err[0] = 0;
  if (!p || !g || !m || !v || !p_out || !m_out || !v_out || !conf) return set_err(err, err_cap, PCPB_E_INVALID, "null argument");
  if (n < 0) return set_err(err, err_cap, PCPB_E_INVALID, "negative element count");
  if (n > MAX_ELEMS) {
    char msg[160];
    snprintf(msg, sizeof msg, "tensor of %lld elements exceeds the fixed scratch of pcpb_adamw_step_noalloc (max %lld)", n,
             (long long)MAX_ELEMS);
    return set_err(err, err_cap, PCPB_E_TOO_LARGE, msg);
  }
  if (n == 0) return PCPB_OK;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return set_err(err, err_cap, PCPB_E_CUDA, "no current CUDA device");
  NoAllocScratch* s = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_dev_ptr[dev]) {
      // one-time set-up for this device (it is the current one): device address of the static array
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess || !ptr) {
        char msg[200];
        snprintf(msg, sizeof msg, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        return set_err(err, err_cap, PCPB_E_CUDA, msg);
      }
      g_dev_ptr[dev] = (NoAllocScratch*)ptr;
    }
    s = g_dev_ptr[dev];
  }
  cudaStream_t st = (cudaStream_t)stream;
  TensorSeg seg;
  seg.p = p; seg.g = g; seg.m = m; seg.v = v; seg.p_out = p_out; seg.m_out = m_out; seg.v_out = v_out;
  seg.shadow = nullptr; seg.n = n; seg.first_chunk = 0;
  seg.num_chunks = (int)((n + ADAM_CHUNK - 1) / ADAM_CHUNK);
  k_noalloc_setup<<<(seg.num_chunks + 255) / 256, 256, 0, st>>>(s, seg, seg.num_chunks);
  e = cudaGetLastError();
  if (e == cudaSuccess) {
    AdamHyper h;
    h.lr = conf->learning_rate; h.beta1 = conf->beta1; h.beta2 = conf->beta2; h.eps = conf->epsilon;
    h.wd = conf->weight_decay; h.max_norm = conf->max_grad_norm;
    h.m_corr = fmaxf(1.f - powf(h.beta1, timestep), h.eps);
    h.v_corr = fmaxf(1.f - powf(h.beta2, timestep), h.eps);
    e = launch_adamw(st, -1, &s->seg, 1, s->chunk2seg, seg.num_chunks, s->partial, s->normsq, h);
  }
  if (e != cudaSuccess) {
    char msg[200];
    snprintf(msg, sizeof msg, "launch failed: %s", cudaGetErrorString(e));
    return set_err(err, err_cap, PCPB_E_CUDA, msg);
  }
  return PCPB_OK;
}
