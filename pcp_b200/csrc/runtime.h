// Backend object behind the C ABI: buffers, artefact, workspace, training step, worker round, outer step.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <string>
#include <vector>

#include "graph_exec.h"
#include "kernels.h"
#include "model.h"

struct pcpb_backend;

namespace pcpb {

struct Block {                     // one device allocation, shared by the buffers that view it
  void* ptr = nullptr;
  size_t bytes = 0;
  std::atomic<int> refs{1};
  int device = 0;
};

struct LayerActs {                 // saved forward values of one transformer layer (model dtype unless noted)
  void *h1, *qkv, *qkn, *o, *xmid, *h2, *u, *a;
  float *t1, *t2, *tq, *mrow, *lrow;
  float *mu1 = nullptr, *mu2 = nullptr;          // nanoGPT: LayerNorm means (f32)
  double *m64_1 = nullptr, *m64_2 = nullptr;     // nanoGPT: LayerNorm means of the f64 variance branch
};

struct Workspace {
  bool ready = false;
  std::vector<void*> allocs;       // everything cudaMalloc'ed for this artefact
  // flat parameter-sized buffers (argument order)
  float *theta = nullptr, *theta0 = nullptr, *mstate = nullptr, *vstate = nullptr, *grads = nullptr,
        *gacc = nullptr, *delta = nullptr;
  void* shadow = nullptr;          // model-dtype copy of theta (== theta for f32 models)
  // activations
  std::vector<void*> xs;           // L+1 residual streams [M,d]
  std::vector<LayerActs> layers;
  float *t0 = nullptr, *tf = nullptr, *rowloss = nullptr, *count = nullptr, *loss = nullptr;
  void *hf = nullptr, *logits = nullptr;
  // backward temporaries
  void *dx = nullptr, *dh = nullptr, *du = nullptr, *dout = nullptr, *dqkn = nullptr, *dqkv = nullptr;
  float* dkv_acc = nullptr;
  float* drow = nullptr;           // [B*H*T] attention-backward row scratch, followed by [B*H*T] float4 row records
  float *muf = nullptr, *ln_partial = nullptr, *cs_partial = nullptr;   // nanoGPT: final LN mean, reduction scratch
  double* m64f = nullptr;
  // data
  long long *ids = nullptr, *targets = nullptr;
  uint16_t *d_cos = nullptr, *d_sin = nullptr;
  // optimiser tables for the flat layout
  TensorSeg* segs = nullptr; int* chunk2seg = nullptr; float* partial = nullptr; float* normsq = nullptr;
  int nchunks = 0;
  int* heal_flags = nullptr;
  void* tc_scratch = nullptr; size_t tc_scratch_bytes = 0; int* tc_err = nullptr;
  // f32 models on the tensor cores: operands split into three bf16 pieces and packed [rows, 6 K] (launch_split3_pack),
  // the f32 result before its epilogue
  void* emb_scratch = nullptr; size_t emb_scratch_bytes = 0;   // sorted embedding-gradient scatter (keys, positions, partials)
  void *pk_a = nullptr, *pk_b = nullptr; float* pk_c = nullptr;
  size_t pk_ab_bytes = 0, pk_c_bytes = 0;
  float* loss_record = nullptr;    // device, one per inner step of a round
  int loss_capacity = 0;
};

}  // namespace pcpb

struct pcpb_buffer {
  pcpb_backend* owner;
  pcpb::Block* block;
  void* ptr;
  size_t nbytes;
  std::vector<int64_t> shape;
  int dtype;
  std::atomic<int> refs{1};
};

struct pcpb_backend {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::string err;
  const void* art_ptr = nullptr;
  size_t art_len = 0;
  bool loaded = false;
  pcpb::ModelConfig cfg;
  pcpb::Graph graph;                         // FAMILY_GRAPH: the tensor program of the artefact (forward + gradients)
  pcpb::GraphExec* gx = nullptr;             // ... and its planned executor
  pcpb::Workspace ws;
  pcpb::AdamHyper adam;
  long long launches = 0;
  bool force_generic = false;
  int attn_path = 0;                         // 0 auto (tcgen05, else mma.sync, else generic), 1 mma.sync, 2 generic
  // worker round state
  bool in_round = false;
  int tau = 0, accumulation_steps = 1, param_dtype = 0, persist_adam = 0, tokens_on_device = 0;
  float timestep = 1.f;
  int steps_done = 0;
  const uint16_t* tokens_src = nullptr;      // host or device pointer given by the caller
  size_t n_tokens = 0, cursor = 0;
  uint16_t* tokens_stage = nullptr;          // device staging for one step's window (host-token mode)
  size_t stage_cap = 0;
  bool have_master = false;                  // theta0 holds the master parameters of the next round
  int sampling = 0;                          // 0 FIFO, 1 random windows
  uint64_t prng_state[4] = {0, 0, 0, 0};     // generator of the random-window starts (pcpb_prng)
  unsigned long long* starts_dev = nullptr;  // device: one window start per batch row
  uint16_t* window_stage = nullptr;          // device staging of the gathered windows (host-token mode)
  size_t window_stage_cap = 0;
  std::vector<uint16_t> window_host;         // host gather buffer
  // outer step
  int rank = 0, world = 1;
  std::vector<float*> peer_delta, peer_theta0;
  std::vector<void*> ipc_opened;
  float *master_shard = nullptr, *velocity = nullptr;
  long long shard_len = 0;
  bool velocity_init = false;
  // streaming DiLoCo
  float* snapshot = nullptr;                 // last synchronised value of every parameter (f32, flat)
  int stream_fragments = 0;
  cudaStream_t side_stream = nullptr;            // fragment outer steps that run under the following training steps
  std::vector<cudaEvent_t> frag_ev;              // [2 * fragment + {0: start, 1: done}]
  std::vector<char> frag_pending;                // an outer step of the fragment was started and not yet waited for
  float stream_alpha = 0.5f, stream_lr = 0.7f, stream_mu = 0.9f;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr, tm0 = nullptr, tm1 = nullptr;
  // tensor-core GEMM profiling
  bool profiling = false;
  std::vector<cudaEvent_t> prof_events;      // pairs
  size_t prof_used = 0;
  double prof_flops = 0.0, prof_ms = 0.0;
  long long prof_launches = 0;
};
